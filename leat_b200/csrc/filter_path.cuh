// The filter path: how large batches reach the memory roofline.  Included inside namespace leat by
// sampler_kernels.cuh.
//
// Three launches instead of one fused kernel doing everything per block:
//
//   filter_kernel       streams every logit exactly once with 128-bit loads and nothing else to do
//                       than compare it with its row's floor; the few hundred logits per row at or
//                       above it are appended, as (logit, index) pairs, to the row's list in the
//                       workspace.  The floor is a raw logit above which, with overwhelming
//                       probability, at least top_k logits of the row lie, and not many more: a low
//                       order statistic of the maxima of a spread-out sample of the row (256 chunks
//                       of 128 bytes in 64 pieces of 512, 32 KB), which every block works out for
//                       itself when it comes to a new row (the sample's lines are the row's own, so
//                       the stream finds them in L2).
//   finish_list_kernel  (finish_list.cuh) one small block per row finishes the row from its list.
//   sample_kernel       takes the rows the list finish does not (rows without a list stream their
//                       logits here) and leaves at once when there are none.
//
// The floor is only a guess, so the finish checks it: the result stands if at least top_k
// candidates score strictly above the floor's score and the cut lies strictly above it too (then no
// logit the filter dropped could have been a survivor or changed the cut); greedy rows need their
// best candidate at or above the floor.  A row that fails the check is redone by the exact
// multi-pass routine.
#pragma once

constexpr int SAMPLE_CHUNKS = 256;   // chunks of the sample, one per thread of floor_kernel
constexpr int SAMPLE_SIDE_BY_SIDE_ROWS = 128;  // batches from here on load the sample a line per instruction (measured: 72 rows 0.4 us slower with it, 256 rows 0.3 us faster, 512 rows 2.5 us)
constexpr int SAMPLE_CHUNK_BYTES = 128;  // a chunk is one 128-byte line: 32 float32 logits, 64 16-bit ones
constexpr int SAMPLE_MAX_ORDER = 96; // deepest order statistic of the chunk maxima that is trusted
constexpr int FILTER_THREADS = 256;
constexpr int FILTER_VECS = 8;       // 128-bit loads in flight per thread
constexpr int FILTER_STAGE = 64;     // pairs a warp collects in shared memory between flushes

constexpr int FL_SORT = 512;            // most candidates finish_list_kernel sorts
constexpr int FL_MAX_K = FL_SORT - 64;  // the largest top_k it takes

__device__ __forceinline__ float pos_inf() { return __uint_as_float(0x7F800000u); }

// What the filter leaves per row for the blocks and kernels that follow, in one 64-bit word (so one
// load or store moves it whole): the row's floor (float32 bits), whether the list finish takes the
// row, and a mark that the word is this call's.  The kernels that take the rows clear the mark.
constexpr unsigned long long INFO_LEAN = 1ull << 32, INFO_READY = 1ull << 33;
__device__ __forceinline__ float info_floor(unsigned long long info) { return __uint_as_float((uint32_t)info); }

// Does finish_list_kernel take this row?  (sample_kernel takes the others.)  Worked out once per
// row, by the filter, and kept in the workspace as the row's flag.
__device__ __forceinline__ bool lean_takes(const KParams& P, const RowCfg& rc, float floor_l) {
  if (!P.lean || !(floor_l < pos_inf())) return false;
  if (P.history && !rc.lowers) return false;  // history tokens must be fetched one by one
  if (rc.mode == M_ARGMAX_L || rc.mode == M_SELECT_MINP) return true;
  return rc.mode == M_SELECT_K && rc.k_eff <= FL_MAX_K;
}

// Which order statistic of the sample bounds the top k of the row from below.  x = k * sample / V
// sample elements are expected among the row's top k; the number that really are is close to
// Poisson(x), and j is chosen so that fewer than j are with probability about 1 - 1e-6.
__device__ __forceinline__ int floor_order(int k, int vocab, int sample) {
  const float x = (float)k * (float)sample / (float)vocab;
  return (int)ceilf(x + 4.75f * sqrtf(x) + 4.0f);
}

// Logits come as float32, bfloat16 or float16 (KParams::dtype 0, 1, 2); a 16-byte vector holds 4 or
// 8 of them.  Both 16-bit formats convert to float32 exactly, so everything downstream of a
// comparison works on the same float32 values the oracle sees.
struct F32 { static constexpr int PER_VEC = 4; };
struct BF16 { static constexpr int PER_VEC = 8; };
struct F16 { static constexpr int PER_VEC = 8; };

template <typename T>
__device__ __forceinline__ void vec_to_floats(const uint4& v, float (&out)[T::PER_VEC]);
template <>
__device__ __forceinline__ void vec_to_floats<F32>(const uint4& v, float (&out)[4]) {
  out[0] = __uint_as_float(v.x); out[1] = __uint_as_float(v.y); out[2] = __uint_as_float(v.z); out[3] = __uint_as_float(v.w);
}
template <>
__device__ __forceinline__ void vec_to_floats<BF16>(const uint4& v, float (&out)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
template <>
__device__ __forceinline__ void vec_to_floats<F16>(const uint4& v, float (&out)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
// the largest of a vector's logits (NaNs dropped); the 16-bit formats compare packed pairs first
template <typename T>
__device__ __forceinline__ float vec_max(const uint4& v);
template <>
__device__ __forceinline__ float vec_max<F32>(const uint4& v) {
  return fmaxf(fmaxf(__uint_as_float(v.x), __uint_as_float(v.y)), fmaxf(__uint_as_float(v.z), __uint_as_float(v.w)));
}
template <>
__device__ __forceinline__ float vec_max<BF16>(const uint4& v) {
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x), b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
  const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(&v.z), d = *reinterpret_cast<const __nv_bfloat162*>(&v.w);
  const __nv_bfloat162 m = __hmax2(__hmax2(a, b), __hmax2(c, d));
  return fmaxf(__bfloat162float(m.x), __bfloat162float(m.y));
}
template <>
__device__ __forceinline__ float vec_max<F16>(const uint4& v) {
  const __half2 a = *reinterpret_cast<const __half2*>(&v.x), b = *reinterpret_cast<const __half2*>(&v.y);
  const __half2 c = *reinterpret_cast<const __half2*>(&v.z), d = *reinterpret_cast<const __half2*>(&v.w);
  const __half2 m = __hmax2(__hmax2(a, b), __hmax2(c, d));
  return fmaxf(__half2float(m.x), __half2float(m.y));
}
// which of a vector's logits reach the floor, one bit each (out of line: it runs for the few
// vectors whose maximum reaches the floor)
template <typename T>
__device__ __noinline__ uint32_t vec_hits(uint4 v, float floor_l) {
  float f[T::PER_VEC];
  vec_to_floats<T>(v, f);
  uint32_t bits = 0u;
#pragma unroll
  for (int e = 0; e < T::PER_VEC; ++e) bits |= (f[e] >= floor_l ? 1u : 0u) << e;
  return bits;
}
// the packed maxima of two vectors, pair by pair
template <typename T>
__device__ __forceinline__ uint4 packed_max(const uint4& a, const uint4& b);
template <>
__device__ __forceinline__ uint4 packed_max<BF16>(const uint4& a, const uint4& b) {
  uint4 r;
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&b);
  __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i] = __hmax2(p[i], q[i]);
  return r;
}
template <>
__device__ __forceinline__ uint4 packed_max<F16>(const uint4& a, const uint4& b) {
  uint4 r;
  const __half2* p = reinterpret_cast<const __half2*>(&a);
  const __half2* q = reinterpret_cast<const __half2*>(&b);
  __half2* o = reinterpret_cast<__half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i] = __hmax2(p[i], q[i]);
  return r;
}
template <>
__device__ __forceinline__ uint4 packed_max<F32>(const uint4& a, const uint4& b) {
  return make_uint4(__float_as_uint(fmaxf(__uint_as_float(a.x), __uint_as_float(b.x))),
                    __float_as_uint(fmaxf(__uint_as_float(a.y), __uint_as_float(b.y))),
                    __float_as_uint(fmaxf(__uint_as_float(a.z), __uint_as_float(b.z))),
                    __float_as_uint(fmaxf(__uint_as_float(a.w), __uint_as_float(b.w))));
}
__device__ __forceinline__ uint4 minus_inf_vec(int dtype) {
  const uint32_t w = dtype == 0 ? 0xFF800000u : (dtype == 1 ? 0xFF80FF80u : 0xFC00FC00u);
  return make_uint4(w, w, w, w);
}
// logit i of row b, whatever the format (scattered single reads: history tokens, the multi-pass routine)
__device__ __forceinline__ float logit_at(const KParams& P, int b, int i) {
  const size_t at = (size_t)b * P.row_stride + i;
  if (P.dtype == 0) return P.logits[at];
  const unsigned short h = reinterpret_cast<const unsigned short*>(P.logits)[at];
  if (P.dtype == 1) return __uint_as_float((uint32_t)h << 16);
  return __half2float(__ushort_as_half(h));
}

// Vectors of 16 bytes per chunk of the sample: eight (a 128-byte line) unless the row is short;
// the sample stays under an eighth of the row (a vocabulary slice of 25 000 tokens gives 2048 of
// them, not 8192).
__device__ __forceinline__ int sample_vecs(int V, int per_vec) {
  int vecs = SAMPLE_CHUNK_BYTES / 16;
  while (vecs > 1 && (long long)SAMPLE_CHUNKS * vecs * per_vec * 8 > V) vecs >>= 1;
  return vecs;
}

// The descending chunk maxima of a row's sample, by the first SAMPLE_CHUNKS threads of the calling
// block (whole warps; every thread of the block must call); `runs` is SAMPLE_CHUNKS 8-byte words of
// shared memory, `sorted` as many floats.  Rows are 16-byte aligned whole vectors, at least twice
// the sample long (so that the chunks do not overlap).
template <typename T, int VECS>
__device__ __forceinline__ float chunk_maximum(const void* row, int V) {
  // four chunks in a row make a piece; piece p starts at a multiple of its own length near p * V / 64
  const int tid = threadIdx.x;
  constexpr long long CHUNK = VECS * T::PER_VEC;  // logits
  constexpr int PIECES = SAMPLE_CHUNKS / 4;
  const long long at = (((long long)(tid >> 2) * V / PIECES) & ~(4 * CHUNK - 1)) + (tid & 3) * CHUNK;
  const uint4* src = reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(row) + at * (16 / T::PER_VEC));
  uint4 x[VECS];
#pragma unroll
  for (int u = 0; u < VECS; ++u) x[u] = __ldg(src + u);
  float m = neg_inf();  // fmaxf drops NaNs
#pragma unroll
  for (int u = 0; u < VECS; ++u) m = fmaxf(m, vec_max<T>(x[u]));
  return m;
}
// The same maximum for batches of many rows, where the sample's loads are a matter of throughput,
// not of latency: thread t still answers for chunk t, but a warp loads its eight pieces side by
// side, a lane one vector of a piece per instruction, so that every instruction asks for whole
// lines; the lanes that share a chunk then merge their maxima, and every lane fetches its chunk's.
template <typename T, int VECS>
__device__ __forceinline__ float chunk_maximum_side_by_side(const void* row, int V) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr long long CHUNK = VECS * T::PER_VEC;  // logits
  constexpr int PIECES = SAMPLE_CHUNKS / 4;
  constexpr int LANES = 4 * VECS;    // lanes (vectors) per piece
  constexpr int SIDE = 32 / LANES;   // pieces per instruction
  constexpr int GROUPS = 32 / VECS;  // chunks per instruction
  uint4 x[VECS];
#pragma unroll
  for (int q = 0; q < VECS; ++q) {
    const int piece = warp * 8 + q * SIDE + lane / LANES;
    const long long at = ((long long)piece * V / PIECES) & ~(4 * CHUNK - 1);
    x[q] = __ldg(reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(row) + at * (16 / T::PER_VEC)) + lane % LANES);
  }
  float m[VECS];
#pragma unroll
  for (int q = 0; q < VECS; ++q) m[q] = vec_max<T>(x[q]);  // fmaxf drops NaNs
#pragma unroll
  for (int d = 1; d < VECS; d <<= 1)
#pragma unroll
    for (int q = 0; q < VECS; ++q) m[q] = fmaxf(m[q], __shfl_xor_sync(FULL, m[q], d));
  // the warp's chunk c was loaded by instruction c / GROUPS, by the lanes from (c % GROUPS) * VECS on
  float mine = neg_inf();
#pragma unroll
  for (int q = 0; q < VECS; ++q) {
    const float v = __shfl_sync(FULL, m[q], (lane % GROUPS) * VECS);
    if (lane / GROUPS == q) mine = v;
  }
  return mine;
}

// `meanwhile` runs once the sample's loads have been waited for, before the first barrier.
template <typename T, typename F>
__device__ __forceinline__ void sample_maxima(const void* row, int V, int vecs, unsigned long long* runs, float* sorted,
                                              bool many_rows, F meanwhile) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned long long key = 0ull;
  if (tid < SAMPLE_CHUNKS) {
    const float m = (many_rows && vecs == 8) ? chunk_maximum_side_by_side<T, 8>(row, V)
                  : vecs == 8 ? chunk_maximum<T, 8>(row, V) : vecs == 4 ? chunk_maximum<T, 4>(row, V)
                  : vecs == 2 ? chunk_maximum<T, 2>(row, V) : chunk_maximum<T, 1>(row, V);
    // ordered like the candidates' keys: value first, the chunk's number breaking ties
    key = make_key(m, (uint32_t)tid);
    // every warp sorts its 32 maxima in registers (a bitonic network over shuffles) ...
#pragma unroll
    for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
      for (int j = k >> 1; j > 0; j >>= 1) {
        const unsigned long long other = __shfl_xor_sync(FULL, key, j);
        const bool keep_max = ((lane & k) == 0) == ((lane & j) == 0);
        const unsigned long long hi = key > other ? key : other, lo = key > other ? other : key;
        key = keep_max ? hi : lo;
      }
    }
    runs[tid] = key;
  }
  meanwhile();
  __syncthreads();
  if (tid < SAMPLE_CHUNKS) {
    // ... and a maximum's place is its place in its run plus the maxima above it in the other runs
    constexpr int RUNS = SAMPLE_CHUNKS / 32;
    int place = lane;
#pragma unroll
    for (int r0 = 0; r0 < RUNS; r0 += 4) {
      int pos[4] = {0, 0, 0, 0};
#pragma unroll
      for (int step = 16; step > 0; step >>= 1) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
          if (runs[(r0 + q) * 32 + pos[q] + step - 1] > key) pos[q] += step;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (pos[q] == 31 && runs[(r0 + q) * 32 + 31] > key) pos[q] = 32;
        if (r0 + q != warp) place += pos[q];
      }
    }
    sorted[place] = key_value(key);
  }
  __syncthreads();
}

// The row's floor from its sorted sample maxima: +inf for rows that do not use a list (whole-row
// Gumbel rows, rows for the multi-pass routine and rows whose list would be long; under a soft cap
// also min-p rows, whose threshold lives in capped scores while the floor is a raw logit).
__device__ __forceinline__ float floor_from_sample(const RowCfg& rc, int V, int sample, int list_cap, const float* sorted,
                                                   bool capped) {
  const int mode = rc.mode;
  float floor_l = pos_inf();
  if (mode == M_SELECT_K) {
    const int j = floor_order(rc.k_eff, V, sample);
    // the list must also fit: about j * V / sample logits lie above the j-th maximum
    if (j <= SAMPLE_MAX_ORDER && (long long)j * V / sample * 4 <= (long long)list_cap * 3) floor_l = sorted[j - 1];
  } else if (mode == M_ARGMAX_L) {
    floor_l = sorted[3];
  } else if (mode == M_SELECT_MINP && !capped) {
    // survivors score at least (true top) + log(min_p), and the true top is at least the sample's
    const float f = logit_floor(scaled(sorted[0], rc) + rc.logm, rc.tf);
    if (f >= sorted[SAMPLE_MAX_ORDER - 1]) floor_l = f;
  }
  if (rc.track && floor_l < pos_inf()) floor_l = fminf(floor_l, sorted[3]);
  if (!(floor_l > neg_inf())) floor_l = pos_inf();  // a row of mostly -inf: everything would be listed
  return floor_l;
}

// The floor of row b for a block of SAMPLE_CHUNKS threads that comes to the row: taken from the
// workspace if a block before it has left it there already, else worked out from the row's sample
// (blocks that start on the same row together all do so, to the same value) and left there for the
// blocks and kernels that follow.
template <typename T>
__device__ __forceinline__ float block_floor(const KParams& P, int b, unsigned long long* runs, float* sorted, RowCfg* rc,
                                             unsigned long long* known, bool look = true) {
  const int tid = threadIdx.x;
  __syncthreads();  // every thread is done with the floor before (`rc` and `known` are about to change)
  if (look) {
    if (tid == 0) *known = __ldcg(&P.list_info[b]);
    __syncthreads();
    const unsigned long long have = *known;
    if (have & INFO_READY) return info_floor(have);
  }
  // the row's options are asked for first and looked at once the sample has come in: one wait for both
  const uint32_t word = tid < 32 ? row_inputs_word(P, b, nullptr) : 0u;
  const unsigned char* row = reinterpret_cast<const unsigned char*>(P.logits) + (size_t)b * P.row_stride * (16 / T::PER_VEC);
  const int vecs = sample_vecs(P.vocab, T::PER_VEC);
  sample_maxima<T>(row, P.vocab, vecs, runs, sorted, P.rows >= SAMPLE_SIDE_BY_SIDE_ROWS, [&]() {
    if (tid < 32) {
      uint32_t unused;
      const RowIn in = row_inputs_from(P, word, unused);
      if (tid == 0) *rc = row_config_from(P, in);
    }
  });
  const float floor_l = floor_from_sample(*rc, P.vocab, SAMPLE_CHUNKS * vecs * T::PER_VEC, P.list_cap, sorted, P.softcap > 0.0f);
  if (tid == 0)
    P.list_info[b] = INFO_READY | (lean_takes(P, *rc, floor_l) ? INFO_LEAN : 0ull) | (unsigned long long)__float_as_uint(floor_l);
  return floor_l;
}

// With few rows the floors are worked out ahead of the filter, one block per row, so that the many
// blocks that then share a row find its floor waiting instead of each working it out.
template <typename T>
__global__ void __launch_bounds__(SAMPLE_CHUNKS) floor_kernel(const __grid_constant__ KParams P) {
  __shared__ unsigned long long runs[SAMPLE_CHUNKS];
  __shared__ float sorted[SAMPLE_CHUNKS];
  __shared__ RowCfg rc;
  __shared__ unsigned long long known;
  grid_dependency_wait();  // (launched as a programmatic dependent of whatever wrote the logits)
  stamp_begin(P.stamps, 3);
  grid_launch_dependents();  // the filter's blocks may ask for their first logits meanwhile
  if (blockIdx.x == 0 && threadIdx.x == 0 && (P.flags & 16u) && P.status) *P.status = 0;
  block_floor<T>(P, blockIdx.x, runs, sorted, &rc, &known, false);
  stamp_end(P.stamps, 3);
}

// A warp's finds on their way to a row's list: collected in shared memory (FILTER_STAGE pairs per
// warp) and appended with one atomic per flush.
struct FilterStage {
  unsigned long long* mine;  // this warp's FILTER_STAGE pairs of shared memory
  int held;                  // pairs collected (the same in every lane)
  int row;                   // the row they belong to
};

__device__ __forceinline__ void filter_flush(const KParams& P, FilterStage& st) {
  const int lane = threadIdx.x & 31;
  if (st.held > 0) {
    int at = 0;
    if (lane == 0) at = atomicAdd(&P.list_count[st.row], st.held);
    at = __shfl_sync(FULL, at, 0);
    unsigned long long* list = P.list + (size_t)st.row * P.list_cap;
    __syncwarp();
    for (int i = lane; i < st.held; i += 32)
      if (at + i < P.list_cap) list[at + i] = st.mine[i];
    __syncwarp();
  }
  st.held = 0;
}

// The block's NT threads load FILTER_VECS 16-byte vectors each of a row, from logit `base` on:
// logit e of vector u has index base + (u * NT + tid) * PER_VEC + e; past the row's end (`limit`)
// they read as -inf.
template <typename T, int NT>
__device__ __forceinline__ void filter_load(uint4 (&x)[FILTER_VECS], const unsigned char* row, int base, int limit,
                                            int dtype) {
  const int tid = threadIdx.x;
#pragma unroll
  for (int u = 0; u < FILTER_VECS; ++u) {
    const int i = base + (u * NT + tid) * T::PER_VEC;
    x[u] = minus_inf_vec(dtype);
    if (i < limit) x[u] = __ldcs(reinterpret_cast<const uint4*>(row + (size_t)i * (16 / T::PER_VEC)));
  }
}

// What a thread does with the logits it holds of row st.row: those at or above the floor go to the
// warp's stage, as (float32 bits, index) pairs.  Whole warps call it together.
template <typename T, int NT>
__device__ __forceinline__ void filter_process(const KParams& P, FilterStage& st, const uint4 (&x)[FILTER_VECS], int base,
                                               float floor_l, const unsigned char* row) {
  const int tid = threadIdx.x, lane = tid & 31;
  // the largest logit this thread holds: vectors are merged pair by pair first (for the 16-bit
  // formats two logits per instruction), one vector is widened at the end
  uint4 top = x[0];
#pragma unroll
  for (int u = 1; u < FILTER_VECS; ++u) top = packed_max<T>(top, x[u]);
  const bool hot = vec_max<T>(top) >= floor_l;
  if (!__any_sync(FULL, hot)) return;
  int count = 0;
  unsigned long long hits = 0ull;  // one bit per logit at or above the floor
  if (hot) {
#pragma unroll
    for (int u = 0; u < FILTER_VECS; ++u)
      if (vec_max<T>(x[u]) >= floor_l) hits |= (unsigned long long)vec_hits<T>(x[u], floor_l) << (T::PER_VEC * u);
    count = __popcll(hits);
  }
  int incl = count;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int o = __shfl_up_sync(FULL, incl, d);
    if (lane >= d) incl += o;
  }
  const int total = __shfl_sync(FULL, incl, 31);
  if (total > FILTER_STAGE) {
    // more than the stage holds from one warp's logits: the floor is useless for this row; the
    // count is pushed past the list's capacity, which sends the row to the multi-pass routine
    if (lane == 0) atomicAdd(&P.list_count[st.row], P.list_cap + 1);
    return;
  }
  if (st.held + total > FILTER_STAGE) filter_flush(P, st);
  if (hot) {
    int at = st.held + incl - count;
    // the few logits that made it go to the stage straight from the registers: every vector and
    // element is looked at under a predicate, so no register array is indexed by a run-time number
    // and nothing is read again
#pragma unroll
    for (int u = 0; u < FILTER_VECS; ++u) {
      const uint32_t bits = (uint32_t)(hits >> (T::PER_VEC * u)) & ((1u << T::PER_VEC) - 1u);
      if (bits) {
        float f[T::PER_VEC];
        vec_to_floats<T>(x[u], f);
        const int i0 = base + (u * NT + tid) * T::PER_VEC;
#pragma unroll
        for (int e = 0; e < T::PER_VEC; ++e)
          if ((bits >> e) & 1u) st.mine[at++] = ((unsigned long long)__float_as_uint(f[e]) << 32) | (uint32_t)(i0 + e);
      }
    }
  }
  st.held += total;
}

// 16 bytes global -> shared without passing through registers; waited for with async_wait_all()
__device__ __forceinline__ void async_copy16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void async_wait_all() {
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// Streams the logits once.  A work item is FILTER_THREADS x FILTER_VECS consecutive vectors of one
// row (8192 float32 logits or 16384 16-bit ones).  With many rows the items are dealt to the blocks
// in contiguous runs, so a block mostly stays within one row and needs one or two floors; with few
// rows (`per` > 0) every row has `per` blocks of its own, which share its items, so that no block
// ever changes rows.  When a block comes to a new row, the item's logits are on their way into
// shared memory while the floor is found.
template <typename T>
__global__ void __launch_bounds__(FILTER_THREADS, 4) filter_kernel(const __grid_constant__ KParams P, int per_row,
                                                                   int items, int per, int floors_first) {
  static_assert(FILTER_THREADS == SAMPLE_CHUNKS, "a block's threads take one chunk of the sample each");
  extern __shared__ __align__(16) unsigned char filter_smem[];
  uint4* ahead = reinterpret_cast<uint4*>(filter_smem);  // FILTER_THREADS x FILTER_VECS vectors
  __shared__ unsigned long long stage[FILTER_THREADS / 32][FILTER_STAGE];
  __shared__ unsigned long long runs[SAMPLE_CHUNKS];
  __shared__ float sorted[SAMPLE_CHUNKS];
  __shared__ RowCfg rc;
  __shared__ unsigned long long known;
  constexpr int SPAN = FILTER_THREADS * FILTER_VECS * T::PER_VEC;
  constexpr int BYTES = 16 / T::PER_VEC;
  int first = (int)((long long)blockIdx.x * items / gridDim.x);
  int last = (int)((long long)(blockIdx.x + 1) * items / gridDim.x);
  if (per > 0) {
    const int r = blockIdx.x / per, j = blockIdx.x - r * per;
    first = r * per_row + j * per_row / per;
    last = r * per_row + (j + 1) * per_row / per;
  }
  const unsigned char* logits = reinterpret_cast<const unsigned char*>(P.logits);
  const int tid = threadIdx.x;
  auto ask_ahead = [&](const unsigned char* row, int base) {
#pragma unroll
    for (int u = 0; u < FILTER_VECS; ++u) {
      const int i = base + (u * FILTER_THREADS + tid) * T::PER_VEC;
      if (i < P.vocab) async_copy16(&ahead[u * FILTER_THREADS + tid], row + (size_t)i * BYTES);
    }
  };
  bool asked = false;
  if (floors_first) {
    // floor_kernel runs before this grid and waited for the logits itself: this block's first
    // logits can be on their way while the floors are written
    if (first < last) {
      const int b = first / per_row;
      ask_ahead(logits + (size_t)b * P.row_stride * BYTES, (first - b * per_row) * SPAN);
      asked = true;
    }
    grid_dependency_wait();
    stamp_begin(P.stamps, 0);
  } else {
    grid_dependency_wait();  // (launched as a programmatic dependent of whatever wrote the logits)
    stamp_begin(P.stamps, 0);
    // every kernel that may OR into the status word waits for this grid to end
    if (blockIdx.x == 0 && tid == 0 && (P.flags & 16u) && P.status) *P.status = 0;
  }
  grid_launch_dependents();  // the blocks that finish rows may queue up behind this grid's
  FilterStage st;
  st.mine = stage[tid >> 5];
  st.held = 0;
  st.row = -1;
  float floor_l = pos_inf();
#pragma unroll 1
  for (int item = first; item < last; ++item) {
    const int b = item / per_row;
    const int base = (item - b * per_row) * SPAN;
    const unsigned char* row = logits + (size_t)b * P.row_stride * BYTES;
    uint4 x[FILTER_VECS];
    if (b != st.row) {
      filter_flush(P, st);
      st.row = b;
      if (!asked) ask_ahead(row, base);
      asked = false;
      // (a handful of rows with one item per block: every block starts on its row at the same time,
      // so no block would find the row's word there yet: no use looking)
      floor_l = block_floor<T>(P, b, runs, sorted, &rc, &known, floors_first || items > (int)gridDim.x);
      async_wait_all();  // (each thread reads back what it asked for itself)
      if (!(floor_l < pos_inf())) continue;  // the row does not use the list
#pragma unroll
      for (int u = 0; u < FILTER_VECS; ++u) {
        const int i = base + (u * FILTER_THREADS + tid) * T::PER_VEC;
        x[u] = i < P.vocab ? ahead[u * FILTER_THREADS + tid] : minus_inf_vec(P.dtype);
      }
    } else {
      if (!(floor_l < pos_inf())) continue;
      filter_load<T, FILTER_THREADS>(x, row, base, P.vocab, P.dtype);
    }
    filter_process<T, FILTER_THREADS>(P, st, x, base, floor_l, row);
  }
  filter_flush(P, st);
  stamp_end(P.stamps, 0);
}

// sample_kernel's replacement for the stream on a row that has a list: the listed logits become
// (score, id) keys in the candidate buffer, history tokens among them penalised, and the greedy
// best among them is tracked.  `listed` is the list's length and first_pair this thread's entry of
// the first round, both loaded by the caller ahead of time; `bitmap`, if not null, marks the
// history tokens (then only membership matters).  False if the list ran over.
template <bool PEN>
__device__ __noinline__ bool list_load(const KParams& P, const RowCfg& rc, const Ctx& c, const History& h,
                                       const unsigned* bitmap, int b, Tracked& t, int listed,
                                       unsigned long long first_pair) {
  Shared& sm = *c.sm;
  const int tid = threadIdx.x, nt = blockDim.x;
  if (listed > P.list_cap) return false;
  const unsigned long long* list = P.list + (size_t)b * P.list_cap;
  const bool select = rc.mode == M_SELECT_K || rc.mode == M_SELECT_MINP;
#pragma unroll 1
  for (int base = 0; base < listed; base += nt) {
    const int i = base + tid;
    bool want = false;
    unsigned long long key = 0ull;
    if (i < listed) {
      const unsigned long long pair = base == 0 ? first_pair : __ldcg(&list[i]);
      const int idx = (int)(uint32_t)pair;
      float l = __uint_as_float((uint32_t)(pair >> 32));
      bool skip = false;
      if (PEN && P.history) {
        // a history token: penalised here if penalties only lower logits (then those that matter are
        // all listed), else left to the history pass, which fetches every history token's logit
        const int count = bitmap ? (int)((bitmap[idx >> 5] >> (idx & 31)) & 1u) : history_count(h, idx);
        if (count) {
          if (rc.lowers) l = penalised(l, count, rc);
          else skip = true;
        }
      }
      if (!skip) {
        if (rc.track && (l > t.gl || (l == t.gl && idx < t.gid))) { t.gl = l; t.gid = idx; }
        const float s = scaled(l, rc);
        want = select && s == s;
        key = make_key(s, (uint32_t)(idx + P.vocab_offset));
      }
    }
    if (select) {
      buffer_push(c, want, key);
      if (sm.overflow) break;
    }
  }
  return true;
}
