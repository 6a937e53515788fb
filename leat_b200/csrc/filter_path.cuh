// The filter path: how large batches reach the memory roofline.  Included inside namespace leat by
// sampler_kernels.cuh.
//
// Three launches instead of one fused kernel doing everything per block:
//
//   floor_kernel   one block per row reads a spread-out sample of the row (256 chunks of 32 logits,
//                  32 KB) and takes a low order statistic of the chunks' maxima as the row's floor:
//                  a raw logit above which, with overwhelming probability, at least top_k logits of
//                  the row lie, and not many more.
//   filter_kernel  streams every logit exactly once with 128-bit loads and nothing else to do than
//                  compare it with its row's floor; the few hundred logits per row at or above it
//                  are appended, as (logit, index) pairs, to the row's list in the workspace.
//   sample_kernel  (one block per row) builds the candidate buffer from the list and from the row's
//                  history tokens instead of streaming, and finishes the row as always.
//
// The floor is only a guess, so the finish checks it: the result stands if at least top_k
// candidates score strictly above the floor's score and the cut lies strictly above it too (then no
// logit the filter dropped could have been a survivor or changed the cut); greedy rows need their
// best candidate at or above the floor.  A row that fails the check is flagged and redone by the
// exact multi-pass kernel.
#pragma once

constexpr int SAMPLE_CHUNKS = 256;   // chunks of the sample, one per thread of floor_kernel
constexpr int SAMPLE_CHUNK = 32;     // logits per chunk (128 bytes)
constexpr int SAMPLE_SIZE = SAMPLE_CHUNKS * SAMPLE_CHUNK;
constexpr int SAMPLE_MAX_ORDER = 96; // deepest order statistic of the chunk maxima that is trusted
constexpr int FILTER_THREADS = 256;
constexpr int FILTER_VECS = 8;       // 128-bit loads in flight per thread
constexpr int FILTER_SPAN = FILTER_THREADS * FILTER_VECS * 4;  // logits of one work item: 8192
constexpr int FILTER_STAGE = 64;     // pairs a warp collects in shared memory between flushes

__device__ __forceinline__ float pos_inf() { return __uint_as_float(0x7F800000u); }

// Which order statistic of the sample bounds the top k of the row from below.  x = k * sample / V
// sample elements are expected among the row's top k; the number that really are is close to
// Poisson(x), and j is chosen so that fewer than j are with probability about 1 - 1e-6.
__device__ __forceinline__ int floor_order(int k, int vocab) {
  const float x = (float)k * (float)SAMPLE_SIZE / (float)vocab;
  return (int)ceilf(x + 4.75f * sqrtf(x) + 4.0f);
}

// The descending chunk maxima of a row's sample, by the first SAMPLE_CHUNKS threads of the calling
// block (every thread of the block must call); `maxima` and `sorted` are SAMPLE_CHUNKS floats of
// shared memory each.  Rows are 16-byte aligned multiples of four floats, at least 2 * SAMPLE_SIZE
// long.
__device__ __forceinline__ void sample_maxima(const float* __restrict__ row, int V, float* maxima, float* sorted) {
  const int tid = threadIdx.x;
  if (tid < SAMPLE_CHUNKS) {
    // chunk tid starts at a multiple of 32 logits near tid * V / 256
    const long long at = ((long long)tid * V / SAMPLE_CHUNKS) & ~31ll;
    const float4* src = reinterpret_cast<const float4*>(row + at);
    float4 x[SAMPLE_CHUNK / 4];
#pragma unroll
    for (int u = 0; u < SAMPLE_CHUNK / 4; ++u) x[u] = __ldg(src + u);
    float m = neg_inf();  // fmaxf drops NaNs
#pragma unroll
    for (int u = 0; u < SAMPLE_CHUNK / 4; ++u) m = fmaxf(fmaxf(m, fmaxf(x[u].x, x[u].y)), fmaxf(x[u].z, x[u].w));
    maxima[tid] = m;
  }
  __syncthreads();
  if (tid < SAMPLE_CHUNKS) {
    // descending order by counting: place = number of maxima ahead of this one
    const float v = maxima[tid];
    int place = 0;
#pragma unroll 8
    for (int j = 0; j < SAMPLE_CHUNKS; ++j) {
      const float o = maxima[j];
      place += (o > v) || (o == v && j < tid);
    }
    sorted[place] = v;
  }
  __syncthreads();
}

// The row's floor from its sorted sample maxima: +inf for rows that do not use a list (whole-row
// Gumbel rows, rows for the multi-pass routine and rows whose list would be long).
__device__ __forceinline__ float floor_from_sample(const RowCfg& rc, int V, int list_cap, const float* sorted) {
  const int mode = rc.mode;
  float floor_l = pos_inf();
  if (mode == M_SELECT_K) {
    const int j = floor_order(rc.k_eff, V);
    // the list must also fit: about j * V / sample logits lie above the j-th maximum
    if (j <= SAMPLE_MAX_ORDER && (long long)j * V / SAMPLE_SIZE * 4 <= (long long)list_cap * 3) floor_l = sorted[j - 1];
  } else if (mode == M_ARGMAX_L) {
    floor_l = sorted[3];
  } else if (mode == M_SELECT_MINP) {
    // survivors score at least (true top) + log(min_p), and the true top is at least the sample's
    const float f = logit_floor(scaled(sorted[0], rc) + rc.logm, rc.tf);
    if (f >= sorted[SAMPLE_MAX_ORDER - 1]) floor_l = f;
  }
  if (rc.track && floor_l < pos_inf()) floor_l = fminf(floor_l, sorted[3]);
  if (!(floor_l > neg_inf())) floor_l = pos_inf();  // a row of mostly -inf: everything would be listed
  return floor_l;
}

// One block of 256 + 32 threads per row.  Writes the row's floor and clears the row's list.
__global__ void __launch_bounds__(SAMPLE_CHUNKS + 32) floor_kernel(const __grid_constant__ KParams P) {
  __shared__ float maxima[SAMPLE_CHUNKS];
  __shared__ float sorted[SAMPLE_CHUNKS];
  __shared__ RowCfg rc;
  const int b = blockIdx.x, tid = threadIdx.x;
  grid_launch_dependents();  // the filter's blocks may take their places; they wait for this grid to end
  if (tid >= SAMPLE_CHUNKS) {  // a warp of its own fetches the row's options while the sample is on its way
    uint32_t unused;
    const RowIn in = row_inputs_warp(P, b, nullptr, unused);
    if (tid == SAMPLE_CHUNKS) rc = row_config_from(P, in);
  }
  sample_maxima(P.logits + (size_t)b * P.row_stride, P.vocab, maxima, sorted);
  if (tid == 0) {
    P.list_floor[b] = floor_from_sample(rc, P.vocab, P.list_cap, sorted);
    P.list_count[b] = 0;
  }
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

// The block's NT threads load the logits [base, base + NT * 32) of a row, below `limit`: logit e of
// vector u has index base + (u * NT + tid) * 4 + e; logits past the row's end read as -inf.
template <int NT>
__device__ __forceinline__ void filter_load(float4 (&x)[FILTER_VECS], const float* __restrict__ row, int base, int limit) {
  const int tid = threadIdx.x;
#pragma unroll
  for (int u = 0; u < FILTER_VECS; ++u) {
    const int i = base + (u * NT + tid) * 4;
    x[u] = make_float4(neg_inf(), neg_inf(), neg_inf(), neg_inf());
    if (i < limit) x[u] = __ldcs(reinterpret_cast<const float4*>(row + i));
  }
}

// What a thread does with the logits it holds of row st.row: those at or above the floor go to the
// warp's stage.  Whole warps call it together.
template <int NT>
__device__ __forceinline__ void filter_process(const KParams& P, FilterStage& st, const float4 (&x)[FILTER_VECS],
                                               int base, float floor_l) {
  const int tid = threadIdx.x, lane = tid & 31;
  float m = neg_inf();
#pragma unroll
  for (int u = 0; u < FILTER_VECS; ++u) m = fmaxf(fmaxf(m, fmaxf(x[u].x, x[u].y)), fmaxf(x[u].z, x[u].w));
  const bool hot = m >= floor_l;
  if (!__any_sync(FULL, hot)) return;
  int count = 0;
  if (hot) {
#pragma unroll
    for (int u = 0; u < FILTER_VECS; ++u)
      count += (x[u].x >= floor_l) + (x[u].y >= floor_l) + (x[u].z >= floor_l) + (x[u].w >= floor_l);
  }
  int incl = count;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int o = __shfl_up_sync(FULL, incl, d);
    if (lane >= d) incl += o;
  }
  const int total = __shfl_sync(FULL, incl, 31);
  if (total > FILTER_STAGE) {
    // more than the stage holds from 1024 logits: the floor is useless for this row; the count is
    // pushed past the list's capacity, which sends the row to the multi-pass routine
    if (lane == 0) atomicAdd(&P.list_count[st.row], P.list_cap + 1);
    return;
  }
  if (st.held + total > FILTER_STAGE) filter_flush(P, st);
  if (hot) {
    int at = st.held + incl - count;
#pragma unroll
    for (int u = 0; u < FILTER_VECS; ++u) {
      const int i = base + (u * NT + tid) * 4;
      const float v[4] = {x[u].x, x[u].y, x[u].z, x[u].w};
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (v[e] >= floor_l) st.mine[at++] = ((unsigned long long)__float_as_uint(v[e]) << 32) | (uint32_t)(i + e);
    }
  }
  st.held += total;
}

// Streams the logits once.  A work item is FILTER_SPAN consecutive logits of one row; the items
// are dealt to the blocks in contiguous runs, so a block mostly stays within one row.
__global__ void __launch_bounds__(FILTER_THREADS, 4) filter_kernel(const __grid_constant__ KParams P, int per_row,
                                                                   int items) {
  __shared__ unsigned long long stage[FILTER_THREADS / 32][FILTER_STAGE];
  const int first = (int)((long long)blockIdx.x * items / gridDim.x);
  const int last = (int)((long long)(blockIdx.x + 1) * items / gridDim.x);
  FilterStage st;
  st.mine = stage[threadIdx.x >> 5];
  st.held = 0;
  st.row = -1;
  // the first item's logits are asked for before the floors are waited for: they are the caller's
  float4 x[FILTER_VECS];
  if (first < last) {
    const int b = first / per_row;
    filter_load<FILTER_THREADS>(x, P.logits + (size_t)b * P.row_stride, (first - b * per_row) * FILTER_SPAN, P.vocab);
  }
  grid_dependency_wait();    // the floors are written
  grid_launch_dependents();  // blocks that finish rows move in as this grid's blocks leave
#pragma unroll 1
  for (int item = first; item < last; ++item) {
    const int b = item / per_row;
    const int base = (item - b * per_row) * FILTER_SPAN;
    if (b != st.row) { filter_flush(P, st); st.row = b; }
    const float floor_l = __ldcg(&P.list_floor[b]);
    if (!(floor_l < pos_inf())) continue;  // the row does not use the list
    if (item > first) filter_load<FILTER_THREADS>(x, P.logits + (size_t)b * P.row_stride, base, P.vocab);
    filter_process<FILTER_THREADS>(P, st, x, base, floor_l);
  }
  filter_flush(P, st);
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
