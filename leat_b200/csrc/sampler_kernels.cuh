// The fused sampler kernel for sm_100a.
//
// One launch samples every row.  A row of logits is cut into `slices` contiguous pieces, one
// thread block each (grid = slices x rows).  A block streams its piece from HBM exactly once with
// 128-bit loads, applies the penalties (history ids are scattered into a shared-memory bitmap and a
// small hash table of counts first) and the temperature, and keeps the piece's candidates -- every
// score at or above the piece's k-th largest -- in a shared-memory buffer guarded by a running
// threshold: an element is appended only if it beats the threshold, and the buffer is reduced by
// an in-register radix select whenever it fills.  Each block publishes its candidates to the
// handle's workspace and takes a ticket; the block that draws the last ticket of a row merges the
// row's candidates with the same select, sorts the few survivors, and finishes the row: top-p inside
// the top-k by a block scan, the min-p floor, the cut, probabilities, and the draw.  No block waits
// for another.
//
// Semantics follow leat/sampler.py:31-73 and leat/ops.py:496-529 (the exact, sort-based cut).
#pragma once
#include "device_util.cuh"

namespace leat {

enum RowMode : int {
  M_ARGMAX_L = 0,   // greedy: first argmax of the penalised logits
  M_ARGMAX_G = 1,   // no cut set, hashed draw: first argmax of score + gumbel over the whole row
  M_SELECT_K = 2,   // candidates = scores >= the k-th largest
  M_SELECT_MINP = 3,  // candidates = scores >= top + log(min_p)
  M_GENERAL = 4     // needs the multi-pass kernel
};

constexpr int EPT = 16;        // buffer entries a thread holds in registers while the buffer is rebuilt
constexpr int UNROLL = 4;      // vectors per thread per streaming step
constexpr int HASH_EMPTY = -1;

struct KParams {
  const float* logits; int rows; int vocab; long long row_stride; int vocab_total;
  const float* options; int options_rows;
  const float* opt_k; const float* opt_p; const float* opt_m;  // leat_cutoff: separate columns, T = 1
  const uint32_t* seed; int seed_rows; const int* position; int position_rows;
  const uint8_t* seen; long long seen_stride;
  const int* history; const int* history_len; int history_cap;
  const float* penalties; int penalties_rows;
  const float* uniform;
  int vocab_offset; unsigned flags; int force_greedy;
  int* out_ids; int* out_greedy; float* out_cut; int* out_kept;
  float* out_probs; int* out_prob_ids; int out_width; int* status;
  // shard mode: publish the row's candidates instead of finishing it
  float* cand_value; int* cand_id; int* cand_count; unsigned long long* cand_best; int cand_cap;
  // gathered candidates (finish-from-candidates kernel)
  const float* g_value; const int* g_id; const int* g_count; const unsigned long long* g_best; int g_parts;
  // launch plan
  int slices; int slice_len; int cap; int keep; int k_max; int bm_words; int ht_size;
  // workspace
  unsigned long long* ws_keys;  // (rows, slices, keep)
  int* ws_count;                // (rows, slices): candidates published, -1 = could not reduce
  unsigned long long* ws_best;  // (rows, slices): greedy / whole-row argmax key
  float* ws_min;                // (rows, slices): smallest score of the slice
  unsigned* ws_ticket;          // (rows)
  int* ws_flag;                 // (rows): 1 = the row needs the multi-pass kernel
};

struct RowCfg {
  float T, k, p, m, rinv, rep, pres, freq, u, logm;
  int mode, k_eff, has_cut, greedy, track;
  uint32_t rkey;
};

struct Shared {
  int n;                 // entries appended to the buffer (may exceed cap until the next rebuild)
  float tau;             // running threshold on scores
  int overflow;          // the slice / row cannot be reduced to `keep` candidates
  int sel_bin, sel_rem;
  unsigned diff, vmax;
  int is_last;
  unsigned long long best;   // block max of an argmax key
  unsigned long long gbest;  // block max of the greedy key
  unsigned smin;             // block min of score bits (ord32)
  int jstar, ns, pick;
  float kept, total, cut;
};

__device__ __forceinline__ float penalised(float l, int count, const RowCfg& rc) {
  float r = l > 0.0f ? l / rc.rep : l * rc.rep;
  float off = rc.pres + rc.freq * (float)count;
  return r - off;
}

__device__ __forceinline__ float scaled(float l, const RowCfg& rc, bool divide, float tfloor) {
  return divide ? l / tfloor : l * rc.rinv;
}

__device__ inline RowCfg row_config(const KParams& P, int b) {
  RowCfg rc;
  if (P.options) {
    const float* o = P.options + (size_t)(P.options_rows == 1 ? 0 : b) * 5;
    rc.T = o[0]; rc.k = o[1]; rc.p = o[2]; rc.m = o[3]; rc.pres = o[4];
  } else if (P.opt_k) {
    rc.T = 1.0f; rc.k = P.opt_k[b]; rc.p = P.opt_p[b]; rc.m = P.opt_m[b]; rc.pres = 0.0f;
  } else {
    rc.T = 0.0f; rc.k = 0.0f; rc.p = 1.0f; rc.m = 0.0f; rc.pres = 0.0f;
  }
  rc.rep = 1.0f; rc.freq = 0.0f;
  if (P.penalties) {
    const float* q = P.penalties + (size_t)(P.penalties_rows == 1 ? 0 : b) * 3;
    rc.rep = q[0]; rc.pres = q[1]; rc.freq = q[2];
  }
  float tf = fmaxf(rc.T, 1e-6f);
  rc.rinv = 1.0f / tf;
  rc.u = P.uniform ? P.uniform[b] : 0.0f;
  rc.logm = log_ref(rc.m);
  rc.greedy = (P.force_greedy || !(rc.T > 0.0f)) ? 1 : 0;
  rc.has_cut = (rc.k > 0.0f || rc.p < 1.0f || rc.m > 0.0f) ? 1 : 0;
  int V = P.vocab;
  rc.k_eff = (rc.k > 0.0f) ? max(1, (int)fminf(floorf(rc.k), (float)V)) : V;
  uint32_t seed = P.seed ? P.seed[P.seed_rows == 1 ? 0 : b] : 0u;
  int pos = P.position ? P.position[P.position_rows == 1 ? 0 : b] : 0;
  rc.rkey = row_key(seed, pos);
  int vt = P.vocab_total > 0 ? P.vocab_total : V;
  if (rc.greedy) rc.mode = M_ARGMAX_L;
  else if (!rc.has_cut && !P.uniform && vt > P.k_max) rc.mode = M_ARGMAX_G;
  else if (rc.k_eff <= P.k_max) rc.mode = M_SELECT_K;
  else if (!(rc.k > 0.0f) && !(rc.p < 1.0f) && rc.m > 0.0f) rc.mode = M_SELECT_MINP;
  else rc.mode = M_GENERAL;
  rc.track = (P.out_greedy != nullptr || P.cand_best != nullptr || rc.mode == M_ARGMAX_L) ? 1 : 0;
  return rc;
}

// ---- candidate buffer -------------------------------------------------------------------------

// Appends `key` from every thread whose `want` is set; returns false for a thread whose entry did
// not fit (the buffer must then be rebuilt and the append retried).  One atomic per warp.
__device__ __forceinline__ bool buffer_append(unsigned long long* buf, Shared& sm, int cap, bool want,
                                              unsigned long long key) {
  unsigned mask = __ballot_sync(FULL, want);
  if (mask == 0) return true;
  int lane = threadIdx.x & 31;
  int leader = __ffs(mask) - 1;
  int base = 0;
  if (lane == leader) base = atomicAdd(&sm.n, __popc(mask));
  base = __shfl_sync(FULL, base, leader);
  if (!want) return true;
  int slot = base + __popc(mask & ((1u << lane) - 1u));
  if (slot < cap) { buf[slot] = key; return true; }
  return false;
}

// Rebuilds the buffer around a new threshold.  All threads of the block call it together, after a
// barrier that made every append visible.  mode M_SELECT_K: the threshold is the k-th largest
// value held (none if fewer than k are held); mode M_SELECT_MINP: the largest value held plus
// log(min_p).  Every entry at or above the threshold stays; sm.tau becomes the threshold.
__device__ inline void buffer_rebuild(unsigned long long* buf, unsigned* hist, Shared& sm, int cap,
                                      int keep, int mode, int k, float logm) {
  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31;
  const int n = min(sm.n, cap);
  unsigned long long e[EPT];
#pragma unroll
  for (int j = 0; j < EPT; ++j) {
    int i = j * nt + tid;
    e[j] = (i < n) ? buf[i] : 0ull;
  }
  if (tid == 0) { sm.diff = 0u; sm.vmax = 0u; }
  __syncthreads();  // every entry is in registers; sm.n may be reset below
  uint32_t thr = 0u;
  if (mode == M_SELECT_MINP) {
    uint32_t mx = 0u;
#pragma unroll
    for (int j = 0; j < EPT; ++j) mx = max(mx, key_vbits(e[j]));
    mx = __reduce_max_sync(FULL, mx);
    if (lane == 0) atomicMax(&sm.vmax, mx);
    __syncthreads();
    thr = ord32(unord32(sm.vmax) + logm + 0.0f);
  } else if (n > k) {
    const uint32_t ref = key_vbits(buf[0]);
    uint32_t d = 0u;
#pragma unroll
    for (int j = 0; j < EPT; ++j)
      if (e[j]) d |= key_vbits(e[j]) ^ ref;
    d = __reduce_or_sync(FULL, d);
    if (lane == 0 && d) atomicOr(&sm.diff, d);
    __syncthreads();
    const uint32_t diff = sm.diff;
    if (diff == 0u) {
      thr = ref;
    } else {
      int shift = ((31 - __clz(diff)) >> 3) << 3;
      uint32_t known = (shift + 8 >= 32) ? 0u : (0xFFFFFFFFu << (shift + 8));
      uint32_t prefix = ref & known;
      int rem = k;
      for (; shift >= 0; shift -= 8) {
        for (int i = tid; i < 256; i += nt) hist[i] = 0u;
        __syncthreads();
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
          uint32_t v = key_vbits(e[j]);
          if (e[j] && (v & known) == prefix) atomicAdd(&hist[(v >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid < 32) {
          // lane L owns bins 255-8L .. 248-8L, highest first
          unsigned c[8];
          unsigned local = 0;
#pragma unroll
          for (int q = 0; q < 8; ++q) { c[q] = hist[255 - 8 * lane - q]; local += c[q]; }
          unsigned incl = local;
#pragma unroll
          for (int dd = 1; dd < 32; dd <<= 1) {
            unsigned o = __shfl_up_sync(FULL, incl, dd);
            if (lane >= dd) incl += o;
          }
          unsigned excl = incl - local;
          if (excl < (unsigned)rem && (unsigned)rem <= incl) {
            unsigned acc = excl;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              if (acc < (unsigned)rem && (unsigned)rem <= acc + c[q]) {
                sm.sel_bin = 255 - 8 * lane - q;
                sm.sel_rem = rem - (int)acc;
              }
              acc += c[q];
            }
          }
        }
        __syncthreads();
        prefix |= ((uint32_t)sm.sel_bin) << shift;
        known |= 255u << shift;
        rem = sm.sel_rem;
      }
      thr = prefix;
    }
  }
  if (tid == 0) sm.n = 0;
  __syncthreads();
#pragma unroll
  for (int j = 0; j < EPT; ++j) {
    if (j * nt < n) {  // uniform across the block
      bool want = e[j] != 0ull && key_vbits(e[j]) >= thr;
      buffer_append(buf, sm, cap, want, e[j]);
    }
  }
  __syncthreads();
  if (tid == 0) {
    if (thr != 0u) sm.tau = fmaxf(sm.tau, unord32(thr));
    if (sm.n > keep) sm.overflow = 1;
  }
  __syncthreads();
}

// Appends one optional entry per thread, rebuilding the buffer as often as it takes.  Block-wide.
__device__ inline void buffer_push(unsigned long long* buf, unsigned* hist, Shared& sm, int cap, int keep,
                                   int mode, int k, float logm, bool want, unsigned long long key) {
  bool pending = want && key_value(key) >= sm.tau;
  while (true) {
    bool ok = buffer_append(buf, sm, cap, pending, key);
    pending = pending && !ok;
    if (!__syncthreads_or(pending ? 1 : 0)) break;
    buffer_rebuild(buf, hist, sm, cap, keep, mode, k, logm);
    if (sm.overflow) break;
    pending = pending && key_value(key) >= sm.tau;
  }
}

// descending bitonic sort of buf[0..p2), p2 a power of two
__device__ inline void block_sort_desc(unsigned long long* buf, int p2) {
  const int tid = threadIdx.x, nt = blockDim.x;
  for (int k = 2; k <= p2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = tid; i < p2; i += nt) {
        int x = i ^ j;
        if (x > i) {
          unsigned long long a = buf[i], c = buf[x];
          bool desc = (i & k) == 0;
          if (desc ? (a < c) : (a > c)) { buf[i] = c; buf[x] = a; }
        }
      }
      __syncthreads();
    }
  }
}

// ---- finishing a row ----------------------------------------------------------------------------

// buf[0..sm.n) holds the row's candidates (unsorted).  Computes the cut and the draw and writes the
// row's outputs.  fw / fi / fs are float scratch of cap, cap and cap/32 entries.
__device__ inline void finish_row(const KParams& P, const RowCfg& rc, int b, unsigned long long* buf,
                                  Shared& sm, float* fw, float* fi, float* fs, float row_min) {
  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = nt >> 5;
  const int n = sm.n;
  int p2 = 1;
  while (p2 < n) p2 <<= 1;
  for (int i = n + tid; i < p2; i += nt) buf[i] = 0ull;
  if (tid == 0) { sm.jstar = 0; sm.ns = 0; sm.pick = 0x7FFFFFFF; sm.best = 0ull; }
  __syncthreads();
  block_sort_desc(buf, p2);
  const float top = key_value(buf[0]);
  const int in_k = min(rc.k_eff, n);
  const int nseg = (n + 31) >> 5;
  for (int s = warp; s < nseg; s += nwarps) {
    int j = s * 32 + lane;
    float w = 0.0f;
    if (j < n) w = exp_ref(key_value(buf[j]) - top);
    float x = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      float y = __shfl_up_sync(FULL, x, d);
      if (lane >= d) x = x + y;
    }
    if (j < n) { fw[j] = w; fi[j] = x; }
    if (lane == 31) fs[s] = x;
  }
  __syncthreads();
  if (tid == 0) {
    float off = 0.0f;
    for (int s = 0; s < nseg; ++s) { float t = fs[s]; fs[s] = off; off = off + t; }
  }
  __syncthreads();
  for (int j = tid; j < n; j += nt) fi[j] = fs[j >> 5] + fi[j];
  __syncthreads();
  const float kept = fi[in_k - 1];
  const float bound_p = rc.p * kept;
  for (int j = tid; j < in_k; j += nt) {
    float likelier = fi[j] - fw[j];
    if (j == 0 || likelier < bound_p) atomicMax(&sm.jstar, j);
  }
  __syncthreads();
  float base = (rc.p < 1.0f) ? key_value(buf[sm.jstar]) : key_value(buf[in_k - 1]);
  if (rc.mode == M_SELECT_MINP) base = row_min;  // k = 0: the k-th score is the row's last
  float cut = fmaxf(base, top + rc.logm);
  if (!rc.has_cut) cut = neg_inf();
  for (int j = tid; j < n; j += nt) {
    float r = key_value(buf[j]);
    if (r >= cut && (j + 1 == n || !(key_value(buf[j + 1]) >= cut))) sm.ns = j + 1;
  }
  __syncthreads();
  const int ns = max(sm.ns, 1);
  const float total = fi[ns - 1];
  if (P.uniform) {
    const float bound_u = rc.u * total;
    for (int j = tid; j < ns; j += nt)
      if (fi[j] > bound_u) atomicMin(&sm.pick, j);
  } else {
    unsigned long long best = 0ull;
    for (int j = tid; j < ns; j += nt) {
      uint32_t id = (uint32_t)key_id(buf[j]);
      float d = key_value(buf[j]) + gumbel(hashed_uniform(id, rc.rkey));
      unsigned long long kk = make_key(d, id);
      best = kk > best ? kk : best;
    }
    best = warp_max_u64(best);
    if (lane == 0) atomicMax(&sm.best, best);
  }
  __syncthreads();
  if (tid == 0) {
    int id;
    if (P.uniform) id = key_id(buf[min(sm.pick, ns - 1)]);
    else id = key_id(sm.best);
    if (P.out_ids) P.out_ids[b] = id;
    if (P.out_cut) P.out_cut[b] = cut;
    if (P.out_kept) P.out_kept[b] = sm.ns;
    if (P.status && P.out_probs && sm.ns > P.out_width) atomicOr(P.status, 2);
  }
  if (P.out_probs || P.out_prob_ids) {
    for (int j = tid; j < P.out_width; j += nt) {
      if (P.out_probs) P.out_probs[(size_t)b * P.out_width + j] = (j < ns) ? fw[j] / total : 0.0f;
      if (P.out_prob_ids) P.out_prob_ids[(size_t)b * P.out_width + j] = (j < ns) ? key_id(buf[j]) : -1;
    }
  }
}

// A row that did not go through the candidate buffer: greedy, whole-row Gumbel argmax, or one the
// single pass could not reduce.
__device__ inline void finish_simple(const KParams& P, const RowCfg& rc, int b, int mode,
                                     unsigned long long best, unsigned long long gbest, bool failed) {
  if (threadIdx.x != 0) return;
  int id = (mode == M_ARGMAX_L) ? key_id(gbest) : key_id(best);
  if (failed) {
    id = -1;
    if (P.ws_flag && !(P.flags & 2u)) P.ws_flag[b] = 1;
    else if (P.status) atomicOr(P.status, 4);
  }
  if (P.out_ids) P.out_ids[b] = id;
  if (failed) return;
  if (P.out_cut) P.out_cut[b] = (mode == M_ARGMAX_G) ? neg_inf() : quiet_nan();
  if (P.out_kept) P.out_kept[b] = (mode == M_ARGMAX_G) ? P.vocab : 0;
  if (mode == M_ARGMAX_G && P.out_probs && P.status) atomicOr(P.status, 2);
}

__device__ inline void clear_probs(const KParams& P, int b) {
  for (int j = threadIdx.x; j < P.out_width; j += blockDim.x) {
    if (P.out_probs) P.out_probs[(size_t)b * P.out_width + j] = 0.0f;
    if (P.out_prob_ids) P.out_prob_ids[(size_t)b * P.out_width + j] = -1;
  }
}

// ---- the kernel ---------------------------------------------------------------------------------

template <int VEC>
struct Chunk {
  float v[UNROLL * VEC];
  uint32_t seen[UNROLL];  // VEC seen bytes per vector, packed
};

template <int VEC, bool PEN>
__device__ __forceinline__ void load_chunk(Chunk<VEC>& c, const float* __restrict__ row,
                                           const uint8_t* __restrict__ seen_row, int first, int stride,
                                           int end) {
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    int idx = first + u * stride;
    bool in = idx < end;
    if (VEC == 4) {
      float4 t = make_float4(quiet_nan(), quiet_nan(), quiet_nan(), quiet_nan());
      if (in) t = __ldcs(reinterpret_cast<const float4*>(row + idx));
      c.v[u * VEC + 0] = t.x; c.v[u * VEC + 1] = t.y; c.v[u * VEC + 2] = t.z; c.v[u * VEC + 3] = t.w;
      if (PEN) c.seen[u] = (in && seen_row) ? __ldcs(reinterpret_cast<const unsigned*>(seen_row + idx)) : 0u;
    } else {
      c.v[u] = in ? __ldcs(row + idx) : quiet_nan();
      if (PEN) c.seen[u] = (in && seen_row) ? (unsigned)__ldcs(seen_row + idx) : 0u;
    }
  }
}

__device__ __forceinline__ int hash_count(const int* hk, const int* hc, int ht_mask, int id) {
  uint32_t slot = lowbias32((uint32_t)id) & ht_mask;
  for (int probe = 0; probe <= ht_mask; ++probe) {
    int k = hk[slot];
    if (k == id) return hc[slot];
    if (k == HASH_EMPTY) return 0;
    slot = (slot + 1) & ht_mask;
  }
  return 0;
}

template <int VEC, bool PEN>
__global__ void __launch_bounds__(512) sample_kernel(const KParams P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned long long* buf = reinterpret_cast<unsigned long long*>(smem_raw);
  unsigned* hist = reinterpret_cast<unsigned*>(smem_raw + (size_t)P.cap * 8);
  Shared& sm = *reinterpret_cast<Shared*>(hist + 256);
  unsigned char* region = reinterpret_cast<unsigned char*>(hist + 256) + 128;
  static_assert(sizeof(Shared) <= 128, "Shared must fit its slot");
  unsigned* bitmap = reinterpret_cast<unsigned*>(region);
  int* hkeys = reinterpret_cast<int*>(bitmap + P.bm_words);
  int* hcnt = hkeys + P.ht_size;
  float* fw = reinterpret_cast<float*>(region);
  float* fi = fw + P.cap;
  float* fs = fi + P.cap;

  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31;
  const int b = blockIdx.y, slice = blockIdx.x, S = P.slices;
  const RowCfg rc = row_config(P, b);
  const int mode = rc.mode;
  const bool divide = (P.flags & 1u) != 0u;
  const float tfloor = fmaxf(rc.T, 1e-6f);
  const int begin = slice * P.slice_len;
  const int end = min(P.vocab, begin + P.slice_len);
  const float* row = P.logits + (size_t)b * P.row_stride;
  const uint8_t* seen_row = (PEN && P.seen) ? P.seen + (size_t)b * P.seen_stride : nullptr;

  if (tid == 0) {
    sm.n = 0; sm.tau = neg_inf(); sm.overflow = 0; sm.best = 0ull; sm.gbest = 0ull;
    sm.smin = 0xFFFFFFFFu; sm.is_last = (S == 1);
  }
  const int ht_mask = P.ht_size - 1;
  if (PEN) {
    for (int i = tid; i < P.bm_words; i += nt) bitmap[i] = 0u;
    for (int i = tid; i < P.ht_size; i += nt) { hkeys[i] = HASH_EMPTY; hcnt[i] = 0; }
  }
  __syncthreads();
  if (PEN && P.history) {
    const int hl = P.history_len ? min(P.history_len[b], P.history_cap) : P.history_cap;
    const int* h = P.history + (size_t)b * P.history_cap;
    for (int i = tid; i < hl; i += nt) {
      int id = h[i] - P.vocab_offset;
      if (id >= begin && id < end) {
        int local = id - begin;
        atomicOr(&bitmap[local >> 5], 1u << (local & 31));
        uint32_t slot = lowbias32((uint32_t)id) & ht_mask;
        for (int probe = 0; probe <= ht_mask; ++probe) {
          int old = atomicCAS(&hkeys[slot], HASH_EMPTY, id);
          if (old == HASH_EMPTY || old == id) { atomicAdd(&hcnt[slot], 1); break; }
          slot = (slot + 1) & ht_mask;
        }
      }
    }
    __syncthreads();
  }

  // ---- stream the slice once ----
  float gl = neg_inf();     // this thread's best penalised logit and where
  int gid = 0x7FFFFFFF;
  float al = neg_inf();     // this thread's best score + gumbel and where
  int aid = 0x7FFFFFFF;
  float mn = __uint_as_float(0x7F800000u);  // this thread's smallest score
  if (mode != M_GENERAL) {
    const int stride = nt * VEC;
    const int span = stride * UNROLL;
    Chunk<VEC> cur, nxt;
    load_chunk<VEC, PEN>(cur, row, seen_row, begin + tid * VEC, stride, end);
    for (int base = begin; base < end; base += span) {
      const int first = base + tid * VEC;
      if (base + span < end) load_chunk<VEC, PEN>(nxt, row, seen_row, first + span, stride, end);
      float tau = sm.tau;
      unsigned pend = 0u;
      float sv[UNROLL * VEC];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int idx = first + u * stride;
        unsigned hbits = 0u;
        if (PEN) {
          int local = idx - begin;
          if (idx < end) {
            if (P.history) hbits = (bitmap[local >> 5] >> (local & 31)) & ((1u << VEC) - 1u);
          }
        }
#pragma unroll
        for (int c = 0; c < VEC; ++c) {
          float l = cur.v[u * VEC + c];
          if (PEN) {
            unsigned sbyte = (cur.seen[u] >> (8 * c)) & 255u;
            if (((hbits >> c) & 1u) | sbyte) {
              int cnt = ((hbits >> c) & 1u) ? hash_count(hkeys, hcnt, ht_mask, idx + c) : 0;
              cnt = max(cnt, sbyte ? 1 : 0);
              l = penalised(l, cnt, rc);
            }
          }
          if (rc.track && l > gl) { gl = l; gid = idx + c; }
          float s = scaled(l, rc, divide, tfloor);
          sv[u * VEC + c] = s;
          if (mode == M_ARGMAX_G) {
            if (idx + c < end) {
              float d = s + gumbel(hashed_uniform((uint32_t)(idx + c + P.vocab_offset), rc.rkey));
              if (d > al) { al = d; aid = idx + c; }
            }
          } else if (mode >= M_SELECT_K) {
            if (s >= tau) pend |= 1u << (u * VEC + c);
            if (mode == M_SELECT_MINP) mn = fminf(mn, s);
          }
        }
      }
      if (mode >= M_SELECT_K) {
        while (true) {
          if (__any_sync(FULL, pend != 0u)) {
#pragma unroll
            for (int q = 0; q < UNROLL * VEC; ++q) {
              bool want = (pend >> q) & 1u;
              int id = first + (q / VEC) * stride + (q % VEC) + P.vocab_offset;
              if (buffer_append(buf, sm, P.cap, want, make_key(sv[q], (uint32_t)id))) pend &= ~(1u << q);
            }
          }
          if (!__syncthreads_or(pend != 0u)) break;
          buffer_rebuild(buf, hist, sm, P.cap, P.keep, mode, rc.k_eff, rc.logm);
          if (sm.overflow) { pend = 0u; break; }
          tau = sm.tau;
#pragma unroll
          for (int q = 0; q < UNROLL * VEC; ++q)
            if (!(sv[q] >= tau)) pend &= ~(1u << q);
        }
        if (sm.overflow) break;
      }
      cur = nxt;
    }
  }
  __syncthreads();

  // ---- reduce what the slice found ----
  if (rc.track) {
    unsigned long long g = (gid != 0x7FFFFFFF) ? make_key(gl, (uint32_t)(gid + P.vocab_offset)) : 0ull;
    g = warp_max_u64(g);
    if (lane == 0) atomicMax(&sm.gbest, g);
  }
  if (mode == M_ARGMAX_G) {
    unsigned long long a = (aid != 0x7FFFFFFF) ? make_key(al, (uint32_t)(aid + P.vocab_offset)) : 0ull;
    a = warp_max_u64(a);
    if (lane == 0) atomicMax(&sm.best, a);
  }
  if (mode == M_SELECT_MINP) {
    unsigned m = __reduce_min_sync(FULL, ord32(mn));
    if (lane == 0) atomicMin(&sm.smin, m);
  }
  __syncthreads();
  if (mode >= M_SELECT_K && mode != M_GENERAL && !sm.overflow) {
    if (mode == M_SELECT_MINP || sm.n > rc.k_eff)
      buffer_rebuild(buf, hist, sm, P.cap, P.keep, mode, rc.k_eff, rc.logm);
  }
  bool failed = (mode == M_GENERAL) || sm.overflow;

  // ---- publish, and let the last block of the row go on ----
  if (S > 1) {
    const size_t cell = (size_t)b * S + slice;
    if (mode >= M_SELECT_K && !failed) {
      const int n = sm.n;
      unsigned long long* dst = P.ws_keys + cell * P.keep;
      for (int i = tid; i < n; i += nt) dst[i] = buf[i];
    }
    if (tid == 0) {
      P.ws_count[cell] = failed ? -1 : sm.n;
      P.ws_best[cell * 2 + 0] = sm.gbest;
      P.ws_best[cell * 2 + 1] = sm.best;
      P.ws_min[cell] = unord32(sm.smin);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      unsigned t = atomicAdd(&P.ws_ticket[b], 1u);
      sm.is_last = (t == (unsigned)(S - 1));
      if (sm.is_last) P.ws_ticket[b] = 0u;
    }
    __syncthreads();
    if (!sm.is_last) return;
    __threadfence();
    // merge the row's slices
    if (tid == 0) { sm.n = 0; sm.tau = neg_inf(); sm.overflow = 0; sm.smin = 0xFFFFFFFFu; }
    __syncthreads();
    unsigned long long g = 0ull, a = 0ull;
    unsigned mnb = 0xFFFFFFFFu;
    int bad = 0;
    for (int j = tid; j < S; j += nt) {
      const size_t c2 = (size_t)b * S + j;
      unsigned long long gj = __ldcg(&P.ws_best[c2 * 2 + 0]), aj = __ldcg(&P.ws_best[c2 * 2 + 1]);
      g = gj > g ? gj : g;
      a = aj > a ? aj : a;
      mnb = min(mnb, ord32(__ldcg(&P.ws_min[c2])));
      if (__ldcg(&P.ws_count[c2]) < 0) bad = 1;
    }
    g = warp_max_u64(g);
    a = warp_max_u64(a);
    mnb = __reduce_min_sync(FULL, mnb);
    if (lane == 0) { atomicMax(&sm.gbest, g); atomicMax(&sm.best, a); atomicMin(&sm.smin, mnb); }
    failed = __syncthreads_or(bad) != 0;
    if (mode >= M_SELECT_K && !failed) {
      const int total_slots = S * P.keep;
      for (int base = 0; base < total_slots; base += nt) {
        int i = base + tid;
        int j = i / P.keep, q = i - j * P.keep;
        bool want = false;
        unsigned long long key = 0ull;
        if (i < total_slots && q < __ldcg(&P.ws_count[(size_t)b * S + j])) {
          key = __ldcg(&P.ws_keys[((size_t)b * S + j) * P.keep + q]);
          want = true;
        }
        buffer_push(buf, hist, sm, P.cap, P.keep, mode, rc.k_eff, rc.logm, want, key);
        if (sm.overflow) break;
      }
      __syncthreads();
      if (!sm.overflow && (mode == M_SELECT_MINP || sm.n > rc.k_eff))
        buffer_rebuild(buf, hist, sm, P.cap, P.keep, mode, rc.k_eff, rc.logm);
      failed = sm.overflow != 0;
    }
  }
  __syncthreads();

  // ---- the row is whole in this block ----
  if (P.cand_count) {  // shard mode: hand the row's candidates to the gather
    const int cap = P.cand_cap;
    int n = 0;
    if (!failed && mode >= M_SELECT_K) {
      n = sm.n;
      if (n > cap) { n = 0; failed = true; }
      for (int i = tid; i < n; i += nt) {
        P.cand_value[(size_t)b * cap + i] = key_value(buf[i]);
        P.cand_id[(size_t)b * cap + i] = key_id(buf[i]);
      }
    } else if (!failed && mode == M_ARGMAX_G) {
      n = 1;
      if (tid == 0) {
        P.cand_value[(size_t)b * cap] = key_value(sm.best);
        P.cand_id[(size_t)b * cap] = key_id(sm.best);
      }
    }
    if (tid == 0) {
      P.cand_count[b] = failed ? -1 : n;
      P.cand_best[b] = sm.gbest;
    }
    return;
  }
  if (tid == 0 && P.out_greedy) P.out_greedy[b] = key_id(sm.gbest);
  if (failed || mode < M_SELECT_K) {
    finish_simple(P, rc, b, mode, sm.best, sm.gbest, failed);
    clear_probs(P, b);
    return;
  }
  finish_row(P, rc, b, buf, sm, fw, fi, fs, unord32(sm.smin));
}

// Finishes rows from candidates gathered from `g_parts` vocabulary slices: one block per row.
__global__ void __launch_bounds__(512) finish_candidates_kernel(const KParams P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned long long* buf = reinterpret_cast<unsigned long long*>(smem_raw);
  unsigned* hist = reinterpret_cast<unsigned*>(smem_raw + (size_t)P.cap * 8);
  Shared& sm = *reinterpret_cast<Shared*>(hist + 256);
  unsigned char* region = reinterpret_cast<unsigned char*>(hist + 256) + 128;
  float* fw = reinterpret_cast<float*>(region);
  float* fi = fw + P.cap;
  float* fs = fi + P.cap;
  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31;
  const int b = blockIdx.x, parts = P.g_parts, cap = P.cand_cap, rows = P.rows;
  const RowCfg rc = row_config(P, b);
  const int mode = rc.mode;
  if (tid == 0) {
    sm.n = 0; sm.tau = neg_inf(); sm.overflow = 0; sm.best = 0ull; sm.gbest = 0ull; sm.smin = 0u;
  }
  __syncthreads();
  unsigned long long g = 0ull;
  int bad = 0;
  for (int j = tid; j < parts; j += nt) {
    unsigned long long gj = P.g_best[(size_t)j * rows + b];
    g = gj > g ? gj : g;
    if (P.g_count[(size_t)j * rows + b] < 0) bad = 1;
  }
  g = warp_max_u64(g);
  if (lane == 0) atomicMax(&sm.gbest, g);
  bool failed = __syncthreads_or(bad) != 0 || mode == M_GENERAL;
  if (tid == 0 && P.out_greedy) P.out_greedy[b] = key_id(sm.gbest);
  if (!failed && mode == M_ARGMAX_G) {
    unsigned long long a = 0ull;
    for (int j = tid; j < parts; j += nt) {
      size_t at = ((size_t)j * rows + b) * cap;
      unsigned long long kk = make_key(P.g_value[at], (uint32_t)P.g_id[at]);
      a = kk > a ? kk : a;
    }
    a = warp_max_u64(a);
    if (lane == 0) atomicMax(&sm.best, a);
    __syncthreads();
  }
  if (!failed && mode >= M_SELECT_K) {
    const int total_slots = parts * cap;
    for (int base = 0; base < total_slots; base += nt) {
      int i = base + tid;
      int j = i / cap, q = i - j * cap;
      bool want = false;
      unsigned long long key = 0ull;
      if (i < total_slots && q < P.g_count[(size_t)j * rows + b]) {
        size_t at = ((size_t)j * rows + b) * cap + q;
        key = make_key(P.g_value[at], (uint32_t)P.g_id[at]);
        want = true;
      }
      buffer_push(buf, hist, sm, P.cap, P.keep, mode, rc.k_eff, rc.logm, want, key);
      if (sm.overflow) break;
    }
    __syncthreads();
    if (!sm.overflow && (mode == M_SELECT_MINP || sm.n > rc.k_eff))
      buffer_rebuild(buf, hist, sm, P.cap, P.keep, mode, rc.k_eff, rc.logm);
    failed = sm.overflow != 0;
  }
  __syncthreads();
  if (failed || mode < M_SELECT_K) {
    KParams Q = P;
    Q.ws_flag = nullptr;
    finish_simple(Q, rc, b, mode, sm.best, sm.gbest, failed);
    clear_probs(P, b);
    return;
  }
  // the smallest score of the whole row is not gathered: with min_p alone the cut reported is
  // top + log(min_p), which keeps the same survivors
  finish_row(P, rc, b, buf, sm, fw, fi, fs, neg_inf());
}

// leat/engine.py:612-626 on the device: one thread per sequence
__global__ void verify_kernel(const int* __restrict__ drafted, const int* __restrict__ sampled,
                              const int* __restrict__ greedy, int n, int drafts, int* accepted,
                              int* tokens) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int ran = drafts + 1;
  const int* against = greedy ? greedy : sampled;
  int kept = drafts;
  for (int j = 0; j < drafts; ++j) {
    if (drafted[(size_t)i * drafts + j] != against[(size_t)i * ran + j]) { kept = j; break; }
  }
  accepted[i] = kept;
  for (int j = 0; j < ran; ++j) {
    int t = -1;
    if (j < kept) t = greedy ? drafted[(size_t)i * drafts + j] : sampled[(size_t)i * ran + j];
    else if (j == kept) t = sampled[(size_t)i * ran + j];
    tokens[(size_t)i * ran + j] = t;
  }
}

}  // namespace leat
