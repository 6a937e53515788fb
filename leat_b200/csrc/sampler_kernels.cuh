// The sampler's kernels for sm_100a.
//
// sample_kernel settles rows.  Its grid is (slices, rows); what a block does depends on the row:
//
//   * A row with a list (filter_path.cuh: a floor per row, every logit compared with it once by
//     filter_kernel, the few at or above it listed in the workspace) needs one block: history
//     tokens are marked in a shared-memory bitmap (or counted in a hash table), the listed logits
//     are penalised, scaled and become (score, id) keys in the candidate buffer, and the row is
//     finished.  The other blocks of the row return at once.
//   * Any other row is cut into `slices` contiguous pieces, one block each.  A block streams its
//     piece from HBM exactly once (through a ring of bulk asynchronous copies, stream_ring.cuh, or
//     with plain loads), comparing raw logits against a conservative threshold; the few that pass
//     go to the candidate buffer, which is rebuilt around the k-th largest score by a
//     coarse-to-fine select whenever it fills.  Each block publishes its candidates to the handle's
//     workspace and takes a ticket; the block that draws a row's last ticket merges them.
//
// Finishing a row (finish_row): sort the few hundred candidates, top-p inside the top-k by a block
// scan, the min-p floor, the cut, probabilities, and the draw.  A row neither way can settle is
// redone exactly by the multi-pass routine (general_kernel.cuh) in the same block.  No block ever
// waits for another block.
//
// Semantics follow leat/sampler.py:31-73 and leat/ops.py:496-529 (the exact, sort-based cut).
#pragma once
#include "device_util.cuh"

namespace leat {

enum RowMode : int {
  M_ARGMAX_L = 0,     // greedy: first argmax of the penalised logits
  M_ARGMAX_G = 1,     // no cut set, hashed draw: first argmax of score + gumbel over the whole row
  M_SELECT_K = 2,     // candidates = scores >= the k-th largest
  M_SELECT_MINP = 3,  // candidates = scores >= top + log(min_p)
  M_GENERAL = 4       // needs the multi-pass kernel
};

constexpr int UNROLL = 4;  // vectors per thread per streaming step
constexpr int BINS = 2048;  // buckets of one select step
constexpr int SMEM_FIXED = 768;  // Shared (256 bytes), Ctx, RowCfg, the ring's mbarriers and History (128 bytes each)
constexpr int MAX_RING_STAGES = 8;
constexpr int HASH_EMPTY = -1;
constexpr int NO_ID = 0x7FFFFFFF;
constexpr float GUMBEL_MAX = 17.0f;  // above -log(-log(1 - 2^-24)) = 16.64

#include "shard_exchange.cuh"

struct KParams {
  const float* logits; int rows; int vocab; long long row_stride; int vocab_total;
  int dtype;  // what `logits` really points at: 0 float32, 1 bfloat16, 2 float16 (row_stride in logits)
  const float* options; int options_rows;
  const float* opt_k; const float* opt_p; const float* opt_m;  // leat_cutoff: separate columns, T = 1
  const uint32_t* seed; int seed_rows; const int* position; int position_rows;
  const uint8_t* seen; long long seen_stride;
  const int* history; const int* history_len; int history_cap;
  const float* penalties; int penalties_rows;
  const float* uniform;
  int vocab_offset; unsigned flags; int force_greedy;
  float softcap;        // the model's soft cap on its logits (0: none)
  int position_scalar;  // every row's position when `position` is null
  int* out_ids; int* out_greedy; float* out_cut; int* out_kept;
  float* out_probs; int* out_prob_ids; int out_width; int* status;
  // shard mode: publish the row's candidates instead of finishing it
  float* cand_value; int* cand_id; int* cand_count; unsigned long long* cand_best; int cand_cap;
  // gathered candidates (finish-from-candidates kernel)
  const float* g_value; const int* g_id; const int* g_count; const unsigned long long* g_best; int g_parts;
  // distance between two parts' arrays, in elements of each array (dense arrays or packed records)
  long long g_stride_value, g_stride_id, g_stride_count, g_stride_best;
  // launch plan
  int slices; int slice_len; int cap; int keep; int k_max; int bm_words; int ht_size; int ring_stages;
  // workspace
  unsigned long long* ws_keys;  // (rows, slices, keep)
  int* ws_count;                // (rows, slices): candidates published, -1 = could not reduce
  unsigned long long* ws_best;  // (rows, slices, 2): greedy key, whole-row argmax key
  float* ws_min;                // (rows, slices): smallest score of the slice
  unsigned* ws_ticket;          // (rows)
  int* ws_flag;                 // (rows): 1 = the row needs the multi-pass kernel
  // the filter path: per row a floor, and the list of (logit, index) pairs at or above it
  unsigned long long* list; int* list_count; int list_cap;
  unsigned long long* list_info;  // (rows): floor, flag and mark of the row (filter_path.cuh)
  // a second pass over the rows a shard's list could not settle: only rows with only_rows[b] == -2
  const int* only_rows;
  // finish_list_kernel runs before sample_kernel and takes the rows lean_takes() names; words of
  // its area behind the keys, slots of its hash table of history tokens
  int lean; int fl_area_words; int fl_ht;
  // measurement aid (device_util.cuh: stamp_begin / stamp_end), or null
  unsigned long long* stamps;
  // vocabulary shards with a peer exchange (shard_exchange.cuh); world = 0: not in use
  ShardView shard;
};

struct RowCfg {
  float T, k, p, m, rinv, tf, rep, pres, freq, u, logm;
  int mode, k_eff, has_cut, greedy, track, divide;
  int lowers;  // the penalties can only lower a logit (repetition >= 1, presence and frequency >= 0)
  uint32_t rkey;
};

struct Shared {
  int n;         // entries in the buffer (may run past cap until the next rebuild)
  int conv;      // entries [0, conv) are (score, id) keys; the rest may be raw (logit, index) pairs
  int valid;     // live entries counted by a rebuild
  int m;         // entries staged by a rebuild
  float tau;     // running threshold on scores
  int overflow;  // the slice / row cannot be reduced to `keep` candidates
  int sel_bin, sel_above, sel_count;
  unsigned vmin, vmax, smin2, rmin, rmax;
  int is_last;
  unsigned long long best;   // block max of an argmax key
  unsigned long long gbest;  // block max of the greedy key
  unsigned smin;             // block min of score bits (ord32)
  int jstar, ns, pick, nstrict;
  int redo;  // the finish found the row's list wanting: the multi-pass routine takes the row
  float floor_l, s_floor;  // the filter's floor of a listed row (+inf otherwise) and its score
  int wcount[32];  // raw entries each warp holds in its own region of the buffer
  // the block's best so far, as order-preserving bits: what a logit must reach to be looked at
  unsigned share_greedy, share_gumbel, share_min;
};

// what the candidate buffer needs, by value in registers
struct Ctx {
  unsigned long long* buf;
  unsigned long long* stage;
  unsigned* hist;
  Shared* sm;
  int cap, keep, mode, k;
  float logm;
  // raw appends: the stream stores (logit bits, index) and the rebuild turns them into keys
  int divide, off, begin;
  int region;  // raw slots per warp, after the first `keep` slots of the buffer
  float rinv, tf;
  const int* hkeys;  // hash table of the slice's history tokens (their raw entries are dropped), or null
  int hmask;
};

// is token `idx` one of the slice's history tokens?  (open addressing, keys only)
__device__ __forceinline__ bool in_history(const int* keys, int mask, int idx) {
  uint32_t slot = lowbias32((uint32_t)idx) & mask;
#pragma unroll 1
  for (int probe = 0; probe <= mask; ++probe) {
    const int k = keys[slot];
    if (k == idx) return true;
    if (k == -1) return false;
    slot = (slot + 1) & mask;
  }
  return false;
}

__device__ __forceinline__ float penalised(float l, int count, const RowCfg& rc) {
  float r = l > 0.0f ? l / rc.rep : l * rc.rep;
  float off = rc.pres + rc.freq * (float)count;
  return r - off;
}

// the model's soft cap, tanh(l / cap) * cap (leat/model.py:419-423), in double precision and rounded
// once, so that the CPU statement of it gives the same float; monotone, so a raw logit under a
// row's floor is, capped, at or under the capped floor
__device__ __forceinline__ float soft_capped(float l, float cap) {
  return cap > 0.0f ? (float)(tanh((double)l / (double)cap) * (double)cap) : l;
}

__device__ __forceinline__ float scaled(float l, const RowCfg& rc) {
  return rc.divide ? l / rc.tf : l * rc.rinv;
}

// a raw logit below this cannot reach score `tau` (conservative: the exact test follows)
__device__ __forceinline__ float logit_floor(float tau, float tf) {
  if (!(tau > neg_inf())) return neg_inf();
  float g = tau * tf;
  return g - fabsf(g) * 9.5367431640625e-07f - 1e-37f;
}

// a row's raw inputs, before anything is derived from them
struct RowIn {
  float T, k, p, m, pres, rep, freq, u;
  uint32_t seed;
  int pos;
};

__device__ inline RowIn row_inputs(const KParams& P, int b) {
  RowIn in;
  if (P.options) {
    const float* o = P.options + (size_t)(P.options_rows == 1 ? 0 : b) * 5;
    in.T = o[0]; in.k = o[1]; in.p = o[2]; in.m = o[3]; in.pres = o[4];
  } else if (P.opt_k) {
    in.T = 1.0f; in.k = P.opt_k[b]; in.p = P.opt_p[b]; in.m = P.opt_m[b]; in.pres = 0.0f;
  } else {
    in.T = 0.0f; in.k = 0.0f; in.p = 1.0f; in.m = 0.0f; in.pres = 0.0f;
  }
  in.rep = 1.0f; in.freq = 0.0f;
  if (P.penalties) {
    const float* q = P.penalties + (size_t)(P.penalties_rows == 1 ? 0 : b) * 3;
    in.rep = q[0]; in.pres = q[1]; in.freq = q[2];
  }
  in.u = P.uniform ? P.uniform[b] : 0.0f;
  in.seed = P.seed ? P.seed[P.seed_rows == 1 ? 0 : b] : 0u;
  in.pos = P.position ? P.position[P.position_rows == 1 ? 0 : b] : P.position_scalar;
  return in;
}

// The same inputs, fetched by a whole warp at once: every word comes from a lane of its own, so
// the loads overlap instead of following one another.  `extra` (may be null) is one more word to
// fetch alongside; it comes back in extra_out.
__device__ inline uint32_t row_inputs_word(const KParams& P, int b, const void* extra) {
  const int lane = threadIdx.x & 31;
  const uint32_t* src = nullptr;
  if (lane < 5) {
    if (P.options) src = reinterpret_cast<const uint32_t*>(P.options + (size_t)(P.options_rows == 1 ? 0 : b) * 5 + lane);
    else if (P.opt_k && lane == 1) src = reinterpret_cast<const uint32_t*>(P.opt_k + b);
    else if (P.opt_k && lane == 2) src = reinterpret_cast<const uint32_t*>(P.opt_p + b);
    else if (P.opt_k && lane == 3) src = reinterpret_cast<const uint32_t*>(P.opt_m + b);
  } else if (lane < 8) {
    if (P.penalties) src = reinterpret_cast<const uint32_t*>(P.penalties + (size_t)(P.penalties_rows == 1 ? 0 : b) * 3 + (lane - 5));
  } else if (lane == 8) {
    if (P.uniform) src = reinterpret_cast<const uint32_t*>(P.uniform + b);
  } else if (lane == 9) {
    if (P.seed) src = P.seed + (P.seed_rows == 1 ? 0 : b);
  } else if (lane == 10) {
    if (P.position) src = reinterpret_cast<const uint32_t*>(P.position + (P.position_rows == 1 ? 0 : b));
  } else if (lane == 11) {
    src = reinterpret_cast<const uint32_t*>(extra);
  }
  // (the extra word is another kernel's output: read past L1)
  return src ? (lane == 11 ? __ldcg(src) : *src) : 0u;
}
// ... and handed round: `w` is what row_inputs_word() gave this lane (a caller with other loads to
// issue puts them between the two, so that one wait covers both)
__device__ inline RowIn row_inputs_from(const KParams& P, uint32_t w, uint32_t& extra_out) {
  uint32_t v[12];
#pragma unroll
  for (int i = 0; i < 12; ++i) v[i] = __shfl_sync(FULL, w, i);
  RowIn in;
  if (P.options) {
    in.T = __uint_as_float(v[0]); in.k = __uint_as_float(v[1]); in.p = __uint_as_float(v[2]);
    in.m = __uint_as_float(v[3]); in.pres = __uint_as_float(v[4]);
  } else if (P.opt_k) {
    in.T = 1.0f; in.k = __uint_as_float(v[1]); in.p = __uint_as_float(v[2]); in.m = __uint_as_float(v[3]); in.pres = 0.0f;
  } else {
    in.T = 0.0f; in.k = 0.0f; in.p = 1.0f; in.m = 0.0f; in.pres = 0.0f;
  }
  in.rep = 1.0f; in.freq = 0.0f;
  if (P.penalties) { in.rep = __uint_as_float(v[5]); in.pres = __uint_as_float(v[6]); in.freq = __uint_as_float(v[7]); }
  in.u = __uint_as_float(v[8]);
  in.seed = v[9];
  in.pos = P.position ? (int)v[10] : P.position_scalar;
  extra_out = v[11];
  return in;
}
__device__ inline RowIn row_inputs_warp(const KParams& P, int b, const void* extra, uint32_t& extra_out) {
  return row_inputs_from(P, row_inputs_word(P, b, extra), extra_out);
}

__device__ inline RowCfg row_config_from(const KParams& P, const RowIn& in) {
  RowCfg rc;
  rc.T = in.T; rc.k = in.k; rc.p = in.p; rc.m = in.m; rc.pres = in.pres; rc.rep = in.rep; rc.freq = in.freq;
  rc.lowers = (rc.rep >= 1.0f && rc.pres >= 0.0f && rc.freq >= 0.0f) ? 1 : 0;
  rc.tf = fmaxf(rc.T, 1e-6f);
  rc.rinv = 1.0f / rc.tf;
  rc.divide = (P.flags & 1u) ? 1 : 0;
  rc.u = in.u;
  rc.logm = log_ref(rc.m);
  rc.greedy = (P.force_greedy || !(rc.T > 0.0f)) ? 1 : 0;
  rc.has_cut = (rc.k > 0.0f || rc.p < 1.0f || rc.m > 0.0f) ? 1 : 0;
  int V = P.vocab;
  rc.k_eff = (rc.k > 0.0f) ? max(1, (int)fminf(floorf(rc.k), (float)V)) : V;
  rc.rkey = row_key(in.seed, in.pos);
  int vt = P.vocab_total > 0 ? P.vocab_total : V;
  if (rc.greedy) rc.mode = M_ARGMAX_L;
  else if (!rc.has_cut && !P.uniform && vt > P.k_max) rc.mode = M_ARGMAX_G;
  else if (rc.k_eff <= P.k_max) rc.mode = M_SELECT_K;
  else if (!(rc.k > 0.0f) && !(rc.p < 1.0f) && rc.m > 0.0f) rc.mode = M_SELECT_MINP;
  else rc.mode = M_GENERAL;
  rc.track = (P.out_greedy != nullptr || P.cand_best != nullptr || P.shard.world > 0 || rc.mode == M_ARGMAX_L) ? 1 : 0;
  return rc;
}

__device__ inline RowCfg row_config(const KParams& P, int b) { return row_config_from(P, row_inputs(P, b)); }

// ---- candidate buffer -------------------------------------------------------------------------

// Appends `key` from every lane whose `want` is set; false for a lane whose entry did not fit.
// The whole warp calls it together.  One shared-memory atomic per warp.
__device__ __forceinline__ bool warp_append(unsigned long long* dst, int* counter, int limit, bool want,
                                            unsigned long long key) {
  unsigned mask = __ballot_sync(FULL, want);
  if (mask == 0) return true;
  int lane = threadIdx.x & 31;
  int leader = __ffs(mask) - 1;
  int base = 0;
  if (lane == leader) base = atomicAdd(counter, __popc(mask));
  base = __shfl_sync(FULL, base, leader);
  if (!want) return true;
  int slot = base + __popc(mask & ((1u << lane) - 1u));
  if (slot < limit) { dst[slot] = key; return true; }
  return false;
}

// One bucket per score: linear in value between `low_v` and the largest score held when `scale` is
// positive, else by the score's bits above `lo`.
__device__ __forceinline__ int bucket_of(uint32_t v, float low_v, float scale, uint32_t lo, int shift) {
  if (scale > 0.0f) return min(BINS - 1, max(0, (int)((unord32(v) - low_v) * scale)));
  return (int)((v - lo) >> shift);
}

// Rebuilds the buffer around a new threshold.  All threads of the block call it together, after a
// barrier that made every append visible.  M_SELECT_K: the threshold is a score with at least k
// and little more than k entries at or above it (at most `keep`), found coarse to fine over 2048
// buckets: by value first, so that scores spread evenly and the counting atomics rarely meet, then
// by the chosen bucket's bits.  M_SELECT_MINP: the largest score held plus log(min_p).  Every entry
// at or above the threshold stays; sm.tau becomes the threshold.
//
// `raw` bit 0 (raw mode): slots [0, conv) hold keys and warp w's raw (logit, index) pairs sit in
// [keep + w * region, ... + wcount[w]); every other slot is ignored.  Otherwise slots [0, n) hold
// keys.  `raw` bit 1: a slice's last rebuild before it publishes: if little more than k entries are
// live they all stay (the row's last block selects among all slices' anyway).  On entry the histogram is zero and vmin / vmax / m / valid are reset (kernel start and the
// end of every rebuild see to that), which keeps the barriers down to five.
__device__ __noinline__ void buffer_rebuild(const Ctx& c, int raw) {
  Shared& sm = *c.sm;
  unsigned long long* buf = c.buf;
  unsigned* hist = c.hist;
  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, nwarps = nt >> 5;
  const int region = c.region;
  const int conv = sm.conv;
  const int n = (raw & 1) ? c.keep + nwarps * region : min(sm.n, c.cap);
  // ---- A: make raw pairs keys; smallest, largest and number of live keys ----
  {
    const float tau = sm.tau;
    uint32_t mx = 0u, mn = 0xFFFFFFFFu;
    int live = 0;
#pragma unroll 1
    for (int i = tid; i < n; i += nt) {
      unsigned long long key = 0ull;
      if (!(raw & 1) || i < conv) {
        key = buf[i];
      } else if (i >= c.keep) {
        // a history token's raw logit is dropped (the history pass gave its penalised one), and
        // so is anything below the threshold it was appended under
        const int w = (i - c.keep) / region;
        if ((i - c.keep) - w * region < sm.wcount[w]) {
          const unsigned long long pair = buf[i];
          const float l = __uint_as_float((uint32_t)(pair >> 32));
          const int idx = (int)(uint32_t)pair;
          bool drop = false;
          if (c.hkeys) drop = in_history(c.hkeys, c.hmask, idx);
          const float sc = c.divide ? l / c.tf : l * c.rinv;
          if (!drop && sc >= tau) key = make_key(sc, (uint32_t)(idx + c.off));
        }
      }
      if (raw & 1) buf[i] = key;
      if (key) {
        const uint32_t v = key_vbits(key);
        mx = max(mx, v);
        mn = min(mn, v);
        live += 1;
      }
    }
    mx = __reduce_max_sync(FULL, mx);
    mn = __reduce_min_sync(FULL, mn);
    live = __reduce_add_sync(FULL, live);
    if (lane == 0 && live) { atomicMax(&sm.vmax, mx); atomicMin(&sm.vmin, mn); atomicAdd(&sm.valid, live); }
  }
  __syncthreads();
  const int live = sm.valid;
  uint32_t lo = sm.vmin, hi = sm.vmax;  // the k-th largest lies in [lo, hi]
  uint32_t thr = 1u;                    // keep every live entry (key bits of any score exceed 0)
  float low_v = 0.0f, scale = 0.0f;     // the bucket function of the accepted step
  int shift = 0, chosen = 0;
  bool by_bucket = false;
  if (live > 0 && c.mode == M_SELECT_MINP) {
    thr = ord32(unord32(hi) + c.logm + 0.0f);
  } else if (live > c.k && !((raw & 2) && live <= c.k + max(8, c.k >> 3))) {
    unsigned above = 0u;           // entries above hi
    unsigned rem = (unsigned)c.k;  // the one sought is the rem-th largest within [lo, hi]
    const float top_v = unord32(hi);
    low_v = fmaxf(unord32(lo), top_v - 64.0f);
    scale = (float)(BINS - 1) / (top_v - low_v);
    if (!(top_v > low_v && scale > 0.0f && scale < 3.0e38f)) scale = 0.0f;
#pragma unroll 1
    for (int pass = 0; pass < 5; ++pass) {
      if (hi == lo) { thr = lo; by_bucket = false; break; }
      const int bits = 32 - __clz(hi - lo);
      shift = bits > 11 ? bits - 11 : 0;
      if (pass > 0) {  // the histogram is dirty and the bucket's own range is wanted: one more barrier
#pragma unroll 1
        for (int i = tid; i < BINS; i += nt) hist[i] = 0u;
        __syncthreads();
      }
      // ---- B: count ----
#pragma unroll 1
      for (int i = tid; i < n; i += nt) {
        const unsigned long long key = buf[i];
        const uint32_t v = key_vbits(key);
        if (key && v >= lo && v <= hi) atomicAdd(&hist[bucket_of(v, low_v, scale, lo, shift)], 1u);
      }
      __syncthreads();
      // ---- C: the block walks the buckets from the top ----
      {
        unsigned* wtot = hist + BINS;
        const int per = BINS / nt;
        const int warp = tid >> 5;
        // thread t owns buckets BINS-1 - t*per - j, j < per: highest first
        unsigned local = 0u;
#pragma unroll 4
        for (int j = 0; j < per; ++j) local += hist[BINS - 1 - tid * per - j];
        unsigned incl = local;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          unsigned o = __shfl_up_sync(FULL, incl, d);
          if (lane >= d) incl += o;
        }
        if (lane == 31) wtot[warp] = incl;
        __syncthreads();
        unsigned before = 0u;
#pragma unroll 1
        for (int w = 0; w < warp; ++w) before += wtot[w];
        unsigned acc = before + incl - local;  // entries in buckets above this thread's
        if (acc < rem && rem <= acc + local) {
#pragma unroll 1
          for (int j = 0; j < per; ++j) {
            const unsigned cnt = hist[BINS - 1 - tid * per - j];
            if (acc < rem && rem <= acc + cnt) {
              sm.sel_bin = BINS - 1 - tid * per - j;
              sm.sel_above = (int)acc;
              sm.sel_count = (int)cnt;
            }
            acc += cnt;
          }
        }
      }
      __syncthreads();
      chosen = sm.sel_bin;
      const unsigned at_or_above = above + (unsigned)sm.sel_above + (unsigned)sm.sel_count;
      const bool finest = scale == 0.0f && shift == 0;
      // accept a threshold that keeps little more than k: a loose one lets too much through later
      if (at_or_above <= (unsigned)min(c.keep, c.k + max(8, c.k >> 3)) || finest) {
        by_bucket = true;
        break;
      }
      // refine inside the chosen bucket: its own smallest and largest score bits
      {
        uint32_t mx = 0u, mn = 0xFFFFFFFFu;
#pragma unroll 1
        for (int i = tid; i < n; i += nt) {
          const unsigned long long key = buf[i];
          const uint32_t v = key_vbits(key);
          if (key && v >= lo && v <= hi && bucket_of(v, low_v, scale, lo, shift) == chosen) {
            mx = max(mx, v);
            mn = min(mn, v);
          }
        }
        mx = __reduce_max_sync(FULL, mx);
        mn = __reduce_min_sync(FULL, mn);
        if (lane == 0 && mx >= mn) { atomicMax(&sm.rmax, mx); atomicMin(&sm.rmin, mn); }
      }
      __syncthreads();
      above += (unsigned)sm.sel_above;
      rem -= (unsigned)sm.sel_above;
      lo = sm.rmin;
      hi = sm.rmax;
      scale = 0.0f;
      __syncthreads();  // everyone has read the range before it is reset for the next step
      if (tid == 0) { sm.rmin = 0xFFFFFFFFu; sm.rmax = 0u; }
    }
  }
  // ---- D: survivors go to the staging area; the smallest of them is the new threshold ----
  {
    uint32_t mn = 0xFFFFFFFFu;
#pragma unroll 1
    for (int base = 0; base < n; base += nt) {
      const int i = base + tid;
      const unsigned long long key = (i < n) ? buf[i] : 0ull;
      const uint32_t v = key_vbits(key);
      bool stay = key != 0ull;
      if (stay && by_bucket) stay = v > hi || (v >= lo && bucket_of(v, low_v, scale, lo, shift) >= chosen);
      else if (stay) stay = v >= thr;
      if (stay) mn = min(mn, v);
      warp_append(c.stage, &sm.m, c.keep, stay, key);
    }
    mn = __reduce_min_sync(FULL, mn);
    if (by_bucket && lane == 0) atomicMin(&sm.smin2, mn);
  }
  __syncthreads();
  // ---- E: back to the front of the buffer ----
  const int m = min(sm.m, c.keep);
  if (by_bucket) thr = sm.smin2;
#pragma unroll 1
  for (int i = tid; i < m; i += nt) buf[i] = c.stage[i];
#pragma unroll 1
  for (int i = tid; i < BINS; i += nt) hist[i] = 0u;
  if (tid < 32) sm.wcount[tid] = 0;
  const bool over = sm.m > c.keep;
  __syncthreads();
  if (tid == 0) {
    if (over) sm.overflow = 1;
    sm.n = m;
    sm.conv = m;
    if (thr > 1u && thr != 0xFFFFFFFFu) sm.tau = fmaxf(sm.tau, unord32(thr));
    sm.vmin = 0xFFFFFFFFu; sm.vmax = 0u; sm.m = 0; sm.valid = 0; sm.smin2 = 0xFFFFFFFFu;
  }
  __syncthreads();
}

// Block-synchronous append of one optional entry per thread (the merge of a row's slices).
__device__ inline void buffer_push(const Ctx& c, bool want, unsigned long long key) {
  Shared& sm = *c.sm;
  bool pending = want && key_value(key) >= sm.tau;
  while (true) {
    bool ok = warp_append(c.buf, &sm.n, c.cap, pending, key);
    pending = pending && !ok;
    if (!__syncthreads_or(pending ? 1 : 0)) break;
    buffer_rebuild(c, 0);
    if (sm.overflow) break;
    pending = pending && key_value(key) >= sm.tau;
  }
}

// descending bitonic sort of buf[0..p2), p2 a power of two
__device__ inline void block_sort_desc(unsigned long long* buf, int p2) {
  const int tid = threadIdx.x, nt = blockDim.x;
#pragma unroll 1
  for (int k = 2; k <= p2; k <<= 1) {
#pragma unroll 1
    for (int j = k >> 1; j > 0; j >>= 1) {
#pragma unroll 1
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

// A row that did not go through the candidate buffer: greedy, whole-row Gumbel argmax, or one the
// single pass could not reduce.
__device__ inline void finish_simple(const KParams& P, int b, int mode, unsigned long long best,
                                     unsigned long long gbest, bool failed) {
#pragma unroll 1
  for (int j = threadIdx.x; j < P.out_width; j += blockDim.x) {
    if (P.out_probs) P.out_probs[(size_t)b * P.out_width + j] = 0.0f;
    if (P.out_prob_ids) P.out_prob_ids[(size_t)b * P.out_width + j] = -1;
  }
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

// buf[0..sm.n) holds the row's candidates (unsorted, or likeliest first with `presorted`).  Computes
// the cut and the draw and writes the row's outputs.  fw / fi / fs are float scratch of n, n and
// 2 * ceil(n / 32) entries.
__device__ inline void finish_row(const KParams& P, const RowCfg& rc, int b, unsigned long long* buf,
                                  Shared& sm, float* fw, float* fi, float* fs, float row_min,
                                  bool listed = false, float s_floor = 0.0f, bool presorted = false) {
  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = nt >> 5;
  const int n = sm.n;
  if (n <= 0) {  // nothing comparable in the row (all NaN)
    finish_simple(P, b, rc.mode, 0ull, 0ull, true);
    return;
  }
  if (tid == 0) { sm.jstar = 0; sm.ns = 0; sm.pick = NO_ID; sm.best = 0ull; sm.nstrict = 0; sm.redo = 0; }
  if (presorted) {
    __syncthreads();
  } else if (n <= nt) {
    // one key per thread: every warp sorts its 32 keys in registers, then a key's place is its place
    // in its own run plus, for every other run, the number of keys there above it (a binary search)
    unsigned long long* runs = buf + P.cap / 2;
    unsigned long long key = tid < n ? buf[tid] : 0ull;
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
    const int nruns = (n + 31) >> 5;
    if (warp < nruns) runs[tid] = key;
    __syncthreads();
    if (key != 0ull) {
      int place = lane;
      // four runs at a time, so that four searches' loads are in flight together
#pragma unroll 1
      for (int r0 = 0; r0 < nruns; r0 += 4) {
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
          if (r0 + q < nruns && r0 + q != warp) place += pos[q];
        }
      }
      buf[place] = key;  // every key is in registers or in `runs` by now: the front is free
    }
    __syncthreads();
  } else if (n <= P.cap / 2) {
    // a key's place is the number of keys above it (keys are distinct), one sweep over shared
    // memory and no barriers, into the buffer's upper half
    unsigned long long* sorted = buf + P.cap / 2;
#pragma unroll 1
    for (int i = tid; i < n; i += nt) {
      const unsigned long long key = buf[i];
      int rank = 0;
      int j = 0;
#pragma unroll 1
      for (; j + 4 <= n; j += 4)
        rank += (buf[j] > key) + (buf[j + 1] > key) + (buf[j + 2] > key) + (buf[j + 3] > key);
#pragma unroll 1
      for (; j < n; ++j) rank += buf[j] > key;
      sorted[rank] = key;
    }
    __syncthreads();
    buf = sorted;
  } else {
    int p2 = 1;
    while (p2 < n) p2 <<= 1;
#pragma unroll 1
    for (int i = n + tid; i < p2; i += nt) buf[i] = 0ull;
    __syncthreads();
    block_sort_desc(buf, p2);
  }
  const float top = key_value(buf[0]);
  const int in_k = min(rc.k_eff, n);
  const int nseg = (n + 31) >> 5;
#pragma unroll 1
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
  if (tid < nseg) {
    // segment tid starts at the sum, in order, of the segments before it
    float off = 0.0f;
#pragma unroll 1
    for (int s = 0; s < tid; ++s) off = off + fs[s];
    fs[nseg + tid] = off;
  }
  __syncthreads();
#pragma unroll 1
  for (int j = tid; j < n; j += nt) fi[j] = fs[nseg + (j >> 5)] + fi[j];
  __syncthreads();
  const float kept = fi[in_k - 1];
  const float bound_p = rc.p * kept;
  {
    // the last place whose likelier mass stays under the bound: one shared atomic per warp
    int last = 0;
#pragma unroll 1
    for (int j = tid; j < in_k; j += nt) {
      float likelier = fi[j] - fw[j];
      if (j == 0 || likelier < bound_p) last = j;
    }
    last = __reduce_max_sync(FULL, last);
    if (lane == 0 && last > 0) atomicMax(&sm.jstar, last);
  }
  __syncthreads();
  float base = (rc.p < 1.0f) ? key_value(buf[sm.jstar]) : key_value(buf[in_k - 1]);
  if (rc.mode == M_SELECT_MINP) base = row_min;  // k = 0: the k-th score is the row's last
  float cut = fmaxf(base, top + rc.logm);
  if (!rc.has_cut) cut = neg_inf();
#pragma unroll 1
  for (int j = tid; j < n; j += nt) {
    float r = key_value(buf[j]);
    if (r >= cut && (j + 1 == n || !(key_value(buf[j + 1]) >= cut))) sm.ns = j + 1;
    if (listed && r > s_floor && (j + 1 == n || !(key_value(buf[j + 1]) > s_floor))) sm.nstrict = j + 1;
  }
  __syncthreads();
  const int ns = max(sm.ns, 1);
  const float total = fi[ns - 1];
  if (P.uniform) {
    const float bound_u = rc.u * total;
    int first = NO_ID;
#pragma unroll 1
    for (int j = tid; j < ns; j += nt)
      if (fi[j] > bound_u) first = min(first, j);
    first = __reduce_min_sync(FULL, first);
    if (lane == 0 && first != NO_ID) atomicMin(&sm.pick, first);
  } else {
    unsigned long long best = 0ull;
#pragma unroll 1
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
    if (listed) {
      // the list stands only if nothing the filter dropped could have mattered: enough candidates
      // strictly above the floor's score, and the cut strictly above it
      const bool enough = rc.mode == M_SELECT_MINP || sm.nstrict >= rc.k_eff;
      if (!(enough && cut > s_floor)) {
        id = -1;
        if (!(P.flags & 2u)) sm.redo = 1;
        else if (P.status) atomicOr(P.status, 4);
      }
    }
    if (P.out_ids) P.out_ids[b] = id;
    if (P.out_cut) P.out_cut[b] = cut;
    if (P.out_kept) P.out_kept[b] = sm.ns;
    if (P.status && P.out_probs && sm.ns > P.out_width) atomicOr(P.status, 2);
  }
  if (P.out_probs || P.out_prob_ids) {
#pragma unroll 1
    for (int j = tid; j < P.out_width; j += nt) {
      if (P.out_probs) P.out_probs[(size_t)b * P.out_width + j] = (j < ns) ? fw[j] / total : 0.0f;
      if (P.out_prob_ids) P.out_prob_ids[(size_t)b * P.out_width + j] = (j < ns) ? key_id(buf[j]) : -1;
    }
  }
}

// ---- streaming a slice --------------------------------------------------------------------------

struct History {
  const float* raw;  // the slice's history tokens' logits, loaded while the table was built
  const int* keys;
  const int* counts;
  int mask;
  int begin;
};

__device__ __forceinline__ int history_count(const History& h, int idx) {
  uint32_t slot = lowbias32((uint32_t)idx) & h.mask;
#pragma unroll 1
  for (int probe = 0; probe <= h.mask; ++probe) {
    int k = h.keys[slot];
    if (k == idx) return h.counts[slot];
    if (k == HASH_EMPTY) return 0;
    slot = (slot + 1) & h.mask;
  }
  return 0;
}

// the penalised logit of element idx, whose raw logit is l
template <bool PEN>
__device__ __noinline__ float exact_logit(const KParams& P, const RowCfg& rc, const History& h,
                                          const uint8_t* seen_row, int idx, float l) {
  if (PEN) {
    int count = P.history ? history_count(h, idx) : 0;
    if (seen_row && seen_row[idx]) count = max(count, 1);
    if (count) l = penalised(l, count, rc);
  }
  return l;
}

struct Tracked {
  float gl; int gid;  // best penalised logit and where (greedy)
  float al; int aid;  // best score + gumbel and where
  float mnl;          // smallest unpenalised logit
  float mns;          // smallest score among penalised elements
};

#include "stream_ring.cuh"

#include "filter_path.cuh"

#include "argmax_kernel.cuh"

// Logit i of the row that begins at `row` (the row's first byte, dressed as a float pointer),
// whatever the logits' format.
__device__ __forceinline__ float row_logit(const KParams& P, const float* __restrict__ row, int i) {
  if (P.dtype == 0) return row[i];
  const unsigned short h = reinterpret_cast<const unsigned short*>(row)[i];
  return P.dtype == 1 ? __uint_as_float((uint32_t)h << 16) : __half2float(__ushort_as_half(h));
}

// The first `cap` scores of a top-k / min-p slice go straight into the candidate buffer (exact,
// penalties applied); one rebuild gives the first threshold.  Returns where the stream starts.
template <bool PEN>
__device__ __noinline__ int slice_fill(const KParams& P, const RowCfg& rc, const Ctx& c, const History& h,
                                       const float* __restrict__ row, const uint8_t* __restrict__ seen_row,
                                       int begin, int end, Tracked& t) {
  Shared& sm = *c.sm;
  const int tid = threadIdx.x, nt = blockDim.x;
  const int fill_end = min(end, begin + c.cap);
  constexpr int FB = 4;  // loads in flight per thread
#pragma unroll 1
  for (int base = begin; base < fill_end; base += nt * FB) {
    float raw[FB];
#pragma unroll
    for (int j = 0; j < FB; ++j) {
      const int i = base + j * nt + tid;
      raw[j] = i < fill_end ? row_logit(P, row, i) : 0.0f;
    }
#pragma unroll 1
    for (int j = 0; j < FB; ++j) {
      const int i = base + j * nt + tid;
      if (i < fill_end) {
        float l = exact_logit<PEN>(P, rc, h, seen_row, i, j == 0 ? raw[0] : j == 1 ? raw[1] : j == 2 ? raw[2] : raw[3]);
        if (rc.track && (l > t.gl || (l == t.gl && i < t.gid))) { t.gl = l; t.gid = i; }
        float s = scaled(l, rc);
        if (!(s == s)) s = neg_inf();
        if (rc.mode == M_SELECT_MINP) t.mns = fminf(t.mns, s);
        c.buf[i - begin] = make_key(s, (uint32_t)(i + P.vocab_offset));
      }
    }
  }
  __syncthreads();
  if (tid == 0) sm.n = fill_end - begin;
  __syncthreads();
  if (end > fill_end) buffer_rebuild(c, 0);
  return fill_end;
}

// The penalised tokens of a slice come from the history table, not from the stream: one scattered
// load each (issued in batches), so the stream never has to penalise a logit.
template <bool PEN>
__device__ __noinline__ void slice_history(const KParams& P, const RowCfg& rc, const Ctx& c, const History& h,
                                           const float* __restrict__ row, const uint8_t* __restrict__ seen_row,
                                           int from, int end, Tracked& t) {
  Shared& sm = *c.sm;
  const int nt = blockDim.x, tid = threadIdx.x;
  const int mode = rc.mode;
  const bool select = mode == M_SELECT_K || mode == M_SELECT_MINP;
  constexpr int HB = 4;  // table slots per thread per batch (kept in registers)
#pragma unroll 1
  for (int base = 0; base < h.mask + 1; base += nt * HB) {
    int idxs[HB], counts[HB];
    float raw[HB];
#pragma unroll
    for (int j = 0; j < HB; ++j) {
      const int slot = base + j * nt + tid;
      int idx = (slot <= h.mask) ? h.keys[slot] : HASH_EMPTY;
      if (idx != HASH_EMPTY && !(idx >= from && idx < end)) idx = HASH_EMPTY;
      idxs[j] = idx;
      counts[j] = idx != HASH_EMPTY ? h.counts[slot] : 0;
      raw[j] = idx != HASH_EMPTY ? h.raw[slot] : 0.0f;
    }
    unsigned long long keys[HB];
    unsigned pending = 0u;
#pragma unroll
    for (int j = 0; j < HB; ++j) {
      const int idx = idxs[j];
      keys[j] = 0ull;
      if (idx != HASH_EMPTY) {
        int count = counts[j];
        if (seen_row && seen_row[idx]) count = max(count, 1);
        float l = penalised(raw[j], count, rc);
        if (rc.track && (l > t.gl || (l == t.gl && idx < t.gid))) { t.gl = l; t.gid = idx; }
        float s = scaled(l, rc);
        if (mode == M_SELECT_MINP) t.mns = fminf(t.mns, s);
        if (mode == M_ARGMAX_G) {
          float d = s + gumbel(hashed_uniform((uint32_t)(idx + P.vocab_offset), rc.rkey));
          if (d > t.al || (d == t.al && idx < t.aid)) { t.al = d; t.aid = idx; }
        }
        if (select && s >= sm.tau) {
          keys[j] = make_key(s, (uint32_t)(idx + P.vocab_offset));
          pending |= 1u << j;
        }
      }
    }
    if (select) {
      // one barrier per batch unless the buffer runs out
      int rounds = 0;
      while (true) {
#pragma unroll
        for (int j = 0; j < HB; ++j) {
          const bool fit = warp_append(c.buf, &sm.n, c.cap, (pending >> j) & 1u, keys[j]);
          if (fit) pending &= ~(1u << j);
        }
        if (!__syncthreads_or(pending != 0u)) break;
        buffer_rebuild(c, 0);
        if (sm.overflow || ++rounds > 64) {  // entries still pending: the row is not settled here
          if (tid == 0) sm.overflow = 1;
          __syncthreads();
          break;
        }
#pragma unroll
        for (int j = 0; j < HB; ++j)
          if (((pending >> j) & 1u) && !(key_value(keys[j]) >= sm.tau)) pending &= ~(1u << j);
      }
      if (sm.overflow) break;
    }
  }
}

// The stream for rows the ring cannot take (a vocabulary or a stride that is not a multiple of four
// floats): scalar loads, eight logits per thread per step, every logit looked at exactly.  Compact
// rather than fast.
template <bool PEN>
__device__ __noinline__ void stream_plain(const KParams& P, const RowCfg& rc, const Ctx& c, const History& h,
                                          const float* __restrict__ row, const uint8_t* __restrict__ seen_row,
                                          int from, int end, Tracked& t) {
  Shared& sm = *c.sm;
  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5;
  const int mode = rc.mode;
  const bool select = mode == M_SELECT_K || mode == M_SELECT_MINP;
  constexpr int PER = 8;
  if (select) {
    if (sm.n > c.keep) buffer_rebuild(c, 0);
#pragma unroll 1
    for (int i = sm.n + tid; i < c.keep; i += nt) c.buf[i] = 0ull;
    if (tid < 32) sm.wcount[tid] = 0;
    if (tid == 0) sm.conv = sm.n;
  }
  __syncthreads();
  const int region = c.region;
  unsigned long long* const mine = c.buf + c.keep + warp * region;
  int held = 0;
  float floor_l = select ? logit_floor(sm.tau, rc.tf) : 0.0f;
  bool stop = select && sm.overflow != 0;
#pragma unroll 1
  for (int base = from; base < end && !stop; base += nt * PER) {
    unsigned todo = (1u << PER) - 1u;  // elements of this step still to be placed
    int rounds = 0;
    while (true) {
      unsigned redo = 0u;
#pragma unroll 1
      for (int j = 0; j < PER; ++j) {
        const int idx = base + j * nt + tid;
        bool want = false;
        float l = 0.0f;
        if (((todo >> j) & 1u) && idx < end) {
          bool in_history = false;
          if (PEN && P.history) in_history = leat::in_history(h.keys, h.mask, idx);
          if (!in_history) {
            l = row_logit(P, row, idx);
            if (PEN && seen_row && seen_row[idx]) l = penalised(l, 1, rc);
            if (rounds == 0) {
              if ((mode == M_ARGMAX_L || rc.track) && (l > t.gl || (l == t.gl && idx < t.gid))) { t.gl = l; t.gid = idx; }
              const float sc = scaled(l, rc);
              if (mode == M_SELECT_MINP) t.mns = fminf(t.mns, sc);
              if (mode == M_ARGMAX_G && sc + GUMBEL_MAX >= t.al) {
                const float d = sc + gumbel(hashed_uniform((uint32_t)(idx + P.vocab_offset), rc.rkey));
                if (d > t.al || (d == t.al && idx < t.aid)) { t.al = d; t.aid = idx; }
              }
            }
            want = select && l >= floor_l;
          }
        }
        if (select) {
          const unsigned mask = __ballot_sync(FULL, want);
          if (want) {
            const int slot = held + __popc(mask & ((1u << lane) - 1u));
            if (slot < region) mine[slot] = ((unsigned long long)__float_as_uint(l) << 32) | (uint32_t)idx;
            else redo |= 1u << j;
          }
          held = min(held + __popc(mask), region);
        }
      }
      if (!select) break;
      if (lane == 0) sm.wcount[warp] = held;
      if (!__syncthreads_or(redo != 0u)) break;
      buffer_rebuild(c, 1);
      held = 0;
      floor_l = logit_floor(sm.tau, rc.tf);
      if (sm.overflow || ++rounds > 64) {
        if (tid == 0) sm.overflow = 1;
        stop = true;
        break;
      }
      todo = redo;
    }
  }
}

// ---- the kernel ---------------------------------------------------------------------------------

struct SmemMap {
  unsigned long long* buf;
  unsigned long long* stage;
  unsigned* hist;
  Shared* sm;
  Ctx* ctx;
  RowCfg* rc;
  unsigned long long* bars;
  History* history;
  unsigned char* region;  // the history tokens' hash keys, then: their counts | the ring | finish scratch
};

__device__ __forceinline__ SmemMap smem_map(unsigned char* raw, int cap, int keep) {
  SmemMap m;
  m.buf = reinterpret_cast<unsigned long long*>(raw);
  m.stage = m.buf + cap;
  m.hist = reinterpret_cast<unsigned*>(m.stage + keep);
  unsigned char* at = reinterpret_cast<unsigned char*>(m.hist + BINS + 32);
  m.sm = reinterpret_cast<Shared*>(at);
  m.ctx = reinterpret_cast<Ctx*>(at + 256);
  m.rc = reinterpret_cast<RowCfg*>(at + 384);
  m.bars = reinterpret_cast<unsigned long long*>(at + 512);
  m.history = reinterpret_cast<History*>(at + 640);
  m.region = at + SMEM_FIXED;
  return m;
}
static_assert(sizeof(Shared) <= 256 && sizeof(Ctx) <= 128 && sizeof(RowCfg) <= 128, "fixed shared-memory slots");

#include "general_kernel.cuh"

#include "finish_list.cuh"

#define LEAT_SHARD_KERNELS
#include "shard_exchange.cuh"

// One (row, slice) of sample_kernel's work, by the whole block.
template <bool PEN>
__device__ __forceinline__ void sample_block(const KParams& P, const int b, const int slice, unsigned char* smem_raw) {
  const SmemMap M = smem_map(smem_raw, P.cap, P.keep);
  unsigned long long* buf = M.buf;
  Shared& sm = *M.sm;
  // the hash keys stay until the last rebuild; their counts share bytes with the ring and with
  // the scratch of the finish, which come later
  int* hkeys = reinterpret_cast<int*>(M.region);
  unsigned char* later = M.region + (((size_t)P.ht_size * 4 + 127) / 128) * 128;
  int* hcnt = reinterpret_cast<int*>(later);
  float* fw = reinterpret_cast<float*>(later);
  float* fi = fw + P.cap;
  float* fs = fi + P.cap;
  // the ring shares its bytes with the hash table, which is dead once the history pass is over
  Ring ring;
  ring.data = reinterpret_cast<float*>(later);
  ring.bars = M.bars;
  ring.stages = P.ring_stages;

  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31;
  if (P.only_rows && P.only_rows[b] != -2) return;
  // a row with a list needs its first block only: the others leave before they set anything up
  if (P.list && slice > 0 && info_floor(__ldcg(&P.list_info[b])) < __uint_as_float(0x7F800000u)) return;
  int S = P.slices;
  const int begin = slice * P.slice_len;
  int end = min(P.vocab, begin + P.slice_len);
  const float* row = P.dtype == 0 ? P.logits + (size_t)b * P.row_stride
                                  : reinterpret_cast<const float*>(reinterpret_cast<const unsigned short*>(P.logits) + (size_t)b * P.row_stride);
  const uint8_t* seen_row = (PEN && P.seen) ? P.seen + (size_t)b * P.seen_stride : nullptr;
  // the row's options and the buffer's description live in shared memory, not in registers
  // loads nothing else depends on go out first: the first history ids, the list's length and entry
  constexpr int IB = 4;
  const int* hist_ids = (PEN && P.history) ? P.history + (size_t)b * P.history_cap : nullptr;
  int pre_ids[IB];
  int pre_hl = 0;
  if (PEN && P.history) {
#pragma unroll
    for (int j = 0; j < IB; ++j) {
      const int i = j * nt + tid;
      pre_ids[j] = i < P.history_cap ? hist_ids[i] : -1;
    }
    pre_hl = P.history_len ? P.history_len[b] : P.history_cap;
  }
  RowCfg& rc = *M.rc;
  Ctx& c = *M.ctx;
  History& h = *M.history;  // in shared memory: the out-of-line stream functions take it by reference
  float* hraw = reinterpret_cast<float*>(hcnt + P.ht_size);
  RowIn in;
  uint32_t floor_bits = 0x7F800000u;
  if (tid < 32) in = row_inputs_warp(P, b, P.list ? P.list_info + b : nullptr, floor_bits);  // (the word's low half: the floor)
  if (tid == 0) {
    rc = row_config_from(P, in);
    c.buf = buf; c.stage = M.stage; c.hist = M.hist; c.sm = M.sm;
    c.cap = P.cap; c.keep = P.keep; c.mode = rc.mode; c.k = rc.k_eff; c.logm = rc.logm;
    c.divide = rc.divide; c.off = P.vocab_offset; c.begin = begin; c.rinv = rc.rinv; c.tf = rc.tf;
    c.hkeys = (PEN && P.history) ? hkeys : nullptr;
    c.hmask = P.ht_size - 1;
    c.region = (P.cap - P.keep) / (nt >> 5);
    sm.n = 0; sm.m = 0; sm.conv = 0; sm.tau = neg_inf(); sm.overflow = 0; sm.best = 0ull; sm.gbest = 0ull;
    sm.vmin = 0xFFFFFFFFu; sm.vmax = 0u; sm.valid = 0; sm.smin2 = 0xFFFFFFFFu; sm.rmin = 0xFFFFFFFFu; sm.rmax = 0u;
    sm.smin = 0xFFFFFFFFu; sm.is_last = (S == 1); sm.nstrict = 0;
    sm.share_greedy = 0u; sm.share_gumbel = 0u; sm.share_min = 0xFFFFFFFFu;
    h.raw = hraw; h.keys = hkeys; h.counts = hcnt; h.mask = P.ht_size - 1; h.begin = begin;
    sm.floor_l = P.list ? __uint_as_float(floor_bits) : __uint_as_float(0x7F800000u);
    // a soft cap is applied where candidates are few: here, by the multi-pass routine
    if (P.softcap > 0.0f) { rc.mode = M_GENERAL; c.mode = M_GENERAL; }
    sm.s_floor = neg_inf();
    if (sm.floor_l < __uint_as_float(0x7F800000u)) {
      // nothing scoring under the floor can matter to a row whose list stands
      sm.s_floor = scaled(sm.floor_l, rc) + 0.0f;
      sm.tau = sm.s_floor;
    }
  }
  // (the other threads clear the tables meanwhile)
#pragma unroll 1
  for (int i = tid; i < BINS; i += nt) M.hist[i] = 0u;
  if (PEN && P.history) {
#pragma unroll 1
    for (int i = tid; i < P.ht_size; i += nt) hkeys[i] = HASH_EMPTY;
    // the counts, or the bitmap a listed row may use in their place: the same bytes
    const int zero = max(P.ht_size, P.list ? min(P.bm_words, (P.vocab + 31) >> 5) : 0);
#pragma unroll 1
    for (int i = tid; i < zero; i += nt) hcnt[i] = 0;
  }
  __syncthreads();
  const int mode = rc.mode;
  // a row whose logits the filter listed needs one block, which owns the whole row
  const bool listed = sm.floor_l < __uint_as_float(0x7F800000u);
  if (P.lean && (__ldcg(&P.list_info[b]) & INFO_LEAN)) return;  // finish_list_kernel's row
  if (P.list && !P.lean && slice == 0 && tid == 0) P.list_info[b] &= ~INFO_READY;  // (the list finish clears it otherwise)
  if (listed) {
    if (slice > 0) return;
    S = 1;
    end = P.vocab;
  } else {
    grid_dependency_wait();  // nothing to gain from an early start: keep the launches in order
  }
  unsigned* bitmap = nullptr;
  if (PEN && P.history) {
    // the slice's history tokens: a hash table of counts, and each token's logit fetched now (one
    // scattered load each, issued in batches) so the later passes never wait on them
    const int hl = min(pre_hl, P.history_cap);
    // a listed row whose penalties only lower logits finds every history token that matters in its
    // list, logit included: nothing to fetch
    const bool fetch = !(listed && rc.lowers);
    // ... and if only membership matters (no frequency penalty), a bitmap over the vocabulary says
    // it with one fire-and-forget atomic per history token instead of a probe sequence
    if (!fetch && rc.freq == 0.0f && P.vocab <= P.bm_words * 32) bitmap = reinterpret_cast<unsigned*>(hcnt);
#pragma unroll 1
    for (int base = 0; base < (bitmap ? hl : 0); base += nt * IB) {
#pragma unroll
      for (int j = 0; j < IB; ++j) {
        const int i = base + j * nt + tid;
        const int id = i < hl ? (base == 0 ? pre_ids[j] : hist_ids[i]) - P.vocab_offset : -1;
        if (id >= 0 && id < end) atomicOr(&bitmap[id >> 5], 1u << (id & 31));
      }
    }
#pragma unroll 1
    for (int base = 0; base < (bitmap ? 0 : hl); base += nt * IB) {
      int ids[IB];
      float raw[IB];
#pragma unroll
      for (int j = 0; j < IB; ++j) {
        const int i = base + j * nt + tid;
        int id = i < hl ? pre_ids[j] - P.vocab_offset : -1;
        if (!(id >= begin && id < end)) id = -1;
        ids[j] = id;
      }
      if (base + nt * IB < hl) {  // the next batch of ids is on its way while this one is inserted
#pragma unroll
        for (int j = 0; j < IB; ++j) {
          const int i = base + nt * IB + j * nt + tid;
          pre_ids[j] = i < hl ? hist_ids[i] : -1;
        }
      }
#pragma unroll
      for (int j = 0; j < IB; ++j) raw[j] = (fetch && ids[j] >= 0) ? logit_at(P, b, ids[j]) : 0.0f;
#pragma unroll
      for (int j = 0; j < IB; ++j) {
        const int id = ids[j];
        if (id >= 0) {
          uint32_t slot = lowbias32((uint32_t)id) & h.mask;
#pragma unroll 1
          for (int probe = 0; probe <= h.mask; ++probe) {
            int old = atomicCAS(&hkeys[slot], HASH_EMPTY, id);
            if (old == HASH_EMPTY || old == id) { atomicAdd(&hcnt[slot], 1); hraw[slot] = raw[j]; break; }
            slot = (slot + 1) & h.mask;
          }
        }
      }
    }
    __syncthreads();
  }

  // ---- stream the slice once ----
  Tracked t;
  t.gl = neg_inf(); t.gid = NO_ID; t.al = neg_inf(); t.aid = NO_ID;
  t.mnl = __uint_as_float(0x7F800000u); t.mns = t.mnl;
  bool list_ok = true;
  if (listed) {
    // the filter already streamed the row: candidates come from its list and from the history
    // everything up to here needed the floors only; the lists are complete when the filter's grid is
    grid_dependency_wait();
    const int pre_count = __ldcg(&P.list_count[b]);
    const unsigned long long pre_pair = __ldcg(&P.list[(size_t)b * P.list_cap + tid]);
    list_ok = list_load<PEN>(P, rc, c, h, bitmap, b, t, pre_count, pre_pair);
    if (PEN && P.history && list_ok && !rc.lowers) slice_history<PEN>(P, rc, c, h, row, seen_row, begin, end, t);
    __syncthreads();
    if (tid == 0) P.list_count[b] = 0;  // the list is taken: empty for the next call's filter
  } else if (mode != M_GENERAL) {
    const bool select = mode == M_SELECT_K || mode == M_SELECT_MINP;
    int from = begin;
    if (select) from = slice_fill<PEN>(P, rc, c, h, row, seen_row, begin, end, t);
    if (PEN && P.history) slice_history<PEN>(P, rc, c, h, row, seen_row, from, end, t);
    if (ring.stages > 0) stream_ring<PEN>(P, rc, c, h, row, seen_row, from, end, t, ring);
    else stream_plain<PEN>(P, rc, c, h, row, seen_row, from, end, t);
  }
  __syncthreads();

  // ---- reduce what the slice found ----
  if (rc.track) {
    unsigned long long g = (t.gid != NO_ID) ? make_key(t.gl, (uint32_t)(t.gid + P.vocab_offset)) : 0ull;
    if (tid == 0 && begin < end) g = max(g, make_key(neg_inf(), (uint32_t)(begin + P.vocab_offset)));
    g = warp_max_u64(g);
    if (lane == 0) atomicMax(&sm.gbest, g);
  }
  if (mode == M_ARGMAX_G) {
    unsigned long long a = (t.aid != NO_ID) ? make_key(t.al, (uint32_t)(t.aid + P.vocab_offset)) : 0ull;
    if (tid == 0 && begin < end) a = max(a, make_key(neg_inf(), (uint32_t)(begin + P.vocab_offset)));
    a = warp_max_u64(a);
    if (lane == 0) atomicMax(&sm.best, a);
  }
  if (mode == M_SELECT_MINP) {
    float mn = fminf(t.mns, scaled(t.mnl, rc));
    unsigned m = __reduce_min_sync(FULL, ord32(mn + 0.0f));
    if (lane == 0) atomicMin(&sm.smin, m);
  }
  __syncthreads();
  if ((mode == M_SELECT_K || mode == M_SELECT_MINP) && !sm.overflow) {
    if (listed) {
      // keys already; a few hundred the finish sorts as they are, more are reduced first
      if (mode == M_SELECT_MINP || sm.n > min(384, P.cap / 2) || (P.cand_count && sm.n > P.cand_cap)) buffer_rebuild(c, 0);
    } else {
      // the stream of a top-k row leaves raw entries behind: the rebuild also turns them into keys
      buffer_rebuild(c, S > 1 ? 3 : 1);
    }
  }
  bool failed = (mode == M_GENERAL) || sm.overflow || !list_ok;
  const float floor_l = listed ? sm.floor_l : neg_inf();
  // a greedy token is only known if the best candidate reaches the floor (nothing dropped beats it)
  if (listed && rc.track && !(sm.gbest != 0ull && key_value(sm.gbest) >= floor_l)) failed = true;
  if (listed && P.cand_count) {
    // A shard hands its candidates on instead of finishing, so the list is checked here: top-k rows
    // need top_k candidates strictly above the floor's score, min-p rows their own threshold strictly
    // above it.  A row that fails is marked for a second launch that streams it (count -2).
    if (!failed && mode == M_SELECT_K) {
      int above = 0;
#pragma unroll 1
      for (int i = tid; i < sm.n; i += nt) above += key_value(buf[i]) > sm.s_floor;
      above = __reduce_add_sync(FULL, above);
      if (lane == 0 && above) atomicAdd(&sm.nstrict, above);
      __syncthreads();
      if (sm.nstrict < rc.k_eff) failed = true;
    }
    if (!failed && mode == M_SELECT_MINP && !(sm.tau > sm.s_floor)) failed = true;
    if (failed) {
      if (tid == 0) { P.cand_count[b] = -2; P.cand_best[b] = 0ull; }
      return;
    }
  }

  // ---- publish, and let the last block of the row go on ----
  if (S > 1) {
    const size_t cell = (size_t)b * S + slice;
    if ((mode == M_SELECT_K || mode == M_SELECT_MINP) && !failed) {
      const int n = sm.n;
      unsigned long long* dst = P.ws_keys + cell * P.keep;
#pragma unroll 1
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
      unsigned ticket = atomicAdd(&P.ws_ticket[b], 1u);
      sm.is_last = (ticket == (unsigned)(S - 1));
      if (sm.is_last) P.ws_ticket[b] = 0u;
    }
    __syncthreads();
    if (!sm.is_last) return;
    __threadfence();
    // merge the row's slices
    if (tid == 0) { sm.n = 0; sm.conv = 0; sm.tau = neg_inf(); sm.overflow = 0; sm.smin = 0xFFFFFFFFu; }
    __syncthreads();
    unsigned long long g = 0ull, a = 0ull;
    unsigned mnb = 0xFFFFFFFFu;
    int bad = 0;
#pragma unroll 1
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
    if ((mode == M_SELECT_K || mode == M_SELECT_MINP) && !failed) {
      // where each slice's candidates go in the buffer: counts, then their running sum (the
      // histogram's words are free here; they are cleared again below)
      unsigned* counts = M.hist;
      unsigned* starts = M.hist + S;
      bool direct = 2 * S + 1 <= BINS;
      if (direct) {
#pragma unroll 1
        for (int j = tid; j < S; j += nt) counts[j] = (unsigned)max(__ldcg(&P.ws_count[(size_t)b * S + j]), 0);
        __syncthreads();
        if (tid == 0) {
          unsigned at = 0u;
#pragma unroll 1
          for (int j = 0; j < S; ++j) { starts[j] = at; at += counts[j]; }
          starts[S] = at;
        }
        __syncthreads();
        direct = starts[S] <= (unsigned)P.cap;
      }
      if (direct) {
        // everything fits: one gather, no barriers in between
        const int total = (int)starts[S];
#pragma unroll 1
        for (int i = tid; i < total; i += nt) {
          int lo = 0, hi = S - 1;  // the slice whose range holds i
          while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (starts[mid] <= (unsigned)i) lo = mid; else hi = mid - 1;
          }
          buf[i] = __ldcg(&P.ws_keys[((size_t)b * S + lo) * P.keep + (i - (int)starts[lo])]);
        }
        __syncthreads();
#pragma unroll 1
        for (int j = tid; j < 2 * S + 1; j += nt) M.hist[j] = 0u;
        if (tid == 0) { sm.n = total; sm.conv = total; }
        __syncthreads();
      } else {
        if (2 * S + 1 <= BINS) {
#pragma unroll 1
          for (int j = tid; j < 2 * S + 1; j += nt) M.hist[j] = 0u;
          __syncthreads();
        }
        const int total_slots = S * P.keep;
#pragma unroll 1
        for (int base = 0; base < total_slots; base += nt) {
          int i = base + tid;
          int j = i / P.keep, q = i - j * P.keep;
          bool want = false;
          unsigned long long key = 0ull;
          if (i < total_slots && q < __ldcg(&P.ws_count[(size_t)b * S + j])) {
            key = __ldcg(&P.ws_keys[((size_t)b * S + j) * P.keep + q]);
            want = true;
          }
          buffer_push(c, want, key);
          if (sm.overflow) break;
        }
        __syncthreads();
      }
      // a few hundred candidates the finish sorts as they are; more are reduced first
      if (!sm.overflow && (mode == M_SELECT_MINP || sm.n > min(384, P.cap / 2) || P.cand_count)) buffer_rebuild(c, 0);
      failed = sm.overflow != 0;
    }
  }
  __syncthreads();

  // ---- the row is whole in this block ----
  if (P.shard.world > 0) {  // shards with a peer exchange: the row's candidates go to its owner
    const unsigned epoch = __ldcg(P.shard.epoch);
    ShardSlot* slot = shard_slot(P.shard, b / P.shard.owned, (int)(epoch & 1u), P.shard.rank, b - (b / P.shard.owned) * P.shard.owned);
    int n = 0;
    if (!failed && (mode == M_SELECT_K || mode == M_SELECT_MINP)) {
      n = sm.n;
      if (n > P.shard.cap) { n = 0; failed = true; }
#pragma unroll 1
      for (int i = tid; i < n; i += nt) slot->keys[i] = buf[i];
    } else if (!failed && mode == M_ARGMAX_G) {
      n = 1;
      if (tid == 0) slot->keys[0] = sm.best;
    }
    if (tid == 0) {
      slot->best = sm.gbest;
      slot->count = (failed || mode == M_GENERAL) ? -1 : n;
    }
    shard_hand_over(P.shard, b, epoch);
    return;
  }
  if (P.cand_count) {  // shard mode: hand the row's candidates to the gather
    const int cap = P.cand_cap;
    int n = 0;
    if (!failed && (mode == M_SELECT_K || mode == M_SELECT_MINP)) {
      n = sm.n;
      if (n > cap) { n = 0; failed = true; }
#pragma unroll 1
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
  // a row this kernel could not settle goes through the exact multi-pass routine, here and now
  const bool may_redo = P.ws_flag != nullptr && !(P.flags & 2u) && !P.cand_count;
  if (failed && may_redo) {
    __syncthreads();
    general_row<PEN>(P, b, smem_raw);
    return;
  }
  if (failed || mode < M_SELECT_K) {
    finish_simple(P, b, mode, sm.best, sm.gbest, failed);
    return;
  }
  finish_row(P, rc, b, buf, sm, fw, fi, fs, listed ? neg_inf() : unord32(sm.smin), listed, sm.s_floor);
  __syncthreads();
  if (sm.redo) {
    __syncthreads();
    general_row<PEN>(P, b, smem_raw);
  }
}

// The grid is (slices, rows) or, with fewer blocks along y than rows, each block takes every
// gridDim.y-th row in turn (after finish_list_kernel most rows need nothing here, and a short grid
// of blocks that look and leave costs less than one block per row).
template <bool PEN>
__global__ void __launch_bounds__(512, 2) sample_kernel(const __grid_constant__ KParams P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  stamp_begin(P.stamps, 2);
  if (P.lean || P.only_rows) {
    // after the list finish most calls leave nothing to do here: the filter's flags (or the marks
    // of the rows a shard's lists could not settle) say so
    int any = 0;
#pragma unroll 1
    for (int i = threadIdx.x; i < P.rows; i += blockDim.x)
      any |= P.only_rows ? (__ldcg(&P.only_rows[i]) == -2) : ((__ldcg(&P.list_info[i]) & INFO_LEAN) == 0ull);
    if (!__syncthreads_or(any)) {
      // this grid must not be over before the list finish is: what follows it in the stream may
      // depend on this grid alone
      grid_dependency_wait();
      stamp_end(P.stamps, 2);
      return;
    }
  }
#pragma unroll 1
  for (int b = blockIdx.y; b < P.rows; b += gridDim.y) {
    sample_block<PEN>(P, b, blockIdx.x, smem_raw);
    __syncthreads();
  }
  stamp_end(P.stamps, 2);
}

// Finishes rows from candidates gathered from `g_parts` vocabulary slices: one block per row.
__global__ void __launch_bounds__(512) finish_candidates_kernel(const __grid_constant__ KParams P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const SmemMap M = smem_map(smem_raw, P.cap, P.keep);
  unsigned long long* buf = M.buf;
  Shared& sm = *M.sm;
  float* fw = reinterpret_cast<float*>(M.region);
  float* fi = fw + P.cap;
  float* fs = fi + P.cap;
  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31;
  const int b = blockIdx.x, parts = P.g_parts, cap = P.cand_cap, rows = P.rows;
  const RowCfg rc = row_config(P, b);
  const int mode = rc.mode;
  Ctx c;
  c.buf = buf; c.stage = M.stage; c.hist = M.hist; c.sm = M.sm;
  c.cap = P.cap; c.keep = P.keep; c.mode = mode; c.k = rc.k_eff; c.logm = rc.logm;
  c.divide = 0; c.off = 0; c.begin = 0; c.rinv = 1.0f; c.tf = 1.0f; c.hkeys = nullptr; c.hmask = 0; c.region = 1;
  if (tid == 0) {
    sm.n = 0; sm.m = 0; sm.conv = 0; sm.tau = neg_inf(); sm.overflow = 0; sm.best = 0ull; sm.gbest = 0ull;
    sm.vmin = 0xFFFFFFFFu; sm.vmax = 0u; sm.valid = 0; sm.smin2 = 0xFFFFFFFFu; sm.rmin = 0xFFFFFFFFu; sm.rmax = 0u;
    sm.smin = 0u;
  }
#pragma unroll 1
  for (int i = tid; i < BINS; i += nt) M.hist[i] = 0u;
  __syncthreads();
  unsigned long long g = 0ull;
  int bad = 0;
#pragma unroll 1
  for (int j = tid; j < parts; j += nt) {
    unsigned long long gj = P.g_best[(size_t)j * P.g_stride_best + b];
    g = gj > g ? gj : g;
    if (P.g_count[(size_t)j * P.g_stride_count + b] < 0) bad = 1;
  }
  g = warp_max_u64(g);
  if (lane == 0) atomicMax(&sm.gbest, g);
  bool failed = __syncthreads_or(bad) != 0 || mode == M_GENERAL;
  if (tid == 0 && P.out_greedy) P.out_greedy[b] = key_id(sm.gbest);
  if (!failed && mode == M_ARGMAX_G) {
    unsigned long long a = 0ull;
#pragma unroll 1
    for (int j = tid; j < parts; j += nt) {
      const size_t at = (size_t)b * cap;
      unsigned long long kk = make_key(P.g_value[(size_t)j * P.g_stride_value + at],
                                       (uint32_t)P.g_id[(size_t)j * P.g_stride_id + at]);
      a = kk > a ? kk : a;
    }
    a = warp_max_u64(a);
    if (lane == 0) atomicMax(&sm.best, a);
    __syncthreads();
  }
  if (!failed && (mode == M_SELECT_K || mode == M_SELECT_MINP)) {
    const int total_slots = parts * cap;
#pragma unroll 1
    for (int base = 0; base < total_slots; base += nt) {
      int i = base + tid;
      int j = i / cap, q = i - j * cap;
      bool want = false;
      unsigned long long key = 0ull;
      if (i < total_slots && q < P.g_count[(size_t)j * P.g_stride_count + b]) {
        const size_t at = (size_t)b * cap + q;
        key = make_key(P.g_value[(size_t)j * P.g_stride_value + at], (uint32_t)P.g_id[(size_t)j * P.g_stride_id + at]);
        want = true;
      }
      buffer_push(c, want, key);
      if (sm.overflow) break;
    }
    __syncthreads();
    if (!sm.overflow && (mode == M_SELECT_MINP || sm.n > rc.k_eff)) buffer_rebuild(c, 0);
    failed = sm.overflow != 0;
  }
  __syncthreads();
  if (failed || mode < M_SELECT_K) {
    KParams Q = P;
    Q.ws_flag = nullptr;
    finish_simple(Q, b, mode, sm.best, sm.gbest, failed);
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
#pragma unroll 1
  for (int j = 0; j < drafts; ++j) {
    if (drafted[(size_t)i * drafts + j] != against[(size_t)i * ran + j]) { kept = j; break; }
  }
  accepted[i] = kept;
#pragma unroll 1
  for (int j = 0; j < ran; ++j) {
    int t = -1;
    if (j < kept) t = greedy ? drafted[(size_t)i * drafts + j] : sampled[(size_t)i * ran + j];
    else if (j == kept) t = sampled[(size_t)i * ran + j];
    tokens[(size_t)i * ran + j] = t;
  }
}


// leat/engine.py:677-686 with the history kept as ids: one thread per sequence
__global__ void settle_kernel(const int* __restrict__ accepted, const int* __restrict__ last, const int* __restrict__ drafted,
                              const int* __restrict__ sampled, const int* __restrict__ slots, int n, int drafts,
                              int* history_ids, int* history_count, int capacity, const uint8_t* __restrict__ text,
                              int vocab, int* next, int* row) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int ran = drafts + 1;
  const int kept = min(max(accepted[i], 0), drafts);
  const int slot = slots ? slots[i] : i;
  int count = history_count[slot];
#pragma unroll 1
  for (int j = 0; j <= kept; ++j) {
    const int token = j == 0 ? last[i] : drafted[(size_t)i * drafts + j - 1];
    if (token < 0 || token >= vocab || (text && !text[token])) continue;
    history_ids[(size_t)slot * capacity + count % capacity] = token;
    count += 1;
  }
  history_count[slot] = count;
  if (next) next[i] = sampled[(size_t)i * ran + kept];
  if (row) row[i] = i * ran + kept;
}

}  // namespace leat
