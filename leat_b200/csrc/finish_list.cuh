// Finishing a row from its list: the third launch of the filter path.  Included inside namespace
// leat by sampler_kernels.cuh.
//
// filter_kernel leaves, per row, the few hundred (logit, index) pairs at or above the row's floor.
// finish_list_kernel turns them into the row's token with one block of 256 threads per row, four
// blocks to an SM, so that 592 rows finish at once:
//
//   before the lists are waited for   the row's options; its history tokens marked in a bitmap
//                                     over the vocabulary (or counted in a hash table when a
//                                     frequency penalty needs counts)
//   keys                              every listed logit penalised, scaled and packed as a
//                                     (score, id) key; the row's top score and greedy token
//   select                            one 2048-bucket histogram over the scores' values finds the
//                                     bucket of the k-th largest; everything from that bucket up is
//                                     a candidate (refined bucket by bucket if too many share it)
//   sort                              runs of 32 sorted in registers by a bitonic network over
//                                     shuffles, then each key placed by binary searches in the
//                                     other runs
//   finish_row                        weights, running sums, top-p, min-p, the cut, the draw
//
// The checks that make a list trustworthy are finish_row's: at least top_k candidates strictly
// above the floor's score and the cut strictly above it.  A row that fails them, or whose list ran
// over, is redone on the spot by the multi-pass routine.  Rows this kernel does not take (no list;
// penalties that can raise a logit, whose history tokens must be fetched one by one; top_k beyond
// what it sorts) are left to sample_kernel, launched after it, which skips the rows taken here: the
// filter leaves a flag per row (lean_takes(), filter_path.cuh) that both follow.
#pragma once

constexpr int FL_THREADS = 256;       // threads of a block when more rows wait than SMs can hold blocks of 512
constexpr int FL_THREADS_WIDE = 512;  // ... and when they can: twice the hands per row
constexpr int FL_KEYS = 2048;  // keys held in shared memory; a longer list is worked on where it lies
// lists up to this long are sorted whole, without the select: longer ones when few rows wait (every
// phase less counts), shorter ones when many do (sorting what the select would drop costs issue slots)
constexpr int FL_DIRECT_WIDE = 384, FL_DIRECT = 128;
constexpr int FL_FIXED = 1024;  // bytes of FLShared's slot at the front of shared memory
constexpr int FL_HIST_WORDS = BINS + 32;
// words of the area behind the keys once the history marks are dead: the candidates, the sorted
// runs, weights and running sums, segment sums
constexpr int FL_AREA_MIN_WORDS = 2 * FL_SORT + 2 * FL_SORT + 2 * FL_SORT + 2 * (FL_SORT / 32) + 32;

struct FLShared {
  RowCfg rc;
  unsigned long long gbest, best;
  unsigned vmin, vmax, rmin, rmax;
  int live, m;
  int sel_bin, sel_above, sel_count;
  int jstar, ns, nstrict, pick, redo;
  unsigned wtot[FL_THREADS_WIDE / 32];
};
static_assert(sizeof(FLShared) <= FL_FIXED, "FLShared's slot");

// Leaves in cbuf every key of keys[0..n) at or above the K-th largest (ties at the K-th included),
// unordered; S.m is their number (more than FL_SORT: they did not fit).  All threads call it, after
// a barrier that made keys, S.live, S.vmin and S.vmax visible.  `hist` is BINS words, all zero.
template <int NT>
__device__ __forceinline__ void fl_select(const unsigned long long* keys, int n, int K, bool minp, float logm,
                                          unsigned* hist, unsigned long long* cbuf, FLShared& S) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t lo = S.vmin, hi = S.vmax;
  uint32_t thr = 1u;  // every live key (their value bits exceed 0)
  float low_v = 0.0f, scale = 0.0f;
  int shift = 0, chosen = 0;
  bool by_bucket = false;
  if (minp) {
    thr = ord32(unord32(hi) + logm + 0.0f);
  } else if (S.live > K + 32) {
    unsigned above = 0u, rem = (unsigned)K;
#pragma unroll 1
    for (int pass = 0; pass < 5; ++pass) {
      if (hi == lo) { thr = lo; by_bucket = false; break; }
      const float top_v = unord32(hi);
      low_v = pass == 0 ? fmaxf(unord32(lo), top_v - 64.0f) : unord32(lo);
      scale = (float)(BINS - 1) / (top_v - low_v);
      if (!(top_v > low_v && scale > 0.0f && scale < 3.0e38f)) scale = 0.0f;
      const int bits = 32 - __clz(hi - lo);
      shift = bits > 11 ? bits - 11 : 0;
      if (pass > 0) {  // the histogram is dirty
#pragma unroll 1
        for (int i = tid; i < BINS; i += NT) hist[i] = 0u;
        __syncthreads();
      }
#pragma unroll 1
      for (int i = tid; i < n; i += NT) {
        const unsigned long long key = keys[i];
        const uint32_t v = key_vbits(key);
        if (key && v >= lo && v <= hi) atomicAdd(&hist[bucket_of(v, low_v, scale, lo, shift)], 1u);
      }
      __syncthreads();
      {
        // thread t owns buckets BINS-1 - t*per - j, j < per: highest first
        constexpr int per = BINS / NT;
        unsigned local = 0u;
#pragma unroll
        for (int j = 0; j < per; ++j) local += hist[BINS - 1 - tid * per - j];
        unsigned incl = local;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const unsigned o = __shfl_up_sync(FULL, incl, d);
          if (lane >= d) incl += o;
        }
        if (lane == 31) S.wtot[warp] = incl;
        __syncthreads();
        unsigned acc = incl - local;
#pragma unroll
        for (int w = 0; w < NT / 32; ++w) acc += w < warp ? S.wtot[w] : 0u;
        if (acc < rem && rem <= acc + local) {
#pragma unroll 1
          for (int j = 0; j < per; ++j) {
            const unsigned cnt = hist[BINS - 1 - tid * per - j];
            if (acc < rem && rem <= acc + cnt) {
              S.sel_bin = BINS - 1 - tid * per - j;
              S.sel_above = (int)acc;
              S.sel_count = (int)cnt;
            }
            acc += cnt;
          }
        }
      }
      __syncthreads();
      chosen = S.sel_bin;
      by_bucket = true;
      const unsigned at_or_above = above + (unsigned)S.sel_above + (unsigned)S.sel_count;
      if (at_or_above <= (unsigned)(K + 64) || (scale == 0.0f && shift == 0)) break;
      // too many share the bucket: its own smallest and largest score bits bound the next step
      {
        uint32_t mx = 0u, mn = 0xFFFFFFFFu;
#pragma unroll 1
        for (int i = tid; i < n; i += NT) {
          const unsigned long long key = keys[i];
          const uint32_t v = key_vbits(key);
          if (key && v >= lo && v <= hi && bucket_of(v, low_v, scale, lo, shift) == chosen) {
            mx = max(mx, v);
            mn = min(mn, v);
          }
        }
        mx = __reduce_max_sync(FULL, mx);
        mn = __reduce_min_sync(FULL, mn);
        if (lane == 0 && mx >= mn) { atomicMax(&S.rmax, mx); atomicMin(&S.rmin, mn); }
      }
      __syncthreads();
      above += (unsigned)S.sel_above;
      rem -= (unsigned)S.sel_above;
      lo = S.rmin;
      hi = S.rmax;
      by_bucket = false;
      thr = lo;  // should the passes run out: everything from the bucket's smallest up
      __syncthreads();
      if (tid == 0) { S.rmin = 0xFFFFFFFFu; S.rmax = 0u; }
    }
  }
  // the keys that stay, four per thread at a time: one count, one scan and one atomic per warp
#pragma unroll 1
  for (int base = 0; base < n; base += NT * 4) {
    unsigned long long key[4];
    int count = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int i = base + q * NT + tid;
      key[q] = i < n ? keys[i] : 0ull;
      const uint32_t v = key_vbits(key[q]);
      bool stay = key[q] != 0ull;
      if (stay && by_bucket) stay = v > hi || (v >= lo && bucket_of(v, low_v, scale, lo, shift) >= chosen);
      else if (stay) stay = v >= thr;
      if (!stay) key[q] = 0ull;
      count += stay ? 1 : 0;
    }
    int incl = count;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(FULL, incl, d);
      if (lane >= d) incl += o;
    }
    int at = 0;
    if (lane == 31 && incl > 0) at = atomicAdd(&S.m, incl);
    at = __shfl_sync(FULL, at, 31) + incl - count;
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (key[q] != 0ull) {
        if (at < FL_SORT) cbuf[at] = key[q];
        ++at;
      }
  }
  __syncthreads();
}

// How many keys of runs r0 .. r0 + W - 1 (descending runs of 32; runs at or past `nruns` and run
// `mine` do not count) lie above `key`: W binary searches side by side.
template <int W>
__device__ __forceinline__ int fl_above(const unsigned long long* runs, unsigned long long key, int r0, int nruns, int mine) {
  int pos[W];
#pragma unroll
  for (int r = 0; r < W; ++r) pos[r] = 0;
#pragma unroll
  for (int step = 16; step > 0; step >>= 1) {
#pragma unroll
    for (int r = 0; r < W; ++r)
      if (runs[((r0 + r) & (FL_SORT / 32 - 1)) * 32 + pos[r] + step - 1] > key) pos[r] += step;
  }
  int total = 0;
#pragma unroll
  for (int r = 0; r < W; ++r) {
    if (pos[r] == 31 && runs[((r0 + r) & (FL_SORT / 32 - 1)) * 32 + 31] > key) pos[r] = 32;
    if (r0 + r < nruns && r0 + r != mine) total += pos[r];
  }
  return total;
}

// Sorts the non-zero keys of src[0..c), c <= FL_SORT, all distinct, likeliest first into dst; `runs`
// is FL_SORT words of scratch.  Runs of 32 are sorted in registers; a key's place is its place in
// its run plus, for every other run, the number of keys there above it (eight searches at a time).
template <int NT>
__device__ __forceinline__ void fl_sort(const unsigned long long* src, int c, unsigned long long* runs,
                                        unsigned long long* dst) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int PER = FL_SORT / NT;
  constexpr int WARPS = NT / 32;
  const int nruns = (c + 31) >> 5;
  unsigned long long key[PER];
#pragma unroll
  for (int q = 0; q < PER; ++q) {
    const int slot = q * NT + tid;
    key[q] = slot < c ? src[slot] : 0ull;
    if (q * WARPS + warp < nruns) {
#pragma unroll
      for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
          const unsigned long long other = __shfl_xor_sync(FULL, key[q], j);
          const bool keep_max = ((lane & k) == 0) == ((lane & j) == 0);
          const unsigned long long hi = key[q] > other ? key[q] : other, lo = key[q] > other ? other : key[q];
          key[q] = keep_max ? hi : lo;
        }
      }
    }
    runs[slot] = key[q];
  }
  __syncthreads();
  int place[PER];
#pragma unroll
  for (int q = 0; q < PER; ++q) place[q] = lane;
  if (nruns <= 4) {  // (a top_k of 64 leaves three runs: no need to search eight)
#pragma unroll
    for (int q = 0; q < PER; ++q)
      if (key[q] != 0ull) place[q] += fl_above<4>(runs, key[q], 0, nruns, q * WARPS + warp);
  } else {
#pragma unroll 1
    for (int r0 = 0; r0 < nruns; r0 += 8) {
#pragma unroll
      for (int q = 0; q < PER; ++q)
        if (key[q] != 0ull) place[q] += fl_above<8>(runs, key[q], r0, nruns, q * WARPS + warp);
    }
  }
#pragma unroll
  for (int q = 0; q < PER; ++q)
    if (key[q] != 0ull) dst[place[q]] = key[q];
  __syncthreads();
}

// is token `idx` in the table (keys hold id + 1, 0 = empty), and how often?
__device__ __forceinline__ int fl_count(const unsigned* hkeys, const unsigned* hcnt, int mask, int idx) {
  uint32_t slot = lowbias32((uint32_t)idx) & mask;
#pragma unroll 1
  for (int probe = 0; probe <= mask; ++probe) {
    const unsigned k = hkeys[slot];
    if (k == (unsigned)idx + 1u) return (int)hcnt[slot];
    if (k == 0u) return 0;
    slot = (slot + 1) & mask;
  }
  return 0;
}

// sorted[0..n) holds the row's candidates, likeliest first.  The cut and the draw, as finish_row
// computes them (the same sums in the same order), with fewer barriers: a segment's offset is summed
// by every thread that needs it instead of being handed round.  fw / fx hold n floats, fs n / 32.
// where a finished row's results go (any but `id` may be null)
struct RowOut {
  int* id; float* cut; int* kept; float* probs; int* prob_ids; int width;
};
__device__ __forceinline__ RowOut row_out(const KParams& P, int b) {
  RowOut o;
  o.id = P.out_ids ? P.out_ids + b : nullptr;
  o.cut = P.out_cut ? P.out_cut + b : nullptr;
  o.kept = P.out_kept ? P.out_kept + b : nullptr;
  o.probs = P.out_probs ? P.out_probs + (size_t)b * P.out_width : nullptr;
  o.prob_ids = P.out_prob_ids ? P.out_prob_ids + (size_t)b * P.out_width : nullptr;
  o.width = P.out_width;
  return o;
}

template <int NT, bool CHECK>
__device__ __forceinline__ void fl_finish(const KParams& P, const RowCfg& rc, const RowOut& out, const unsigned long long* sorted,
                                          int n, FLShared& S, float* fw, float* fx, float* fs, float s_floor) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float top = key_value(sorted[0]);
  const int in_k = min(rc.k_eff, n);
  const int nseg = (n + 31) >> 5;
  if (tid == 0) { S.jstar = 0; S.ns = 0; S.pick = NO_ID; S.best = 0ull; S.nstrict = 0; S.redo = 0; }
#pragma unroll 1
  for (int s = warp; s < nseg; s += NT / 32) {
    const int j = s * 32 + lane;
    float w = 0.0f;
    if (j < n) w = exp_ref(key_value(sorted[j]) - top);
    float x = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float y = __shfl_up_sync(FULL, x, d);
      if (lane >= d) x = x + y;
    }
    if (j < n) { fw[j] = w; fx[j] = x; }
    if (lane == 31) fs[s] = x;
  }
  __syncthreads();
  // the running sum at place j: the segments before j's summed left to right, then j's own
  auto offset = [&](int seg) {
    float off = 0.0f;
#pragma unroll 1
    for (int s = 0; s < seg; ++s) off = off + fs[s];
    return off;
  };
  const float kept = offset((in_k - 1) >> 5) + fx[in_k - 1];
  const float bound_p = rc.p * kept;
  {
    int last = 0;
#pragma unroll 1
    for (int j = tid; j < in_k; j += NT) {
      const float likelier = (offset(j >> 5) + fx[j]) - fw[j];
      if (j == 0 || likelier < bound_p) last = j;
    }
    last = __reduce_max_sync(FULL, last);
    if (lane == 0 && last > 0) atomicMax(&S.jstar, last);
  }
  __syncthreads();
  float base = (rc.p < 1.0f) ? key_value(sorted[S.jstar]) : key_value(sorted[in_k - 1]);
  if (rc.mode == M_SELECT_MINP) base = neg_inf();  // k = 0: the k-th score is the row's last
  float cut = fmaxf(base, top + rc.logm);
  if (!rc.has_cut) cut = neg_inf();
#pragma unroll 1
  for (int j = tid; j < n; j += NT) {
    const float r = key_value(sorted[j]);
    const float next = j + 1 < n ? key_value(sorted[j + 1]) : neg_inf();
    if (r >= cut && (j + 1 == n || !(next >= cut))) S.ns = j + 1;
    if (CHECK && r > s_floor && (j + 1 == n || !(next > s_floor))) S.nstrict = j + 1;
  }
  __syncthreads();
  const int ns = max(S.ns, 1);
  const float total = offset((ns - 1) >> 5) + fx[ns - 1];
  if (P.uniform) {
    const float bound_u = rc.u * total;
    int first = NO_ID;
#pragma unroll 1
    for (int j = tid; j < ns; j += NT)
      if (offset(j >> 5) + fx[j] > bound_u) first = min(first, j);
    first = __reduce_min_sync(FULL, first);
    if (lane == 0 && first != NO_ID) atomicMin(&S.pick, first);
  } else {
    unsigned long long best = 0ull;
#pragma unroll 1
    for (int j = tid; j < ns; j += NT) {
      const uint32_t id = (uint32_t)key_id(sorted[j]);
      const float d = key_value(sorted[j]) + gumbel(hashed_uniform(id, rc.rkey));
      const unsigned long long kk = make_key(d, id);
      best = kk > best ? kk : best;
    }
    best = warp_max_u64(best);
    if (lane == 0) atomicMax(&S.best, best);
  }
  __syncthreads();
  if (tid == 0) {
    int id = P.uniform ? key_id(sorted[min(S.pick, ns - 1)]) : key_id(S.best);
    if (CHECK) {
      // the list stands only if nothing the filter dropped could have mattered: enough candidates
      // strictly above the floor's score, and the cut strictly above it
      const bool enough = rc.mode == M_SELECT_MINP || S.nstrict >= rc.k_eff;
      if (!(enough && cut > s_floor)) {
        id = -1;
        if (!(P.flags & 2u)) S.redo = 1;
        else if (P.status) atomicOr(P.status, 4);
      }
    }
    if (out.id) *out.id = id;
    if (out.cut) *out.cut = cut;
    if (out.kept) *out.kept = S.ns;
    if (P.status && out.probs && S.ns > out.width) atomicOr(P.status, 2);
  }
  if (out.probs || out.prob_ids) {
#pragma unroll 1
    for (int j = tid; j < out.width; j += NT) {
      if (out.probs) out.probs[j] = (j < ns) ? fw[j] / total : 0.0f;
      if (out.prob_ids) out.prob_ids[j] = (j < ns) ? key_id(sorted[j]) : -1;
    }
  }
  __syncthreads();
}

// SHARD: the row is one slice of a vocabulary shared out over ranks: instead of being finished, its
// candidates (everything at or above the slice's top_k-th score) are handed to the rank that owns
// the row (shard_exchange.cuh); a row the list cannot vouch for is marked for the streaming kernel.
template <int NT, bool SHARD>
__device__ __forceinline__ void finish_list_block(const KParams& P, unsigned char* smem_raw) {
  FLShared& S = *reinterpret_cast<FLShared*>(smem_raw);
  unsigned* hist = reinterpret_cast<unsigned*>(smem_raw + FL_FIXED);
  unsigned long long* skeys = reinterpret_cast<unsigned long long*>(hist + FL_HIST_WORDS);
  unsigned* area = reinterpret_cast<unsigned*>(skeys + FL_KEYS);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = blockIdx.x;
  const int V = P.vocab;
  RowCfg& rc = S.rc;

  // ---- what needs no list: the row's options, its history tokens marked, tables cleared ----
  const int* hist_ids = P.history ? P.history + (size_t)b * P.history_cap : nullptr;
  constexpr int IB = 2048 / NT;
  int pre_ids[IB];
  int hl = 0;
  if (P.history) {
#pragma unroll
    for (int j = 0; j < IB; ++j) {
      const int i = j * NT + tid;
      pre_ids[j] = i < P.history_cap ? hist_ids[i] : -1;
    }
    hl = P.history_len ? min(P.history_len[b], P.history_cap) : P.history_cap;
  }
  if (warp == 0) {
    uint32_t unused;
    const RowIn in = row_inputs_warp(P, b, nullptr, unused);
    if (lane == 0) {
      rc = row_config_from(P, in);
      S.gbest = 0ull; S.vmin = 0xFFFFFFFFu; S.vmax = 0u; S.rmin = 0xFFFFFFFFu; S.rmax = 0u;
      S.live = 0; S.m = 0; S.redo = 0; S.nstrict = 0;
    }
  }
  const int bm_words = (V + 31) >> 5;
  const int ht = P.fl_ht;  // slots of the hash table (a power of two), keys then counts
  {
    uint4* h4 = reinterpret_cast<uint4*>(hist);
#pragma unroll 1
    for (int i = tid; i < BINS / 4; i += NT) h4[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  if (P.history) {
    uint4* a4 = reinterpret_cast<uint4*>(area);
    const int zero4 = (max(bm_words <= P.fl_area_words ? bm_words : 0, 2 * ht) + 3) >> 2;
#pragma unroll 1
    for (int i = tid; i < zero4; i += NT) a4[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  __syncthreads();
  // membership is enough without a frequency penalty: a bitmap over the vocabulary, one
  // fire-and-forget atomic per history token; counts go to a hash table
  const bool bitmap = P.history && rc.freq == 0.0f && bm_words <= P.fl_area_words;
  unsigned* hkeys = area;
  unsigned* hcnt = area + ht;
  if (P.history) {
#pragma unroll 1
    for (int base = 0; base < hl; base += NT * IB) {
#pragma unroll
      for (int j = 0; j < IB; ++j) {
        const int i = base + j * NT + tid;
        const int id = i < hl ? (base == 0 ? pre_ids[j] : hist_ids[i]) - P.vocab_offset : -1;
        if (id < 0 || id >= V) continue;
        if (bitmap) {
          atomicOr(&area[id >> 5], 1u << (id & 31));
        } else {
          uint32_t slot = lowbias32((uint32_t)id) & (ht - 1);
#pragma unroll 1
          for (int probe = 0; probe < ht; ++probe) {
            const unsigned old = atomicCAS(&hkeys[slot], 0u, (unsigned)id + 1u);
            if (old == 0u || old == (unsigned)id + 1u) { atomicAdd(&hcnt[slot], 1u); break; }
            slot = (slot + 1) & (ht - 1);
          }
        }
      }
    }
  }

  // ---- the lists are complete when the filter's grid is: everything wanted of them is asked for at once ----
  grid_dependency_wait();
  grid_launch_dependents();
  unsigned long long* list = P.list + (size_t)b * P.list_cap;
  constexpr int PRE = 1024 / NT;  // list entries per thread fetched before the list's length is known
  const unsigned long long info = __ldcg(&P.list_info[b]);
  const int n = __ldcg(&P.list_count[b]);
  unsigned long long pre[PRE];
#pragma unroll
  for (int q = 0; q < PRE; ++q) pre[q] = __ldcg(&list[q * NT + tid]);
  __syncthreads();  // the history marks are in; every thread has the list's length
  const bool lean = (info & INFO_LEAN) != 0ull;
  const float floor_l = soft_capped(info_floor(info), P.softcap);  // (what a logit under the floor is at most, capped)
  // the next call's filter must find the row's list empty and its word unmarked
  if (tid == 0) {
    P.list_info[b] = info & ~INFO_READY;
    if (lean) P.list_count[b] = 0;
    if (SHARD) P.shard.marks[b] = lean ? 0 : -2;
  }
  if (!lean) return;  // sample_kernel's row
  const int mode = rc.mode;
  const float s_floor = scaled(floor_l, rc) + 0.0f;
  const bool may_redo = P.ws_flag != nullptr && !(P.flags & 2u);
  bool failed = n > P.list_cap;
  unsigned long long* keys = n <= FL_KEYS ? skeys : list;
  if (!failed) {
    unsigned long long gbest = 0ull;
    uint32_t mn = 0xFFFFFFFFu, mx = 0u;
    int live = 0;
    auto visit = [&](int i, unsigned long long pair) {
      const int idx = (int)(uint32_t)pair;
      float l = soft_capped(__uint_as_float((uint32_t)(pair >> 32)), P.softcap);
      if (P.history) {
        const int count = bitmap ? (int)((area[idx >> 5] >> (idx & 31)) & 1u) : fl_count(hkeys, hcnt, ht - 1, idx);
        if (count) l = penalised(l, count, rc);
      }
      if (rc.track && l == l) {
        const unsigned long long g = make_key(l, (uint32_t)(idx + P.vocab_offset));
        gbest = g > gbest ? g : gbest;
      }
      const float s = scaled(l, rc);
      unsigned long long key = 0ull;
      if (mode != M_ARGMAX_L && s == s && s >= s_floor) {
        key = make_key(s, (uint32_t)(idx + P.vocab_offset));
        mx = max(mx, key_vbits(key));
        mn = min(mn, key_vbits(key));
        live += 1;
      }
      if (mode != M_ARGMAX_L) keys[i] = key;
    };
#pragma unroll
    for (int q = 0; q < PRE; ++q)
      if (q * NT + tid < n) visit(q * NT + tid, pre[q]);
#pragma unroll 1
    for (int i = PRE * NT + tid; i < n; i += NT) visit(i, __ldcg(&list[i]));
    if (rc.track) {
      gbest = warp_max_u64(gbest);
      if (lane == 0 && gbest) atomicMax(&S.gbest, gbest);
    }
    mx = __reduce_max_sync(FULL, mx);
    mn = __reduce_min_sync(FULL, mn);
    live = __reduce_add_sync(FULL, live);
    if (lane == 0 && live) { atomicMax(&S.vmax, mx); atomicMin(&S.vmin, mn); atomicAdd(&S.live, live); }
  }
  __syncthreads();  // keys are in; the history marks are dead, their area is free
  // a greedy token is only known if the best candidate reaches the floor (nothing dropped beats it)
  // (under a soft cap it must beat the floor: distinct logits may be capped to the same float, and
  // the first index wins a tie)
  if (rc.track && !(S.gbest != 0ull && (P.softcap > 0.0f ? key_value(S.gbest) > floor_l : key_value(S.gbest) >= floor_l)))
    failed = true;
  if (tid == 0 && P.out_greedy) P.out_greedy[b] = key_id(S.gbest);
  unsigned long long* cbuf = reinterpret_cast<unsigned long long*>(area);
  unsigned long long* runs = cbuf + FL_SORT;
  float* fw = reinterpret_cast<float*>(runs + FL_SORT);
  float* fx = fw + FL_SORT;
  float* fseg = fx + FL_SORT;
  int c = 0;
  if (SHARD) {
    const unsigned epoch = __ldcg(P.shard.epoch);
    const int owner = b / P.shard.owned;
    ShardSlot* slot = shard_slot(P.shard, owner, (int)(epoch & 1u), P.shard.rank, b - owner * P.shard.owned);
    if (!failed && mode != M_ARGMAX_L) {
      if (S.live == 0) {
        failed = true;
      } else {
        fl_select<NT>(keys, n, rc.k_eff, mode == M_SELECT_MINP, rc.logm, hist, cbuf, S);
        c = S.m;
        // the list stands for the slice only if nothing the filter dropped could be a candidate:
        // top_k candidates strictly above the floor's score (min-p: the threshold itself above it)
        if (c > P.shard.cap) {
          failed = true;
        } else if (mode == M_SELECT_K) {
          int above = 0;
#pragma unroll 1
          for (int i = tid; i < c; i += NT) above += key_value(cbuf[i]) > s_floor ? 1 : 0;
          above = __reduce_add_sync(FULL, above);
          if (lane == 0 && above) atomicAdd(&S.nstrict, above);
          __syncthreads();
          if (S.nstrict < rc.k_eff) failed = true;
        } else if (!(unord32(S.vmax) + rc.logm + 0.0f > s_floor)) {
          failed = true;
        }
      }
    }
    if (failed) {
      if (tid == 0) P.shard.marks[b] = -2;  // the streaming kernel takes the row
      return;
    }
#pragma unroll 1
    for (int i = tid; i < c; i += NT) slot->keys[i] = cbuf[i];
    if (tid == 0) { slot->best = S.gbest; slot->count = c; }
    shard_hand_over(P.shard, b, epoch);
    return;
  }
  if (!failed && mode != M_ARGMAX_L) {
    c = S.live;
    if (c == 0) {
      failed = true;
    } else if (n <= (NT == FL_THREADS_WIDE ? FL_DIRECT_WIDE : FL_DIRECT) && mode == M_SELECT_K) {
      // few enough to sort as they are (dead entries are zero keys, which the sort drops)
      fl_sort<NT>(keys, n, runs, cbuf);
    } else {
      fl_select<NT>(keys, n, rc.k_eff, mode == M_SELECT_MINP, rc.logm, hist, cbuf, S);
      c = S.m;
      if (c > FL_SORT) failed = true;
      else fl_sort<NT>(cbuf, c, runs, cbuf);  // (the sort reads the candidates into registers first)
    }
  }
  if (failed) {
    if (may_redo) {
      __syncthreads();
      general_row<true>(P, b, smem_raw);
    } else {
      finish_simple(P, b, mode, 0ull, S.gbest, true);
    }
    return;
  }
  if (mode == M_ARGMAX_L) {
    finish_simple(P, b, mode, 0ull, S.gbest, false);
    return;
  }
  fl_finish<NT, true>(P, rc, row_out(P, b), cbuf, c, S, fw, fx, fseg, s_floor);
  if (S.redo) general_row<true>(P, b, smem_raw);
}

template <int NT>
__global__ void __launch_bounds__(NT, 1024 / NT) finish_list_kernel(const __grid_constant__ KParams P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  stamp_begin(P.stamps, 1);
  finish_list_block<NT, false>(P, smem_raw);
  stamp_end(P.stamps, 1);
}

// The same block per row for a vocabulary shard: the slice's candidates go to the row's owner.
template <int NT>
__global__ void __launch_bounds__(NT, 1024 / NT) shard_select_kernel(const __grid_constant__ KParams P) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  stamp_begin(P.stamps, 1);
  finish_list_block<NT, true>(P, smem_raw);
  stamp_end(P.stamps, 1);
}
