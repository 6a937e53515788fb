// The exact multi-pass path, for the rows the single pass cannot take: top_p < 1 with top_k = 0 on
// a vocabulary wider than the candidate buffer, top_k beyond the buffer, more ties at the k-th
// score than the buffer has room for, and the supplied-uniform draw with no cut at all.  Included
// inside namespace leat by sampler_kernels.cuh.
//
// One block per flagged row (rows that need nothing return at once).  The row is read several
// times (it sits in L2 after the first pass): a pass for the top score, then radix descents over
// the scores' order-preserving bits, eleven bits a level, with a histogram of counts and of
// softmax mass per bucket.  Mass is accumulated as 64-bit fixed point (2^-40 of the top score's
// weight), so sums do not depend on the order threads arrive in and results are reproducible.
//
//   k-th score      descent by count
//   top-p boundary  descent by mass: the lowest score whose likelier ones weigh less than p * kept
//                   (leat/ops.py:518-529: likelier < top_p * kept, the likeliest always kept)
//   uniform draw    descent by mass: the first score, from the top, at which the running mass
//                   exceeds u * total; ties at that score are taken in ascending id
#pragma once

constexpr int G_BINS = 2048;
constexpr float G_FIXED = 1099511627776.0f;  // 2^40

struct GShared {
  unsigned top_bits, min_bits;
  unsigned long long greedy_key, best_key;
  unsigned valid, live;
  unsigned long long live_mass;
  int bin;
  unsigned bin_count, count_above;
  unsigned long long mass_above, bin_mass;
  unsigned found_id;
  unsigned scan[32];
};

struct GRow {
  const KParams* P;
  const RowCfg* rc;
  int b;  // the row
  const uint8_t* seen_row;
  History h;
  int vocab;
};

// score of token i (penalties, temperature) and whether it counts (NaN scores do not)
__device__ __forceinline__ bool g_score(const GRow& g, int i, float& l_out, float& s_out) {
  float l = soft_capped(logit_at(*g.P, g.b, i), g.P->softcap);
  int count = g.P->history ? history_count(g.h, i) : 0;
  if (g.seen_row && g.seen_row[i]) count = max(count, 1);
  if (count) l = penalised(l, count, *g.rc);
  const float s = scaled(l, *g.rc) + 0.0f;
  l_out = l;
  s_out = s;
  return s == s;
}

__device__ __forceinline__ unsigned long long g_weight(float s, float top) {
  return __float2ull_rn(exp_ref(s - top) * G_FIXED);
}

// One warp picks a bucket.  rule 0: the bucket holding the k_rem-th entry from the top.  rule 1:
// the lowest non-empty bucket whose mass above (base + buckets above it) is below `bound`, else the
// topmost non-empty one.  rule 2: the first non-empty bucket from the top where mass above plus its
// own exceeds `bound`, else the lowest non-empty one.
__device__ inline void g_choose(GShared& gs, int rule, const unsigned* cnt, const unsigned long long* mass,
                                int nb, unsigned long long base_mass, unsigned k_rem, double bound) {
  const int lane = threadIdx.x & 31;
  const int per = nb / 32;
  const int hi = nb - 1 - lane * per;  // lane 0 owns the highest buckets
  unsigned c = 0u;
  unsigned long long m = 0ull;
#pragma unroll 4
  for (int j = 0; j < per; ++j) { c += cnt[hi - j]; m += mass[hi - j]; }
  unsigned ci = c;
  unsigned long long mi = m;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const unsigned oc = __shfl_up_sync(FULL, ci, d);
    const unsigned long long om = __shfl_up_sync(FULL, mi, d);
    if (lane >= d) { ci += oc; mi += om; }
  }
  unsigned acc_c = ci - c;
  unsigned long long acc_m = mi - m;
  int pick = -1;
  unsigned pick_c = 0u;
  unsigned long long pick_m = 0ull;
  int top_nonempty = -1, low_nonempty = -1;
  unsigned tn_c = 0u, ln_c = 0u;
  unsigned long long tn_m = 0ull, ln_m = 0ull;
#pragma unroll 1
  for (int j = 0; j < per; ++j) {
    const int b = hi - j;
    const unsigned cb = cnt[b];
    const unsigned long long mb = mass[b];
    if (cb) {
      if (top_nonempty < 0) { top_nonempty = b; tn_c = acc_c; tn_m = acc_m; }
      low_nonempty = b; ln_c = acc_c; ln_m = acc_m;
      bool hit = false;
      if (rule == 0) hit = acc_c < k_rem && k_rem <= acc_c + cb;
      if (rule == 1) hit = (double)(base_mass + acc_m) < bound;
      if (rule == 2) hit = pick < 0 && (double)(base_mass + acc_m + mb) > bound;
      if (hit) { pick = b; pick_c = acc_c; pick_m = acc_m; }
    }
    acc_c += cb;
    acc_m += mb;
  }
  // across lanes: rule 1 wants the lowest hit (highest lane), rules 0 and 2 the highest hit
  const unsigned hits = __ballot_sync(FULL, pick >= 0);
  int src = -1;
  if (hits) src = (rule == 1) ? 31 - __clz(hits) : __ffs(hits) - 1;
  if (src < 0) {  // fallbacks
    const unsigned any = __ballot_sync(FULL, top_nonempty >= 0);
    if (any) {
      src = (rule == 2) ? 31 - __clz(any) : __ffs(any) - 1;
      if (rule == 2) { pick = low_nonempty; pick_c = ln_c; pick_m = ln_m; }
      else { pick = top_nonempty; pick_c = tn_c; pick_m = tn_m; }
    }
  }
  if (src >= 0 && lane == src) {
    gs.bin = pick;
    gs.count_above = pick_c;
    gs.mass_above = pick_m;
    gs.bin_count = cnt[pick];
    gs.bin_mass = mass[pick];
  }
  if (src < 0 && lane == 0) { gs.bin = 0; gs.count_above = 0u; gs.mass_above = 0ull; gs.bin_count = 0u; gs.bin_mass = 0ull; }
}

// A three-level descent over the score bits (11 + 11 + 10).  Only scores with bits >= floor_bits
// take part.  On return gs.bin_* describe the single score found: value bits in *value, count and
// mass above it in *count_above / *mass_above, its own multiplicity and mass in gs.bin_count /
// gs.bin_mass.
__device__ inline void g_descend(const GRow& g, GShared& gs, unsigned* cnt, unsigned long long* mass, int rule,
                                 float top, unsigned floor_bits, unsigned k, double bound, unsigned* value,
                                 unsigned* count_above, unsigned long long* mass_above) {
  const int tid = threadIdx.x, nt = blockDim.x;
  unsigned prefix = 0u;
  unsigned ca = 0u;
  unsigned long long ma = 0ull;
#pragma unroll 1
  for (int level = 0; level < 3; ++level) {
    const int shift = level == 0 ? 21 : level == 1 ? 10 : 0;
    const int nb = level == 2 ? 1024 : 2048;
    const int known = level == 0 ? 32 : level == 1 ? 21 : 10;  // bits below `known` are still open
#pragma unroll 1
    for (int i = tid; i < G_BINS; i += nt) { cnt[i] = 0u; mass[i] = 0ull; }
    __syncthreads();
#pragma unroll 1
    for (int i = tid; i < g.vocab; i += nt) {
      float l, s;
      if (!g_score(g, i, l, s)) continue;
      const unsigned v = ord32(s);
      if (v < floor_bits) continue;
      if (known < 32 && (v >> known) != (prefix >> known)) continue;
      const int b = (int)((v >> shift) & (unsigned)(nb - 1));
      atomicAdd(&cnt[b], 1u);
      atomicAdd(&mass[b], g_weight(s, top));
    }
    __syncthreads();
    if (tid < 32) g_choose(gs, rule, cnt, mass, nb, ma, k - ca, bound);
    __syncthreads();
    prefix |= (unsigned)gs.bin << shift;
    ca += gs.count_above;
    ma += gs.mass_above;
    __syncthreads();
  }
  *value = prefix;
  *count_above = ca;
  *mass_above = ma;
}

// One row, by the whole block that calls it (512 threads), in shared memory it may overwrite:
// G_BINS * 12 + 384 + ht_size * 8 bytes.
template <bool PEN>
__device__ __noinline__ void general_row(const KParams& P, int b, unsigned char* smem_raw) {
  unsigned long long* mass = reinterpret_cast<unsigned long long*>(smem_raw);
  unsigned* cnt = reinterpret_cast<unsigned*>(mass + G_BINS);
  GShared& gs = *reinterpret_cast<GShared*>(cnt + G_BINS);
  RowCfg& rc = *reinterpret_cast<RowCfg*>(reinterpret_cast<unsigned char*>(&gs) + 256);
  int* hkeys = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(&gs) + 384);
  int* hcnt = hkeys + P.ht_size;
  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31;
  const int V = P.vocab;
  if (tid == 0) {
    rc = row_config(P, b);
    gs.top_bits = 0u; gs.min_bits = 0xFFFFFFFFu; gs.greedy_key = 0ull; gs.best_key = 0ull;
    gs.valid = 0u; gs.live = 0u; gs.live_mass = 0ull; gs.found_id = 0xFFFFFFFFu;
  }
  GRow g;
  g.P = &P; g.rc = &rc; g.b = b; g.vocab = V;
  g.seen_row = (PEN && P.seen) ? P.seen + (size_t)b * P.seen_stride : nullptr;
  g.h.raw = nullptr; g.h.keys = hkeys; g.h.counts = hcnt; g.h.mask = P.ht_size - 1; g.h.begin = 0;
  if (PEN && P.history) {
#pragma unroll 1
    for (int i = tid; i < P.ht_size; i += nt) { hkeys[i] = HASH_EMPTY; hcnt[i] = 0; }
  }
  __syncthreads();
  if (PEN && P.history) {
    const int hl = P.history_len ? min(P.history_len[b], P.history_cap) : P.history_cap;
    const int* ids = P.history + (size_t)b * P.history_cap;
#pragma unroll 1
    for (int i = tid; i < hl; i += nt) {
      const int id = ids[i] - P.vocab_offset;
      if (id >= 0 && id < V) {
        uint32_t slot = lowbias32((uint32_t)id) & g.h.mask;
#pragma unroll 1
        for (int probe = 0; probe <= g.h.mask; ++probe) {
          const int old = atomicCAS(&hkeys[slot], HASH_EMPTY, id);
          if (old == HASH_EMPTY || old == id) { atomicAdd(&hcnt[slot], 1); break; }
          slot = (slot + 1) & g.h.mask;
        }
      }
    }
    __syncthreads();
  }
  // ---- pass 1: top score, smallest score, greedy token ----
  {
    unsigned tb = 0u, mb = 0xFFFFFFFFu, n = 0u;
    unsigned long long gk = 0ull;
#pragma unroll 1
    for (int i = tid; i < V; i += nt) {
      float l, s;
      const bool ok = g_score(g, i, l, s);
      if (l == l) { const unsigned long long k2 = make_key(l, (uint32_t)(i + P.vocab_offset)); gk = k2 > gk ? k2 : gk; }
      if (ok) { const unsigned v = ord32(s); tb = max(tb, v); mb = min(mb, v); n += 1u; }
    }
    tb = __reduce_max_sync(FULL, tb);
    mb = __reduce_min_sync(FULL, mb);
    n = __reduce_add_sync(FULL, n);
    gk = warp_max_u64(gk);
    if (lane == 0) { atomicMax(&gs.top_bits, tb); atomicMin(&gs.min_bits, mb); atomicAdd(&gs.valid, n); atomicMax(&gs.greedy_key, gk); }
  }
  __syncthreads();
  const int greedy_id = gs.greedy_key ? key_id(gs.greedy_key) : P.vocab_offset;
  if (tid == 0) {
    if (P.out_greedy) P.out_greedy[b] = greedy_id;
    if (P.status) atomicOr(P.status, 1);
  }
#pragma unroll 1
  for (int j = tid; j < P.out_width; j += nt) {
    if (P.out_probs) P.out_probs[(size_t)b * P.out_width + j] = 0.0f;
    if (P.out_prob_ids) P.out_prob_ids[(size_t)b * P.out_width + j] = -1;
  }
  const unsigned valid = gs.valid;
  if (valid == 0u || rc.greedy) {
    if (tid == 0) {
      if (P.out_ids) P.out_ids[b] = valid == 0u && !rc.greedy ? -1 : greedy_id;
      if (P.out_cut) P.out_cut[b] = quiet_nan();
      if (P.out_kept) P.out_kept[b] = 0;
    }
    return;
  }
  const float top = unord32(gs.top_bits);
  // ---- the k-th score (ranks beyond the row's length are the row's last) ----
  const unsigned K = (rc.k > 0.0f) ? (unsigned)min((float)valid, fmaxf(floorf(rc.k), 1.0f)) : valid;
  unsigned kth_bits, count_gt;
  unsigned long long mass_gt;
  g_descend(g, gs, cnt, mass, 0, top, 0u, K, 0.0, &kth_bits, &count_gt, &mass_gt);
  const unsigned ties_in = K - count_gt;  // how many of the k-th score's ties are inside the top k
  const unsigned long long kept = mass_gt + (unsigned long long)ties_in * g_weight(unord32(kth_bits), top);
  // ---- top-p inside the top k ----
  unsigned by_bits = kth_bits;
  if (rc.p < 1.0f) {
    unsigned ca;
    unsigned long long ma;
    g_descend(g, gs, cnt, mass, 1, top, kth_bits, 0u, (double)rc.p * (double)kept, &by_bits, &ca, &ma);
  }
  float cut = fmaxf(unord32(by_bits), top + rc.logm);
  if (!rc.has_cut) cut = neg_inf();
  const unsigned cut_bits = ord32(cut + 0.0f);
  // ---- survivors: how many, how much mass; the hashed draw over them ----
  {
    unsigned n = 0u;
    unsigned long long m = 0ull, best = 0ull;
#pragma unroll 1
    for (int i = tid; i < V; i += nt) {
      float l, s;
      if (!g_score(g, i, l, s) || ord32(s) < cut_bits) continue;
      n += 1u;
      m += g_weight(s, top);
      if (!P.uniform) {
        const uint32_t id = (uint32_t)(i + P.vocab_offset);
        const unsigned long long k2 = make_key(s + gumbel(hashed_uniform(id, rc.rkey)), id);
        best = k2 > best ? k2 : best;
      }
    }
    n = __reduce_add_sync(FULL, n);
    best = warp_max_u64(best);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m += __shfl_xor_sync(FULL, m, d);
    if (lane == 0) { atomicAdd(&gs.live, n); atomicAdd(&gs.live_mass, m); atomicMax(&gs.best_key, best); }
  }
  __syncthreads();
  int id = key_id(gs.best_key);
  if (P.uniform) {
    // ---- inverse CDF: the score at which the running mass passes u * total, then the tie ----
    const double bound = (double)rc.u * (double)gs.live_mass;
    unsigned pick_bits, ca;
    unsigned long long ma;
    g_descend(g, gs, cnt, mass, 2, top, cut_bits, 0u, bound, &pick_bits, &ca, &ma);
    const unsigned ties = gs.bin_count;
    const unsigned long long w = g_weight(unord32(pick_bits), top);
    // the first tie (by ascending id) whose running mass exceeds the bound; the last if none does
    unsigned want = ties;
    if (w > 0ull && (double)ma + (double)w * (double)ties > bound) {
      const double need = (bound - (double)ma) / (double)w;
      want = need < 0.0 ? 1u : (unsigned)need + 1u;
      if (want > ties) want = ties;
      if (want < 1u) want = 1u;
    }
    // the want-th smallest id among the ties: threads take contiguous chunks, count, scan, rescan
    const int chunk = (V + nt - 1) / nt;
    const int from = tid * chunk, to = min(V, from + chunk);
    unsigned mine = 0u;
#pragma unroll 1
    for (int i = from; i < to; ++i) {
      float l, s;
      if (g_score(g, i, l, s) && ord32(s) == pick_bits) mine += 1u;
    }
    unsigned incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const unsigned o = __shfl_up_sync(FULL, incl, d);
      if (lane >= d) incl += o;
    }
    if (lane == 31) gs.scan[tid >> 5] = incl;
    __syncthreads();
    unsigned before = 0u;
#pragma unroll 1
    for (int w2 = 0; w2 < (tid >> 5); ++w2) before += gs.scan[w2];
    const unsigned excl = before + incl - mine;
    if (excl < want && want <= excl + mine) {
      unsigned seen_ties = excl;
#pragma unroll 1
      for (int i = from; i < to; ++i) {
        float l, s;
        if (g_score(g, i, l, s) && ord32(s) == pick_bits) {
          seen_ties += 1u;
          if (seen_ties == want) gs.found_id = (unsigned)(i + P.vocab_offset);
        }
      }
    }
    __syncthreads();
    id = gs.found_id == 0xFFFFFFFFu ? -1 : (int)gs.found_id;
  }
  if (tid == 0) {
    if (P.out_ids) P.out_ids[b] = id;
    if (P.out_cut) P.out_cut[b] = cut;
    if (P.out_kept) P.out_kept[b] = (int)gs.live;
    if (P.status && P.out_probs) atomicOr(P.status, 2);
  }
}
