// Streaming a slice through a shared-memory ring filled by bulk asynchronous copies (the TMA
// engine's untiled form, cp.async.bulk), included inside namespace leat by sampler_kernels.cuh.
//
// One elected thread keeps `stages` copies of `threads x 16` logits in flight; each completes on an
// mbarrier.  The block consumes a stage per step: every thread reads its sixteen logits with four
// conflict-free 128-bit shared loads, so no logit waits in a register for the next step, and the
// depth of the pipeline does not depend on occupancy.  The step's closing barrier is also what
// frees the stage for the next copy.  Every wait on an mbarrier is bounded; a wait that runs out
// marks the row as failed and the block leaves through the normal path.
#pragma once

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}
// untiled bulk copy global -> shared: both addresses 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}
// One poll; the thread may be suspended up to about a microsecond while the phase is pending, so
// waiting warps leave the issue slots to the warps that have work.
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity), "r"(1000u)
      : "memory");
  return ok != 0u;
}
// false if the copy has not landed after about a million polls (far beyond any real latency)
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, uint32_t parity) {
#pragma unroll 1
  for (int spin = 0; spin < (1 << 20); ++spin)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

constexpr int RING_PER_THREAD = 16;  // logits a thread takes from a stage

struct Ring {
  float* data;              // stages x (threads x 16) floats
  unsigned long long* bars; // one mbarrier per stage
  int stages;
};

// One lane's look at a logit the cheap tests singled out: penalties if a dense seen mask marks it,
// greedy tracking, and whether it goes on to the candidate buffer.  Kept out of line: it runs for a
// few logits per step and must not bloat the loop around it.
template <bool PEN>
__device__ __noinline__ void ring_visit(const KParams& P, const RowCfg& rc, const History& h, Shared& sm,
                                        const uint8_t* seen_row, Tracked& t, int idx, float raw, int what) {
  // what: 1 = greedy candidate, 2 = whole-row gumbel candidate, 4 = smallest-score candidate
  bool in_history = false;
  if (PEN && P.history) in_history = leat::in_history(h.keys, h.mask, idx);
  if (in_history) return;  // its penalised logit came from the history table
  float l = raw;
  if (PEN && seen_row && seen_row[idx]) l = penalised(raw, 1, rc);
  if ((what & 1) && (l > t.gl || (l == t.gl && idx < t.gid))) {
    t.gl = l; t.gid = idx;
    atomicMax(&sm.share_greedy, ord32(l + 0.0f));
  }
  if (what & 2) {
    const float sc = scaled(l, rc);
    if (sc + GUMBEL_MAX >= t.al) {
      const float d = sc + gumbel(hashed_uniform((uint32_t)(idx + P.vocab_offset), rc.rkey));
      if (d > t.al || (d == t.al && idx < t.aid)) {
        t.al = d; t.aid = idx;
        atomicMax(&sm.share_gumbel, ord32(d + 0.0f));
      }
    }
  }
  if (what & 4) {
    t.mns = fminf(t.mns, scaled(l, rc));
    t.mnl = fminf(t.mnl, l);
    atomicMin(&sm.share_min, ord32(l + 0.0f));
  }
}

// Streams [from, end) of `row` in the row's mode (rc.mode: M_SELECT_K, M_SELECT_MINP, M_ARGMAX_L or
// M_ARGMAX_G).  `row + from` is 16-byte aligned and end - from is a multiple of 4.
template <bool PEN>
__device__ __noinline__ void stream_ring(const KParams& P, const RowCfg& rc, const Ctx& c, const History& h,
                                         const float* __restrict__ row, const uint8_t* __restrict__ seen_row,
                                         int from, int end, Tracked& t, Ring ring) {
  Shared& sm = *c.sm;
  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5;
  constexpr int N = RING_PER_THREAD;
  const int mode = rc.mode;
  const bool select = mode == M_SELECT_K || mode == M_SELECT_MINP;
  const bool greedy = mode == M_ARGMAX_L || rc.track != 0;
  const bool dense = PEN && seen_row != nullptr;
  const bool want_hi = greedy || mode == M_ARGMAX_G, want_lo = mode == M_SELECT_MINP;
  const int stage_elems = nt * N;
  const int steps = (end - from + stage_elems - 1) / stage_elems;
  const int stride = nt * 4;

  if (tid == 0) {
#pragma unroll 1
    for (int s = 0; s < ring.stages; ++s) mbar_init(&ring.bars[s], 1);
    mbar_fence_init();
  }
  if (select) {
    // keys so far fit the first `keep` slots; the rest of the buffer is one raw region per warp
    if (sm.n > c.keep) buffer_rebuild(c, 0);
#pragma unroll 1
    for (int i = sm.n + tid; i < c.keep; i += nt) c.buf[i] = 0ull;
    if (tid < 32) sm.wcount[tid] = 0;
    if (tid == 0) sm.conv = sm.n;
  }
  __syncthreads();
  int issued = 0;  // steps whose copy has been issued (the same in every thread)
  {
    const int first = min(ring.stages, steps);
    if (tid == 0) {
#pragma unroll 1
      for (int s = 0; s < first; ++s) {
        const int at = from + s * stage_elems;
        const uint32_t bytes = (uint32_t)(min(end, at + stage_elems) - at) * 4u;
        mbar_expect_tx(&ring.bars[s], bytes);
        bulk_load(ring.data + (size_t)s * stage_elems, row + at, bytes, &ring.bars[s]);
      }
    }
    issued = first;
  }
  const int region = c.region;
  unsigned long long* const mine = c.buf + c.keep + warp * region;
  int held = 0;
  float floor_l = select ? logit_floor(sm.tau, rc.tf) : __uint_as_float(0x7F800000u);
  bool stop = select && sm.overflow != 0;
  int it = 0;
#pragma unroll 1
  for (; it < steps && !stop; ++it) {
    const int s = it % ring.stages;
    const bool landed = mbar_wait_bounded(&ring.bars[s], (uint32_t)(it / ring.stages) & 1u);
    const int first = from + it * stage_elems + tid * 4;
    const float* stage = ring.data + (size_t)s * stage_elems;
    const float4* src = reinterpret_cast<const float4*>(stage) + tid;
    // sixteen logits, kept only as: which reach the floor, which a dense mask marks, max and min
    unsigned pm = 0u, xm = 0u;
    float hi = neg_inf(), lo = __uint_as_float(0x7F800000u);
#pragma unroll
    for (int u = 0; u < N / 4; ++u) {
      float4 x = make_float4(quiet_nan(), quiet_nan(), quiet_nan(), quiet_nan());
      const bool in = landed && first + u * stride < end;
      if (in) x = src[u * nt];
      pm |= (x.x >= floor_l ? 1u : 0u) << (u * 4 + 0);
      pm |= (x.y >= floor_l ? 1u : 0u) << (u * 4 + 1);
      pm |= (x.z >= floor_l ? 1u : 0u) << (u * 4 + 2);
      pm |= (x.w >= floor_l ? 1u : 0u) << (u * 4 + 3);
      if (want_hi) hi = fmaxf(fmaxf(hi, fmaxf(x.x, x.y)), fmaxf(x.z, x.w));
      if (want_lo) lo = fminf(fminf(lo, fminf(x.x, x.y)), fminf(x.z, x.w));
      if (dense && in) {
        const unsigned bytes = *reinterpret_cast<const unsigned*>(seen_row + first + u * stride);
        if (bytes) {
          xm |= ((bytes & 0xFFu) ? 1u : 0u) << (u * 4 + 0);
          xm |= ((bytes & 0xFF00u) ? 1u : 0u) << (u * 4 + 1);
          xm |= ((bytes & 0xFF0000u) ? 1u : 0u) << (u * 4 + 2);
          xm |= ((bytes & 0xFF000000u) ? 1u : 0u) << (u * 4 + 3);
        }
      }
    }
    // logits that may beat the greedy best, the whole-row gumbel best or the smallest score so far
    // The bounds are the block's, not the thread's: a thread's own best rises with every few
    // logits it sees, the block's only a dozen times per slice.  Ties with the bound still count
    // (the lower index wins), hence >= and <=.
    int what = 0;
    float bound_g = 0.0f, bound_a = 0.0f, bound_m = 0.0f;
    if (greedy) {
      bound_g = unord32(*reinterpret_cast<volatile unsigned*>(&sm.share_greedy));
      if (!(bound_g == bound_g)) bound_g = neg_inf();
      if (hi >= bound_g) what |= 1;
    }
    if (mode == M_ARGMAX_G) {
      bound_a = unord32(*reinterpret_cast<volatile unsigned*>(&sm.share_gumbel));
      if (!(bound_a == bound_a)) bound_a = neg_inf();
      if (scaled(hi, rc) + GUMBEL_MAX >= bound_a) what |= 2;
    }
    if (mode == M_SELECT_MINP) {
      bound_m = unord32(*reinterpret_cast<volatile unsigned*>(&sm.share_min));
      if (!(bound_m == bound_m)) bound_m = __uint_as_float(0x7F800000u);
      if (lo <= bound_m) what |= 4;
    }
    if (what) {
#pragma unroll 1
      for (int q = 0; q < N; ++q) {
        const int at = (q >> 2) * stride + (q & 3);
        if (first + at < end && !((xm >> q) & 1u)) {
          const float raw = stage[at + tid * 4];
          if (((what & 1) && raw >= bound_g) || ((what & 2) && scaled(raw, rc) + GUMBEL_MAX >= bound_a) ||
              ((what & 4) && raw <= bound_m))
            ring_visit<PEN>(P, rc, h, sm, seen_row, t, first + at, raw, what);
        }
      }
    }
    // what goes to the candidate buffer: logits at the floor, but under a dense mask only if the
    // penalised logit still reaches it
    unsigned am = select ? (pm & ~xm) : 0u;
    if (dense && xm) {
      const int all = (greedy ? 1 : 0) | (mode == M_ARGMAX_G ? 2 : 0) | (mode == M_SELECT_MINP ? 4 : 0);
      unsigned left = xm;
      while (left) {
        const int q = __ffs(left) - 1;
        left &= left - 1u;
        const int at = (q >> 2) * stride + (q & 3);
        const float raw = stage[at + tid * 4];
        if (all) ring_visit<PEN>(P, rc, h, sm, seen_row, t, first + at, raw, all);
        bool in_history = false;
        if (P.history) in_history = leat::in_history(h.keys, h.mask, first + at);
        if (select && !in_history && penalised(raw, 1, rc) >= floor_l) am |= 1u << q;
      }
    }
    int rounds = 0;
    while (true) {
      unsigned redo = 0u;
      if (select && __any_sync(FULL, am != 0u)) {
        // the warp's entries go to its own region: no atomics, one scan over the lanes; each lane
        // then walks its own few set bits and fetches the logit back from the stage
        const int count = __popc(am);
        int incl = count;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int o = __shfl_up_sync(FULL, incl, d);
          if (lane >= d) incl += o;
        }
        const int total = __shfl_sync(FULL, incl, 31);
        int slot = held + incl - count;
        unsigned left = am;
        while (left) {
          const int q = __ffs(left) - 1;
          left &= left - 1u;
          if (slot < region) {
            const int at = (q >> 2) * stride + (q & 3);
            float l = stage[at + tid * 4];
            if (dense && ((xm >> q) & 1u)) l = penalised(l, 1, rc);
            mine[slot] = ((unsigned long long)__float_as_uint(l) << 32) | (uint32_t)(first + at);
          } else {
            redo |= 1u << q;
          }
          ++slot;
        }
        held = min(held + total, region);
        if (lane == 0) sm.wcount[warp] = held;
      }
      // the step's barrier: every thread is done with the stage unless it has entries to redo;
      // did any warp run out of room, and did every copy land?
      const int verdict = __syncthreads_or((redo != 0u ? 1 : 0) | (landed ? 0 : 2));
      if (verdict & 2) {  // a copy never landed: give the row up
        if (tid == 0) { sm.overflow = 1; if (P.status) atomicOr(P.status, 4); }
        stop = true;
        break;
      }
      if (!(verdict & 1)) break;
      buffer_rebuild(c, 1);
      held = 0;
      floor_l = logit_floor(sm.tau, rc.tf);
      if (sm.overflow || ++rounds > 64) {
        if (tid == 0) sm.overflow = 1;
        stop = true;
        break;
      }
      // what did not fit is taken again from the stage, against the new floor
      am = 0u;
      while (redo) {
        const int q = __ffs(redo) - 1;
        redo &= redo - 1u;
        float l = stage[(q >> 2) * stride + tid * 4 + (q & 3)];
        if (dense && ((xm >> q) & 1u)) l = penalised(l, 1, rc);
        if (l >= floor_l) am |= 1u << q;
      }
    }
    // the stage is free: start the copy of the step that will use it next
    {
      const int next = it + ring.stages;
      if (next < steps && !stop) {
        if (tid == 0) {
          const int at = from + next * stage_elems;
          const uint32_t bytes = (uint32_t)(min(end, at + stage_elems) - at) * 4u;
          mbar_expect_tx(&ring.bars[s], bytes);
          bulk_load(ring.data + (size_t)s * stage_elems, row + at, bytes, &ring.bars[s]);
        }
        issued = next + 1;
      }
    }
  }
  // copies still in flight (the loop stopped early) must land before the ring is reused
#pragma unroll 1
  for (int j = it; j < issued; ++j)
    mbar_wait_bounded(&ring.bars[j % ring.stages], (uint32_t)(j / ring.stages) & 1u);
  __syncthreads();
}
