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
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0u;
}
// false if the copy has not landed after about a million polls (far beyond any real latency)
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, uint32_t parity) {
  for (int spin = 0; spin < (1 << 20); ++spin)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

#ifdef LEAT_PHASE_CLOCKS
#define RING_CLOCK(x) long long x = clock64()
#define RING_ADD(i, d) do { if (threadIdx.x == 0) atomicAdd(&g_phase_cycles[i], (unsigned long long)(d)); } while (0)
#define RING_SET(x, y) x = y
#else
#define RING_CLOCK(x) do { } while (0)
#define RING_ADD(i, d) do { } while (0)
#define RING_SET(x, y) do { } while (0)
#endif

constexpr int RING_PER_THREAD = 16;  // logits a thread takes from a stage

struct Ring {
  float* data;              // stages x (threads x 16) floats
  unsigned long long* bars; // one mbarrier per stage
  int stages;
};

// MODE is M_SELECT_K, M_ARGMAX_L or M_ARGMAX_G.  Streams [from, end) of `row`; `from` and the row
// are 16-byte aligned and end - from is a multiple of 4.
template <bool PEN, int MODE>
__device__ __noinline__ void stream_ring(const KParams& P, const RowCfg& rc, const Ctx& c, const History& h,
                                         const float* __restrict__ row, int from, int end, Tracked& t,
                                         Ring ring) {
  Shared& sm = *c.sm;
  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5;
  constexpr int N = RING_PER_THREAD;
  constexpr bool SELECT = MODE == M_SELECT_K;
  const int off = P.vocab_offset;
  const int stage_elems = nt * N;
  const int steps = (end - from + stage_elems - 1) / stage_elems;
  const int stride = nt * 4;

  if (tid == 0) {
    for (int s = 0; s < ring.stages; ++s) mbar_init(&ring.bars[s], 1);
    mbar_fence_init();
  }
  if (SELECT) {
    // keys so far fit the first `keep` slots; the rest of the buffer is one raw region per warp
    if (sm.n > c.keep) buffer_rebuild(c, 0);
    for (int i = sm.n + tid; i < c.keep; i += nt) c.buf[i] = 0ull;
    if (tid < 32) sm.wcount[tid] = 0;
    if (tid == 0) sm.conv = sm.n;
  }
  __syncthreads();
  int issued = 0;  // steps whose copy has been issued (the same in every thread)
  {
    const int first = min(ring.stages, steps);
    if (tid == 0) {
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
  float floor_l = SELECT ? logit_floor(sm.tau, rc.tf) : 0.0f;
  bool stop = SELECT && sm.overflow != 0;
  int it = 0;
  for (; it < steps && !stop; ++it) {
    RING_CLOCK(a0);
    const int s = it % ring.stages;
    const bool landed = mbar_wait_bounded(&ring.bars[s], (uint32_t)(it / ring.stages) & 1u);
    RING_CLOCK(a1);
    const int base = from + it * stage_elems;
    const int first = base + tid * 4;
    const float* stage = ring.data + (size_t)s * stage_elems;
    const float4* src = reinterpret_cast<const float4*>(stage) + tid;
    // sixteen logits: kept only as a mask of those at or above the floor, and their maximum
    unsigned pm = 0u;
    float m = neg_inf();
#pragma unroll
    for (int u = 0; u < N / 4; ++u) {
      float4 x = make_float4(quiet_nan(), quiet_nan(), quiet_nan(), quiet_nan());
      if (landed && first + u * stride < end) x = src[u * nt];
      if (SELECT) {
        pm |= (x.x >= floor_l ? 1u : 0u) << (u * 4 + 0);
        pm |= (x.y >= floor_l ? 1u : 0u) << (u * 4 + 1);
        pm |= (x.z >= floor_l ? 1u : 0u) << (u * 4 + 2);
        pm |= (x.w >= floor_l ? 1u : 0u) << (u * 4 + 3);
      }
      if (MODE != M_SELECT_K || rc.track) m = fmaxf(fmaxf(m, fmaxf(x.x, x.y)), fmaxf(x.z, x.w));
    }
    // greedy tracking: the largest raw logit that no history entry penalises
    if ((MODE == M_ARGMAX_L || rc.track) && m > t.gl) {
      for (int q = 0; q < N; ++q) {
        const int idx = first + (q >> 2) * stride + (q & 3);
        const float l = idx < end ? stage[(q >> 2) * stride + tid * 4 + (q & 3)] : quiet_nan();
        if (l > t.gl) {
          bool penalised_elsewhere = false;
          if (PEN && P.history) {
            const int local = idx - h.begin;
            penalised_elsewhere = (h.bitmap[local >> 5] >> (local & 31)) & 1u;
          }
          if (!penalised_elsewhere) { t.gl = l; t.gid = idx; }
        }
      }
    }
    // score + gumbel can only win if score + the largest gumbel reaches the best so far
    if (MODE == M_ARGMAX_G && scaled(m, rc) + GUMBEL_MAX >= t.al) {
      for (int q = 0; q < N; ++q) {
        const int idx = first + (q >> 2) * stride + (q & 3);
        const float l = idx < end ? stage[(q >> 2) * stride + tid * 4 + (q & 3)] : quiet_nan();
        const float sc = scaled(l, rc);
        if (sc + GUMBEL_MAX >= t.al) {
          bool penalised_elsewhere = false;
          if (PEN && P.history) {
            const int local = idx - h.begin;
            penalised_elsewhere = (h.bitmap[local >> 5] >> (local & 31)) & 1u;
          }
          if (!penalised_elsewhere) {
            const float d = sc + gumbel(hashed_uniform((uint32_t)(idx + off), rc.rkey));
            if (d > t.al) { t.al = d; t.aid = idx; }
          }
        }
      }
    }
    int rounds = 0;
    while (true) {
      unsigned redo = 0u;
      if (SELECT && __any_sync(FULL, pm != 0u)) {
        // the warp's passing logits go to its own region: no atomics, one scan over the lanes;
        // each lane then walks its own few set bits and fetches the logit back from the stage
        const int count = __popc(pm);
        int incl = count;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int o = __shfl_up_sync(FULL, incl, d);
          if (lane >= d) incl += o;
        }
        const int total = __shfl_sync(FULL, incl, 31);
        int slot = held + incl - count;
        unsigned left = pm;
        while (left) {
          const int q = __ffs(left) - 1;
          left &= left - 1u;
          if (slot < region) {
            const int at = (q >> 2) * stride + (q & 3);
            const float l = stage[at + tid * 4];
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
      RING_CLOCK(a2);
      const int verdict = __syncthreads_or((redo != 0u ? 1 : 0) | (landed ? 0 : 2));
      RING_CLOCK(a3);
      RING_ADD(8, a1 - a0); RING_ADD(9, a2 - a1); RING_ADD(10, a3 - a2); RING_ADD(13, 1);
      if (verdict & 2) {  // a copy never landed: give the row up
        if (tid == 0) { sm.overflow = 1; if (P.status) atomicOr(P.status, 4); }
        stop = true;
        break;
      }
      if (!(verdict & 1)) break;
      buffer_rebuild(c, 1);
      RING_CLOCK(a4);
      RING_ADD(11, a4 - a3); RING_ADD(12, 1);
      RING_SET(a1, a4);
      held = 0;
      floor_l = logit_floor(sm.tau, rc.tf);
      if (sm.overflow || ++rounds > 64) {
        if (tid == 0) sm.overflow = 1;
        stop = true;
        break;
      }
      // what did not fit is taken again from the stage, against the new floor
      pm = 0u;
      while (redo) {
        const int q = __ffs(redo) - 1;
        redo &= redo - 1u;
        if (stage[(q >> 2) * stride + tid * 4 + (q & 3)] >= floor_l) pm |= 1u << q;
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
  for (int j = it; j < issued; ++j)
    mbar_wait_bounded(&ring.bars[j % ring.stages], (uint32_t)(j / ring.stages) & 1u);
  __syncthreads();
}
