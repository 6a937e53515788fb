// Device helpers shared by the sampler kernels: order-preserving keys, the hashed uniform of the
// reference draw, and float32 elementary functions evaluated the way the reference's runtime
// lowers them (exp as exp2(x * log2 e), log as log2(x) * ln 2).  Built with -fmad=false: every
// product and sum below is rounded separately, as the CPU statement of the algorithm does.
#pragma once
#include <cuda_bf16.h>
#include <type_traits>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace leat {

constexpr unsigned FULL = 0xFFFFFFFFu;

__device__ __forceinline__ float log2e() { return __uint_as_float(0x3FB8AA3Bu); }  // f32(1 / ln 2)
__device__ __forceinline__ float ln2() { return __uint_as_float(0x3F317218u); }    // f32(ln 2)
__device__ __forceinline__ float neg_inf() { return __uint_as_float(0xFF800000u); }
__device__ __forceinline__ float quiet_nan() { return __uint_as_float(0x7FC00000u); }

// float -> uint32 whose unsigned order is the float order (-inf lowest, +inf highest)
__device__ __forceinline__ uint32_t ord32(float f) {
  uint32_t b = __float_as_uint(f);
  return b ^ ((b >> 31) ? 0xFFFFFFFFu : 0x80000000u);
}
__device__ __forceinline__ float unord32(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}
// (value, id) -> 64-bit key: larger value first, then smaller id.  -0 is folded onto +0 so that
// equal floats give equal value bits.
__device__ __forceinline__ unsigned long long make_key(float value, uint32_t id) {
  return ((unsigned long long)ord32(value + 0.0f) << 32) | (unsigned long long)(~id);
}
__device__ __forceinline__ float key_value(unsigned long long k) { return unord32((uint32_t)(k >> 32)); }
__device__ __forceinline__ uint32_t key_vbits(unsigned long long k) { return (uint32_t)(k >> 32); }
__device__ __forceinline__ int key_id(unsigned long long k) { return (int)(~(uint32_t)k); }

// lowbias32 (leat/sampler.py:67-73); unsigned arithmetic wraps to 32 bits by definition
__device__ __forceinline__ uint32_t lowbias32(uint32_t x) {
  x = (x ^ (x >> 16)) * 0x7FEB352Du;
  x = (x ^ (x >> 15)) * 0x846CA68Bu;
  return x ^ (x >> 16);
}
// key of a row: h(h(seed) + u32(position))  (leat/sampler.py:62)
__device__ __forceinline__ uint32_t row_key(uint32_t seed, int position) {
  return lowbias32(lowbias32(seed) + (uint32_t)position);
}
// the uniform of token `id` in a row (leat/sampler.py:63-64): 23 bits, in (0, 1)
__device__ __forceinline__ float hashed_uniform(uint32_t id, uint32_t key) {
  uint32_t bits = lowbias32(id ^ key);
  return ((float)(bits >> 9) + 0.5f) * 1.1920928955078125e-07f;  // 2^-23
}
__device__ __forceinline__ float exp_ref(float x) { return exp2f(x * log2e()); }
__device__ __forceinline__ float log_ref(float x) { return log2f(x) * ln2(); }
// Gumbel noise of leat/sampler.py:53: -log(-log(u))
__device__ __forceinline__ float gumbel(float u) { return -log_ref(-log_ref(u)); }

__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    unsigned long long o = __shfl_xor_sync(FULL, v, d);
    v = o > v ? o : v;
  }
  return v;
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may
// start while the kernel before it in the stream still runs; it must not touch what that kernel
// writes before grid_dependency_wait() returns (the earlier grid complete, its writes visible).
// grid_launch_dependents() lets the next kernel's blocks be scheduled from here on.  Both do nothing
// in a kernel launched the ordinary way.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Measurement aid: with a stamps array (16 words, zeroed before the call) a kernel's blocks record
// the earliest begin and the latest end of kernel `k` on the GPU's nanosecond timer.  Begins are kept
// complemented, so that one atomicMax serves both and zero means "never ran".
__device__ __forceinline__ unsigned long long global_nanoseconds() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void stamp_begin(unsigned long long* stamps, int k) {
  if (stamps && threadIdx.x == 0) atomicMax(&stamps[2 * k], ~global_nanoseconds());
}
__device__ __forceinline__ void stamp_end(unsigned long long* stamps, int k) {
  if (stamps && threadIdx.x == 0) atomicMax(&stamps[2 * k + 1], global_nanoseconds());
}

}  // namespace leat
