// ops.argmax (leat/ops.py:496-500; the reference's two launches are leat/kernels/argmax.py:14-61)
// as one launch that streams the rows once.  Included inside namespace leat by sampler_kernels.cuh.
//
// A row is cut into `slices` spans of `span` logits, one block each.  A thread holds eight 128-bit
// loads at a time and keeps its largest value with the first index that had it (a NaN never beats
// anything); the block's best goes, as a (value, ~index) key whose maximum is the largest value at
// its smallest index, to the row's partials in the workspace; the block that arrives last for a row
// (one ticket per block) takes the largest partial and writes the row's index.  The ticket word is
// zero between calls: the last block clears it.
#pragma once

constexpr int AM_THREADS = 256;
constexpr int AM_VECS = 8;                          // 128-bit loads in flight per thread
constexpr int AM_ROUND = AM_THREADS * AM_VECS * 4;  // logits a block takes per round
constexpr int AM_MAX_SLICES = 64;

// rows of a multiple of four floats, 16-byte aligned; span a multiple of four
__global__ void __launch_bounds__(AM_THREADS, 4) argmax_kernel(const float* __restrict__ x, int vocab, long long row_stride,
                                                               int slices, int span, unsigned long long* partial,
                                                               unsigned* ticket, int* __restrict__ out) {
  __shared__ unsigned long long best[AM_THREADS / 32];
  __shared__ int last;
  const int b = blockIdx.y, slice = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int begin = slice * span, end = min(vocab, begin + span);
  const float* row = x + (size_t)b * row_stride;
  grid_dependency_wait();  // (launched as a programmatic dependent of whatever wrote x)
  grid_launch_dependents();
  float bv = neg_inf();
  int bi = NO_ID;
#pragma unroll 1
  for (int base = begin; base < end; base += AM_ROUND) {
    uint4 v[AM_VECS];
#pragma unroll
    for (int u = 0; u < AM_VECS; ++u) {
      const int i = base + (u * AM_THREADS + tid) * 4;
      v[u] = make_uint4(0xFF800000u, 0xFF800000u, 0xFF800000u, 0xFF800000u);
      if (i < end) v[u] = __ldcs(reinterpret_cast<const uint4*>(row + i));
    }
#pragma unroll
    for (int u = 0; u < AM_VECS; ++u) {
      const int i = base + (u * AM_THREADS + tid) * 4;
      const float f[4] = {__uint_as_float(v[u].x), __uint_as_float(v[u].y), __uint_as_float(v[u].z), __uint_as_float(v[u].w)};
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (f[e] > bv) { bv = f[e]; bi = i + e; }  // (a thread's indices only grow: the first of equals stays)
    }
  }
  unsigned long long key = bi != NO_ID ? make_key(bv, (uint32_t)bi) : 0ull;
  key = warp_max_u64(key);
  if (lane == 0) best[warp] = key;
  __syncthreads();
  if (tid == 0) {
    // a span of nothing but -inf and NaN answers with its first index
    unsigned long long k = make_key(neg_inf(), (uint32_t)begin);
#pragma unroll
    for (int w = 0; w < AM_THREADS / 32; ++w) k = best[w] > k ? best[w] : k;
    __stcg(&partial[(size_t)b * slices + slice], k);
    __threadfence();
    last = atomicAdd(&ticket[b], 1u) == (unsigned)(slices - 1) ? 1 : 0;
  }
  __syncthreads();
  if (last && tid < 32) {
    __threadfence();
    unsigned long long k = 0ull;
#pragma unroll 1
    for (int s = lane; s < slices; s += 32) {
      const unsigned long long p = __ldcg(&partial[(size_t)b * slices + s]);
      k = p > k ? p : k;
    }
    k = warp_max_u64(k);
    if (lane == 0) {
      out[b] = key_id(k);
      ticket[b] = 0u;
    }
  }
}
