// Helpers shared by the kernels of the layer-list decoders (csrc/seq): dtype conversion, warp / block reductions,
// row -> sequence lookup, paged-cache indexing. Each .cu file pulls them in with `using namespace seqk`.
#pragma once
#include <cuda_bf16.h>

namespace seqk {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// sum over a block of NT threads (NT multiple of 32, <= 1024); every thread gets the total
template <int NT> __device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) scratch[w] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < NT / 32; ++i) t += scratch[i];
  return t;
}
// sequence that owns batch row t: largest s with qsl[s] <= t
__device__ __forceinline__ int find_seq(const int* __restrict__ qsl, int nseq, int t) {
  int lo = 0, hi = nseq - 1;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (qsl[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ size_t cache_index(int slot, int head, int d, int nheads, int dim, int ps, int slab) {
  const int page = slot / ps, off = slot - page * ps;
  return (((size_t)page * nheads + head) * (dim / slab) + d / slab) * ((size_t)ps * slab) + (size_t)off * slab + d % slab;
}

}  // namespace seqk
