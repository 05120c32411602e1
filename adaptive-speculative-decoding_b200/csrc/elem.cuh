// Element access for kernels that are instantiated for bf16 and for fp32 buffers, and block-wide sums.
#pragma once
#include <cuda_bf16.h>

namespace asd {

template <typename T>
__device__ __forceinline__ float ldf(const T* p) {
    return (float)*p;
}
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) {
    return __bfloat162float(*p);
}
template <typename T>
__device__ __forceinline__ void stf(T* p, float v) {
    *p = v;
}
template <>
__device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) {
    *p = __float2bfloat16(v);
}
// runtime-typed forms (f32 flag: 0 = bf16, 1 = fp32) for kernels whose arithmetic dwarfs the branch
__device__ __forceinline__ float ldx(const void* p, long long i, int f32) {
    return f32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ void stx(void* p, long long i, int f32, float v) {
    if (f32)
        ((float*)p)[i] = v;
    else
        ((__nv_bfloat16*)p)[i] = __float2bfloat16(v);
}

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
// sum over the block in a fixed order (warp sums, then the warps in index order); red: >= 33 floats of shared memory
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int i = 0; i < nw; ++i) t += red[i];
        red[32] = t;
    }
    __syncthreads();
    return red[32];
}

}  // namespace asd
