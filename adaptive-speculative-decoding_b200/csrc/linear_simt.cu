// Batched / grouped linear layer on the CUDA cores: fp32 FMA accumulation in increasing k (slices of 16 summed on their
// own, then added up in order), any shape, any of
// {bf16, fp32} for the activations, the weights and the result.  It is the arithmetic of the fp32 engines (no tensor
// core has a true fp32 mode) and the fallback of the bf16 engines for shapes outside the tcgen05 GEMM's contract.
// 64 x 64 output tile per CTA, 16-deep k slices through shared memory, 4 x 4 results per thread.
#include <cuda_bf16.h>

#include "asd_internal.h"
#include "blocks.h"
#include "elem.cuh"

namespace asd {

namespace {

constexpr int TM = 64, TN = 64, TK = 16, PAD = 4;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) simt_linear_kernel(SimtLinear L) {
    __shared__ float As[TK][TM + PAD];
    __shared__ float Ws[TK][TN + PAD];
    const int z = blockIdx.z;
    int row0 = 0, rows = L.M;
    const TA* A = (const TA*)L.a;
    TC* C = (TC*)L.c;
    if (L.group_off) {
        row0 = L.group_off[z];
        rows = L.group_off[z + 1] - row0;
    } else {
        A += (long long)z * L.a_zs;
        C += (long long)z * L.c_zs;
    }
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    if (m0 >= rows) return;
    const TW* W = (const TW*)L.w + (long long)z * L.w_zs;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    // loader mapping: 256 threads fetch 64 rows x 16 k, four elements each (k fastest: rows are k-contiguous)
    const int lk = tid & 15, lr = tid >> 4;
    long long arow[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + lr + 16 * i;
        long long r = -1;
        if (m < rows) r = L.group_off ? (L.gather ? L.gather[row0 + m] : row0 + m) : m;
        arow[i] = r;
    }
    for (int k0 = 0; k0 < L.K; k0 += TK) {
        const int k = k0 + lk;
#pragma unroll
        for (int i = 0; i < 4; ++i)
            As[lk][lr + 16 * i] = (arow[i] >= 0 && k < L.K) ? ldf(A + arow[i] * L.lda + k) : 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int n = n0 + lr + 16 * i;
            Ws[lk][lr + 16 * i] = (n < L.N && k < L.K) ? ldf(W + (long long)n * L.ldw + k) : 0.f;
        }
        __syncthreads();
        // a slice's 16 products are summed on their own and then added to the total: the rounding error of a long sum
        // grows with sqrt(16) + sqrt(K / 16) instead of sqrt(K) steps, still in one fixed order
        float part[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) part[i][j] = 0.f;
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) part[i][j] = fmaf(a[i], b[j], part[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] += part[i][j];
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty + 16 * i;
        if (m >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx + 16 * j;
            if (n >= L.N) continue;
            float v = acc[i][j];
            if (L.epilogue == 1) {
                v = fmaxf(v, 0.f);
                v = v * v;
            }
            stf(C + (long long)(row0 + m) * L.ldc + n, v);
        }
    }
}

template <typename TA, typename TW>
int launch_c(const SimtLinear& L, dim3 grid, cudaStream_t s) {
    if (L.c_f32)
        simt_linear_kernel<TA, TW, float><<<grid, 256, 0, s>>>(L);
    else
        simt_linear_kernel<TA, TW, __nv_bfloat16><<<grid, 256, 0, s>>>(L);
    return 0;
}

}  // namespace

int launch_simt_linear(const SimtLinear& L, cudaStream_t stream) {
    if (L.M <= 0 || L.N <= 0 || L.Z <= 0) return 0;
    if (L.K <= 0 || !L.a || !L.w || !L.c) return set_error("simt_linear: bad arguments");
    dim3 grid((L.N + TN - 1) / TN, (L.M + TM - 1) / TM, L.Z);
    if (grid.y > 65535 || grid.z > 65535) return set_error("simt_linear: too many row tiles or batches");
    if (L.a_f32 && L.w_f32)
        launch_c<float, float>(L, grid, stream);
    else if (L.a_f32)
        launch_c<float, __nv_bfloat16>(L, grid, stream);
    else if (L.w_f32)
        launch_c<__nv_bfloat16, float>(L, grid, stream);
    else
        launch_c<__nv_bfloat16, __nv_bfloat16>(L, grid, stream);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace asd
