// Batched / grouped linear layer on tcgen05 for operands a tensor map cannot describe: rows gathered through an index
// (mixture-of-experts groups whose sizes only the device knows), per-head slices with their own weights, fp32
// activations that are rounded to bf16 on the way in.  Same operation and descriptor as linear_simt.cu:
//   C[z][m][n] = epilogue( sum_k bf16(A[z][row(m)][k]) * W[z][n][k] ),  fp32 accumulation in TMEM.
//
//   * swap-AB like gemm.cu: the 128 weight rows of a tile are the UMMA A operand (M = 128), the token tile (MT = 16 ..
//     128 rows) the B operand (N = MT), one accumulator [128 lanes x MT columns] in TMEM;
//   * operands go global -> registers -> shared memory in the K-major 128-byte-swizzled layout the MMA descriptors
//     expect (what TMA would have produced): 16-byte chunk c of row r lands at (r / 8) * 1024 + (r % 8) * 128 +
//     ((c ^ (r % 8)) * 16).  All 256 threads load; the registers of k-blocks i + 1 and i + 2 are in flight while k-block
//     i is stored, fenced to the async proxy and issued;
//   * three shared-memory stages; tcgen05.commit frees a stage when the MMAs that read it have retired;
//   * epilogue: the eight warps read their TMEM lane quarter 16 token columns at a time; lane = weight row, so the 32
//     lanes of a warp write 32 consecutive outputs of one token.
// Every wait on an mbarrier is bounded: on expiry the kernel raises the caller's error flag, stops waiting and still
// frees its TMEM.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "asd_internal.h"
#include "blocks.h"
#include "ptx.cuh"

namespace asd {

namespace {

constexpr int kRowsW = 128, kBK = 64, kThreads = 256, kStages = 3;
constexpr int kWBytes = kRowsW * kBK * 2;
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t swz(int r, int c) { return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4)); }

__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
// 8 consecutive k elements of one row as bf16 (16 bytes)
__device__ __forceinline__ uint4 load8(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint4 load8(const float* p) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    return make_uint4(pack2(a.x, a.y), pack2(a.z, a.w), pack2(b.x, b.y), pack2(b.z, b.w));
}

__device__ __forceinline__ bool wait_bounded(uint64_t* bar, uint32_t parity, volatile int* failed, int* err) {
    if (*failed) return false;
    for (uint32_t i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    *failed = 1;
    if (err) atomicExch(err, 1);
    return false;
}

template <typename TA, typename TC>
__global__ void __launch_bounds__(kThreads) tc_linear_kernel(SimtLinear L, int MT, uint32_t tmem_cols, int* err) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t empty_bar[kStages];
    __shared__ uint64_t acc_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int failed;
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
    const int m0 = blockIdx.y * MT, n0 = blockIdx.x * kRowsW;
    if (m0 >= rows) return;                                   // the whole CTA leaves before it owns anything
    const __nv_bfloat16* W = (const __nv_bfloat16*)L.w + (long long)z * L.w_zs;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int stage_bytes = kWBytes + MT * kBK * 2;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&empty_bar[s], 1);
        mbar_init(&acc_bar, 1);
        failed = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(&tmem_slot, tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    // loader mapping: thread -> 16-byte chunk c of rows r0 + 32 i
    const int c = tid & 7, r0 = tid >> 3;
    const __nv_bfloat16* wrow[4];
    const TA* xrow[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + 32 * i, n = n0 + r;
        wrow[i] = n < L.N ? W + (long long)n * L.ldw : nullptr;
        const int m = m0 + r;
        xrow[i] = nullptr;
        if (r < MT && m < rows) {
            const long long ar = L.group_off ? (L.gather ? L.gather[row0 + m] : row0 + m) : m;
            xrow[i] = A + ar * L.lda;
        }
    }
    const int nkb = (L.K + kBK - 1) / kBK;
    // two register sets: the loads of k-blocks i + 1 and i + 2 are in flight while k-block i is stored and issued
    uint4 wr[2][4], xr[2][4];
    const uint4 zero4 = make_uint4(0, 0, 0, 0);
    auto fetch = [&](int kb, uint4 (&w4)[4], uint4 (&x4)[4]) {
        const int k = kb * kBK + c * 8;
        const bool in = k < L.K;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            w4[i] = (in && wrow[i]) ? load8(wrow[i] + k) : zero4;
            x4[i] = (in && xrow[i]) ? load8(xrow[i] + k) : zero4;
        }
    };
    const uint32_t idesc = umma_idesc_bf16(kRowsW, MT);
    auto step = [&](int kb, uint4 (&w4)[4], uint4 (&x4)[4]) {
        const int s = kb % kStages, round = kb / kStages;
        if (round > 0) wait_bounded(&empty_bar[s], (round - 1) & 1, &failed, err);
        uint8_t* st = smem + (size_t)s * stage_bytes;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = r0 + 32 * i;
            *reinterpret_cast<uint4*>(st + swz(r, c)) = w4[i];
            if (r < MT) *reinterpret_cast<uint4*>(st + kWBytes + swz(r, c)) = x4[i];
        }
        if (kb + 2 < nkb) fetch(kb + 2, w4, x4);
        fence_proxy_async_smem();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            const uint32_t sa = smem_u32(st);
            const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sa + kWBytes);
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k) umma_f16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
            umma_commit(&empty_bar[s]);
            if (kb == nkb - 1) umma_commit(&acc_bar);
        }
    };
    fetch(0, wr[0], xr[0]);
    if (nkb > 1) fetch(1, wr[1], xr[1]);
    for (int kb = 0; kb < nkb; kb += 2) {
        step(kb, wr[0], xr[0]);
        if (kb + 1 < nkb) step(kb + 1, wr[1], xr[1]);
    }
    const bool ok = wait_bounded(&acc_bar, 0, &failed, err);
    tc_fence_after();
    if (ok) {
        const int q = warp & 3, n = n0 + q * 32 + lane;
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
        for (int j = warp >> 2; j * 16 < MT; j += 2) {
            if (m0 + j * 16 >= rows) break;                    // warp-uniform
            uint32_t r[16];
            tmem_ld_32x16(taddr + j * 16, r);
            tmem_ld_wait();
            if (n < L.N) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int m = m0 + j * 16 + i;
                    if (m >= rows) break;
                    float v = __uint_as_float(r[i]);
                    if (L.epilogue == 1) {
                        v = fmaxf(v, 0.f);
                        v = v * v;
                    }
                    TC* dst = C + (long long)(row0 + m) * L.ldc + n;
                    if constexpr (sizeof(TC) == 4)
                        *dst = v;
                    else
                        *dst = __float2bfloat16(v);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_cols);
    }
}

template <typename TA, typename TC>
int launch_t(const SimtLinear& L, dim3 grid, int MT, uint32_t cols, size_t smem, int* err, cudaStream_t s) {
    auto fn = tc_linear_kernel<TA, TC>;
    ASD_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    fn<<<grid, kThreads, smem, s>>>(L, MT, cols, err);
    return 0;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

bool tc_linear_supports(const SimtLinear& L) {
    if (L.w_f32 || L.K <= 0 || (L.K & 7) || (L.ldw & 7) || (L.w_zs & 7) || !aligned16(L.w) || !aligned16(L.a)) return false;
    const int am = L.a_f32 ? 3 : 7;
    if ((L.lda & am) || (!L.group_off && (L.a_zs & am))) return false;
    return true;
}

int launch_tc_linear(const SimtLinear& L, int* err_flag, cudaStream_t stream) {
    if (L.M <= 0 || L.N <= 0 || L.Z <= 0) return 0;
    if (!L.a || !L.w || !L.c || !tc_linear_supports(L)) return set_error("tc_linear: shape or alignment outside the kernel's contract");
    int MT = ((L.M < 128 ? L.M : 128) + 15) & ~15;
    uint32_t cols = 32;
    while ((int)cols < MT) cols <<= 1;
    const size_t smem = (size_t)kStages * (kWBytes + MT * kBK * 2) + 1024;
    dim3 grid((L.N + kRowsW - 1) / kRowsW, (L.M + MT - 1) / MT, L.Z);
    if (grid.y > 65535 || grid.z > 65535) return set_error("tc_linear: too many row tiles or batches");
    int rc;
    if (L.a_f32)
        rc = L.c_f32 ? launch_t<float, float>(L, grid, MT, cols, smem, err_flag, stream)
                     : launch_t<float, __nv_bfloat16>(L, grid, MT, cols, smem, err_flag, stream);
    else
        rc = L.c_f32 ? launch_t<__nv_bfloat16, float>(L, grid, MT, cols, smem, err_flag, stream)
                     : launch_t<__nv_bfloat16, __nv_bfloat16>(L, grid, MT, cols, smem, err_flag, stream);
    if (rc) return rc;
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace asd
