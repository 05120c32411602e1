// Dense projection of an engine's activations, y fp32 [M][ldc] = x [M][K] * w[N][K]^T, routed by shape and element
// type: the weight-streaming tcgen05 GEMM (gemm.cu) for bf16 operands it accepts, its tensor-bound CTA-pair form
// (gemm_tc.cu) from `tc_min_rows` tokens on, the CUDA-core kernel (linear_simt.cu) for fp32 engines and every other
// shape.  Plans and tensor maps are cached per (call site, token count); a call site always passes the same buffers.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <unordered_map>

#include "blocks.h"
#include "gemm.h"

namespace asd {

struct DenseRunner {
    int f32 = 0;                 // 1: fp32 operands (always the CUDA-core kernel)
    int tc_linear = 1;
    int tc_min_rows = 257;       // token count from which the tensor-bound CTA-pair GEMM runs
    struct Entry {
        GemmPlan pl;
        TcPlan big;
        CUtensorMap tw, tx;
    };
    std::unordered_map<unsigned long long, Entry> cache;

    void clear() { cache.clear(); }

    int run(const void* x, const void* w, float* y, int M, int N, int K, int ldc, int key, cudaStream_t s) {
        if (!f32 && tc_linear && (K % 8) == 0 && (ldc % 4) == 0 && K >= 64 && N >= 8 &&
            (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
            (reinterpret_cast<uintptr_t>(y) & 15) == 0) {
            const unsigned long long k = ((unsigned long long)key << 32) | (unsigned)M;
            auto it = cache.find(k);
            if (it == cache.end()) {
                Entry t;
                if (make_tmap_bf16(&t.tw, w, N, K, K, 128)) return -1;
                if (M >= tc_min_rows) {   // above the HBM / tensor ridge: 256 weight rows x MT tokens on a CTA pair
                    if (gemm_tc_plan(&t.big, M, N, K, GEMM_OUT_F32, 1, 0)) return -1;
                    if (make_tmap_bf16(&t.tx, x, M, K, K, t.big.MT / 2)) return -1;
                } else {
                    if (gemm_plan(&t.pl, M, N, K, GEMM_OUT_F32, 0, 0, 1)) return -1;
                    if (make_tmap_bf16(&t.tx, x, M, K, K, t.pl.MT)) return -1;
                }
                it = cache.emplace(k, t).first;
            }
            if (M >= tc_min_rows)
                return gemm_tc_launch(it->second.big, it->second.tw, it->second.tx, y, ldc, N, 0, false, s, false, nullptr);
            return gemm_launch(it->second.pl, it->second.tw, it->second.tx, y, ldc, N, false, s, false);
        }
        SimtLinear L;
        L.a = x, L.a_f32 = f32, L.lda = K;
        L.w = w, L.w_f32 = f32, L.ldw = K;
        L.c = y, L.c_f32 = 1, L.ldc = ldc;
        L.M = M, L.N = N, L.K = K;
        return launch_simt_linear(L, s);
    }
};

}  // namespace asd
