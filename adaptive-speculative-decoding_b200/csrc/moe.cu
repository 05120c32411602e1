// Mixture-of-experts routing: fp32 softmax over all experts, the `top` largest probabilities kept as gates (as they
// are, no renormalisation), then the (token, choice) pairs grouped by expert so that each expert's rows are contiguous
// for the grouped linear layers.  Which slot inside an expert's group a pair gets does not matter for the result: every
// slot is computed on its own and a token's choices are summed in choice order by the layer close.
#include <cuda_runtime.h>
#include <math.h>

#include "asd_internal.h"
#include "blocks.h"
#include "elem.cuh"

namespace asd {

namespace {

// one warp per token; probs of the token live in shared memory (E floats per warp)
__global__ void moe_route_kernel(const float* logits, int M, int E, int top, int* expert_of, float* gate, int* counts) {
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m = blockIdx.x * (blockDim.x >> 5) + warp;
    if (m >= M) return;
    float* pr = sm + (size_t)warp * E;
    const float* z = logits + (long long)m * E;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float s = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float v = expf(z[e] - mx);
        pr[e] = v;
        s += v;
    }
    s = warp_sum(s);
    const float inv = 1.f / s;
    __syncwarp();
    for (int k = 0; k < top; ++k) {
        float best = -1.f;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = pr[e];
            if (v > best) {        // increasing e per lane: the first maximum wins
                best = v;
                bi = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) {
                best = ob;
                bi = oi;
            }
        }
        if (lane == 0) {
            expert_of[(long long)m * top + k] = bi;
            gate[(long long)m * top + k] = best * inv;
            atomicAdd(&counts[bi], 1);
            pr[bi] = -2.f;         // taken
        }
        __syncwarp();
    }
}

__global__ void moe_offsets_kernel(int* counters, int* group_off, int E) {
    if (threadIdx.x == 0) {
        int o = 0;
        for (int e = 0; e < E; ++e) {
            group_off[e] = o;
            o += counters[e];
            counters[E + e] = 0;   // fill counters of the scatter pass
        }
        group_off[E] = o;
    }
}

__global__ void moe_scatter_kernel(const int* expert_of, int n, int top, int E, const int* group_off, int* counters,
                                   int* sorted_tok, int* slot_of) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int e = expert_of[i];
    const int slot = group_off[e] + atomicAdd(&counters[E + e], 1);
    sorted_tok[slot] = i / top;
    slot_of[i] = slot;
}

}  // namespace

int launch_moe_route(const float* logits, int M, int E, int top, int* expert_of, float* gate, int* counters,
                     int* group_off, int* sorted_tok, int* slot_of, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E) return set_error("moe: need 0 < top <= experts (top %d, experts %d)", top, E);
    if ((size_t)E * 4 * sizeof(float) > 48 * 1024) return set_error("moe: more than 3072 experts");
    ASD_CUDA(cudaMemsetAsync(counters, 0, sizeof(int) * E, stream));
    moe_route_kernel<<<(M + 3) / 4, 128, (size_t)E * 4 * sizeof(float), stream>>>(logits, M, E, top, expert_of, gate,
                                                                                 counters);
    moe_offsets_kernel<<<1, 32, 0, stream>>>(counters, group_off, E);
    const int n = M * top;
    moe_scatter_kernel<<<(n + 255) / 256, 256, 0, stream>>>(expert_of, n, top, E, group_off, counters, sorted_tok, slot_of);
    count_launch(3);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace asd
