// Residual-stream kernels that are not contractions: embedding with a hashed token-pair table, scalar-gain RMS norm,
// token shift with carried state, the close of a parallel layer with depth-weighted averaging, row selection.
// One CTA per token row; the residual stream, the norms and the carried state are fp32 whatever the engine's type.
#include <cuda_bf16.h>

#include "asd_internal.h"
#include "blocks.h"
#include "elem.cuh"

namespace asd {

namespace {

// the row above is this sequence's previous position
__device__ __forceinline__ bool follows(const SeqIndex& ix, int m) {
    return m > 0 && ix.token_slot[m - 1] == ix.token_slot[m] && ix.positions[m - 1] == ix.positions[m] - 1;
}
// row m is one of the last `ring` rows of its run of consecutive positions: no later row of the batch lands on the
// same ring entry
__device__ __forceinline__ bool owns_ring_entry(const SeqIndex& ix, int m, int ring) {
    const int o = m + ring;
    return !(o < ix.M && ix.token_slot[o] == ix.token_slot[m] && ix.positions[o] == ix.positions[m] + ring);
}

__global__ void embed_pair_kernel(SeqIndex ix, const void* embed, const void* table, int wf32, int buckets, int mul_prev,
                                  int mul_cur, const int* tok_ring, int ring, float* x0, const void* g, float eps,
                                  float* hn, int D) {
    __shared__ float red[33];
    const int m = blockIdx.x;
    const int tok = ix.tokens[m], pos = ix.positions[m], slot = ix.token_slot[m];
    long long row;
    if (pos == 0) {
        row = buckets;
    } else {
        const int prev = follows(ix, m) ? ix.tokens[m - 1] : tok_ring[(long long)slot * ring + (pos - 1) % ring];
        row = (long long)(((unsigned long long)prev * (unsigned long long)mul_prev +
                           (unsigned long long)tok * (unsigned long long)mul_cur) % (unsigned long long)buckets);
    }
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float v = ldx(embed, (long long)tok * D + d, wf32) + ldx(table, row * D + d, wf32);
        x0[(long long)m * D + d] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float r = ldx(g, 0, wf32) / sqrtf(ss / (float)D + eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x) hn[(long long)m * D + d] = x0[(long long)m * D + d] * r;
}

__global__ void commit_tokens_kernel(SeqIndex ix, int* tok_ring, int ring) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= ix.M || !owns_ring_entry(ix, m, ring)) return;
    tok_ring[(long long)ix.token_slot[m] * ring + ix.positions[m] % ring] = ix.tokens[m];
}

__global__ void token_shift_kernel(SeqIndex ix, const float* hn, const float* state, int ring, const void* mu, int wf32,
                                   void* h, void* hs, int of32, int D) {
    const int m = blockIdx.x;
    const int pos = ix.positions[m];
    const float* prev = nullptr;
    if (pos > 0)
        prev = follows(ix, m) ? hn + (long long)(m - 1) * D
                              : state + ((long long)ix.token_slot[m] * ring + (pos - 1) % ring) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float v = hn[(long long)m * D + d];
        const float p = prev ? prev[d] : 0.f;
        stx(h, (long long)m * D + d, of32, v);
        stx(hs, (long long)m * D + d, of32, v + (p - v) * ldx(mu, d, wf32));
    }
}

__global__ void commit_shift_kernel(SeqIndex ix, const float* hn, float* state, int ring, int D) {
    const int m = blockIdx.x;
    if (!owns_ring_entry(ix, m, ring)) return;
    float* dst = state + ((long long)ix.token_slot[m] * ring + ix.positions[m] % ring) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) dst[d] = hn[(long long)m * D + d];
}

__global__ void layer_close_kernel(LayerClose L, SeqIndex ix) {
    __shared__ float red[33];
    const int m = blockIdx.x, D = L.D;
    const long long base = (long long)m * D;
    if (L.state_ring && owns_ring_entry(ix, m, L.ring)) {
        float* dst = L.state_ring + ((long long)ix.token_slot[m] * L.ring + ix.positions[m] % L.ring) * D;
        for (int d = threadIdx.x; d < D; d += blockDim.x) dst[d] = L.hn[base + d];
    }
    float* xnew = L.stack + (size_t)(L.layer + 1) * L.stack_stride + base;
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float y = L.mix[base + d];
        if (L.top > 0) {
            float f = 0.f;
            for (int k = 0; k < L.top; ++k)
                f += L.gate[(long long)m * L.top + k] * L.expert_out[(long long)L.slot_of[(long long)m * L.top + k] * D + d];
            y += f;
        }
        const float xn = L.x_in[base + d] + y;
        xnew[d] = xn;
        float a = 0.f;
        for (int j = 0; j <= L.layer; ++j) a += ldx(L.coeff, j, L.wf32) * L.stack[(size_t)j * L.stack_stride + base + d];
        a += ldx(L.coeff, L.layer + 1, L.wf32) * xn;
        L.x_next[base + d] = a;
        ss += a * a;
    }
    ss = block_sum(ss, red);
    const float r = ldx(L.g_next, 0, L.wf32) / sqrtf(ss / (float)D + L.eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x) L.hn[base + d] = L.x_next[base + d] * r;
}

__global__ void select_rows_kernel(const float* src, const int* rows, void* dst, int of32, int D) {
    const int r = blockIdx.x;
    const long long s = (long long)(rows ? rows[r] : r) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) stx(dst, (long long)r * D + d, of32, src[s + d]);
}

inline int row_threads(int D) { return D >= 1024 ? 256 : (D >= 256 ? 128 : 64); }

}  // namespace

int launch_embed_pair(const SeqIndex& ix, const void* embed, const void* pair_table, int wf32, int buckets, int mul_prev,
                      int mul_cur, const int* tok_ring, int ring, float* x0, const void* g, float eps, float* hn, int D,
                      cudaStream_t stream) {
    if (ix.M <= 0) return 0;
    if (buckets <= 0 || ring <= 0) return set_error("embed_pair: buckets and ring must be positive");
    embed_pair_kernel<<<ix.M, row_threads(D), 0, stream>>>(ix, embed, pair_table, wf32, buckets, mul_prev, mul_cur,
                                                           tok_ring, ring, x0, g, eps, hn, D);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_commit_tokens(const SeqIndex& ix, int* tok_ring, int ring, cudaStream_t stream) {
    if (ix.M <= 0) return 0;
    commit_tokens_kernel<<<(ix.M + 127) / 128, 128, 0, stream>>>(ix, tok_ring, ring);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_token_shift(const SeqIndex& ix, const float* hn, const float* state_ring, int ring, const void* mu, int wf32,
                       void* h, void* hs, int of32, int D, cudaStream_t stream) {
    if (ix.M <= 0) return 0;
    token_shift_kernel<<<ix.M, row_threads(D), 0, stream>>>(ix, hn, state_ring, ring, mu, wf32, h, hs, of32, D);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_commit_shift_state(const SeqIndex& ix, const float* hn, float* state_ring, int ring, int D,
                              cudaStream_t stream) {
    if (ix.M <= 0) return 0;
    commit_shift_kernel<<<ix.M, row_threads(D), 0, stream>>>(ix, hn, state_ring, ring, D);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_layer_close(const LayerClose& L, cudaStream_t stream) {
    if (L.M <= 0) return 0;
    if (L.state_ring && (!L.ix || L.ring <= 0)) return set_error("layer_close: the carried state needs the batch index and a ring");
    layer_close_kernel<<<L.M, row_threads(L.D), 0, stream>>>(L, L.ix ? *L.ix : SeqIndex{nullptr, nullptr, nullptr, 0});
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_select_rows(const float* src, const int* rows, void* dst, int of32, int n, int D, cudaStream_t stream) {
    if (n <= 0) return 0;
    select_rows_kernel<<<n, row_threads(D), 0, stream>>>(src, rows, dst, of32, D);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace asd
