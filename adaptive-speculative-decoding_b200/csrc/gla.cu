// Gated linear attention: a recurrence with a [dk][dv] state per head and a decay per key channel,
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,   alpha_t = sigmoid(z_t)^(1 / tau).
// gla_decay_kernel:  alpha from the inner decay projection (one thread per channel, fp32).
// gla_recurrence_kernel: one CTA per (sequence, head, 32 value columns).  Columns of S never mix, so a CTA owns its
//   columns for the whole run of new positions: lane = column, warp = a slice of RS = ceil(dk / 32) consecutive key
//   rows' worth of state held in registers.  The new positions are staged CH at a time in shared memory (q, k, alpha
//   rows and the CTA's 32 value columns); per position every thread updates its rows and forms its slice's part of
//   o, and after the chunk the slices are added in index order.  The arithmetic per position is the same whatever the
//   chunking or the batch, so a sequence's outputs do not depend on how its tokens were cut into forwards.
//   The state lives in fp32 [slot][ring][head][dk][dv]; entry p % ring is the state after position p.
// gla_out_kernel: RMS norm of every head's o over dv (plain weight), times silu(gate).
#include <cuda_bf16.h>

#include "asd_internal.h"
#include "blocks.h"
#include "elem.cuh"

namespace asd {

namespace {

constexpr int GLA_CH = 16;   // positions staged per chunk
constexpr int GLA_NR = 32;   // state rows per thread at most

__global__ void gla_decay_kernel(const float* a, long long lda, const float* w_decay, const float* b_decay, GlaDims d,
                                 float* alpha) {
    extern __shared__ float av[];   // [low]
    const int m = blockIdx.x, n = d.heads * d.dk;
    for (int r = threadIdx.x; r < d.low; r += blockDim.x) av[r] = a[(long long)m * lda + r];
    __syncthreads();
    const float inv_tau = 1.f / d.tau;
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        const float* wr = w_decay + (long long)c * d.low;
        float z = 0.f;
        for (int r = 0; r < d.low; ++r) z = fmaf(wr[r], av[r], z);
        z += b_decay[c];
        // log sigmoid(z) = min(z, 0) - log1p(exp(-|z|))
        const float ls = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
        alpha[(long long)m * n + c] = expf(ls * inv_tau);
    }
}

__global__ void __launch_bounds__(256) gla_recurrence_kernel(SeqIndex ix, const int* cu_q, const int* seq_slot,
                                                             const float* q, const float* k, const float* v,
                                                             long long ld, const float* alpha, GlaDims d, float* state,
                                                             int ring, float* out) {
    extern __shared__ float sm[];
    const int seq = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * 32;
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    if (t0 >= t1) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, RS = blockDim.x >> 5;
    const int rows_per = (d.dk + RS - 1) / RS;          // <= GLA_NR
    const int r0 = warp * rows_per;
    const int col = col0 + lane;
    const bool col_ok = col < d.dv;
    const int slot = seq_slot[seq];
    const int p0 = ix.positions[t0];
    // shared: q, k, alpha [CH][dk] each, v [CH][32], partial o [RS][CH][32]
    float* qs = sm;
    float* ks = qs + GLA_CH * d.dk;
    float* as = ks + GLA_CH * d.dk;
    float* vs = as + GLA_CH * d.dk;
    float* part = vs + GLA_CH * 32;
    const long long st_head = ((long long)head * d.dk) * d.dv;
    const long long st_entry = (long long)d.heads * d.dk * d.dv;
    float* st_slot = state + (long long)slot * ring * st_entry;
    float S[GLA_NR];
#pragma unroll
    for (int r = 0; r < GLA_NR; ++r) S[r] = 0.f;
    if (p0 > 0 && col_ok) {
        const float* src = st_slot + (long long)((p0 - 1) % ring) * st_entry + st_head;
#pragma unroll
        for (int r = 0; r < GLA_NR; ++r)
            if (r < rows_per && r0 + r < d.dk) S[r] = src[(long long)(r0 + r) * d.dv + col];
    }
    const int hq = head * d.dk, hv = head * d.dv;
    const int n_alpha = d.heads * d.dk;
    for (int c0 = t0; c0 < t1; c0 += GLA_CH) {
        const int nt = min(GLA_CH, t1 - c0);
        __syncthreads();   // the previous chunk's partial sums have been read
        for (int i = threadIdx.x; i < nt * d.dk; i += blockDim.x) {
            const int t = i / d.dk, c = i % d.dk;
            const long long row = (long long)(c0 + t) * ld;
            qs[t * d.dk + c] = q[row + hq + c] * d.q_scale;
            ks[t * d.dk + c] = k[row + hq + c];
            as[t * d.dk + c] = alpha[(long long)(c0 + t) * n_alpha + hq + c];
        }
        for (int i = threadIdx.x; i < nt * 32; i += blockDim.x) {
            const int t = i >> 5, c = i & 31;
            vs[i] = col0 + c < d.dv ? v[(long long)(c0 + t) * ld + hv + col0 + c] : 0.f;
        }
        __syncthreads();
        for (int t = 0; t < nt; ++t) {
            const float vt = vs[t * 32 + lane];
            const float* qt = qs + t * d.dk + r0;
            const float* kt = ks + t * d.dk + r0;
            const float* at = as + t * d.dk + r0;
            float o = 0.f;
#pragma unroll
            for (int r = 0; r < GLA_NR; ++r) {
                if (r < rows_per && r0 + r < d.dk) {
                    S[r] = fmaf(at[r], S[r], kt[r] * vt);
                    o = fmaf(S[r], qt[r], o);
                }
            }
            part[(warp * GLA_CH + t) * 32 + lane] = o;
            // the last `ring` new positions leave their state behind
            const int m = c0 + t;
            if (t1 - m <= ring && col_ok) {
                float* dst = st_slot + (long long)((p0 + (m - t0)) % ring) * st_entry + st_head;
#pragma unroll
                for (int r = 0; r < GLA_NR; ++r)
                    if (r < rows_per && r0 + r < d.dk) dst[(long long)(r0 + r) * d.dv + col] = S[r];
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < nt * 32; i += blockDim.x) {
            const int t = i >> 5, c = i & 31;
            if (col0 + c >= d.dv) continue;
            float o = 0.f;
            for (int w = 0; w < RS; ++w) o += part[(w * GLA_CH + t) * 32 + c];
            out[(long long)(c0 + t) * d.heads * d.dv + hv + col0 + c] = o;
        }
    }
}

__global__ void gla_out_kernel(const float* o, const float* gate, long long ldg, const float* w, float eps, void* y,
                               int of32, int heads, int dv) {
    // one warp per (token, head)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * (blockDim.x >> 5) + warp;
    if (h >= heads) return;
    const long long m = blockIdx.x;
    const float* src = o + (m * heads + h) * dv;
    const float* g = gate + m * ldg + (long long)h * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss += src[i] * src[i];
    ss = warp_sum(ss);
    const float r = 1.f / sqrtf(ss / (float)dv + eps);
    for (int i = lane; i < dv; i += 32) {
        const float gv = g[i];
        stx(y, (m * heads + h) * dv + i, of32, src[i] * r * w[i] * (gv / (1.f + expf(-gv))));
    }
}

}  // namespace

int launch_gla_decay(const float* a, long long lda, const float* w_decay, const float* b_decay, const GlaDims& d,
                     float* alpha, int M, cudaStream_t stream) {
    if (M <= 0) return 0;
    if (d.low <= 0 || !(d.tau > 0.f)) return set_error("gla: decay projection of size %d, tau %f", d.low, d.tau);
    gla_decay_kernel<<<M, 128, d.low * sizeof(float), stream>>>(a, lda, w_decay, b_decay, d, alpha);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_gla_recurrence(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, const float* q,
                          const float* k, const float* v, long long ld, const float* alpha, const GlaDims& d,
                          float* state, int ring, float* out, cudaStream_t stream) {
    if (ix.M <= 0 || nseq <= 0) return 0;
    if (d.dk <= 0 || d.dk > 8 * GLA_NR) return set_error("gla: key size %d outside 1..%d", d.dk, 8 * GLA_NR);
    if (ring <= 0 || !state) return set_error("gla: no state");
    const int RS = (d.dk + GLA_NR - 1) / GLA_NR;     // warps: slices of at most GLA_NR key rows
    const size_t smem = (size_t)(3 * GLA_CH * d.dk + GLA_CH * 32 + RS * GLA_CH * 32) * sizeof(float);
    if (smem > 48 * 1024)
        ASD_CUDA(cudaFuncSetAttribute(gla_recurrence_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(nseq, d.heads, (d.dv + 31) / 32);
    if (grid.y > 65535 || grid.z > 65535) return set_error("gla: too many heads or value columns");
    gla_recurrence_kernel<<<grid, RS * 32, smem, stream>>>(ix, cu_q, seq_slot, q, k, v, ld, alpha, d, state, ring, out);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_gla_out(const float* o, const float* gate, long long ldg, const float* w, float eps, void* y, int of32, int M,
                   int heads, int dv, cudaStream_t stream) {
    if (M <= 0) return 0;
    const int wpb = heads < 8 ? heads : 8;
    dim3 grid(M, (heads + wpb - 1) / wpb);
    gla_out_kernel<<<grid, wpb * 32, 0, stream>>>(o, gate, ldg, w, eps, y, of32, heads, dv);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace asd
