// Gated linear attention: a recurrence with a [dk][dv] state per head and a decay per key channel,
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,   alpha_t = sigmoid(z_t)^(1 / tau).
// gla_decay_kernel:  alpha from the inner decay projection (one thread per channel and 32 tokens, fp32).
// gla_recurrence_kernel: one CTA per (sequence, head, 32 value columns).  Columns of S never mix, so a CTA owns its
//   columns for the whole run of new positions: lane = column, warp = a slice of 4 to 32 consecutive key rows' worth of
//   state held in registers (up to eight warps).  The new positions are staged CH at a time in shared memory (q, k,
//   decay rows and the CTA's 32 value columns) by cp.async, one chunk ahead; per position every thread
//   updates its rows and forms its slice's part of o, and after the chunk the slices are added in index order.  The arithmetic per position is the same whatever the
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

__device__ __forceinline__ void cp_async4(float* dst, const float* src, bool valid) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(dst);
    const int sz = valid ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(addr), "l"(src), "r"(sz) : "memory");
}

constexpr int GD_TOK = 32, GD_CH = 256;   // tokens x channels per CTA of the decay kernel

// One CTA = 256 channels x 32 tokens: the channels' projection rows are staged transposed ([low][256], so that the
// threads of a warp read consecutive words) and reused for all the tile's tokens, whose inner vectors every thread
// reads as broadcasts.
__global__ void __launch_bounds__(GD_CH) gla_decay_kernel(const float* a, long long lda, const float* w_decay,
                                                          const float* b_decay, GlaDims d, float* alpha, int M) {
    extern __shared__ float sm[];
    float* wT = sm;                      // [low][GD_CH]
    float* av = sm + d.low * GD_CH;      // [GD_TOK][low]
    const int n = d.heads * d.dk;
    const int c0 = blockIdx.x * GD_CH, m0 = blockIdx.y * GD_TOK;
    const int nt = min(GD_TOK, M - m0);
    for (int i = threadIdx.x; i < GD_CH * d.low; i += GD_CH) {
        const int c = i / d.low, r = i - c * d.low;
        wT[r * GD_CH + c] = c0 + c < n ? w_decay[(long long)(c0 + c) * d.low + r] : 0.f;
    }
    for (int i = threadIdx.x; i < GD_TOK * d.low; i += GD_CH) {
        const int t = i / d.low, r = i - t * d.low;
        av[i] = t < nt ? a[(long long)(m0 + t) * lda + r] : 0.f;
    }
    __syncthreads();
    const int c = c0 + threadIdx.x;
    if (c >= n) return;
    float z[GD_TOK];
#pragma unroll
    for (int t = 0; t < GD_TOK; ++t) z[t] = 0.f;
    for (int r = 0; r < d.low; ++r) {
        const float w = wT[r * GD_CH + threadIdx.x];
#pragma unroll
        for (int t = 0; t < GD_TOK; ++t) z[t] = fmaf(w, av[t * d.low + r], z[t]);
    }
    const float bias = b_decay[c], inv_tau = 1.f / d.tau;
#pragma unroll
    for (int t = 0; t < GD_TOK; ++t) {
        if (t < nt) {
            const float zz = z[t] + bias;
            // log sigmoid(z) = min(z, 0) - log1p(exp(-|z|)).  A slow decay lies just below 1, where expf's two units in
            // the last place are a relative error of 1e-7 that hundreds of steps multiply; 1 + expm1 is rounded once
            const float ls = fminf(zz, 0.f) - log1pf(expf(-fabsf(zz)));
            alpha[(long long)(m0 + t) * n + c] = 1.f + expm1f(ls * inv_tau);
        }
    }
}

// ROWS state rows per thread (a multiple of 4: the staged q, k and decay rows are read as float4); the staged rows are
// padded with zeros up to warps x ROWS, so rows beyond dk keep a zero state and add nothing.
// CH positions are staged per chunk; MAXT bounds the CTA's threads (32 per slice of ROWS key rows).
template <int ROWS, int MAXT, int CH>
__global__ void __launch_bounds__(MAXT, MAXT <= 256 ? 2 : 1) gla_recurrence_kernel(SeqIndex ix, const int* cu_q, const int* seq_slot,
                                                            const float* q, const float* k, const float* v, long long ld,
                                                            const float* alpha, GlaDims d, float* state, int ring,
                                                            float* out) {
    extern __shared__ __align__(16) float sm[];
    const int seq = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * 32;
    const int t0 = cu_q[seq], t1 = cu_q[seq + 1];
    if (t0 >= t1) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, RS = blockDim.x >> 5, nthr = blockDim.x;
    const int dkp = RS * ROWS;                          // padded key size
    const int r0 = warp * ROWS;
    const int col = col0 + lane;
    const bool col_ok = col < d.dv;
    const int slot = seq_slot[seq];
    const int p0 = ix.positions[t0];
    // shared: two buffers of { q, k, decay [CH][dkp] each, v [CH][32] }, then the partial o [RS][CH][32]
    const int buf_elems = 3 * CH * dkp + CH * 32;
    float* part = sm + 2 * buf_elems;
    const long long st_head = ((long long)head * d.dk) * d.dv;
    const long long st_entry = (long long)d.heads * d.dk * d.dv;
    float* st_slot = state + (long long)slot * ring * st_entry;
    float S[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) S[r] = 0.f;
    if (p0 > 0 && col_ok) {
        const float* src = st_slot + (long long)((p0 - 1) % ring) * st_entry + st_head;
#pragma unroll
        for (int r = 0; r < ROWS; ++r)
            if (r0 + r < d.dk) S[r] = src[(long long)(r0 + r) * d.dv + col];
    }
    const int hq = head * d.dk, hv = head * d.dv;
    const int n_alpha = d.heads * d.dk;
    // a chunk's rows arrive by 4-byte cp.async (any alignment), one chunk ahead of the arithmetic; rows beyond the
    // chunk's positions and key channels beyond dk are filled with zeros
    auto fetch = [&](int buf, int c0) {
        const int nt = min(CH, t1 - c0);
        float* qd = sm + buf * buf_elems;
        float* kd = qd + CH * dkp;
        float* ad = kd + CH * dkp;
        float* vd = ad + CH * dkp;
        for (int i = threadIdx.x; i < nt * dkp; i += nthr) {        // rows beyond the chunk's positions are never read
            const int t = i / dkp, c = i - t * dkp;
            const bool ok = c < d.dk;
            const long long row = ok ? (long long)(c0 + t) * ld + hq + c : 0;
            cp_async4(qd + i, q + row, ok);
            cp_async4(kd + i, k + row, ok);
            cp_async4(ad + i, alpha + (ok ? (long long)(c0 + t) * n_alpha + hq + c : 0), ok);
        }
        for (int i = threadIdx.x; i < nt * 32; i += nthr) {
            const int t = i >> 5, c = i & 31;
            const bool ok = col0 + c < d.dv;
            cp_async4(vd + i, v + (ok ? (long long)(c0 + t) * ld + hv + col0 + c : 0), ok);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(0, t0);
    int it = 0;
    for (int c0 = t0; c0 < t1; c0 += CH, ++it) {
        const int nt = min(CH, t1 - c0);
        if (c0 + CH < t1) {
            fetch((it + 1) & 1, c0 + CH);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();   // this chunk's rows have landed for every thread; the previous partial sums have been read
        const float* qs = sm + (it & 1) * buf_elems;
        const float* ks = qs + CH * dkp;
        const float* as = ks + CH * dkp;
        const float* vs = as + CH * dkp;
        for (int t = 0; t < nt; ++t) {
            const float vt = vs[t * 32 + lane];
            const float4* qt = reinterpret_cast<const float4*>(qs + t * dkp + r0);
            const float4* kt = reinterpret_cast<const float4*>(ks + t * dkp + r0);
            const float4* at = reinterpret_cast<const float4*>(as + t * dkp + r0);
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
            for (int r = 0; r < ROWS; r += 4) {
                const float4 a4 = at[r >> 2], k4 = kt[r >> 2], q4 = qt[r >> 2];
                S[r] = fmaf(a4.x, S[r], k4.x * vt);
                S[r + 1] = fmaf(a4.y, S[r + 1], k4.y * vt);
                S[r + 2] = fmaf(a4.z, S[r + 2], k4.z * vt);
                S[r + 3] = fmaf(a4.w, S[r + 3], k4.w * vt);
                o0 = fmaf(S[r], q4.x, o0);
                o1 = fmaf(S[r + 1], q4.y, o1);
                o2 = fmaf(S[r + 2], q4.z, o2);
                o3 = fmaf(S[r + 3], q4.w, o3);
            }
            part[(warp * CH + t) * 32 + lane] = (o0 + o1) + (o2 + o3);
            // the last `ring` new positions leave their state behind
            const int m = c0 + t;
            if (t1 - m <= ring && col_ok) {
                float* dst = st_slot + (long long)((p0 + (m - t0)) % ring) * st_entry + st_head;
#pragma unroll
                for (int r = 0; r < ROWS; ++r)
                    if (r0 + r < d.dk) dst[(long long)(r0 + r) * d.dv + col] = S[r];
            }
        }
        __syncthreads();   // the chunk is consumed (its buffer may be refilled) and the partial sums are complete
        for (int i = threadIdx.x; i < nt * 32; i += nthr) {
            const int t = i >> 5, c = i & 31;
            if (col0 + c >= d.dv) continue;
            float o = 0.f;
            for (int w = 0; w < RS; ++w) o += part[(w * CH + t) * 32 + c];
            out[(long long)(c0 + t) * d.heads * d.dv + hv + col0 + c] = o * d.q_scale;
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
    const size_t smem = (size_t)d.low * (GD_CH + GD_TOK) * sizeof(float);
    if (smem > 200 * 1024) return set_error("gla: decay projection of size %d does not fit shared memory", d.low);
    static PerDeviceOnce once;
    if (once.need()) ASD_CUDA(cudaFuncSetAttribute(gla_decay_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    dim3 grid((d.heads * d.dk + GD_CH - 1) / GD_CH, (M + GD_TOK - 1) / GD_TOK);
    if (grid.y > 65535) return set_error("gla: too many tokens");
    gla_decay_kernel<<<grid, GD_CH, smem, stream>>>(a, lda, w_decay, b_decay, d, alpha, M);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_gla_recurrence(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, const float* q,
                          const float* k, const float* v, long long ld, const float* alpha, const GlaDims& d,
                          float* state, int ring, float* out, cudaStream_t stream) {
    if (ix.M <= 0 || nseq <= 0) return 0;
    if (d.dk <= 0 || d.dk > 32 * GLA_NR) return set_error("gla: key size %d outside 1..%d", d.dk, 32 * GLA_NR);
    if (ring <= 0 || !state) return set_error("gla: no state");
    // the fewest state rows per thread (4, 8, 16 or 32) that at most eight warps cover
    int rows = 4;
    while (rows < GLA_NR && rows * 8 < d.dk) rows *= 2;
    const int RS = (d.dk + rows - 1) / rows;              // more than eight warps only for key sizes above 256
    const int dkp = RS * rows;
    const int ch = RS <= 8 ? GLA_CH : GLA_CH / 4;         // shorter chunks keep the staged rows of a large head in shared memory
    const size_t smem = (size_t)(2 * (3 * ch * dkp + ch * 32) + RS * ch * 32) * sizeof(float);
    dim3 grid(nseq, d.heads, (d.dv + 31) / 32);
    if (grid.y > 65535 || grid.z > 65535) return set_error("gla: too many heads or value columns");
#define ASD_GLA_CASE(R, T, C)                                                                                         \
    {                                                                                                                 \
        auto fn = gla_recurrence_kernel<R, T, C>;                                                                        \
        static PerDeviceOnce once;                                                                                    \
        if (once.need()) ASD_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)); \
        fn<<<grid, RS * 32, smem, stream>>>(ix, cu_q, seq_slot, q, k, v, ld, alpha, d, state, ring, out);             \
    }
    if (RS > 8) ASD_GLA_CASE(32, 1024, GLA_CH / 4)
    else if (rows == 4) ASD_GLA_CASE(4, 256, GLA_CH)
    else if (rows == 8) ASD_GLA_CASE(8, 256, GLA_CH)
    else if (rows == 16) ASD_GLA_CASE(16, 256, GLA_CH)
    else ASD_GLA_CASE(32, 256, GLA_CH)
#undef ASD_GLA_CASE
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
