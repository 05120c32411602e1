// Latent key/value attention in latent space over a paged cache of [R latent | dr rotated key] rows, with a
// sliding window.  Scores, softmax weights and the weighted sum are fp32; the cache rows are the engine's element type.
//
// latent_post_kernel: one CTA per token.  RMS-norms the latent (vector weight), rotates the shared key part and the
// rotated part of every head's query (rotate-half pairing inside the first rot_dims coordinates), appends the cache row.
// latent_attn_kernel: one CTA per (tile of TQ consecutive query tokens, group of HG heads); every warp owns one (token,
// head) pair for the whole key loop, the CTA stages 32 keys at a time in shared memory and all its warps share them,
// so a prefill tile reads each key once per TQ x HG pairs and a decode step (TQ = 1) once per HG heads.  Lane j scores
// key j (fp32 dot over R + dr), the warp keeps a running maximum / sum (online softmax) and lane l accumulates the
// latent coordinates l, l + 32, ...
#include <cuda_bf16.h>

#include "asd_internal.h"
#include "blocks.h"
#include "elem.cuh"

namespace asd {

namespace {

__device__ __forceinline__ long long cache_row(const PagedRows& c, int slot, int pos) {
    const int page = c.page_table[(long long)slot * c.max_pages + pos / c.page_size];
    return (long long)page * c.page_size + pos % c.page_size;
}

__global__ void latent_post_kernel(SeqIndex ix, const float* qd, LatentDims d, const void* c_norm, int wf32, float eps,
                                   const float* inv_freq, PagedRows cache, float* q_lat) {
    __shared__ float red[33];
    const int m = blockIdx.x;
    const int pos = ix.positions[m], slot = ix.token_slot[m];
    const int qw = d.dn + d.dr, nq = d.heads * qw, ld = nq + d.R + d.dr, rw = d.R + d.dr;
    const float* row = qd + (long long)m * ld;
    const long long crow = cache_row(cache, slot, pos) * rw;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d.R; i += blockDim.x) {
        const float v = row[nq + i];
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float r = 1.f / sqrtf(ss / (float)d.R + eps);
    for (int i = threadIdx.x; i < d.R; i += blockDim.x)
        stx(cache.pool, crow + i, cache.f32, row[nq + i] * r * ldx(c_norm, i, wf32));
    // rotated parts: vector 0 is the shared key, vectors 1 .. heads the queries
    const int half = d.rot_dims / 2;
    for (int t = threadIdx.x; t < (d.heads + 1) * d.dr; t += blockDim.x) {
        const int vec = t / d.dr, i = t % d.dr;
        const float* src = vec == 0 ? row + nq + d.R : row + (long long)(vec - 1) * qw + d.dn;
        float out;
        if (i < d.rot_dims) {
            const int j = i < half ? i : i - half;
            float sn, cs;
            sincosf((float)pos * inv_freq[j], &sn, &cs);
            const float u = src[j], v = src[j + half];
            out = i < half ? u * cs - v * sn : v * cs + u * sn;
        } else {
            out = src[i];
        }
        if (vec == 0)
            stx(cache.pool, crow + d.R + i, cache.f32, out);
        else
            q_lat[((long long)m * d.heads + (vec - 1)) * rw + d.R + i] = out;
    }
}

template <typename T, int ACC>   // ACC = ceil(R / 32) accumulators per lane
__global__ void __launch_bounds__(512) latent_attn_kernel(SeqIndex ix, const int* cu_q, const int* seq_slot, int TQ,
                                                          int HG, const float* q_lat, LatentDims d, PagedRows cache,
                                                          float* out_lat) {
    extern __shared__ float smem[];
    const int rw = d.R + d.dr, LD = rw | 1;          // odd row stride: lanes reading one column hit 32 banks
    float* ks = smem;                                 // [32][LD]
    float* qs = smem + 32 * LD;                       // [warps][rw]
    const int seq = blockIdx.y, t0 = cu_q[seq] + blockIdx.x * TQ, t_end = cu_q[seq + 1];
    if (t0 >= t_end) return;
    const int slot = seq_slot[seq];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nthreads = blockDim.x;
    const int tq = warp / HG, head = blockIdx.z * HG + warp % HG;
    const int m = t0 + tq;
    const bool live = m < t_end && head < d.heads;
    const int p = live ? ix.positions[m] : -1;
    const int p_first = ix.positions[t0], n_tok = min(TQ, t_end - t0);
    const int p_last = ix.positions[t0 + n_tok - 1];
    int j_lo = p_first - d.window + 1;
    if (j_lo < 0) j_lo = 0;
    if (live) {
        const float* q = q_lat + ((long long)m * d.heads + head) * rw;
        for (int i = lane; i < rw; i += 32) qs[warp * rw + i] = q[i];
    }
    float mx = -INFINITY, sum = 0.f, acc[ACC];
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[i] = 0.f;
    const T* pool = (const T*)cache.pool;
    for (int j0 = j_lo; j0 <= p_last; j0 += 32) {
        __syncthreads();   // the previous tile has been consumed (and qs is written before the first use)
        for (int r = warp; r < 32; r += nthreads >> 5) {
            const int kp = j0 + r;
            if (kp <= p_last) {
                const T* src = pool + cache_row(cache, slot, kp) * rw;
                for (int i = lane; i < rw; i += 32) ks[r * LD + i] = ldf(src + i);
            }
        }
        __syncthreads();
        if (!live) continue;
        const int kp = j0 + lane;
        const bool seen = kp <= p && p - kp < d.window;
        float s = -INFINITY;
        if (seen) {
            const float* kr = ks + lane * LD;
            const float* qv = qs + warp * rw;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            int i = 0;
            for (; i + 4 <= rw; i += 4) {
                a0 = fmaf(qv[i], kr[i], a0);
                a1 = fmaf(qv[i + 1], kr[i + 1], a1);
                a2 = fmaf(qv[i + 2], kr[i + 2], a2);
                a3 = fmaf(qv[i + 3], kr[i + 3], a3);
            }
            for (; i < rw; ++i) a0 = fmaf(qv[i], kr[i], a0);
            s = ((a0 + a1) + (a2 + a3)) * d.scale;
        }
        const float tile_max = warp_max(s);
        if (tile_max == -INFINITY) continue;          // no key of this tile is in this token's window
        const float mx_new = fmaxf(mx, tile_max);
        const float corr = expf(mx - mx_new);          // exp(-inf) = 0 on the first live tile
        const float w = seen ? expf(s - mx_new) : 0.f;
        sum = sum * corr + warp_sum(w);
        mx = mx_new;
#pragma unroll
        for (int i = 0; i < ACC; ++i) acc[i] *= corr;
        for (int j = 0; j < 32; ++j) {
            const float wj = __shfl_sync(0xffffffffu, w, j);
            if (wj == 0.f) continue;                   // uniform across the warp
            const float* kr = ks + j * LD;
#pragma unroll
            for (int i = 0; i < ACC; ++i) {
                const int c = lane + 32 * i;
                if (c < d.R) acc[i] = fmaf(wj, kr[c], acc[i]);
            }
        }
    }
    if (!live) return;
    float* o = out_lat + ((long long)m * d.heads + head) * d.R;
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < ACC; ++i) {
        const int c = lane + 32 * i;
        if (c < d.R) o[c] = acc[i] * inv;
    }
}

template <typename T>
int launch_attn_t(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen, const float* q_lat,
                  const LatentDims& d, const PagedRows& cache, float* out_lat, cudaStream_t stream) {
    int HG = 1;
    while (HG * 2 <= d.heads && HG < 16) HG *= 2;
    int TQ = 1;
    if (max_qlen > 1) {
        if (HG > 4) HG = 4;
        TQ = 16 / HG;
        while (TQ > 1 && TQ / 2 >= max_qlen) TQ /= 2;
    }
    const int warps = TQ * HG, rw = d.R + d.dr;
    const size_t smem = (size_t)(32 * (rw | 1) + warps * rw) * sizeof(float);
    dim3 grid((max_qlen + TQ - 1) / TQ, nseq, (d.heads + HG - 1) / HG);
    const int acc = (d.R + 31) / 32;
#define ASD_LAT_CASE(A)                                                                                              \
    {                                                                                                                \
        auto fn = latent_attn_kernel<T, A>;                                                                          \
        if (smem > 48 * 1024) ASD_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        fn<<<grid, warps * 32, smem, stream>>>(ix, cu_q, seq_slot, TQ, HG, q_lat, d, cache, out_lat);                \
    }
    if (smem > 220 * 1024) return set_error("latent attention: latent + rotated size %d does not fit shared memory", rw);
    if (acc <= 2) ASD_LAT_CASE(2)
    else if (acc <= 4) ASD_LAT_CASE(4)
    else if (acc <= 8) ASD_LAT_CASE(8)
    else if (acc <= 16) ASD_LAT_CASE(16)
    else if (acc <= 32) ASD_LAT_CASE(32)
    else return set_error("latent attention: latent size %d > 1024", d.R);
#undef ASD_LAT_CASE
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace

int launch_latent_post(const SeqIndex& ix, const float* qd, const LatentDims& d, const void* c_norm, int wf32, float eps,
                       const float* inv_freq, const PagedRows& cache, float* q_lat, cudaStream_t stream) {
    if (ix.M <= 0) return 0;
    if (d.rot_dims < 0 || d.rot_dims > d.dr || (d.rot_dims & 1))
        return set_error("latent attention: rot_dims %d must be even and <= %d", d.rot_dims, d.dr);
    latent_post_kernel<<<ix.M, 128, 0, stream>>>(ix, qd, d, c_norm, wf32, eps, inv_freq, cache, q_lat);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_latent_attention(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen,
                            const float* q_lat, const LatentDims& d, const PagedRows& cache, float* out_lat,
                            cudaStream_t stream) {
    if (ix.M <= 0 || nseq <= 0) return 0;
    if (d.window <= 0) return set_error("latent attention: window must be positive");
    return cache.f32 ? launch_attn_t<float>(ix, cu_q, seq_slot, nseq, max_qlen, q_lat, d, cache, out_lat, stream)
                     : launch_attn_t<__nv_bfloat16>(ix, cu_q, seq_slot, nseq, max_qlen, q_lat, d, cache, out_lat, stream);
}

}  // namespace asd
