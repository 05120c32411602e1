// Grouped-query softmax attention over a sliding window plus kept first positions, with a learned sink in the
// denominator and position-rotated values, over a paged cache of [kv_heads * dk keys | kv_heads * dv values] rows.
// window_post_kernel: one CTA per token; rotates the queries in place and appends the rotated keys and values.
// window_attn_kernel: one CTA per (tile of TQ consecutive query tokens, key/value head); its warps are the TQ x group
//   (token, query head) pairs that share that key/value head, so a staged tile of 32 keys and values is read once
//   for all of them.  The keys a tile of queries can see are two ranges, the kept first positions and the window
//   behind the tile; each pair masks per key.  Lane j scores key j (fp32 dot over dk), the warp keeps a running maximum
//   and sum (online softmax) and lane l accumulates the value columns l, l + 32, ...  The sink enters the denominator
//   once, at the end; the result is turned back by the query's position and stored in the engine's element type.
#include <cuda_bf16.h>

#include "asd_internal.h"
#include "blocks.h"
#include "elem.cuh"

namespace asd {

namespace {

__device__ __forceinline__ long long wcache_row(const PagedRows& c, int slot, int pos) {
    const int page = c.page_table[(long long)slot * c.max_pages + pos / c.page_size];
    return (long long)page * c.page_size + pos % c.page_size;
}

// turns the first n coordinates of src by angle pos * freq[pair] (sign -1 turns back); returns coordinate i
__device__ __forceinline__ float turned(const float* src, int i, int n, int interleaved, float pos, const float* freq,
                                        float sign) {
    if (i >= n) return src[i];
    const int half = n >> 1;
    const int j = interleaved ? i >> 1 : (i < half ? i : i - half);
    const int a = interleaved ? 2 * j : j, b = interleaved ? 2 * j + 1 : j + half;
    float sn, cs;
    sincosf(pos * freq[j], &sn, &cs);
    sn *= sign;
    const float u = src[a], v = src[b];
    return i == a ? u * cs - v * sn : v * cs + u * sn;
}

__global__ void window_post_kernel(SeqIndex ix, float* qkv, long long ld, WindowDims d, const float* freq_k,
                                   const float* freq_v, PagedRows cache) {
    extern __shared__ float row[];   // the token's q | k | v as projected
    const int m = blockIdx.x;
    const int pos = ix.positions[m], slot = ix.token_slot[m];
    const int nq = d.heads * d.dk, nk = d.kv_heads * d.dk, nv = d.kv_heads * d.dv;
    float* src = qkv + (long long)m * ld;
    for (int i = threadIdx.x; i < nq + nk + nv; i += blockDim.x) row[i] = src[i];
    __syncthreads();
    const long long crow = wcache_row(cache, slot, pos) * (nk + nv);
    const float p = (float)pos;
    for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
        const int h = i / d.dk, c = i % d.dk;
        const float v = turned(row + (long long)h * d.dk, c, d.rot_dims, d.interleaved, p, freq_k, 1.f);
        if (i < nq)
            src[i] = v;
        else
            stx(cache.pool, crow + (i - nq), cache.f32, v);
    }
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const int h = i / d.dv, c = i % d.dv;
        stx(cache.pool, crow + nk + i, cache.f32,
            turned(row + nq + nk + (long long)h * d.dv, c, d.dv, d.interleaved, p, freq_v, 1.f));
    }
}

template <typename T, int ACC>   // ACC = ceil(dv / 32) accumulators per lane
__global__ void __launch_bounds__(512) window_attn_kernel(SeqIndex ix, const int* cu_q, const int* seq_slot, int TQ,
                                                           const float* q, long long ldq, WindowDims d, const float* sink,
                                                           const float* freq_v, PagedRows cache, void* out, int of32) {
    extern __shared__ float smem[];
    const int group = d.heads / d.kv_heads;
    const int LDK = d.dk | 1;                          // odd row stride: lanes reading one column hit 32 banks
    const int nwarps = blockDim.x >> 5;
    float* ks = smem;                                  // [32][LDK]
    float* vs = ks + 32 * LDK;                         // [32][dv]
    float* qs = vs + 32 * d.dv;                        // [warps][dk]
    float* os = qs + nwarps * d.dk;                    // [warps][dv]
    const int seq = blockIdx.y, g = blockIdx.z;
    const int t0 = cu_q[seq] + blockIdx.x * TQ, t_end = cu_q[seq + 1];
    if (t0 >= t_end) return;
    const int slot = seq_slot[seq];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tq = warp / group, head = g * group + warp % group;
    const int m = t0 + tq;
    const bool live = m < t_end;
    const int p = live ? ix.positions[m] : -1;
    const int n_tok = min(TQ, t_end - t0);
    const int p_first = ix.positions[t0], p_last = p_first + n_tok - 1;
    // visible keys of the tile: [0, first_end) and [lo, p_last]
    int lo = p_first - d.window + 1;
    if (lo < 0) lo = 0;
    int first_end = d.keep_first < lo ? d.keep_first : lo;
    if (live) {
        const float* qr = q + (long long)m * ldq + (long long)head * d.dk;
        for (int i = lane; i < d.dk; i += 32) qs[warp * d.dk + i] = qr[i];
    }
    float mx = -INFINITY, sum = 0.f, acc[ACC];
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[i] = 0.f;
    const T* pool = (const T*)cache.pool;
    const int nk = d.kv_heads * d.dk, rowlen = nk + d.kv_heads * d.dv;
    const long long koff = (long long)g * d.dk, voff = nk + (long long)g * d.dv;
    for (int range = 0; range < 2; ++range) {
        const int j_begin = range == 0 ? 0 : lo, j_end = range == 0 ? first_end : p_last + 1;
        for (int j0 = j_begin; j0 < j_end; j0 += 32) {
            __syncthreads();   // the previous tile has been consumed (and qs is written before the first use)
            for (int r = warp; r < 32; r += nwarps) {
                const int kp = j0 + r;
                if (kp < j_end) {
                    const T* src = pool + wcache_row(cache, slot, kp) * rowlen;
                    for (int i = lane; i < d.dk; i += 32) ks[r * LDK + i] = ldf(src + koff + i);
                    for (int i = lane; i < d.dv; i += 32) vs[r * d.dv + i] = ldf(src + voff + i);
                }
            }
            __syncthreads();
            if (!live) continue;
            const int kp = j0 + lane;
            const bool seen = kp < j_end && kp <= p && (p - kp < d.window || kp < d.keep_first);
            float s = -INFINITY;
            if (seen) {
                const float* kr = ks + lane * LDK;
                const float* qv = qs + warp * d.dk;
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
                int i = 0;
                for (; i + 4 <= d.dk; i += 4) {
                    a0 = fmaf(qv[i], kr[i], a0);
                    a1 = fmaf(qv[i + 1], kr[i + 1], a1);
                    a2 = fmaf(qv[i + 2], kr[i + 2], a2);
                    a3 = fmaf(qv[i + 3], kr[i + 3], a3);
                }
                for (; i < d.dk; ++i) a0 = fmaf(qv[i], kr[i], a0);
                s = ((a0 + a1) + (a2 + a3)) * d.scale;
            }
            const float tile_max = warp_max(s);
            if (tile_max == -INFINITY) continue;          // no key of this tile is visible to this token
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
                const float* vr = vs + j * d.dv;
#pragma unroll
                for (int i = 0; i < ACC; ++i) {
                    const int c = lane + 32 * i;
                    if (c < d.dv) acc[i] = fmaf(wj, vr[c], acc[i]);
                }
            }
        }
    }
    if (!live) return;
    // the sink: one more term of the denominator, without a value
    float scale_o = 1.f;
    if (sink) {
        const float sk = sink[head];
        const float mf = fmaxf(mx, sk);
        scale_o = expf(mx - mf);
        sum = sum * scale_o + expf(sk - mf);
    }
    const float inv = scale_o / sum;
    float* ow = os + warp * d.dv;
#pragma unroll
    for (int i = 0; i < ACC; ++i) {
        const int c = lane + 32 * i;
        if (c < d.dv) ow[c] = acc[i] * inv;
    }
    __syncwarp();
    const long long obase = ((long long)m * d.heads + head) * d.dv;
    for (int c = lane; c < d.dv; c += 32)
        stx(out, obase + c, of32, turned(ow, c, d.dv, d.interleaved, (float)p, freq_v, -1.f));
}

template <typename T>
int launch_simple(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen, const float* q,
                  long long ldq, const WindowDims& d, const float* sink, const float* freq_v, const PagedRows& cache,
                  void* out, int of32, cudaStream_t stream) {
    const int group = d.heads / d.kv_heads;
    if (group > 16) return set_error("windowed attention: %d query heads per key/value head (at most 16)", group);
    int TQ = 16 / group;
    if (TQ < 1) TQ = 1;
    while (TQ > 1 && TQ / 2 >= max_qlen) TQ /= 2;
    const int warps = TQ * group;
    const size_t smem = (size_t)(32 * (d.dk | 1) + 32 * d.dv + warps * (d.dk + d.dv)) * sizeof(float);
    if (smem > 220 * 1024) return set_error("windowed attention: head sizes %d / %d do not fit shared memory", d.dk, d.dv);
    dim3 grid((max_qlen + TQ - 1) / TQ, nseq, d.kv_heads);
    if (grid.y > 65535 || grid.z > 65535) return set_error("windowed attention: too many sequences or heads");
    const int acc = (d.dv + 31) / 32;
#define ASD_WIN_CASE(A)                                                                                              \
    {                                                                                                                \
        auto fn = window_attn_kernel<T, A>;                                                                          \
        if (smem > 48 * 1024) ASD_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        fn<<<grid, warps * 32, smem, stream>>>(ix, cu_q, seq_slot, TQ, q, ldq, d, sink, freq_v, cache, out, of32);   \
    }
    if (acc <= 1) ASD_WIN_CASE(1)
    else if (acc <= 2) ASD_WIN_CASE(2)
    else if (acc <= 4) ASD_WIN_CASE(4)
    else if (acc <= 8) ASD_WIN_CASE(8)
    else if (acc <= 16) ASD_WIN_CASE(16)
    else return set_error("windowed attention: value size %d > 512", d.dv);
#undef ASD_WIN_CASE
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int check_dims(const WindowDims& d) {
    if (d.heads <= 0 || d.kv_heads <= 0 || d.heads % d.kv_heads || d.dk <= 0 || d.dv <= 0 || (d.dv & 1) ||
        d.rot_dims < 0 || d.rot_dims > d.dk || (d.rot_dims & 1) || d.window <= 0 || d.keep_first < 0)
        return set_error("windowed attention: bad sizes (heads %d / %d, dk %d, dv %d, rot %d, window %d, kept %d)",
                         d.heads, d.kv_heads, d.dk, d.dv, d.rot_dims, d.window, d.keep_first);
    return 0;
}

}  // namespace

int launch_window_post(const SeqIndex& ix, float* qkv, long long ld, const WindowDims& d, const float* freq_k,
                       const float* freq_v, const PagedRows& cache, cudaStream_t stream) {
    if (ix.M <= 0) return 0;
    if (check_dims(d)) return -1;
    const size_t smem = (size_t)(d.heads * d.dk + d.kv_heads * (d.dk + d.dv)) * sizeof(float);
    if (smem > 200 * 1024) return set_error("windowed attention: a token's q | k | v row does not fit shared memory");
    if (smem > 48 * 1024)
        ASD_CUDA(cudaFuncSetAttribute(window_post_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    window_post_kernel<<<ix.M, 256, smem, stream>>>(ix, qkv, ld, d, freq_k, freq_v, cache);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_window_attention(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen,
                            int max_kv_len, const float* q, long long ldq, const WindowDims& d, const float* sink,
                            const float* freq_v, const PagedRows& cache, void* out, int of32, int tiled,
                            cudaStream_t stream) {
    if (ix.M <= 0 || nseq <= 0) return 0;
    if (check_dims(d)) return -1;
    (void)max_kv_len;
    (void)tiled;
    return cache.f32 ? launch_simple<float>(ix, cu_q, seq_slot, nseq, max_qlen, q, ldq, d, sink, freq_v, cache, out, of32, stream)
                     : launch_simple<__nv_bfloat16>(ix, cu_q, seq_slot, nseq, max_qlen, q, ldq, d, sink, freq_v, cache, out, of32, stream);
}

}  // namespace asd
