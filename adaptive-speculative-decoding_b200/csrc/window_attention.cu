// Grouped-query softmax attention over a sliding window plus kept first positions, with a learned sink in the
// denominator and position-rotated values, over a paged cache of [kv_heads * dk keys | kv_heads * dv values] rows.
// window_post_kernel: one CTA per token; rotates the queries in place and appends the rotated keys and values.
// window_attn_kernel: one CTA per (tile of TQ consecutive query tokens, key/value head); its warps are the TQ x group
//   (token, query head) pairs that share that key/value head, so a staged tile of 32 keys and values is read once
//   for all of them.  The keys a tile of queries can see are two ranges, the kept first positions and the window
//   behind the tile; each pair masks per key.  Lane j scores key j (fp32 dot over dk), the warp keeps a running maximum
//   and sum (online softmax) and lane l accumulates the value columns l, l + 32, ...  The sink enters the denominator
//   once, at the end; the result is turned back by the query's position and stored in the engine's element type.
// window_attn_mma: the same on the tensor cores for bf16 cache rows (mma.sync m16n8k16, fp32 accumulation).  One CTA of
//   four warps per (64 query rows = tokens x query heads of one key/value head); tiles of 64 keys and values arrive by
//   cp.async, two in flight.  The fp32 queries and the fp32 softmax weights enter the products as the sum of two bf16
//   terms each, so scores and weights keep fp32 accuracy; maxima, sums and the sink are fp32.
#include <cuda_bf16.h>

#include "asd_internal.h"
#include "blocks.h"
#include "elem.cuh"
#include "mma_sync.cuh"

namespace asd {

namespace {

__device__ __forceinline__ int warp_of(unsigned tid) { return (int)(tid >> 5); }

__device__ __forceinline__ long long wcache_row(const PagedRows& c, int slot, int pos) {
    int pi, in_page;
    if ((c.page_size & (c.page_size - 1)) == 0) {      // a power of two: shift and mask instead of a division
        pi = pos >> (__ffs(c.page_size) - 1);
        in_page = pos & (c.page_size - 1);
    } else {
        pi = pos / c.page_size;
        in_page = pos - pi * c.page_size;
    }
    return (long long)c.page_table[(long long)slot * c.max_pages + pi] * c.page_size + in_page;
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
                                                           int hpc, const float* q, long long ldq, WindowDims d,
                                                           const float* sink, const float* freq_v, PagedRows cache, void* out,
                                                           int of32) {
    extern __shared__ float smem[];
    const int group = d.heads / d.kv_heads;
    const int LDK = d.dk | 1;                          // odd row stride: lanes reading one column hit 32 banks
    const int nwarps = blockDim.x >> 5;
    float* ks = smem;                                  // [32][LDK]
    float* vs = ks + 32 * LDK;                         // [32][dv]
    float* qs = vs + 32 * d.dv;                        // [warps][dk]
    float* os = qs + nwarps * d.dk;                    // [warps][dv]
    // a CTA takes hpc query heads of one key/value head (all of them unless there are more than 16)
    const int nsub = (group + hpc - 1) / hpc;
    const int seq = blockIdx.y, g = blockIdx.z / nsub, h_in_group = (blockIdx.z % nsub) * hpc + warp_of(threadIdx.x) % hpc;
    const int t0 = cu_q[seq] + blockIdx.x * TQ, t_end = cu_q[seq + 1];
    if (t0 >= t_end) return;
    const int slot = seq_slot[seq];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tq = warp / hpc, head = g * group + h_in_group;
    const int m = t0 + tq;
    const bool live = m < t_end && h_in_group < group;
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
    const int hpc = group < 16 ? group : 16;     // query heads per CTA
    const int nsub = (group + hpc - 1) / hpc;
    int TQ = 16 / hpc;
    while (TQ > 1 && TQ / 2 >= max_qlen) TQ /= 2;
    const int warps = TQ * hpc;
    const size_t smem = (size_t)(32 * (d.dk | 1) + 32 * d.dv + warps * (d.dk + d.dv)) * sizeof(float);
    if (smem > 220 * 1024) return set_error("windowed attention: head sizes %d / %d do not fit shared memory", d.dk, d.dv);
    dim3 grid((max_qlen + TQ - 1) / TQ, nseq, d.kv_heads * nsub);
    if (grid.y > 65535 || grid.z > 65535) return set_error("windowed attention: too many sequences or heads");
    const int acc = (d.dv + 31) / 32;
#define ASD_WIN_CASE(A)                                                                                              \
    {                                                                                                                \
        auto fn = window_attn_kernel<T, A>;                                                                          \
        static PerDeviceOnce once;                                                                                   \
        if (once.need()) ASD_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)); \
        fn<<<grid, warps * 32, smem, stream>>>(ix, cu_q, seq_slot, TQ, hpc, q, ldq, d, sink, freq_v, cache, out, of32); \
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

// ---------------------------------------------------------------------------------------------------------------
// Tensor-core form.  Row r of the CTA's 64 is (token r / group, query head r % group of key/value head g).
constexpr int WM_ROWS = 64, WM_KEYS = 64;
constexpr int kMaxSmem = 220 * 1024;   // dynamic shared memory a CTA may ask for (the opt-in limit less the static part)

__device__ __forceinline__ void split2(float x, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16(x);
    lo = __float2bfloat16(x - __bfloat162float(hi));
}

// STAGES key/value tiles are in flight.  When the CTA has at most 16 rows (single-token steps), all four warps take
// those rows and a quarter of every tile's keys each, and their partial results are merged at the end.
// SINGLE: every CTA of the launch is of that kind (single-token steps); the query fragments then stay in registers.
// SQ: key and value size are both exactly 8 * NV (64 or 128 in practice): every loop bound and row stride is then a
// compile-time constant.
template <int NV, int STAGES, bool SINGLE, bool SQ>   // value column tiles of 8: dv <= 8 * NV
__global__ void __launch_bounds__(128) window_attn_mma(SeqIndex ix, const int* cu_q, const int* seq_slot, int TQ,
                                                       const float* q, long long ldq, WindowDims d, const float* sink,
                                                       const float* freq_v, PagedRows cache, void* out, int of32,
                                                       int nsplit, float* ws_o, float* ws_ml, int q_alloc) {
    extern __shared__ __align__(16) unsigned char smraw[];
    const int dk = SQ ? 8 * NV : d.dk, dv = SQ ? 8 * NV : d.dv;
    const int LDQ = dk + 8, LDV = dv + 8;   // bf16 elements; 16 bytes of padding keep ldmatrix rows on distinct banks
    // queries: [q_alloc][LDQ] twice (64 rows, or 16 for single-token steps); q_alloc == 0: the 16 rows of a single-token
    // step only pass through shared memory on their way into registers and borrow the last key buffer, which the first
    // iteration of the tile loop fills
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smraw) + 2 * q_alloc * LDQ;   // [STAGES][64][LDQ]
    __nv_bfloat16* Vs = Ks + STAGES * WM_KEYS * LDQ;               // [STAGES][64][LDV]
    __nv_bfloat16* Qh = q_alloc ? reinterpret_cast<__nv_bfloat16*>(smraw) : Ks + (STAGES - 1) * WM_KEYS * LDQ;
    __nv_bfloat16* Ql = Qh + (q_alloc ? q_alloc : 16) * LDQ;
    float* stage = reinterpret_cast<float*>(Ks);                   // [64][dv] once the last tile is consumed
    float* stage_ml = stage + WM_ROWS * dv;                      // [64][2]: maximum and sum of every warp's share
    const int group = d.heads / d.kv_heads;
    const int seq = blockIdx.y, g = blockIdx.z;
    const int split = blockIdx.x % nsplit;       // this CTA's share of the key tiles (single-token steps only)
    const int t0 = cu_q[seq] + (blockIdx.x / nsplit) * TQ, t_end = cu_q[seq + 1];
    if (t0 >= t_end) return;
    const int slot = seq_slot[seq];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_tok = min(TQ, t_end - t0), n_rows = n_tok * group;
    const int p_first = ix.positions[t0], p_last = p_first + n_tok - 1;
    int lo = p_first - d.window + 1;
    if (lo < 0) lo = 0;
    const int first_end = d.keep_first < lo ? d.keep_first : lo;
    const int nA = (first_end + WM_KEYS - 1) / WM_KEYS, nB = (p_last + 1 - lo + WM_KEYS - 1) / WM_KEYS;
    const int all_tiles = nA + nB, per_split = (all_tiles + nsplit - 1) / nsplit;
    const int tile0 = split * per_split;
    const int ntiles = max(0, min(all_tiles, tile0 + per_split) - tile0);      // tiles tile0 .. tile0 + ntiles - 1 are this CTA's
    // queries as hi + lo bf16 terms
    const int q_rows = n_rows <= 16 ? 16 : WM_ROWS;      // rows the products read (the rest of a single-token tile is unused)
    for (int r = warp; r < q_rows; r += 4) {
        const float* src = r < n_rows ? q + (long long)(t0 + r / group) * ldq + (long long)(g * group + r % group) * dk : nullptr;
        for (int c = lane; c < dk; c += 32) {
            __nv_bfloat16 hi, lw;
            split2(src ? src[c] : 0.f, hi, lw);
            Qh[r * LDQ + c] = hi;
            Ql[r * LDQ + c] = lw;
        }
    }
    const __nv_bfloat16* pool = reinterpret_cast<const __nv_bfloat16*>(cache.pool);
    const int nk = d.kv_heads * dk, rowlen = nk + d.kv_heads * dv;
    const int ck = dk >> 3, cpr = (dk + dv) >> 3;
    auto tile_range = [&](int i, int& j0, int& j_end) {
        i += tile0;
        if (i < nA) {
            j0 = i * WM_KEYS;
            j_end = first_end;
        } else {
            j0 = lo + (i - nA) * WM_KEYS;
            j_end = p_last + 1;
        }
    };
    // two threads per key row: one page lookup each (made a tile ahead of the copies that need it), then every other
    // 16-byte chunk of the row's keys and values.  (Consecutive lanes on consecutive chunks of a row, with the row
    // offsets handed over through shared memory, measured slower: 99 against 78 us at 64 sequences.)
    auto lookup = [&](int i) -> long long {
        if (i >= ntiles) return 0;
        int j0, j_end;
        tile_range(i, j0, j_end);
        const int kp = j0 + (tid >> 1);
        return wcache_row(cache, slot, kp < j_end ? kp : j_end - 1) * rowlen;
    };
    auto load_tile = [&](int buf, int i, long long row_off) {
        int j0, j_end;
        tile_range(i, j0, j_end);
        __nv_bfloat16* kd = Ks + buf * WM_KEYS * LDQ;
        __nv_bfloat16* vd = Vs + buf * WM_KEYS * LDV;
        const int r = tid >> 1;
        const bool ok = j0 + r < j_end;
        const __nv_bfloat16* src = pool + row_off;
        const __nv_bfloat16* ksrc = src + (long long)g * dk;
        const __nv_bfloat16* vsrc = src + nk + (long long)g * dv;
        for (int cc = tid & 1; cc < ck; cc += 2)
            cp_async16((uint32_t)__cvta_generic_to_shared(kd + r * LDQ + cc * 8), ksrc + cc * 8, ok);
        for (int cc = tid & 1; cc < cpr - ck; cc += 2)
            cp_async16((uint32_t)__cvta_generic_to_shared(vd + r * LDV + cc * 8), vsrc + cc * 8, ok);
    };
    constexpr int NP = SINGLE ? 1 : 4;                    // pairs of 8-key score tiles per warp and tile at most
    const bool ksplit = SINGLE || n_rows <= 16;           // every warp: rows 0 .. 15, keys [16 warp, 16 warp + 16) of a tile
    const int row0 = ksplit ? 0 : warp * 16, key0 = ksplit ? warp * 16 : 0, npw = ksplit ? 1 : 4;
    const int rA = row0 + (lane >> 2), rB = rA + 8;
    const bool okA = rA < n_rows, okB = rB < n_rows;
    const int pA = p_first + rA / group, pB = p_first + rB / group;
    const bool warp_live = row0 < n_rows;
    float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;
    float o[NV][4];
#pragma unroll
    for (int i = 0; i < NV; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const int nvt = SQ ? NV : dv >> 3;
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) {
        if (i < ntiles) load_tile(i, i, lookup(i));
        cp_async_commit();
    }
    long long next_off = lookup(STAGES - 1);
    // single-token steps: the 16 query rows are the same for every tile and warp, their fragments are loaded once
    uint32_t qh[SINGLE ? 8 : 1][4], ql[SINGLE ? 8 : 1][4];
    const bool q_regs = SINGLE && dk <= 128;
    if (q_regs) {
        __syncthreads();   // the queries are in place
#pragma unroll
        for (int k8 = 0; k8 < (SINGLE ? 8 : 1); ++k8) {
            if (k8 * 16 < dk) {
                const int qoff = (lane & 15) * LDQ + k8 * 16 + (lane >> 4) * 8;
                ldsm_x4((uint32_t)__cvta_generic_to_shared(Qh + qoff), qh[k8]);
                ldsm_x4((uint32_t)__cvta_generic_to_shared(Ql + qoff), ql[k8]);
            }
        }
        if (!q_alloc) __syncthreads();   // every warp has its fragments before the borrowed buffer is filled with keys
    }
    for (int it = 0; it < ntiles; ++it) {
        if (it + STAGES - 1 < ntiles) load_tile((it + STAGES - 1) % STAGES, it + STAGES - 1, next_off);
        cp_async_commit();                 // (an empty group keeps the count of groups in flight uniform)
        next_off = lookup(it + STAGES);    // its latency passes behind this tile's arithmetic
        cp_async_wait<STAGES - 1>();
        __syncthreads();   // tile `it` has landed for every thread (and the queries are in place)
        if (warp_live) {
            int j0, j_end;
            tile_range(it, j0, j_end);
            const __nv_bfloat16* kb = Ks + ((it % STAGES) * WM_KEYS + key0) * LDQ;
            const __nv_bfloat16* vb = Vs + ((it % STAGES) * WM_KEYS + key0) * LDV;
            float s[2 * NP][4];
#pragma unroll
            for (int i = 0; i < 2 * NP; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
            if (q_regs) {
#pragma unroll
                for (int k8 = 0; k8 < (SINGLE ? 8 : 1); ++k8) {
                    if (k8 * 16 < dk) {
                        uint32_t b[4];
                        ldsm_x4((uint32_t)__cvta_generic_to_shared(kb + ((lane & 7) + ((lane >> 4) & 1) * 8) * LDQ + k8 * 16 +
                                                                    ((lane >> 3) & 1) * 8), b);
                        mma_bf16(s[0], qh[k8], b[0], b[1]);
                        mma_bf16(s[0], ql[k8], b[0], b[1]);
                        mma_bf16(s[1], qh[k8], b[2], b[3]);
                        mma_bf16(s[1], ql[k8], b[2], b[3]);
                    }
                }
            } else {
                for (int ks = 0; ks < dk; ks += 16) {
                    uint32_t ah[4], al[4];
                    const int qoff = (row0 + (lane & 15)) * LDQ + ks + (lane >> 4) * 8;
                    ldsm_x4((uint32_t)__cvta_generic_to_shared(Qh + qoff), ah);
                    ldsm_x4((uint32_t)__cvta_generic_to_shared(Ql + qoff), al);
#pragma unroll
                    for (int np = 0; np < NP; ++np) {
                        if (np >= npw) break;
                        uint32_t b[4];
                        ldsm_x4((uint32_t)__cvta_generic_to_shared(kb + (np * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * LDQ + ks +
                                                                    ((lane >> 3) & 1) * 8), b);
                        mma_bf16(s[2 * np], ah, b[0], b[1]);
                        mma_bf16(s[2 * np], al, b[0], b[1]);
                        mma_bf16(s[2 * np + 1], ah, b[2], b[3]);
                        mma_bf16(s[2 * np + 1], al, b[2], b[3]);
                    }
                }
            }
            // mask, running maxima.  Steps of one or a few tokens: most of a warp's 16-key shares lie wholly inside every
            // row's window (or the kept range) and before every row's position: those take the scale alone
            float txA = -INFINITY, txB = -INFINITY;
            const int k_lo = j0 + key0, k_hi = k_lo + 15;
            const bool whole = SINGLE && k_hi < j_end && k_hi <= p_first && (p_last - k_lo < d.window || k_hi < d.keep_first);
            if (whole) {
#pragma unroll
                for (int nt = 0; nt < 2 * NP; ++nt) {
                    s[nt][0] = okA ? s[nt][0] * d.scale : -INFINITY;
                    s[nt][1] = okA ? s[nt][1] * d.scale : -INFINITY;
                    s[nt][2] = okB ? s[nt][2] * d.scale : -INFINITY;
                    s[nt][3] = okB ? s[nt][3] * d.scale : -INFINITY;
                    txA = fmaxf(txA, fmaxf(s[nt][0], s[nt][1]));
                    txB = fmaxf(txB, fmaxf(s[nt][2], s[nt][3]));
                }
            } else {
#pragma unroll
                for (int nt = 0; nt < 2 * NP; ++nt) {
                    if (nt >= 2 * npw) break;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int kp = j0 + key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                        const int p = e < 2 ? pA : pB;
                        const bool seen = (e < 2 ? okA : okB) && kp < j_end && kp <= p && (p - kp < d.window || kp < d.keep_first);
                        const float v = seen ? s[nt][e] * d.scale : -INFINITY;
                        s[nt][e] = v;
                        if (e < 2)
                            txA = fmaxf(txA, v);
                        else
                            txB = fmaxf(txB, v);
                    }
                }
            }
            txA = fmaxf(txA, __shfl_xor_sync(0xffffffffu, txA, 1));
            txA = fmaxf(txA, __shfl_xor_sync(0xffffffffu, txA, 2));
            txB = fmaxf(txB, __shfl_xor_sync(0xffffffffu, txB, 1));
            txB = fmaxf(txB, __shfl_xor_sync(0xffffffffu, txB, 2));
            const float nA_ = fmaxf(mA, txA), nB_ = fmaxf(mB, txB);
            const float sA = nA_ == -INFINITY ? 0.f : nA_, sB = nB_ == -INFINITY ? 0.f : nB_;   // nothing seen yet: weights 0
            // (rows beyond the CTA's own keep factor 1, so that they never ask for a rescale)
            const float cA = okA ? __expf(mA - sA) : 1.f, cB = okB ? __expf(mB - sB) : 1.f;
            mA = nA_, mB = nB_;
            float sumA = 0.f, sumB = 0.f;
#pragma unroll
            for (int nt = 0; nt < 2 * NP; ++nt) {
                if (nt >= 2 * npw) break;
                s[nt][0] = __expf(s[nt][0] - sA);
                s[nt][1] = __expf(s[nt][1] - sA);
                s[nt][2] = __expf(s[nt][2] - sB);
                s[nt][3] = __expf(s[nt][3] - sB);
                sumA += s[nt][0] + s[nt][1];
                sumB += s[nt][2] + s[nt][3];
            }
            lA = lA * cA + sumA;
            lB = lB * cB + sumB;
            if (__any_sync(0xffffffffu, cA != 1.f || cB != 1.f)) {      // no row of the warp met a new maximum: nothing to rescale
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    o[i][0] *= cA, o[i][1] *= cA;
                    o[i][2] *= cB, o[i][3] *= cB;
                }
            }
            // weights x values: 16 keys at a time, the weights as hi + lo bf16 terms
#pragma unroll
            for (int j = 0; j < NP; ++j) {
                if (j >= npw) break;
                uint32_t ph[4], pl[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float x0 = s[2 * j + (u >> 1)][(u & 1) * 2], x1 = s[2 * j + (u >> 1)][(u & 1) * 2 + 1];
                    __nv_bfloat16 h0, l0, h1, l1;
                    split2(x0, h0, l0);
                    split2(x1, h1, l1);
                    __nv_bfloat162 hh = __halves2bfloat162(h0, h1), ll = __halves2bfloat162(l0, l1);
                    ph[u] = *reinterpret_cast<uint32_t*>(&hh);
                    pl[u] = *reinterpret_cast<uint32_t*>(&ll);
                }
#pragma unroll
                for (int vp = 0; vp < NV / 2; ++vp) {
                    if (2 * vp < nvt) {
                        uint32_t b[4];
                        ldsm_x4_t((uint32_t)__cvta_generic_to_shared(vb + (j * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV +
                                                                      (2 * vp + (lane >> 4)) * 8), b);
                        mma_bf16(o[2 * vp], ph, b[0], b[1]);
                        mma_bf16(o[2 * vp], pl, b[0], b[1]);
                        mma_bf16(o[2 * vp + 1], ph, b[2], b[3]);
                        mma_bf16(o[2 * vp + 1], pl, b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();   // tile `it` is consumed: its buffer may be refilled (and, after the last tile, reused as staging)
    }
    lA += __shfl_xor_sync(0xffffffffu, lA, 1);
    lA += __shfl_xor_sync(0xffffffffu, lA, 2);
    lB += __shfl_xor_sync(0xffffffffu, lB, 1);
    lB += __shfl_xor_sync(0xffffffffu, lB, 2);
    if (ksplit) {
        // every warp leaves its unnormalised share of rows 0 .. 15; the shares are merged per element, then the sink
        if ((lane & 3) == 0) {
            stage_ml[(warp * 16 + (lane >> 2)) * 2] = mA, stage_ml[(warp * 16 + (lane >> 2)) * 2 + 1] = lA;
            stage_ml[(warp * 16 + (lane >> 2) + 8) * 2] = mB, stage_ml[(warp * 16 + (lane >> 2) + 8) * 2 + 1] = lB;
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (i < nvt) {
                const int c = i * 8 + (lane & 3) * 2;
                float* sa = stage + (warp * 16 + (lane >> 2)) * dv + c;
                float* sb = sa + 8 * dv;
                sa[0] = o[i][0], sa[1] = o[i][1];
                sb[0] = o[i][2], sb[1] = o[i][3];
            }
        }
        __syncthreads();
        if (nsplit > 1) {
            // this CTA saw a share of the keys: its merged maximum, sum and unnormalised result wait for the combine kernel
            for (int i = tid; i < n_rows * dv; i += 128) {
                const int r = i / dv, c = i % dv;
                float mx = -INFINITY;
#pragma unroll
                for (int w = 0; w < 4; ++w) mx = fmaxf(mx, stage_ml[(w * 16 + r) * 2]);
                float num = 0.f, den = 0.f;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const float f = mx == -INFINITY ? 0.f : expf(stage_ml[(w * 16 + r) * 2] - mx);
                    den += stage_ml[(w * 16 + r) * 2 + 1] * f;
                    num += stage[(w * 16 + r) * dv + c] * f;
                }
                const long long pair = ((long long)(t0 + r / group) * d.heads + g * group + r % group) * nsplit + split;
                ws_o[pair * dv + c] = num;
                if (c == 0) ws_ml[pair * 2] = mx, ws_ml[pair * 2 + 1] = den;
            }
            return;
        }
        for (int i = tid; i < n_rows * dv; i += 128) {
            const int r = i / dv, c = i % dv;
            float mx = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) mx = fmaxf(mx, stage_ml[(w * 16 + r) * 2]);
            if (sink) mx = fmaxf(mx, sink[g * group + r % group]);
            float num = 0.f, den = sink ? expf(sink[g * group + r % group] - mx) : 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = expf(stage_ml[(w * 16 + r) * 2] - mx);       // a share that saw no key: exp(-inf) = 0
                den += stage_ml[(w * 16 + r) * 2 + 1] * f;
                num += stage[(w * 16 + r) * dv + c] * f;
            }
            stage[r * dv + c] = num / den;       // only this thread reads column c of row r's shares
        }
    } else {
        float invA = 1.f / lA, invB = 1.f / lB;
        if (sink) {   // one more term of the denominator, without a value
            if (okA) {
                const float sk = sink[g * group + rA % group], mf = fmaxf(mA, sk), so = expf(mA - mf);
                invA = so / (lA * so + expf(sk - mf));
            }
            if (okB) {
                const float sk = sink[g * group + rB % group], mf = fmaxf(mB, sk), so = expf(mB - mf);
                invB = so / (lB * so + expf(sk - mf));
            }
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (i < nvt) {
                const int c = i * 8 + (lane & 3) * 2;
                if (okA) stage[rA * dv + c] = o[i][0] * invA, stage[rA * dv + c + 1] = o[i][1] * invA;
                if (okB) stage[rB * dv + c] = o[i][2] * invB, stage[rB * dv + c + 1] = o[i][3] * invB;
            }
        }
    }
    __syncthreads();
    for (int i = tid; i < n_rows * dv; i += 128) {
        const int r = i / dv, c = i % dv;
        const long long m = t0 + r / group;
        stx(out, (m * d.heads + g * group + r % group) * dv + c, of32,
            turned(stage + r * dv, c, dv, d.interleaved, (float)(p_first + r / group), freq_v, -1.f));
    }
}

// merges the shares of a (token, head) pair's keys: one CTA per pair, one thread per value column; then the sink, the
// normalisation and the turn back by the token's position
__global__ void window_combine_kernel(SeqIndex ix, WindowDims d, const float* sink, const float* freq_v, int nsplit,
                                      const float* ws_o, const float* ws_ml, void* out, int of32) {
    extern __shared__ float row[];   // [dv]
    const long long pair = blockIdx.x;
    const int m = (int)(pair / d.heads), head = (int)(pair % d.heads);
    float mx = sink ? sink[head] : -INFINITY;
    for (int sp = 0; sp < nsplit; ++sp) mx = fmaxf(mx, ws_ml[(pair * nsplit + sp) * 2]);
    float den = sink ? expf(sink[head] - mx) : 0.f;
    for (int sp = 0; sp < nsplit; ++sp) den += ws_ml[(pair * nsplit + sp) * 2 + 1] * expf(ws_ml[(pair * nsplit + sp) * 2] - mx);
    for (int c = threadIdx.x; c < d.dv; c += blockDim.x) {
        float num = 0.f;
        for (int sp = 0; sp < nsplit; ++sp)
            num += ws_o[(pair * nsplit + sp) * d.dv + c] * expf(ws_ml[(pair * nsplit + sp) * 2] - mx);
        row[c] = num / den;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < d.dv; c += blockDim.x)
        stx(out, pair * d.dv + c, of32, turned(row, c, d.dv, d.interleaved, (float)ix.positions[m], freq_v, -1.f));
}

bool mma_supports(const WindowDims& d, const PagedRows& cache) {
    const int group = d.heads / d.kv_heads;
    return !cache.f32 && (d.dk % 16) == 0 && (d.dv % 16) == 0 && d.dv <= 128 && d.dk <= 256 && group <= WM_ROWS &&
           (reinterpret_cast<uintptr_t>(cache.pool) & 15) == 0;
}

int launch_mma(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen, int max_kv_len,
               const float* q, long long ldq, const WindowDims& d, const float* sink, const float* freq_v,
               const PagedRows& cache, void* out, int of32, const AttnSplit& ws, cudaStream_t stream) {
    const int group = d.heads / d.kv_heads;
    const int TQ = WM_ROWS / group;
    dim3 grid((max_qlen + TQ - 1) / TQ, nseq, d.kv_heads);
    // Single-token steps with few sequences leave most SMs without a CTA and every CTA with one long chain of tiles: the
    // key tiles are then cut into shares for several CTAs, whose partial results the combine kernel merges.
    static const int sms = []() {
        int n = 148, dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        return n;
    }();
    int nsplit = 1;
    if (max_qlen * group <= 16 && ws.o && ws.ml) {
        const long long ctas = (long long)nseq * d.kv_heads;
        const long long keys = (long long)(d.window < max_kv_len ? d.window : max_kv_len) + d.keep_first;
        const int tiles = (int)((keys + WM_KEYS - 1) / WM_KEYS) + 1;
        // as many shares as still fit one wave of two CTAs per SM: a second, partly filled wave would cost more than it saves
        while (nsplit < 8 && ctas * nsplit * 2 <= 2LL * sms && tiles >= 4 * nsplit) nsplit *= 2;
        while (nsplit > 1 && ((long long)ix.M * d.heads * nsplit > ws.rows || (long long)ix.M * d.heads * nsplit * d.dv > ws.o_elems))
            nsplit /= 2;
    }
    grid.x *= nsplit;
    // single-token steps are bound by the latency of the key/value stream: four tiles in flight when the grid leaves an
    // SM to one CTA anyway, two (and two CTAs per SM) otherwise
    const bool single = max_qlen * group <= 16;          // every CTA has at most 16 rows: a small query buffer, more tiles in flight
    // ... and when the key size lets the query fragments live in registers, no query buffer at all: with two tiles in
    // flight three CTAs then share an SM
    const bool q_in_regs = single && d.dk <= 128;
    const int stages = !single ? 2 : ((long long)grid.x * grid.y * grid.z <= sms ? 4 : (q_in_regs ? 2 : 3));
    const int q_alloc = q_in_regs ? 0 : (single ? 16 : WM_ROWS);
    const size_t smem = (size_t)(2 * q_alloc * (d.dk + 8) + stages * WM_KEYS * (d.dk + 8 + d.dv + 8)) * 2;
    if (smem > (size_t)kMaxSmem) return set_error("windowed attention: head sizes %d / %d do not fit shared memory", d.dk, d.dv);
    if (grid.y > 65535 || grid.z > 65535) return set_error("windowed attention: too many sequences or heads");
#define ASD_WM_LAUNCH(N, S, G, Q)                                                                                    \
    {                                                                                                                \
        auto fn = window_attn_mma<N, S, G, Q>;                                                                           \
        static PerDeviceOnce once;   /* the attribute is set once per device: a host call per launch costs microseconds */ \
        if (once.need()) ASD_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem)); \
        fn<<<grid, 128, smem, stream>>>(ix, cu_q, seq_slot, TQ, q, ldq, d, sink, freq_v, cache, out, of32, nsplit,   \
                                        ws.o, ws.ml, q_alloc);                                                       \
    }
#define ASD_WM_CASE(N, Q)         \
    {                             \
        if (stages == 4)                   \
            ASD_WM_LAUNCH(N, 4, true, Q)   \
        else if (stages == 3)              \
            ASD_WM_LAUNCH(N, 3, true, Q)   \
        else if (single)                   \
            ASD_WM_LAUNCH(N, 2, true, Q)   \
        else                               \
            ASD_WM_LAUNCH(N, 2, false, false) /* prompts: the constant sizes cost registers and measured 7 % slower */ \
    }
    if (d.dk == 128 && d.dv == 128) ASD_WM_CASE(16, true)
    else if (d.dk == 64 && d.dv == 64) ASD_WM_CASE(8, true)
    else if (d.dv <= 32) ASD_WM_CASE(4, false)
    else if (d.dv <= 64) ASD_WM_CASE(8, false)
    else ASD_WM_CASE(16, false)
#undef ASD_WM_CASE
#undef ASD_WM_LAUNCH
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    if (nsplit > 1) {
        window_combine_kernel<<<ix.M * d.heads, d.dv < 128 ? 64 : 128, d.dv * sizeof(float), stream>>>(
            ix, d, sink, freq_v, nsplit, ws.o, ws.ml, out, of32);
        count_launch(1);
        ASD_CUDA(cudaGetLastError());
    }
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
    static PerDeviceOnce once;
    if (once.need()) ASD_CUDA(cudaFuncSetAttribute(window_post_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    window_post_kernel<<<ix.M, 256, smem, stream>>>(ix, qkv, ld, d, freq_k, freq_v, cache);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_window_attention(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen,
                            int max_kv_len, const float* q, long long ldq, const WindowDims& d, const float* sink,
                            const float* freq_v, const PagedRows& cache, void* out, int of32, int tiled,
                            const AttnSplit& ws, cudaStream_t stream) {
    if (ix.M <= 0 || nseq <= 0) return 0;
    if (check_dims(d)) return -1;
    if (tiled && mma_supports(d, cache))
        return launch_mma(ix, cu_q, seq_slot, nseq, max_qlen, max_kv_len, q, ldq, d, sink, freq_v, cache, out, of32, ws, stream);
    return cache.f32 ? launch_simple<float>(ix, cu_q, seq_slot, nseq, max_qlen, q, ldq, d, sink, freq_v, cache, out, of32, stream)
                     : launch_simple<__nv_bfloat16>(ix, cu_q, seq_slot, nseq, max_qlen, q, ldq, d, sink, freq_v, cache, out, of32, stream);
}

}  // namespace asd
