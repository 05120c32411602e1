// Latent key/value attention in latent space over a paged cache of [R latent | dr rotated key] rows, with a
// sliding window.  Scores, softmax weights and the weighted sum are fp32; the cache rows are the engine's element type.
//
// latent_post_kernel: one CTA per token.  RMS-norms the latent (vector weight), rotates the shared key part and the
// rotated part of every head's query (pairs (i, i + rot_dims / 2) or (2 i, 2 i + 1) inside the first rot_dims coordinates),
// appends the cache row.
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

__global__ void latent_post_kernel(SeqIndex ix, const float* q, long long ldq, const float* kvp, long long ldkv,
                                   LatentDims d, const void* c_norm, int wf32, float eps, const float* inv_freq,
                                   PagedRows cache, float* q_lat) {
    __shared__ float red[33];
    const int m = blockIdx.x;
    const int pos = ix.positions[m], slot = ix.token_slot[m];
    const int qw = d.dn + d.dr, rw = d.R + d.dr;
    const float* qrow = q + (long long)m * ldq;
    const float* kv = kvp + (long long)m * ldkv;
    const long long crow = cache_row(cache, slot, pos) * rw;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d.R; i += blockDim.x) {
        const float v = kv[i];
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float r = 1.f / sqrtf(ss / (float)d.R + eps);
    for (int i = threadIdx.x; i < d.R; i += blockDim.x)
        stx(cache.pool, crow + i, cache.f32, kv[i] * r * ldx(c_norm, i, wf32));
    // rotated parts: vector 0 is the shared key, vectors 1 .. heads the queries
    const int half = d.rot_dims / 2;
    for (int t = threadIdx.x; t < (d.heads + 1) * d.dr; t += blockDim.x) {
        const int vec = t / d.dr, i = t % d.dr;
        const float* src = vec == 0 ? kv + d.R : qrow + (long long)(vec - 1) * qw + d.dn;
        float out;
        if (i < d.rot_dims) {
            // pair j = (a, b): coordinate a becomes u cos - v sin, coordinate b becomes v cos + u sin
            const int j = d.interleaved ? i >> 1 : (i < half ? i : i - half);
            const int a = d.interleaved ? 2 * j : j, b = d.interleaved ? 2 * j + 1 : j + half;
            float sn, cs;
            sincosf((float)pos * inv_freq[j], &sn, &cs);
            const float u = src[a], v = src[b];
            out = i == a ? u * cs - v * sn : v * cs + u * sn;
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

// ---------------------------------------------------------------------------------------------------------------
// Register-tiled form for latent sizes that are multiples of 4 and at most 512 (RC = ceil(R / 256) <= 2).
// One CTA = QT = 4 * RPT query rows (TQ consecutive tokens x HG heads of one sequence) x one share of the key tiles.
// Per tile of 32 keys (fp32 in shared memory, row stride rw + 4 so that float4 reads of 8 different keys hit 32 banks):
//   scores   warp w owns rows w * QT / 8 .., lane = key: float4 steps over R + dr, the query values one broadcast read;
//   softmax  in the same registers: running maximum and sum per row, weights written transposed as [key][row];
//   update   thread (qg, rg) = (warp / 2, (warp % 2) * 32 + lane): rows qg * RPT .. x latent columns {4 rg + 256 i}:
//            RPT x 4 RC accumulators fed by one float4 of weights (broadcast) and RC float4 of the key row per key.
// A long key range is cut into shares (blockIdx.y = sequence * nsplit + share) so that few query rows still fill the
// GPU; every share writes its unnormalised sum, maximum and weight sum, and latent_combine_kernel merges them.
// 8 consecutive cache elements as fp32 (16-byte load for bf16 rows)
__device__ __forceinline__ void widen8(const uint4& v, float* dst) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        dst[2 * i] = __uint_as_float(u[i] << 16);
        dst[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}

// vec = 1 (bf16 rows of a multiple of 8 elements, 16-byte aligned pool): the next tile's rows are fetched into registers
// with 16-byte loads while the current tile is computed, and widened to fp32 on the way into shared memory.
template <typename T, int RPT, int RC>
__global__ void __launch_bounds__(256, 1) latent_attn_tiled(SeqIndex ix, const int* cu_q, const int* seq_slot, int TQ,
                                                            int HG, int nsplit, int vec, const float* q_lat, LatentDims d,
                                                            PagedRows cache, float* out_lat, float* ws_o, float* ws_ml) {
    constexpr int QT = 4 * RPT, KT = 32, RW = QT / 8;
    extern __shared__ float smem[];
    const int rw = d.R + d.dr, LD = rw + 4;
    float* Ks = smem;                        // [KT][LD]
    float* Qs = Ks + KT * LD;                // [QT][LD]
    float* Pt = Qs + QT * LD;                // [KT][QT] softmax weights of the tile, transposed
    float* Cs = Pt + KT * QT;                // [QT] rescale of this tile, then the final weight sums
    float* Ms = Cs + QT;                     // [QT] final maxima
    __shared__ int row_pos[32];
    __shared__ long long key_row[2][32];     // pool rows of the keys of tile t in key_row[t & 1] (-1: past the last position)
    const int seq = blockIdx.y / nsplit, split = blockIdx.y % nsplit;
    const int t0 = cu_q[seq] + blockIdx.x * TQ, t_end = cu_q[seq + 1];
    if (t0 >= t_end) return;
    const int slot = seq_slot[seq];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_tok = min(TQ, t_end - t0), h0 = blockIdx.z * HG;
    const int p_first = ix.positions[t0], p_last = ix.positions[t0 + n_tok - 1];
    int j_lo = p_first - d.window + 1;
    if (j_lo < 0) j_lo = 0;
    const int nt = (p_last - j_lo) / KT + 1, per = (nt + nsplit - 1) / nsplit;
    const int ts = split * per, te = min(nt, ts + per);
    // row r of the tile = (token t0 + r / HG, head h0 + r % HG)
    if (tid < QT) {
        const int tq = tid / HG, h = h0 + tid % HG;
        row_pos[tid] = (tq < n_tok && h < d.heads && tid < TQ * HG) ? ix.positions[t0 + tq] : -1;
    }
    for (int i = tid; i < QT * (rw / 4); i += 256) {
        const int r = i / (rw / 4), c = i % (rw / 4);
        const int tq = r / HG, h = h0 + r % HG;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (tq < n_tok && h < d.heads && r < TQ * HG)
            v = *reinterpret_cast<const float4*>(q_lat + ((long long)(t0 + tq) * d.heads + h) * rw + 4 * c);
        *reinterpret_cast<float4*>(Qs + r * LD + 4 * c) = v;
    }
    float4 acc[RPT][RC];
#pragma unroll
    for (int i = 0; i < RPT; ++i)
#pragma unroll
        for (int j = 0; j < RC; ++j) acc[i][j] = make_float4(0.f, 0.f, 0.f, 0.f);
    float m_run[RW], l_run[RW];
#pragma unroll
    for (int i = 0; i < RW; ++i) m_run[i] = -INFINITY, l_run[i] = 0.f;
    const int qg = warp >> 1, rg = (warp & 1) * 32 + lane;
    const T* pool = (const T*)cache.pool;
    constexpr int MAXCH = 13;                // 32 rows x (rw / 8) chunks over 256 threads, rw <= 828
    uint4 pre[MAXCH];
    const int cpr = rw >> 3, nch = KT * cpr;
    auto fetch = [&](int t) {
#pragma unroll
        for (int i = 0; i < MAXCH; ++i) {
            const int idx = tid + 256 * i;
            if (idx < nch) {
                const int r = idx / cpr, c = idx - r * cpr;
                const long long row = key_row[t & 1][r];
                pre[i] = row >= 0 ? *reinterpret_cast<const uint4*>(pool + row * rw + 8 * c) : make_uint4(0, 0, 0, 0);
            }
        }
    };
    // the page-table lookups run one tile ahead of the loads that need them
    auto locate = [&](int t) {
        if (tid < KT) {
            const int kp = j_lo + t * KT + tid;
            key_row[t & 1][tid] = (t < te && kp <= p_last) ? cache_row(cache, slot, kp) : -1;
        }
    };
    if (vec && ts < te) {
        locate(ts);
        locate(ts + 1);
        __syncthreads();
        fetch(ts);
    }
    for (int t = ts; t < te; ++t) {
        const int j0 = j_lo + t * KT;
        __syncthreads();                     // the previous tile is consumed; Qs and row_pos are written
        if (vec) {
#pragma unroll
            for (int i = 0; i < MAXCH; ++i) {
                const int idx = tid + 256 * i;
                if (idx < nch) {
                    const int r = idx / cpr, c = idx - r * cpr;
                    float f[8];
                    widen8(pre[i], f);
                    *reinterpret_cast<float4*>(Ks + r * LD + 8 * c) = make_float4(f[0], f[1], f[2], f[3]);
                    *reinterpret_cast<float4*>(Ks + r * LD + 8 * c + 4) = make_float4(f[4], f[5], f[6], f[7]);
                }
            }
            if (t + 1 < te) fetch(t + 1);    // in flight while this tile is computed
            locate(t + 2);                   // key_row[t & 1] was last read by fetch(t), before this tile's first barrier
        } else {
            for (int r = warp; r < KT; r += 8) {
                const int kp = j0 + r;
                const T* src = kp <= p_last ? pool + cache_row(cache, slot, kp) * rw : nullptr;
                for (int i = lane; i < rw; i += 128) {      // four loads in flight per lane
                    float v[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) v[u] = (src && i + 32 * u < rw) ? ldf(src + i + 32 * u) : 0.f;
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (i + 32 * u < rw) Ks[r * LD + i + 32 * u] = v[u];
                }
            }
        }
        __syncthreads();
        // scores and softmax bookkeeping: warp w owns rows w * RW .., lane = key of the tile.  The query values are the
        // same address for the whole warp (one shared-memory wavefront); the 32 key rows are 32 different bank groups.
        {
            float s[RW][4];                  // four partial sums per row: independent FMA chains
#pragma unroll
            for (int a = 0; a < RW; ++a) s[a][0] = s[a][1] = s[a][2] = s[a][3] = 0.f;
            const float* kr = Ks + lane * LD;
            const float* qr = Qs + warp * RW * LD;
#pragma unroll 4
            for (int i = 0; i < rw; i += 4) {
                const float4 kv = *reinterpret_cast<const float4*>(kr + i);
#pragma unroll
                for (int a = 0; a < RW; ++a) {
                    const float4 q = *reinterpret_cast<const float4*>(qr + a * LD + i);
                    s[a][0] = fmaf(q.x, kv.x, s[a][0]), s[a][1] = fmaf(q.y, kv.y, s[a][1]);
                    s[a][2] = fmaf(q.z, kv.z, s[a][2]), s[a][3] = fmaf(q.w, kv.w, s[a][3]);
                }
            }
            const int kp = j0 + lane;
#pragma unroll
            for (int a = 0; a < RW; ++a) {
                const int r = warp * RW + a, p = row_pos[r];
                const bool seen = p >= 0 && kp <= p && p - kp < d.window;
                const float sv = seen ? ((s[a][0] + s[a][1]) + (s[a][2] + s[a][3])) * d.scale : -INFINITY;
                const float m_new = fmaxf(m_run[a], warp_max(sv));
                float corr = 1.f, w = 0.f;
                if (m_new != -INFINITY) {
                    corr = expf(m_run[a] - m_new);      // exp(-inf) = 0 on the row's first visible tile
                    w = seen ? expf(sv - m_new) : 0.f;
                }
                l_run[a] = l_run[a] * corr + warp_sum(w);
                m_run[a] = m_new;
                Pt[lane * QT + r] = w;
                if (lane == 0) Cs[r] = corr;
            }
        }
        __syncthreads();
        {   // update
            float cr[RPT];
#pragma unroll
            for (int i = 0; i < RPT; ++i) cr[i] = Cs[qg * RPT + i];
#pragma unroll
            for (int i = 0; i < RPT; ++i)
#pragma unroll
                for (int j = 0; j < RC; ++j)
                    acc[i][j].x *= cr[i], acc[i][j].y *= cr[i], acc[i][j].z *= cr[i], acc[i][j].w *= cr[i];
#pragma unroll 2
            for (int k = 0; k < KT; ++k) {
                float w[RPT];
#pragma unroll
                for (int i = 0; i < RPT; i += 4) {
                    const float4 v = *reinterpret_cast<const float4*>(Pt + k * QT + qg * RPT + i);
                    w[i] = v.x, w[i + 1] = v.y, w[i + 2] = v.z, w[i + 3] = v.w;
                }
#pragma unroll
                for (int j = 0; j < RC; ++j) {
                    const int c = 4 * rg + 256 * j;
                    if (c < d.R) {
                        const float4 kv = *reinterpret_cast<const float4*>(Ks + k * LD + c);
#pragma unroll
                        for (int i = 0; i < RPT; ++i) {
                            acc[i][j].x = fmaf(w[i], kv.x, acc[i][j].x), acc[i][j].y = fmaf(w[i], kv.y, acc[i][j].y);
                            acc[i][j].z = fmaf(w[i], kv.z, acc[i][j].z), acc[i][j].w = fmaf(w[i], kv.w, acc[i][j].w);
                        }
                    }
                }
            }
        }
    }
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < RW; ++i) Cs[warp * RW + i] = l_run[i], Ms[warp * RW + i] = m_run[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int r = qg * RPT + i;
        if (row_pos[r] < 0) continue;
        const int tq = r / HG, h = h0 + r % HG;
        const long long row = (long long)(t0 + tq) * d.heads + h;
        if (nsplit == 1) {
            const float inv = 1.f / Cs[r];
#pragma unroll
            for (int j = 0; j < RC; ++j) {
                const int c = 4 * rg + 256 * j;
                if (c < d.R)
                    *reinterpret_cast<float4*>(out_lat + row * d.R + c) =
                        make_float4(acc[i][j].x * inv, acc[i][j].y * inv, acc[i][j].z * inv, acc[i][j].w * inv);
            }
        } else {
            const long long part = row * nsplit + split;
#pragma unroll
            for (int j = 0; j < RC; ++j) {
                const int c = 4 * rg + 256 * j;
                if (c < d.R) *reinterpret_cast<float4*>(ws_o + part * d.R + c) = acc[i][j];
            }
            if (rg == 0) ws_ml[part * 2] = Ms[r], ws_ml[part * 2 + 1] = Cs[r];
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Tensor-core form for bf16 cache rows (latent size a multiple of 8 and at most 512, row length a multiple of 16):
// the two products of a tile run as mma.sync m16n8k16 with fp32 accumulation, and the fp32 operand of each (the query
// in latent space, the softmax weights) enters as a sum of bf16 terms, x = hi + mid + lo with hi = bf16(x), mid =
// bf16(x - hi), lo = bf16(x - hi - mid): three terms carry all 24 bits of the query, so a score is the same fp32 sum of
// exact products the CUDA-core kernel forms; the weights take two terms (16 bits) into the product with the bf16 values.  One CTA = 16 query rows (tokens x heads of one sequence) x one share of the keys,
// 64 keys per tile: warp w scores keys 8 w .. 8 w + 7 over the whole row length, the scores meet in shared memory for
// the running softmax (warp w owns rows 2 w, 2 w + 1), and warp w then updates the latent columns of the 8-wide tiles
// w, w + 8, ... with the key rows read through ldmatrix.trans.
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& b0, uint32_t& b1, const void* smem_row) {
    const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
}
// A fragment (16 rows x 16 k) of a row-major bf16 tile: lane l names row l % 16 at column 8 * (l / 16)
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&a)[4], const void* smem_row) {
    const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
                 : "r"(addr));
}
// B fragment (16 k x 8 n) of a tile stored [n][k]: lanes 0-7 name rows n at column 0, lanes 8-15 at column 8
__device__ __forceinline__ void ldmatrix_x2(uint32_t& b0, uint32_t& b1, const void* smem_row) {
    const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
}
__device__ __forceinline__ void split_bf16(float x, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16(x);
    lo = __float2bfloat16(x - __bfloat162float(hi));
}

template <int MT>   // 16-row tiles per CTA: 1 (few rows: decode) or 2 (prompts: a key tile serves twice the rows)
__global__ void __launch_bounds__(256, 1) latent_attn_mma(SeqIndex ix, const int* cu_q, const int* seq_slot, int TQ, int HG,
                                                          int nsplit, const float* q_lat, LatentDims d, PagedRows cache,
                                                          float* out_lat, float* ws_o, float* ws_ml) {
    constexpr int QT = 16 * MT, KT = 64, NTW = 8, RW = 2 * MT;                  // NTW: 8-wide latent tiles per warp (R <= 512)
    extern __shared__ __align__(16) uint8_t smem_b[];
    const int rw = d.R + d.dr, LDK = rw + 8;                  // bf16 elements per staged row (16-byte multiple)
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_b);          // [KT][LDK]
    __nv_bfloat16* Qh = Ks + KT * LDK;                                     // [QT][LDK]
    __nv_bfloat16* Qm = Qh + QT * LDK;                                     // [QT][LDK]
    __nv_bfloat16* Ql = Qm + QT * LDK;                                     // [QT][LDK]
    __nv_bfloat16* Ph = Ql + QT * LDK;                                     // [QT][KT + 8]
    __nv_bfloat16* Pl = Ph + QT * (KT + 8);                                // [QT][KT + 8]
    float* Ss = reinterpret_cast<float*>(Pl + QT * (KT + 8));              // [QT][KT + 1]
    float* Cs = Ss + QT * (KT + 1);                                        // [QT]
    float* Ms = Cs + QT;                                                   // [QT]
    __shared__ int row_pos[QT];
    __shared__ long long key_row[2][KT];
    const int seq = blockIdx.y / nsplit, split = blockIdx.y % nsplit;
    const int t0 = cu_q[seq] + blockIdx.x * TQ, t_end = cu_q[seq + 1];
    if (t0 >= t_end) return;
    const int slot = seq_slot[seq];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq4 = lane & 3;
    const int n_tok = min(TQ, t_end - t0), h0 = blockIdx.z * HG;
    const int p_first = ix.positions[t0], p_last = ix.positions[t0 + n_tok - 1];
    int j_lo = p_first - d.window + 1;
    if (j_lo < 0) j_lo = 0;
    const int nt = (p_last - j_lo) / KT + 1, per = (nt + nsplit - 1) / nsplit;
    const int ts = split * per, te = min(nt, ts + per);
    if (tid < QT) {
        const int tq = tid / HG, h = h0 + tid % HG;
        row_pos[tid] = (tq < n_tok && h < d.heads && tid < TQ * HG) ? ix.positions[t0 + tq] : -1;
    }
    {   // the query rows as three bf16 terms (24 bits); four 16-byte loads in flight per thread
        const int cpq = rw >> 2, total = QT * cpq;
        for (int base = 0; base < total; base += 1024) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = base + tid + 256 * u;
                v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i < total) {
                    const int r = i / cpq, c = i - r * cpq;
                    const int tq = r / HG, h = h0 + r % HG;
                    if (tq < n_tok && h < d.heads && r < TQ * HG)
                        v[u] = *reinterpret_cast<const float4*>(q_lat + ((long long)(t0 + tq) * d.heads + h) * rw + 4 * c);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = base + tid + 256 * u;
                if (i < total) {
                    const int r = i / cpq, c = i - r * cpq;
                    const float x[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int o = r * LDK + 4 * c + e;
                        split_bf16(x[e], Qh[o], Qm[o]);
                        const float rest = (x[e] - __bfloat162float(Qh[o])) - __bfloat162float(Qm[o]);
                        Ql[o] = __float2bfloat16(rest);
                    }
                }
            }
        }
    }
    float acc[MT][NTW][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int i = 0; i < NTW; ++i) acc[mt][i][0] = acc[mt][i][1] = acc[mt][i][2] = acc[mt][i][3] = 0.f;
    float m_run[RW], l_run[RW];
#pragma unroll
    for (int i = 0; i < RW; ++i) m_run[i] = -INFINITY, l_run[i] = 0.f;
    const __nv_bfloat16* pool = (const __nv_bfloat16*)cache.pool;
    // key rows of a tile -> registers: warp w takes rows 8 w .. 8 w + 7, lane l the 16-byte chunks l, l + 32, l + 64 of
    // each (a warp reads 512 contiguous bytes; no index arithmetic beyond adds)
    constexpr int CPL = 3;                                    // chunks per lane and row: row length <= 768 elements
    uint4 pre[8][CPL];
    const int cpr = rw >> 3;
    auto fetch = [&](int t) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const long long row = key_row[t & 1][warp * 8 + j];
#pragma unroll
            for (int u = 0; u < CPL; ++u) {
                const int c = lane + 32 * u;
                pre[j][u] = (row >= 0 && c < cpr) ? *reinterpret_cast<const uint4*>(pool + row * rw + 8 * c) : make_uint4(0, 0, 0, 0);
            }
        }
    };
    auto locate = [&](int t) {
        if (tid < KT) {
            const int kp = j_lo + t * KT + tid;
            key_row[t & 1][tid] = (t < te && kp <= p_last) ? cache_row(cache, slot, kp) : -1;
        }
    };
    if (ts < te) {
        locate(ts);
        locate(ts + 1);
        __syncthreads();
        fetch(ts);
    }
    const int n_tiles_r = d.R >> 3;
    for (int t = ts; t < te; ++t) {
        const int j0 = j_lo + t * KT;
        __syncthreads();
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int u = 0; u < CPL; ++u) {
                const int c = lane + 32 * u;
                if (c < cpr) *reinterpret_cast<uint4*>(Ks + (warp * 8 + j) * LDK + 8 * c) = pre[j][u];
            }
        if (t + 1 < te) fetch(t + 1);
        locate(t + 2);
        __syncthreads();
        {   // scores of keys 8 warp .. 8 warp + 7 for all rows: a key fragment serves 3 MT products
            float st[MT][3][4];              // one accumulator per row tile and term: independent MMA chains
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int u = 0; u < 3; ++u) st[mt][u][0] = st[mt][u][1] = st[mt][u][2] = st[mt][u][3] = 0.f;
            const __nv_bfloat16* kb = Ks + (warp * 8 + (lane & 7)) * LDK + 8 * ((lane >> 3) & 1);
            const int qoff = (lane & 15) * LDK + 8 * (lane >> 4);
            const __nv_bfloat16* qt[3] = {Qh + qoff, Qm + qoff, Ql + qoff};
#pragma unroll 2
            for (int k0 = 0; k0 < rw; k0 += 16) {
                uint32_t b0, b1;
                ldmatrix_x2(b0, b1, kb + k0);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int u = 0; u < 3; ++u) {
                        uint32_t a[4];
                        ldmatrix_x4(a, qt[u] + mt * 16 * LDK + k0);
                        mma_bf16(st[mt][u], a, b0, b1);
                    }
            }
            const int col = warp * 8 + 2 * tq4;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                float sc[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[e] = st[mt][0][e] + (st[mt][1][e] + st[mt][2][e]);
                float* dst = Ss + (mt * 16 + g) * (KT + 1) + col;
                dst[0] = sc[0], dst[1] = sc[1];
                dst[8 * (KT + 1)] = sc[2], dst[8 * (KT + 1) + 1] = sc[3];
            }
        }
        __syncthreads();
#pragma unroll
        for (int a = 0; a < RW; ++a) {       // running softmax of rows RW warp ..; lane = keys lane, lane + 32
            const int r = warp * RW + a, p = row_pos[r];
            float sv[2], w[2];
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                const int kp = j0 + lane + 32 * b;
                const bool seen = p >= 0 && kp <= p && p - kp < d.window;
                sv[b] = seen ? Ss[r * (KT + 1) + lane + 32 * b] * d.scale : -INFINITY;
            }
            const float m_new = fmaxf(m_run[a], warp_max(fmaxf(sv[0], sv[1])));
            float corr = 1.f;
            w[0] = w[1] = 0.f;
            if (m_new != -INFINITY) {
                corr = expf(m_run[a] - m_new);
                w[0] = sv[0] == -INFINITY ? 0.f : expf(sv[0] - m_new);
                w[1] = sv[1] == -INFINITY ? 0.f : expf(sv[1] - m_new);
            }
            l_run[a] = l_run[a] * corr + warp_sum(w[0] + w[1]);
            m_run[a] = m_new;
#pragma unroll
            for (int b = 0; b < 2; ++b) split_bf16(w[b], Ph[r * (KT + 8) + lane + 32 * b], Pl[r * (KT + 8) + lane + 32 * b]);
            if (lane == 0) Cs[r] = corr;
        }
        __syncthreads();
        {   // update of the latent columns of tiles warp, warp + 8, ...: a key fragment serves 2 MT products
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const float c_lo = Cs[mt * 16 + g], c_hi = Cs[mt * 16 + g + 8];
#pragma unroll
                for (int i = 0; i < NTW; ++i)
                    acc[mt][i][0] *= c_lo, acc[mt][i][1] *= c_lo, acc[mt][i][2] *= c_hi, acc[mt][i][3] *= c_hi;
            }
#pragma unroll
            for (int ks = 0; ks < KT / 16; ++ks) {
                uint32_t ah[MT][4], al[MT][4];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int poff = (mt * 16 + (lane & 15)) * (KT + 8) + 16 * ks + 8 * (lane >> 4);
                    ldmatrix_x4(ah[mt], Ph + poff);
                    ldmatrix_x4(al[mt], Pl + poff);
                }
#pragma unroll
                for (int i = 0; i < NTW; ++i) {
                    const int ntile = warp + 8 * i;
                    if (ntile < n_tiles_r) {
                        uint32_t b0, b1;
                        ldmatrix_x2_trans(b0, b1, Ks + (16 * ks + (lane & 15)) * LDK + 8 * ntile);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            mma_bf16(acc[mt][i], ah[mt], b0, b1);
                            mma_bf16(acc[mt][i], al[mt], b0, b1);
                        }
                    }
                }
            }
        }
    }
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < RW; ++i) Cs[warp * RW + i] = l_run[i], Ms[warp * RW + i] = m_run[i];
    }
    __syncthreads();
#pragma unroll
    for (int mh = 0; mh < 2 * MT; ++mh) {
        const int mt = mh >> 1, hh = mh & 1, r = mt * 16 + g + 8 * hh;
        if (row_pos[r] < 0) continue;
        const int tq = r / HG, h = h0 + r % HG;
        const long long row = (long long)(t0 + tq) * d.heads + h;
        const float inv = nsplit == 1 ? 1.f / Cs[r] : 1.f;
        float* dst = nsplit == 1 ? out_lat + row * d.R : ws_o + (row * nsplit + split) * d.R;
#pragma unroll
        for (int i = 0; i < NTW; ++i) {
            const int ntile = warp + 8 * i;
            if (ntile < n_tiles_r)
                *reinterpret_cast<float2*>(dst + 8 * ntile + 2 * tq4) =
                    make_float2(acc[mt][i][2 * hh] * inv, acc[mt][i][2 * hh + 1] * inv);
        }
        if (nsplit > 1 && warp == 0 && tq4 == 0) {
            ws_ml[(row * nsplit + split) * 2] = Ms[r];
            ws_ml[(row * nsplit + split) * 2 + 1] = Cs[r];
        }
    }
}

// out[row] = sum_s o_s exp(m_s - m) / sum_s l_s exp(m_s - m) over the shares of one (token, head)
__global__ void latent_combine_kernel(const float* ws_o, const float* ws_ml, int nsplit, int R, float* out_lat) {
    const long long row = blockIdx.x;
    float m = -INFINITY;
    for (int s = 0; s < nsplit; ++s) m = fmaxf(m, ws_ml[(row * nsplit + s) * 2]);
    float l = 0.f;
    for (int s = 0; s < nsplit; ++s) {
        const float ms = ws_ml[(row * nsplit + s) * 2];
        if (ms != -INFINITY) l += ws_ml[(row * nsplit + s) * 2 + 1] * expf(ms - m);
    }
    for (int c = threadIdx.x; c < R; c += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < nsplit; ++s) {
            const float ms = ws_ml[(row * nsplit + s) * 2];
            if (ms != -INFINITY) o += ws_o[(row * nsplit + s) * R + c] * expf(ms - m);
        }
        out_lat[row * R + c] = o / l;
    }
}

template <typename T, int RPT, int RC>
int launch_tiled_t(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen, int max_kv_len,
                   const float* q_lat, const LatentDims& d, const PagedRows& cache, float* out_lat, const AttnSplit& ws,
                   cudaStream_t stream) {
    constexpr int QT = 4 * RPT;
    const int HG = d.heads < QT ? d.heads : QT;
    int TQ = QT / HG;
    if (TQ > max_qlen) TQ = max_qlen;
    const int rw = d.R + d.dr, LD = rw + 4;
    const size_t smem = (size_t)(32 * LD + QT * LD + 32 * QT + 2 * QT) * sizeof(float);
    const int q_tiles = (max_qlen + TQ - 1) / TQ, hgs = (d.heads + HG - 1) / HG;
    // shares of the key range: at most two full waves of one CTA per SM (a third, mostly empty wave costs more than the
    // longer key loop of fewer shares), at least four key tiles each, within the workspace
    long long keys = (long long)(d.window < max_kv_len ? d.window : max_kv_len) + TQ;
    const int kv_tiles = (int)((keys + 31) / 32);
    int nsplit = 1;
    const long long ctas = (long long)q_tiles * nseq * hgs, rows = (long long)ix.M * d.heads;
    static const int two_waves = []() {
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        return 2 * sms;
    }();
    if (ws.o && ws.ml && ctas < two_waves) {
        nsplit = (int)(two_waves / ctas);
        if (nsplit > kv_tiles / 4) nsplit = kv_tiles / 4;
        if ((long long)nsplit * rows > ws.rows) nsplit = (int)(ws.rows / rows);
        if ((long long)nsplit * rows * d.R > ws.o_elems) nsplit = (int)(ws.o_elems / (rows * d.R));
        if (nsplit < 1) nsplit = 1;
        if (nsplit > 64) nsplit = 64;
    }
    auto fn = latent_attn_tiled<T, RPT, RC>;
    ASD_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(q_tiles, nseq * nsplit, hgs);
    const int vec = sizeof(T) == 2 && (rw & 7) == 0 && (reinterpret_cast<uintptr_t>(cache.pool) & 15) == 0;
    fn<<<grid, 256, smem, stream>>>(ix, cu_q, seq_slot, TQ, HG, nsplit, vec, q_lat, d, cache, out_lat, ws.o, ws.ml);
    count_launch(1);
    if (nsplit > 1) {
        latent_combine_kernel<<<(unsigned)rows, 128, 0, stream>>>(ws.o, ws.ml, nsplit, d.R, out_lat);
        count_launch(1);
    }
    ASD_CUDA(cudaGetLastError());
    return 0;
}

template <int MT>
int launch_mma_t(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen, int max_kv_len,
                 const float* q_lat, const LatentDims& d, const PagedRows& cache, float* out_lat, const AttnSplit& ws,
                 cudaStream_t stream) {
    constexpr int QT = 16 * MT, KT = 64;
    const int HG = d.heads < QT ? d.heads : QT;
    int TQ = QT / HG;
    if (TQ > max_qlen) TQ = max_qlen;
    const int rw = d.R + d.dr, LDK = rw + 8;
    const size_t smem = (size_t)(KT + 3 * QT) * LDK * 2 + (size_t)2 * QT * (KT + 8) * 2 + (size_t)(QT * (KT + 1) + 2 * QT) * 4;
    const int q_tiles = (max_qlen + TQ - 1) / TQ, hgs = (d.heads + HG - 1) / HG;
    long long keys = (long long)(d.window < max_kv_len ? d.window : max_kv_len) + TQ;
    const int kv_tiles = (int)((keys + KT - 1) / KT);
    int nsplit = 1;
    const long long ctas = (long long)q_tiles * nseq * hgs, rows = (long long)ix.M * d.heads;
    static const int two_waves = []() {
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        return 2 * sms;
    }();
    if (ws.o && ws.ml && ctas < two_waves) {
        nsplit = (int)(two_waves / ctas);
        if (nsplit > kv_tiles / 2) nsplit = kv_tiles / 2;      // at least two key tiles (128 keys) per share
        if ((long long)nsplit * rows > ws.rows) nsplit = (int)(ws.rows / rows);
        if ((long long)nsplit * rows * d.R > ws.o_elems) nsplit = (int)(ws.o_elems / (rows * d.R));
        if (nsplit < 1) nsplit = 1;
        if (nsplit > 64) nsplit = 64;
    }
    ASD_CUDA(cudaFuncSetAttribute(latent_attn_mma<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(q_tiles, nseq * nsplit, hgs);
    latent_attn_mma<MT><<<grid, 256, smem, stream>>>(ix, cu_q, seq_slot, TQ, HG, nsplit, q_lat, d, cache, out_lat, ws.o, ws.ml);
    count_launch(1);
    if (nsplit > 1) {
        latent_combine_kernel<<<(unsigned)rows, 128, 0, stream>>>(ws.o, ws.ml, nsplit, d.R, out_lat);
        count_launch(1);
    }
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_mma(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen, int max_kv_len,
               const float* q_lat, const LatentDims& d, const PagedRows& cache, float* out_lat, const AttnSplit& ws,
               cudaStream_t stream) {
    const long long need = (long long)(d.heads < 32 ? d.heads : 32) * (max_qlen < 32 ? max_qlen : 32);
    const int LDK = d.R + d.dr + 8;
    const size_t smem2 = (size_t)(64 + 3 * 32) * LDK * 2 + (size_t)2 * 32 * 72 * 2 + (size_t)(32 * 65 + 64) * 4;
    if (need >= 32 && smem2 <= 220 * 1024)
        return launch_mma_t<2>(ix, cu_q, seq_slot, nseq, max_qlen, max_kv_len, q_lat, d, cache, out_lat, ws, stream);
    return launch_mma_t<1>(ix, cu_q, seq_slot, nseq, max_qlen, max_kv_len, q_lat, d, cache, out_lat, ws, stream);
}

template <typename T>
int launch_tiled(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen, int max_kv_len,
                 const float* q_lat, const LatentDims& d, const PagedRows& cache, float* out_lat, const AttnSplit& ws,
                 cudaStream_t stream) {
    const long long need = (long long)(d.heads < 32 ? d.heads : 32) * (max_qlen < 32 ? max_qlen : 32);
    const bool small = need <= 16;
#define ASD_TILED(RPT, RC) \
    return launch_tiled_t<T, RPT, RC>(ix, cu_q, seq_slot, nseq, max_qlen, max_kv_len, q_lat, d, cache, out_lat, ws, stream)
    if (d.R <= 256) {
        if (small) ASD_TILED(4, 1);
        ASD_TILED(8, 1);
    }
    if (small) ASD_TILED(4, 2);
    ASD_TILED(8, 2);
#undef ASD_TILED
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

int launch_latent_post_split(const SeqIndex& ix, const float* q, long long ldq, const float* kv, long long ldkv,
                             const LatentDims& d, const void* c_norm, int wf32, float eps, const float* inv_freq,
                             const PagedRows& cache, float* q_lat, cudaStream_t stream) {
    if (ix.M <= 0) return 0;
    if (d.rot_dims < 0 || d.rot_dims > d.dr || (d.rot_dims & 1))
        return set_error("latent attention: rot_dims %d must be even and <= %d", d.rot_dims, d.dr);
    latent_post_kernel<<<ix.M, 128, 0, stream>>>(ix, q, ldq, kv, ldkv, d, c_norm, wf32, eps, inv_freq, cache, q_lat);
    count_launch(1);
    ASD_CUDA(cudaGetLastError());
    return 0;
}

int launch_latent_post(const SeqIndex& ix, const float* qd, const LatentDims& d, const void* c_norm, int wf32, float eps,
                       const float* inv_freq, const PagedRows& cache, float* q_lat, cudaStream_t stream) {
    const int nq = d.heads * (d.dn + d.dr), ld = nq + d.R + d.dr;
    return launch_latent_post_split(ix, qd, ld, qd + nq, ld, d, c_norm, wf32, eps, inv_freq, cache, q_lat, stream);
}

int launch_latent_attention(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen,
                            int max_kv_len, const float* q_lat, const LatentDims& d, const PagedRows& cache,
                            float* out_lat, const AttnSplit& ws, cudaStream_t stream) {
    if (ix.M <= 0 || nseq <= 0) return 0;
    if (d.window <= 0) return set_error("latent attention: window must be positive");
    const int rw = d.R + d.dr;
    const bool tiled = ws.tiled && (d.R % 4) == 0 && (rw % 4) == 0 && d.R <= 512 &&
                       (size_t)(64 * (rw + 4)) * sizeof(float) <= 200 * 1024 &&
                       (reinterpret_cast<uintptr_t>(q_lat) & 15) == 0 && (reinterpret_cast<uintptr_t>(out_lat) & 15) == 0;
    const bool mma = ws.tiled >= 2 && !cache.f32 && (d.R % 8) == 0 && (rw % 16) == 0 && d.R <= 512 && rw <= 768 &&
                     (reinterpret_cast<uintptr_t>(cache.pool) & 15) == 0 && (reinterpret_cast<uintptr_t>(out_lat) & 7) == 0;
    if (mma) return launch_mma(ix, cu_q, seq_slot, nseq, max_qlen, max_kv_len, q_lat, d, cache, out_lat, ws, stream);
    if (tiled)
        return cache.f32 ? launch_tiled<float>(ix, cu_q, seq_slot, nseq, max_qlen, max_kv_len, q_lat, d, cache, out_lat, ws, stream)
                         : launch_tiled<__nv_bfloat16>(ix, cu_q, seq_slot, nseq, max_qlen, max_kv_len, q_lat, d, cache, out_lat, ws, stream);
    return cache.f32 ? launch_attn_t<float>(ix, cu_q, seq_slot, nseq, max_qlen, q_lat, d, cache, out_lat, stream)
                     : launch_attn_t<__nv_bfloat16>(ix, cu_q, seq_slot, nseq, max_qlen, q_lat, d, cache, out_lat, stream);
}

}  // namespace asd
