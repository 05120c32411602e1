// Mezilix family forward engine: one opaque handle per model.  asd_mezilix_forward runs, on the caller's stream and
// with no host synchronisation,
//   token-pair embedding (+ first norm) -> L x [ token shift, q | latent projection, latent norm + rotation + cache
//   append, query into latent space, windowed latent attention, value up-projection, output projection, router,
//   grouped expert up (squared ReLU) / down, layer close: residual + depth-weighted average + next norm ] -> head.
// Every step is a building block of blocks.h that takes its sizes from the layer's configuration; dense bf16
// projections go to the tcgen05 weight-streaming GEMM of gemm.cu when their shape fits its contract.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <string.h>

#include <unordered_map>
#include <vector>

#include "../../include/asd_b200.h"
#include "asd_internal.h"
#include "blocks.h"
#include "dense.h"
#include "gemm.h"
#include "prof.h"

struct asd_mezilix_engine {};

namespace asd {

struct MzLayer {
    asd_mezilix_layer_config c;
    const void *gain = nullptr, *shift = nullptr, *coeff = nullptr, *wqd = nullptr, *latent_gain = nullptr, *wuk = nullptr,
               *wuv = nullptr, *wo = nullptr, *router = nullptr, *w_up = nullptr, *w_down = nullptr;
    float* inv_freq = nullptr;   // owned, [rot_dims / 2]
    size_t cache_off = 0;        // elements from the pool start (set by set_cache)
    int nq, nqd, rw;
};

struct MzEngine : asd_mezilix_engine {
    asd_mezilix_config c;
    std::vector<MzLayer> layers;
    const void *embed = nullptr, *pair_table = nullptr, *final_gain = nullptr, *head = nullptr;
    int f32 = 0, esz = 2;
    // cache / state (caller owned)
    char* pool = nullptr;
    const int* page_table = nullptr;
    int num_pages = 0, max_seqs = 0, max_pages = 0;
    int* tok_ring = nullptr;
    float* shift_ring = nullptr;
    // owned activations
    float *stack = nullptr, *xavg = nullptr, *hn = nullptr, *qd = nullptr, *qlat = nullptr, *olat = nullptr, *mix = nullptr,
          *rlog = nullptr, *gate = nullptr, *eout = nullptr;
    void *h = nullptr, *hs = nullptr, *vout = nullptr, *act = nullptr, *xsel = nullptr;
    int *expert_of = nullptr, *counters = nullptr, *group_off = nullptr, *sorted_tok = nullptr, *slot_of = nullptr;
    std::vector<void*> owned;
    DenseRunner dn;              // dense projections: tcgen05 GEMMs or the CUDA-core kernel, by shape and type
    EventProfiler prof;
    AttnSplit attn_ws;           // partial sums of the attention kernel's key-range shares
    int* dev_error = nullptr;    // raised by a kernel whose bounded wait ran out
    int device = 0;
};

template <typename T>
static int dev_alloc(MzEngine* e, T** p, size_t n) {
    void* q = nullptr;
    ASD_CUDA(cudaMalloc(&q, (n ? n : 1) * sizeof(T)));
    e->owned.push_back(q);
    *p = (T*)q;
    return 0;
}

// y fp32 [M][ldc] = x [M][K] (engine type, contiguous rows) * w[N][K]^T
static int dense(MzEngine* e, const void* x, const void* w, float* y, int M, int N, int K, int ldc, int key,
                 cudaStream_t s) {
    return e->dn.run(x, w, y, M, N, K, ldc, key, s);
}

enum MzProf { MZ_DENSE = 0, MZ_HEADS = 1, MZ_ATTN = 2, MZ_EXPERTS = 3, MZ_ROUTER = 4, MZ_GLUE = 5, MZ_HEAD = 6, MZ_NCLASS = 7 };
#define MZ_PROF(cls) ProfRegion _region(e->prof, cls, s)

// batched / grouped linear: tcgen05 in the bf16 engine when the shape allows, CUDA cores otherwise
static int linear(MzEngine* e, const SimtLinear& L, cudaStream_t s) {
    if (!e->f32 && e->dn.tc_linear && tc_linear_supports(L)) return launch_tc_linear(L, e->dev_error, s);
    return launch_simt_linear(L, s);
}

static int forward(MzEngine* e, const int* tokens, const int* positions, const int* token_slot, int M, const int* cu_q,
                   const int* seq_slot, int nseq, int max_qlen, int max_kv_len, const int* logit_rows, int n_rows,
                   float* logits, long long ld, float* layer_out, cudaStream_t s) {
    const int D = e->c.width, ring = e->c.ring, f32 = e->f32;
    const SeqIndex ix{tokens, positions, token_slot, M};
    const size_t stride = (size_t)e->c.max_tokens * D;
    const int nl = e->c.n_layers;
    const void* first_gain = nl ? e->layers[0].gain : e->final_gain;
    {
        MZ_PROF(MZ_GLUE);
        if (launch_embed_pair(ix, e->embed, e->pair_table, f32, e->c.buckets, e->c.mul_prev, e->c.mul_cur, e->tok_ring,
                              ring, e->stack, first_gain, e->c.eps, e->hn, D, s))
            return -1;
        if (launch_commit_tokens(ix, e->tok_ring, ring, s)) return -1;
    }
    for (int l = 0; l < nl; ++l) {
        MzLayer& ly = e->layers[l];
        const asd_mezilix_layer_config& c = ly.c;
        float* ring_l = e->shift_ring + (size_t)l * e->max_seqs * ring * D;
        {
            MZ_PROF(MZ_GLUE);
            if (launch_token_shift(ix, e->hn, ring_l, ring, ly.shift, f32, e->h, e->hs, f32, D, s)) return -1;
        }
        {   // queries | latent | rotated key in one projection
            MZ_PROF(MZ_DENSE);
            if (dense(e, e->hs, ly.wqd, e->qd, M, ly.nqd, D, ly.nqd, l * 8 + 0, s)) return -1;
        }
        const LatentDims dm{c.heads, c.dim, c.rot_dim, c.vdim, c.kv_rank, c.rot_dims, c.window, c.scale};
        const PagedRows cache{e->pool + ly.cache_off * e->esz, f32, e->page_table, e->max_pages, e->c.page_size};
        {
            MZ_PROF(MZ_GLUE);
            if (launch_latent_post(ix, e->qd, dm, ly.latent_gain, f32, e->c.eps, ly.inv_freq, cache, e->qlat, s)) return -1;
        }
        {   // q_lat[m][h][r] = sum_d q[m][h][d] * WukT[h][r][d]
            MZ_PROF(MZ_HEADS);
            SimtLinear L;
            L.a = e->qd, L.a_f32 = 1, L.lda = ly.nqd, L.a_zs = c.dim + c.rot_dim;
            L.w = ly.wuk, L.w_f32 = f32, L.ldw = c.dim, L.w_zs = (long long)c.dim * c.kv_rank;
            L.c = e->qlat, L.c_f32 = 1, L.ldc = (long long)c.heads * ly.rw, L.c_zs = ly.rw;
            L.M = M, L.N = c.kv_rank, L.K = c.dim, L.Z = c.heads;
            if (linear(e, L, s)) return -1;
        }
        {
            MZ_PROF(MZ_ATTN);
            if (launch_latent_attention(ix, cu_q, seq_slot, nseq, max_qlen, max_kv_len, e->qlat, dm, cache, e->olat,
                                        e->attn_ws, s))
                return -1;
        }
        {   // v[m][h][:] = Wuv[h] * out_lat[m][h][:]
            MZ_PROF(MZ_HEADS);
            SimtLinear L;
            L.a = e->olat, L.a_f32 = 1, L.lda = (long long)c.heads * c.kv_rank, L.a_zs = c.kv_rank;
            L.w = ly.wuv, L.w_f32 = f32, L.ldw = c.kv_rank, L.w_zs = (long long)c.vdim * c.kv_rank;
            L.c = e->vout, L.c_f32 = f32, L.ldc = (long long)c.heads * c.vdim, L.c_zs = c.vdim;
            L.M = M, L.N = c.vdim, L.K = c.kv_rank, L.Z = c.heads;
            if (linear(e, L, s)) return -1;
        }
        {
            MZ_PROF(MZ_DENSE);
            if (dense(e, e->vout, ly.wo, e->mix, M, D, c.heads * c.vdim, D, l * 8 + 1, s)) return -1;
        }
        if (c.experts > 0) {
            {   // router logits in fp32 on the CUDA cores in both modes, fused with the softmax and the choice
                MZ_PROF(MZ_ROUTER);
                const MoeRouterInput in{e->h, f32, ly.router, f32, D, e->rlog};
                if (launch_moe_route(nullptr, &in, M, c.experts, c.top, e->expert_of, e->gate, e->counters, e->group_off,
                                     e->sorted_tok, e->slot_of, s))
                    return -1;
            }
            MZ_PROF(MZ_EXPERTS);
            SimtLinear U;
            U.a = e->h, U.a_f32 = f32, U.lda = D;
            U.w = ly.w_up, U.w_f32 = f32, U.ldw = D, U.w_zs = (long long)c.ff * D;
            U.c = e->act, U.c_f32 = f32, U.ldc = c.ff;
            U.M = M, U.N = c.ff, U.K = D, U.Z = c.experts;
            U.group_off = e->group_off, U.gather = e->sorted_tok, U.epilogue = 1;
            if (linear(e, U, s)) return -1;
            SimtLinear W;
            W.a = e->act, W.a_f32 = f32, W.lda = c.ff;
            W.w = ly.w_down, W.w_f32 = f32, W.ldw = c.ff, W.w_zs = (long long)D * c.ff;
            W.c = e->eout, W.c_f32 = 1, W.ldc = D;
            W.M = M, W.N = D, W.K = c.ff, W.Z = c.experts;
            W.group_off = e->group_off;
            if (linear(e, W, s)) return -1;
        }
        MZ_PROF(MZ_GLUE);
        LayerClose C;
        C.x_in = l == 0 ? e->stack : e->xavg;
        C.mix = e->mix;
        C.expert_out = e->eout, C.slot_of = e->slot_of, C.gate = e->gate, C.top = c.experts > 0 ? c.top : 0;
        C.stack = e->stack, C.stack_stride = stride, C.layer = l;
        C.coeff = ly.coeff;
        C.g_next = l + 1 < nl ? e->layers[l + 1].gain : e->final_gain;
        C.wf32 = f32, C.eps = e->c.eps;
        C.x_next = e->xavg, C.hn = e->hn, C.M = M, C.D = D;
        C.ix = &ix, C.state_ring = ring_l, C.ring = ring;     // this layer's normed input becomes the shift's carried state
        if (launch_layer_close(C, s)) return -1;
        if (layer_out)
            ASD_CUDA(cudaMemcpyAsync(layer_out + (size_t)l * M * D, e->xavg, sizeof(float) * M * D,
                                     cudaMemcpyDeviceToDevice, s));
    }
    if (n_rows > 0) {
        MZ_PROF(MZ_HEAD);
        if (launch_select_rows(e->hn, logit_rows, e->xsel, f32, n_rows, D, s)) return -1;
        const int V = e->c.vocab;
        if (dense(e, e->xsel, e->head, logits, n_rows, V, D, ld ? (int)ld : V, nl * 8 + 2, s)) return -1;
    }
    return 0;
}

}  // namespace asd

using namespace asd;

extern "C" {

asd_mezilix_engine_t* asd_mezilix_create(const asd_mezilix_config* cfg, const asd_mezilix_layer_config* layers) {
    if (!cfg || (cfg->n_layers > 0 && !layers)) {
        set_error("asd_mezilix_create: NULL config");
        return nullptr;
    }
    if (cfg->width <= 0 || cfg->vocab <= 0 || cfg->n_layers < 0 || cfg->max_tokens <= 0 || cfg->page_size <= 0 ||
        cfg->ring <= 0 || cfg->buckets <= 0 || (cfg->dtype != 0 && cfg->dtype != 1)) {
        set_error("asd_mezilix_create: bad sizes");
        return nullptr;
    }
    MzEngine* e = new MzEngine();
    e->c = *cfg;
    e->f32 = cfg->dtype;
    e->dn.f32 = cfg->dtype;
    e->esz = cfg->dtype ? 4 : 2;
    cudaGetDevice(&e->device);
    const size_t MT = cfg->max_tokens, D = cfg->width;
    size_t nqd = 1, qlat = 1, olat = 1, hv = 1, E = 1, top = 1, ff = 1;
    for (int l = 0; l < cfg->n_layers; ++l) {
        MzLayer ly;
        ly.c = layers[l];
        const auto& c = ly.c;
        if (c.heads <= 0 || c.dim <= 0 || c.rot_dim < 0 || c.vdim <= 0 || c.kv_rank <= 0 || c.window <= 0 ||
            c.rot_dims < 0 || c.rot_dims > c.rot_dim || (c.rot_dims & 1) || c.experts < 0 ||
            (c.experts > 0 && (c.top <= 0 || c.top > c.experts || c.ff <= 0))) {
            set_error("asd_mezilix_create: bad sizes in layer %d", l);
            asd_mezilix_destroy(e);
            return nullptr;
        }
        ly.nq = c.heads * (c.dim + c.rot_dim);
        ly.nqd = ly.nq + c.kv_rank + c.rot_dim;
        ly.rw = c.kv_rank + c.rot_dim;
        const int half = c.rot_dims / 2;
        std::vector<float> f(half > 0 ? half : 1);
        for (int i = 0; i < half; ++i) f[i] = (float)pow((double)c.rot_base, -2.0 * i / (double)c.rot_dims);
        if (dev_alloc(e, &ly.inv_freq, f.size()) ||
            cudaMemcpy(ly.inv_freq, f.data(), f.size() * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) {
            set_error("asd_mezilix_create: device allocation failed");
            asd_mezilix_destroy(e);
            return nullptr;
        }
        nqd = std::max(nqd, (size_t)ly.nqd);
        qlat = std::max(qlat, (size_t)c.heads * ly.rw);
        olat = std::max(olat, (size_t)c.heads * c.kv_rank);
        hv = std::max(hv, (size_t)c.heads * c.vdim);
        E = std::max(E, (size_t)c.experts);
        top = std::max(top, (size_t)c.top);
        ff = std::max(ff, (size_t)c.ff);
        e->layers.push_back(ly);
    }
    int rc = 0;
    rc |= dev_alloc(e, &e->stack, (size_t)(cfg->n_layers + 1) * MT * D);
    rc |= dev_alloc(e, &e->xavg, MT * D);
    rc |= dev_alloc(e, &e->hn, MT * D);
    rc |= dev_alloc(e, &e->qd, MT * nqd);
    rc |= dev_alloc(e, &e->qlat, MT * qlat);
    rc |= dev_alloc(e, &e->olat, MT * olat);
    rc |= dev_alloc(e, &e->mix, MT * D);
    rc |= dev_alloc(e, &e->rlog, MT * E);
    rc |= dev_alloc(e, &e->gate, MT * top);
    rc |= dev_alloc(e, &e->eout, MT * top * D);
    rc |= dev_alloc(e, (char**)&e->h, MT * D * e->esz);
    rc |= dev_alloc(e, (char**)&e->hs, MT * D * e->esz);
    rc |= dev_alloc(e, (char**)&e->vout, MT * hv * e->esz);
    rc |= dev_alloc(e, (char**)&e->act, MT * top * ff * e->esz);
    rc |= dev_alloc(e, (char**)&e->xsel, MT * D * e->esz);
    rc |= dev_alloc(e, &e->expert_of, MT * top);
    rc |= dev_alloc(e, &e->counters, 2 * E + 1);
    rc |= dev_alloc(e, &e->group_off, E + 1);
    rc |= dev_alloc(e, &e->sorted_tok, MT * top);
    rc |= dev_alloc(e, &e->slot_of, MT * top);
    e->attn_ws.rows = 16384;
    e->attn_ws.o_elems = e->attn_ws.rows * 512;
    rc |= dev_alloc(e, &e->attn_ws.o, (size_t)e->attn_ws.o_elems);
    rc |= dev_alloc(e, &e->attn_ws.ml, (size_t)e->attn_ws.rows * 2);
    rc |= dev_alloc(e, &e->dev_error, 1);
    if (!rc && cudaMemset(e->dev_error, 0, sizeof(int)) != cudaSuccess) rc = -1;
    if (rc) {
        asd_mezilix_destroy(e);
        return nullptr;
    }
    return e;
}

void asd_mezilix_destroy(asd_mezilix_engine_t* h) {
    MzEngine* e = static_cast<MzEngine*>(h);
    if (!e) return;
    for (void* p : e->owned) cudaFree(p);
    delete e;
}

int asd_mezilix_set_globals(asd_mezilix_engine_t* h, const void* embed, const void* pair_table, const void* final_gain,
                            const void* head) {
    MzEngine* e = static_cast<MzEngine*>(h);
    if (!e || !embed || !pair_table || !final_gain || !head) return set_error("asd_mezilix_set_globals: NULL argument");
    e->embed = embed, e->pair_table = pair_table, e->final_gain = final_gain, e->head = head;
    e->dn.clear();
    return 0;
}

int asd_mezilix_set_layer(asd_mezilix_engine_t* h, int layer, const void* gain, const void* shift, const void* depth_coeff,
                          const void* wqd, const void* latent_gain, const void* wuk, const void* wuv, const void* wo,
                          const void* router, const void* w_up, const void* w_down) {
    MzEngine* e = static_cast<MzEngine*>(h);
    if (!e || layer < 0 || layer >= (int)e->layers.size()) return set_error("asd_mezilix_set_layer: bad layer");
    MzLayer& ly = e->layers[layer];
    if (!gain || !shift || !depth_coeff || !wqd || !latent_gain || !wuk || !wuv || !wo)
        return set_error("asd_mezilix_set_layer: NULL weight");
    if (ly.c.experts > 0 && (!router || !w_up || !w_down)) return set_error("asd_mezilix_set_layer: NULL expert weight");
    ly.gain = gain, ly.shift = shift, ly.coeff = depth_coeff, ly.wqd = wqd, ly.latent_gain = latent_gain, ly.wuk = wuk;
    ly.wuv = wuv, ly.wo = wo, ly.router = router, ly.w_up = w_up, ly.w_down = w_down;
    e->dn.clear();
    return 0;
}

size_t asd_mezilix_cache_bytes(const asd_mezilix_engine_t* h, int num_pages) {
    const MzEngine* e = static_cast<const MzEngine*>(h);
    if (!e) return 0;
    size_t n = 0;
    for (const MzLayer& ly : e->layers) n += (size_t)num_pages * e->c.page_size * ly.rw;
    return n * e->esz;
}

int asd_mezilix_set_cache(asd_mezilix_engine_t* h, void* pool, int num_pages, const int32_t* page_table, int max_seqs,
                          int max_pages_per_seq, int32_t* token_ring, float* shift_ring) {
    MzEngine* e = static_cast<MzEngine*>(h);
    if (!e || !pool || !page_table || !token_ring || !shift_ring || num_pages <= 0 || max_seqs <= 0 ||
        max_pages_per_seq <= 0)
        return set_error("asd_mezilix_set_cache: bad arguments");
    e->pool = static_cast<char*>(pool);
    e->num_pages = num_pages, e->page_table = page_table, e->max_seqs = max_seqs, e->max_pages = max_pages_per_seq;
    e->tok_ring = token_ring, e->shift_ring = shift_ring;
    size_t off = 0;
    for (MzLayer& ly : e->layers) {
        ly.cache_off = off;
        off += (size_t)num_pages * e->c.page_size * ly.rw;
    }
    return 0;
}

int asd_mezilix_set_option(asd_mezilix_engine_t* h, const char* name, int value) {
    MzEngine* e = static_cast<MzEngine*>(h);
    if (!e || !name) return set_error("asd_mezilix_set_option: NULL argument");
    if (!strcmp(name, "tc_linear")) {
        e->dn.tc_linear = value;
        return 0;
    }
    if (!strcmp(name, "tc_min_rows")) {
        e->dn.tc_min_rows = value > 0 ? value : 1 << 30;
        e->dn.clear();
        return 0;
    }
    if (!strcmp(name, "attn_tiled")) {
        e->attn_ws.tiled = value;
        return 0;
    }
    if (!strcmp(name, "profile")) {
        e->prof.on = value;
        e->prof.reset();
        return 0;
    }
    return set_error("asd_mezilix_set_option: unknown option %s", name);
}

int asd_mezilix_forward(asd_mezilix_engine_t* h, const int32_t* tokens, const int32_t* positions,
                        const int32_t* token_slot, int M, const int32_t* cu_q, const int32_t* seq_slot, int nseq,
                        int max_qlen, int max_kv_len, const int32_t* logit_rows, int n_logit_rows, float* logits_out,
                        long long logits_ld, float* layer_out, void* stream) {
    MzEngine* e = static_cast<MzEngine*>(h);
    if (!e) return set_error("asd_mezilix_forward: NULL engine");
    if (M <= 0 || M > e->c.max_tokens) return set_error("asd_mezilix_forward: M = %d outside 1..%d", M, e->c.max_tokens);
    if (!e->embed || !e->pool) return set_error("asd_mezilix_forward: weights or cache not set");
    for (const MzLayer& ly : e->layers)
        if (!ly.wqd) return set_error("asd_mezilix_forward: a layer has no weights");
    if (!tokens || !positions || !token_slot || !cu_q || !seq_slot || nseq <= 0 || max_qlen <= 0)
        return set_error("asd_mezilix_forward: bad index arguments");
    if (max_kv_len > e->max_pages * e->c.page_size)
        return set_error("asd_mezilix_forward: length bound %d exceeds the page table", max_kv_len);
    if (n_logit_rows > 0 && !logits_out) return set_error("asd_mezilix_forward: logits_out is NULL");
    if (n_logit_rows > e->c.max_tokens) return set_error("asd_mezilix_forward: too many logit rows");
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != e->device) return set_error("asd_mezilix_forward: called on device %d, engine lives on %d", dev, e->device);
    return forward(e, tokens, positions, token_slot, M, cu_q, seq_slot, nseq, max_qlen, max_kv_len, logit_rows,
                   logit_rows ? n_logit_rows : (n_logit_rows > 0 ? M : 0), logits_out, logits_ld, layer_out,
                   static_cast<cudaStream_t>(stream));
}

int asd_mezilix_profile_read(asd_mezilix_engine_t* h, float* ms_by_class, int* launches_by_class, int nclass) {
    MzEngine* e = static_cast<MzEngine*>(h);
    if (!e || !ms_by_class || nclass < MZ_NCLASS) return set_error("asd_mezilix_profile_read: bad argument");
    ASD_CUDA(e->prof.read(ms_by_class, launches_by_class, nclass));
    return 0;
}

int asd_mezilix_device_error(asd_mezilix_engine_t* h) {
    MzEngine* e = static_cast<MzEngine*>(h);
    if (!e) return set_error("asd_mezilix_device_error: NULL engine");
    int v = 0;
    ASD_CUDA(cudaMemcpy(&v, e->dev_error, sizeof(int), cudaMemcpyDeviceToHost));
    if (v) return set_error("a Mezilix kernel gave up a bounded wait (tcgen05 linear)");
    return 0;
}

int asd_linear_tc(const void* x, int x_f32, const void* w, void* y, int y_f32, int M, int N, int K, int Z,
                  const int32_t* group_off, const int32_t* gather, int relu_sq, int32_t* err_flag, void* stream) {
    SimtLinear L;
    L.a = x, L.a_f32 = x_f32, L.lda = K, L.a_zs = (long long)M * K;
    L.w = w, L.w_f32 = 0, L.ldw = K, L.w_zs = (long long)N * K;
    L.c = y, L.c_f32 = y_f32, L.ldc = N, L.c_zs = (long long)M * N;
    L.M = M, L.N = N, L.K = K, L.Z = Z, L.epilogue = relu_sq ? 1 : 0;
    L.group_off = group_off, L.gather = gather;
    return launch_tc_linear(L, err_flag, static_cast<cudaStream_t>(stream));
}

int asd_linear_simt(const void* x, int x_f32, const void* w, int w_f32, void* y, int y_f32, int M, int N, int K,
                    void* stream) {
    SimtLinear L;
    L.a = x, L.a_f32 = x_f32, L.lda = K;
    L.w = w, L.w_f32 = w_f32, L.ldw = K;
    L.c = y, L.c_f32 = y_f32, L.ldc = N;
    L.M = M, L.N = N, L.K = K;
    return launch_simt_linear(L, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
