// Rivetar family forward engine: one opaque handle per model.  asd_rivetar_forward runs, on the caller's stream and
// with no host synchronisation,
//   scaled embedding -> for every layer execution [ (pass entry: projection of [x | x0] + pass vector) norm, mixer,
//   close (norm after, residual, norm before the feed-forward), up projection, polynomial activation, down projection,
//   close ] -> final norm of the wanted rows, head, tanh cap.
// A layer's mixer is latent attention, gated linear attention or windowed attention; layers of a repeated span execute
// several times with the same weights and a cache or state per execution.  Every step is a building block of blocks.h
// that takes its sizes from the layer's configuration; dense bf16 projections go to the tcgen05 GEMMs when their
// shape fits (dense.h).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <string.h>

#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/asd_b200.h"
#include "asd_internal.h"
#include "blocks.h"
#include "dense.h"
#include "prof.h"

struct asd_rivetar_engine {};

namespace asd {

enum RvType { RV_LATENT = 0, RV_GLA = 1, RV_WINDOW = 2 };

struct RvLayer {
    asd_rivetar_layer_config c;
    std::unordered_map<std::string, const void*> t;   // weights by engine tensor name
    float* freq_k = nullptr;   // owned, [rot_dims / 2]
    float* freq_v = nullptr;   // owned, [vdim / 2] (windowed attention)
    int n_in = 0;              // rows of the stacked input projection
    int cache_row = 0;         // cached elements per position (0: none)
    size_t state_elems = 0;    // recurrent state per (sequence, ring entry)
    const void* w(const char* name) const {
        auto it = t.find(name);
        return it == t.end() ? nullptr : it->second;
    }
    const float* f(const char* name) const { return static_cast<const float*>(w(name)); }
};

struct RvRun {
    int layer, pass;           // pass -1: outside the repeated span
    bool enters;               // first layer of a pass
    size_t cache_off = 0;      // elements from the pool start
    size_t state_off = 0;      // floats from the state start
};

struct RvEngine : asd_rivetar_engine {
    asd_rivetar_config c;
    std::vector<RvLayer> layers;
    std::vector<RvRun> runs;
    std::unordered_map<std::string, const void*> g;   // global weights
    int f32 = 0, esz = 2;
    char* pool = nullptr;
    const int* page_table = nullptr;
    int num_pages = 0, max_seqs = 0, max_pages = 0;
    float* state = nullptr;
    // owned activations
    float *x = nullptr, *x0 = nullptr, *y = nullptr, *proj = nullptr, *qbuf = nullptr, *qlat = nullptr, *olat = nullptr,
          *alpha = nullptr, *orec = nullptr, *up = nullptr;
    void *hn = nullptr, *cq = nullptr, *mixed = nullptr, *act = nullptr, *xsel = nullptr;
    std::vector<void*> owned;
    DenseRunner dn;
    EventProfiler prof;
    AttnSplit attn_ws;
    int fused_attn = 1;
    int* dev_error = nullptr;
    int device = 0;
    const void* gw(const char* name) const {
        auto it = g.find(name);
        return it == g.end() ? nullptr : it->second;
    }
};

template <typename T>
static int dev_alloc(RvEngine* e, T** p, size_t n) {
    void* q = nullptr;
    ASD_CUDA(cudaMalloc(&q, (n ? n : 1) * sizeof(T)));
    e->owned.push_back(q);
    *p = (T*)q;
    return 0;
}

static int upload_freq(RvEngine* e, float** dst, int dims, double base) {
    const int half = dims / 2;
    std::vector<float> f(half > 0 ? half : 1, 0.f);
    for (int i = 0; i < half; ++i) f[i] = (float)pow(base, -2.0 * i / (double)dims);
    if (dev_alloc(e, dst, f.size())) return -1;
    ASD_CUDA(cudaMemcpy(*dst, f.data(), f.size() * sizeof(float), cudaMemcpyHostToDevice));
    return 0;
}

enum RvProf { RV_DENSE = 0, RV_HEADS, RV_LATENT_ATTN, RV_WINDOW_ATTN, RV_RECUR, RV_ACT, RV_GLUE, RV_HEAD, RV_NCLASS };
#define RV_PROF(cls) ProfRegion _region(e->prof, cls, s)

static int linear(RvEngine* e, const SimtLinear& L, cudaStream_t s) {
    if (!e->f32 && e->dn.tc_linear && tc_linear_supports(L)) return launch_tc_linear(L, e->dev_error, s);
    return launch_simt_linear(L, s);
}

struct Batch {
    SeqIndex ix;
    const int* cu_q;
    const int* seq_slot;
    int nseq, max_qlen, max_kv_len;
};

// mixer input hn [M][D] (engine type) -> y fp32 [M][D]
static int mix_latent(RvEngine* e, const RvLayer& ly, const RvRun& run, int li, const Batch& b, cudaStream_t s) {
    const asd_rivetar_layer_config& c = ly.c;
    const int M = b.ix.M, D = e->c.width, f32 = e->f32;
    const int nq = c.heads * (c.dim + c.rot_dim), rw = c.kv_rank + c.rot_dim;
    {   // query latent | cached latent | rotated key in one projection
        RV_PROF(RV_DENSE);
        if (e->dn.run(e->hn, ly.w("w_in"), e->proj, M, ly.n_in, D, ly.n_in, li * 16 + 0, s)) return -1;
    }
    {
        RV_PROF(RV_GLUE);
        if (launch_rms_rows(e->proj, ly.n_in, ly.f("q_norm"), 0, e->c.eps, e->cq, f32, c.q_rank, M, c.q_rank, s)) return -1;
    }
    {
        RV_PROF(RV_DENSE);
        if (e->dn.run(e->cq, ly.w("w_uq"), e->qbuf, M, nq, c.q_rank, nq, li * 16 + 1, s)) return -1;
    }
    LatentDims dm{c.heads, c.dim, c.rot_dim, c.vdim, c.kv_rank, c.rot_dims, c.window, c.scale};
    dm.interleaved = c.rot_interleaved;
    const PagedRows cache{e->pool + run.cache_off * e->esz, f32, e->page_table, e->max_pages, e->c.page_size};
    {
        RV_PROF(RV_GLUE);
        if (launch_latent_post_split(b.ix, e->qbuf, nq, e->proj + c.q_rank, ly.n_in, dm, ly.f("kv_norm"), 1, e->c.eps,
                                     ly.freq_k, cache, e->qlat, s))
            return -1;
    }
    {   // q_lat[m][h][r] = sum_d q[m][h][d] * WukT[h][r][d]
        RV_PROF(RV_HEADS);
        SimtLinear L;
        L.a = e->qbuf, L.a_f32 = 1, L.lda = nq, L.a_zs = c.dim + c.rot_dim;
        L.w = ly.w("w_uk"), L.w_f32 = f32, L.ldw = c.dim, L.w_zs = (long long)c.dim * c.kv_rank;
        L.c = e->qlat, L.c_f32 = 1, L.ldc = (long long)c.heads * rw, L.c_zs = rw;
        L.M = M, L.N = c.kv_rank, L.K = c.dim, L.Z = c.heads;
        if (linear(e, L, s)) return -1;
    }
    {
        RV_PROF(RV_LATENT_ATTN);
        if (launch_latent_attention(b.ix, b.cu_q, b.seq_slot, b.nseq, b.max_qlen, b.max_kv_len, e->qlat, dm, cache, e->olat,
                                    e->attn_ws, s))
            return -1;
    }
    {   // v[m][h][:] = Wuv[h] * out_lat[m][h][:]
        RV_PROF(RV_HEADS);
        SimtLinear L;
        L.a = e->olat, L.a_f32 = 1, L.lda = (long long)c.heads * c.kv_rank, L.a_zs = c.kv_rank;
        L.w = ly.w("w_uv"), L.w_f32 = f32, L.ldw = c.kv_rank, L.w_zs = (long long)c.vdim * c.kv_rank;
        L.c = e->mixed, L.c_f32 = f32, L.ldc = (long long)c.heads * c.vdim, L.c_zs = c.vdim;
        L.M = M, L.N = c.vdim, L.K = c.kv_rank, L.Z = c.heads;
        if (linear(e, L, s)) return -1;
    }
    return 0;
}

static int mix_gla(RvEngine* e, const RvLayer& ly, const RvRun& run, int li, const Batch& b, cudaStream_t s) {
    const asd_rivetar_layer_config& c = ly.c;
    const int M = b.ix.M, D = e->c.width, f32 = e->f32;
    const int nk = c.heads * c.dim, nv = c.heads * c.vdim;
    {   // q | k | v | gate | decay-in in one projection
        RV_PROF(RV_DENSE);
        if (e->dn.run(e->hn, ly.w("w_in"), e->proj, M, ly.n_in, D, ly.n_in, li * 16 + 0, s)) return -1;
    }
    const GlaDims gd{c.heads, c.dim, c.vdim, c.decay_rank, c.tau, 1.f / sqrtf((float)c.dim)};
    {
        RV_PROF(RV_GLUE);
        if (launch_gla_decay(e->proj + 2 * nk + 2 * nv, ly.n_in, ly.f("w_decay"), ly.f("b_decay"), gd, e->alpha, M, s))
            return -1;
    }
    {
        RV_PROF(RV_RECUR);
        if (launch_gla_recurrence(b.ix, b.cu_q, b.seq_slot, b.nseq, e->proj, e->proj + nk, e->proj + 2 * nk, ly.n_in,
                                  e->alpha, gd, e->state + run.state_off, e->c.ring, e->orec, s))
            return -1;
    }
    RV_PROF(RV_GLUE);
    return launch_gla_out(e->orec, e->proj + 2 * nk + nv, ly.n_in, ly.f("out_norm"), e->c.eps, e->mixed, f32, M, c.heads,
                          c.vdim, s);
}

static int mix_window(RvEngine* e, const RvLayer& ly, const RvRun& run, int li, const Batch& b, cudaStream_t s) {
    const asd_rivetar_layer_config& c = ly.c;
    const int M = b.ix.M, D = e->c.width, f32 = e->f32;
    {
        RV_PROF(RV_DENSE);
        if (e->dn.run(e->hn, ly.w("w_in"), e->proj, M, ly.n_in, D, ly.n_in, li * 16 + 0, s)) return -1;
    }
    const WindowDims wd{c.heads, c.kv_heads, c.dim, c.vdim, c.rot_dims, c.rot_interleaved, c.window, c.keep_first, c.scale};
    const PagedRows cache{e->pool + run.cache_off * e->esz, f32, e->page_table, e->max_pages, e->c.page_size};
    {
        RV_PROF(RV_GLUE);
        if (launch_window_post(b.ix, e->proj, ly.n_in, wd, ly.freq_k, ly.freq_v, cache, s)) return -1;
    }
    RV_PROF(RV_WINDOW_ATTN);
    return launch_window_attention(b.ix, b.cu_q, b.seq_slot, b.nseq, b.max_qlen, b.max_kv_len, e->proj, ly.n_in, wd,
                                   ly.f("sink"), ly.freq_v, cache, e->mixed, f32, e->fused_attn, e->attn_ws, s);
}

static int forward(RvEngine* e, const Batch& b, const int* logit_rows, int n_rows, float* logits, long long ld,
                   float* layer_out, cudaStream_t s) {
    const int D = e->c.width, M = b.ix.M, f32 = e->f32;
    const float eps = e->c.eps;
    const int nruns = (int)e->runs.size();
    {
        RV_PROF(RV_GLUE);
        if (launch_embed_scaled(b.ix, e->gw("embed"), f32, e->c.embed_scale, e->x0, e->x, D, s)) return -1;
    }
    // hn holds what the next dense projection reads: the next layer's first norm, or [x | x0] before a pass entry
    auto open_next = [&](int r, RowClose& C) {
        if (r >= nruns) return;   // the final norm runs on the wanted rows only
        if (e->runs[r].enters)
            C.cat = e->x0;
        else
            C.next_w = e->layers[e->runs[r].layer].f("norm1");
        C.hn = e->hn, C.hn_f32 = f32;
    };
    if (nruns) {
        RV_PROF(RV_GLUE);
        RowClose C;
        C.x_in = e->x, C.eps = eps, C.M = M, C.D = D;
        open_next(0, C);
        if (launch_row_close(C, s)) return -1;
    }
    for (int r = 0; r < nruns; ++r) {
        const RvRun& run = e->runs[r];
        const RvLayer& ly = e->layers[run.layer];
        const asd_rivetar_layer_config& c = ly.c;
        const int li = run.layer;
        if (run.enters) {   // x <- W [x | x0] + step[pass], then this layer's first norm
            {
                RV_PROF(RV_DENSE);
                if (e->dn.run(e->hn, e->gw("loop_in"), e->y, M, D, 2 * D, D, (int)e->layers.size() * 16 + 1, s)) return -1;
            }
            RV_PROF(RV_GLUE);
            RowClose C;
            C.y = e->y, C.bias = static_cast<const float*>(e->gw("loop_step")) + (size_t)run.pass * D;
            C.x_out = e->x, C.next_w = ly.f("norm1"), C.hn = e->hn, C.hn_f32 = f32, C.eps = eps, C.M = M, C.D = D;
            if (launch_row_close(C, s)) return -1;
        }
        int rc = 0;
        if (c.type == RV_LATENT)
            rc = mix_latent(e, ly, run, li, b, s);
        else if (c.type == RV_GLA)
            rc = mix_gla(e, ly, run, li, b, s);
        else
            rc = mix_window(e, ly, run, li, b, s);
        if (rc) return -1;
        {
            RV_PROF(RV_DENSE);
            if (e->dn.run(e->mixed, ly.w("w_o"), e->y, M, D, c.heads * c.vdim, D, li * 16 + 2, s)) return -1;
        }
        {   // x += norm1b(y); then the feed-forward's norm, or what the next execution reads
            RV_PROF(RV_GLUE);
            RowClose C;
            C.x_in = e->x, C.y = e->y, C.post_w = ly.f("norm1b"), C.x_out = e->x, C.eps = eps, C.M = M, C.D = D;
            if (c.ff > 0)
                C.next_w = ly.f("norm2"), C.hn = e->hn, C.hn_f32 = f32;
            else
                open_next(r + 1, C);
            if (launch_row_close(C, s)) return -1;
        }
        if (c.ff > 0) {
            {
                RV_PROF(RV_DENSE);
                if (e->dn.run(e->hn, ly.w("w_up"), e->up, M, c.ff, D, c.ff, li * 16 + 3, s)) return -1;
            }
            {
                RV_PROF(RV_ACT);
                if (launch_polynorm(e->up, ly.f("act"), eps, e->act, f32, M, c.ff, s)) return -1;
            }
            {
                RV_PROF(RV_DENSE);
                if (e->dn.run(e->act, ly.w("w_down"), e->y, M, D, c.ff, D, li * 16 + 4, s)) return -1;
            }
            RV_PROF(RV_GLUE);
            RowClose C;
            C.x_in = e->x, C.y = e->y, C.post_w = ly.f("norm2b"), C.x_out = e->x, C.eps = eps, C.M = M, C.D = D;
            open_next(r + 1, C);
            if (launch_row_close(C, s)) return -1;
        }
        if (layer_out)
            ASD_CUDA(cudaMemcpyAsync(layer_out + (size_t)r * M * D, e->x, sizeof(float) * M * D, cudaMemcpyDeviceToDevice, s));
    }
    if (n_rows > 0) {
        RV_PROF(RV_HEAD);
        RowClose C;
        C.x_in = e->x, C.rows = logit_rows, C.next_w = static_cast<const float*>(e->gw("final_norm"));
        C.hn = e->xsel, C.hn_f32 = f32, C.eps = eps, C.M = n_rows, C.D = D;
        if (launch_row_close(C, s)) return -1;
        const int V = e->c.vocab;
        const int ldl = ld ? (int)ld : V;
        if (e->dn.run(e->xsel, e->gw("head"), logits, n_rows, V, D, ldl, (int)e->layers.size() * 16 + 2, s)) return -1;
        if (launch_softcap(logits, ldl, n_rows, V, e->c.logit_softcap, s)) return -1;
    }
    return 0;
}

// elements one execution's rows take in the pool, rounded up so that every execution starts on a 16-byte boundary
static size_t pool_elems(const RvEngine* e, const RvRun& r, int num_pages) {
    const size_t n = (size_t)num_pages * e->c.page_size * e->layers[r.layer].cache_row;
    return (n + 7) & ~(size_t)7;
}

static const char* const kLayerNames[] = {"norm1", "norm1b", "norm2", "norm2b", "w_up", "w_down", "act", "w_o", "w_in",
                                          "q_norm", "kv_norm", "w_uq", "w_uk", "w_uv", "w_decay", "b_decay", "out_norm",
                                          "sink"};
static const char* const kGlobalNames[] = {"embed", "final_norm", "head", "loop_in", "loop_step"};

static std::vector<const char*> required(const RvEngine* e, const RvLayer& ly) {
    std::vector<const char*> n = {"norm1", "norm1b", "w_in", "w_o"};
    if (ly.c.ff > 0) n.insert(n.end(), {"norm2", "norm2b", "w_up", "w_down", "act"});
    if (ly.c.type == RV_LATENT) n.insert(n.end(), {"q_norm", "kv_norm", "w_uq", "w_uk", "w_uv"});
    if (ly.c.type == RV_GLA) n.insert(n.end(), {"w_decay", "b_decay", "out_norm"});
    (void)e;
    return n;
}

}  // namespace asd

using namespace asd;

extern "C" {

asd_rivetar_engine_t* asd_rivetar_create(const asd_rivetar_config* cfg, const asd_rivetar_layer_config* layers) {
    if (!cfg || (cfg->n_layers > 0 && !layers)) {
        set_error("asd_rivetar_create: NULL config");
        return nullptr;
    }
    if (cfg->width <= 0 || cfg->vocab <= 0 || cfg->n_layers < 0 || cfg->max_tokens <= 0 || cfg->page_size <= 0 ||
        cfg->ring <= 0 || (cfg->dtype != 0 && cfg->dtype != 1) || cfg->loop_times < 0 ||
        (cfg->loop_times > 0 && !(0 <= cfg->loop_start && cfg->loop_start < cfg->loop_stop && cfg->loop_stop <= cfg->n_layers))) {
        set_error("asd_rivetar_create: bad sizes");
        return nullptr;
    }
    RvEngine* e = new RvEngine();
    e->c = *cfg;
    e->f32 = e->dn.f32 = cfg->dtype;
    e->esz = cfg->dtype ? 4 : 2;
    cudaGetDevice(&e->device);
    const size_t MT = cfg->max_tokens, D = cfg->width;
    size_t n_in = 1, nq = 1, qlat = 1, olat = 1, hv = 1, qr = 1, nk = 1, ff = 1;
    auto fail = [&](const char* what, int l) {
        set_error("asd_rivetar_create: %s (layer %d)", what, l);
        asd_rivetar_destroy(e);
        return nullptr;
    };
    for (int l = 0; l < cfg->n_layers; ++l) {
        RvLayer ly;
        ly.c = layers[l];
        const auto& c = ly.c;
        if (c.type < 0 || c.type > 2 || c.heads <= 0 || c.dim <= 0 || c.vdim <= 0 || c.ff < 0)
            return fail("bad sizes", l);
        if (c.type == RV_LATENT) {
            if (c.rot_dim < 0 || c.kv_rank <= 0 || c.q_rank <= 0 || c.rot_dims < 0 || c.rot_dims > c.rot_dim ||
                (c.rot_dims & 1) || c.window <= 0)
                return fail("bad latent attention sizes", l);
            ly.n_in = c.q_rank + c.kv_rank + c.rot_dim;
            ly.cache_row = c.kv_rank + c.rot_dim;
            nq = std::max(nq, (size_t)c.heads * (c.dim + c.rot_dim));
            qlat = std::max(qlat, (size_t)c.heads * ly.cache_row);
            olat = std::max(olat, (size_t)c.heads * c.kv_rank);
            qr = std::max(qr, (size_t)c.q_rank);
            if (upload_freq(e, &ly.freq_k, c.rot_dims, c.rot_base)) return fail("device allocation failed", l);
        } else if (c.type == RV_GLA) {
            if (c.decay_rank <= 0 || !(c.tau > 0.f)) return fail("bad gated linear attention sizes", l);
            ly.n_in = 2 * c.heads * c.dim + 2 * c.heads * c.vdim + c.decay_rank;
            ly.state_elems = (size_t)c.heads * c.dim * c.vdim;
            nk = std::max(nk, (size_t)c.heads * c.dim);
        } else {
            if (c.kv_heads <= 0 || c.heads % c.kv_heads || (c.vdim & 1) || c.rot_dims < 0 || c.rot_dims > c.dim ||
                (c.rot_dims & 1) || c.window <= 0 || c.keep_first < 0)
                return fail("bad windowed attention sizes", l);
            ly.n_in = c.heads * c.dim + c.kv_heads * (c.dim + c.vdim);
            ly.cache_row = c.kv_heads * (c.dim + c.vdim);
            if (upload_freq(e, &ly.freq_k, c.rot_dims, c.rot_base) || upload_freq(e, &ly.freq_v, c.vdim, c.rot_base))
                return fail("device allocation failed", l);
        }
        n_in = std::max(n_in, (size_t)ly.n_in);
        hv = std::max(hv, (size_t)c.heads * c.vdim);
        ff = std::max(ff, (size_t)c.ff);
        e->layers.push_back(ly);
    }
    // executions in order
    auto add = [&](int l, int pass, bool enters) { e->runs.push_back(RvRun{l, pass, enters}); };
    if (cfg->loop_times == 0) {
        for (int l = 0; l < cfg->n_layers; ++l) add(l, -1, false);
    } else {
        for (int l = 0; l < cfg->loop_start; ++l) add(l, -1, false);
        for (int t = 0; t < cfg->loop_times; ++t)
            for (int l = cfg->loop_start; l < cfg->loop_stop; ++l) add(l, t, l == cfg->loop_start);
        for (int l = cfg->loop_stop; l < cfg->n_layers; ++l) add(l, -1, false);
    }
    int rc = 0;
    rc |= dev_alloc(e, &e->x, MT * D);
    rc |= dev_alloc(e, &e->x0, MT * D);
    rc |= dev_alloc(e, &e->y, MT * D);
    rc |= dev_alloc(e, &e->proj, MT * n_in);
    rc |= dev_alloc(e, &e->qbuf, MT * nq);
    rc |= dev_alloc(e, &e->qlat, MT * qlat);
    rc |= dev_alloc(e, &e->olat, MT * olat);
    rc |= dev_alloc(e, &e->alpha, MT * nk);
    rc |= dev_alloc(e, &e->orec, MT * hv);
    rc |= dev_alloc(e, &e->up, MT * ff);
    rc |= dev_alloc(e, (char**)&e->hn, MT * 2 * D * e->esz);
    rc |= dev_alloc(e, (char**)&e->cq, MT * qr * e->esz);
    rc |= dev_alloc(e, (char**)&e->mixed, MT * hv * e->esz);
    rc |= dev_alloc(e, (char**)&e->act, MT * ff * e->esz);
    rc |= dev_alloc(e, (char**)&e->xsel, MT * D * e->esz);
    e->attn_ws.rows = 16384;
    e->attn_ws.o_elems = e->attn_ws.rows * 512;
    rc |= dev_alloc(e, &e->attn_ws.o, (size_t)e->attn_ws.o_elems);
    rc |= dev_alloc(e, &e->attn_ws.ml, (size_t)e->attn_ws.rows * 2);
    rc |= dev_alloc(e, &e->dev_error, 1);
    if (!rc && cudaMemset(e->dev_error, 0, sizeof(int)) != cudaSuccess) rc = -1;
    if (rc) {
        asd_rivetar_destroy(e);
        return nullptr;
    }
    return e;
}

void asd_rivetar_destroy(asd_rivetar_engine_t* h) {
    RvEngine* e = static_cast<RvEngine*>(h);
    if (!e) return;
    for (void* p : e->owned) cudaFree(p);
    delete e;
}

int asd_rivetar_set_tensor(asd_rivetar_engine_t* h, int layer, const char* name, const void* data) {
    RvEngine* e = static_cast<RvEngine*>(h);
    if (!e || !name || !data) return set_error("asd_rivetar_set_tensor: NULL argument");
    if (layer >= (int)e->layers.size() || layer < -1) return set_error("asd_rivetar_set_tensor: bad layer %d", layer);
    bool known = false;
    if (layer < 0) {
        for (const char* n : kGlobalNames) known |= !strcmp(n, name);
        if (known) e->g[name] = data;
    } else {
        for (const char* n : kLayerNames) known |= !strcmp(n, name);
        if (known) e->layers[layer].t[name] = data;
    }
    if (!known) return set_error("asd_rivetar_set_tensor: unknown tensor %s (layer %d)", name, layer);
    e->dn.clear();
    return 0;
}

size_t asd_rivetar_cache_bytes(const asd_rivetar_engine_t* h, int num_pages) {
    const RvEngine* e = static_cast<const RvEngine*>(h);
    if (!e) return 0;
    size_t n = 0;
    for (const RvRun& r : e->runs) n += pool_elems(e, r, num_pages);
    return n * e->esz;
}

size_t asd_rivetar_state_bytes(const asd_rivetar_engine_t* h, int max_seqs) {
    const RvEngine* e = static_cast<const RvEngine*>(h);
    if (!e) return 0;
    size_t n = 0;
    for (const RvRun& r : e->runs) n += (size_t)max_seqs * e->c.ring * e->layers[r.layer].state_elems;
    return n * sizeof(float);
}

int asd_rivetar_set_cache(asd_rivetar_engine_t* h, void* pool, int num_pages, const int32_t* page_table, int max_seqs,
                          int max_pages_per_seq, float* state) {
    RvEngine* e = static_cast<RvEngine*>(h);
    if (!e || !pool || !page_table || !state || num_pages <= 0 || max_seqs <= 0 || max_pages_per_seq <= 0)
        return set_error("asd_rivetar_set_cache: bad arguments");
    e->pool = static_cast<char*>(pool);
    e->num_pages = num_pages, e->page_table = page_table, e->max_seqs = max_seqs, e->max_pages = max_pages_per_seq;
    e->state = state;
    size_t off = 0, soff = 0;
    for (RvRun& r : e->runs) {
        r.cache_off = off;
        r.state_off = soff;
        off += pool_elems(e, r, num_pages);
        soff += (size_t)max_seqs * e->c.ring * e->layers[r.layer].state_elems;
    }
    return 0;
}

int asd_rivetar_set_option(asd_rivetar_engine_t* h, const char* name, int value) {
    RvEngine* e = static_cast<RvEngine*>(h);
    if (!e || !name) return set_error("asd_rivetar_set_option: NULL argument");
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
    if (!strcmp(name, "fused_attn")) {
        e->fused_attn = value;
        return 0;
    }
    if (!strcmp(name, "profile")) {
        e->prof.on = value;
        e->prof.reset();
        return 0;
    }
    return set_error("asd_rivetar_set_option: unknown option %s", name);
}

int asd_rivetar_forward(asd_rivetar_engine_t* h, const int32_t* tokens, const int32_t* positions,
                        const int32_t* token_slot, int M, const int32_t* cu_q, const int32_t* seq_slot, int nseq,
                        int max_qlen, int max_kv_len, const int32_t* logit_rows, int n_logit_rows, float* logits_out,
                        long long logits_ld, float* layer_out, void* stream) {
    RvEngine* e = static_cast<RvEngine*>(h);
    if (!e) return set_error("asd_rivetar_forward: NULL engine");
    if (M <= 0 || M > e->c.max_tokens) return set_error("asd_rivetar_forward: M = %d outside 1..%d", M, e->c.max_tokens);
    if (!e->pool) return set_error("asd_rivetar_forward: cache not set");
    for (const char* n : {"embed", "final_norm", "head"})
        if (!e->gw(n)) return set_error("asd_rivetar_forward: tensor %s not set", n);
    if (e->c.loop_times > 0 && (!e->gw("loop_in") || !e->gw("loop_step")))
        return set_error("asd_rivetar_forward: the repeated span's tensors are not set");
    for (size_t l = 0; l < e->layers.size(); ++l)
        for (const char* n : required(e, e->layers[l]))
            if (!e->layers[l].w(n)) return set_error("asd_rivetar_forward: layer %d has no tensor %s", (int)l, n);
    if (!tokens || !positions || !token_slot || !cu_q || !seq_slot || nseq <= 0 || max_qlen <= 0)
        return set_error("asd_rivetar_forward: bad index arguments");
    if (max_kv_len > e->max_pages * e->c.page_size)
        return set_error("asd_rivetar_forward: length bound %d exceeds the page table", max_kv_len);
    if (n_logit_rows > 0 && !logits_out) return set_error("asd_rivetar_forward: logits_out is NULL");
    if (n_logit_rows > e->c.max_tokens) return set_error("asd_rivetar_forward: too many logit rows");
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != e->device) return set_error("asd_rivetar_forward: called on device %d, engine lives on %d", dev, e->device);
    const Batch b{SeqIndex{tokens, positions, token_slot, M}, cu_q, seq_slot, nseq, max_qlen, max_kv_len};
    return forward(e, b, logit_rows, logit_rows ? n_logit_rows : (n_logit_rows > 0 ? M : 0), logits_out, logits_ld,
                   layer_out, static_cast<cudaStream_t>(stream));
}

int asd_rivetar_profile_read(asd_rivetar_engine_t* h, float* ms_by_class, int* launches_by_class, int nclass) {
    RvEngine* e = static_cast<RvEngine*>(h);
    if (!e || !ms_by_class || nclass < RV_NCLASS) return set_error("asd_rivetar_profile_read: bad argument");
    ASD_CUDA(e->prof.read(ms_by_class, launches_by_class, nclass));
    return 0;
}

int asd_rivetar_device_error(asd_rivetar_engine_t* h) {
    RvEngine* e = static_cast<RvEngine*>(h);
    if (!e) return set_error("asd_rivetar_device_error: NULL engine");
    int v = 0;
    ASD_CUDA(cudaMemcpy(&v, e->dev_error, sizeof(int), cudaMemcpyDeviceToHost));
    if (v) return set_error("a Rivetar kernel gave up a bounded wait (tcgen05 linear)");
    return 0;
}

}  // extern "C"
