// Fazolorn.cpp -- config parsing, construction and the per-layer step of the Fazolorn stack (see Fazolorn.hpp).
#include "Fazolorn.hpp"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <stdexcept>

namespace koifish {

#define KF_TRY(expr)                                                                       \
    do {                                                                                   \
        int _rc = (expr);                                                                  \
        if (_rc != KF_OK) {                                                                \
            *hFishErr = std::string(#expr) + " -> " + kf_status_string(_rc);               \
            return _rc;                                                                    \
        }                                                                                  \
    } while (0)

// ------------------------------------------------------------------------------------------------------------ config
static int need_int(const JSON& j, const char* key, const std::string& where) {
    const JSON* p = j.find(key);
    if (!p || !p->is_number()) throw std::runtime_error("config: " + where + "." + key + " is missing");
    return p->as_int();
}
static double need_num(const JSON& j, const char* key, const std::string& where) {
    const JSON* p = j.find(key);
    if (!p || !p->is_number()) throw std::runtime_error("config: " + where + "." + key + " is missing");
    return p->as_double(0.0);
}
static const JSON* present(const JSON& j, const char* key) {  // the value of a key that is there and not null
    const JSON* p = j.find(key);
    return (p && !p->is_null()) ? p : nullptr;
}
// "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}; dims defaults to dflt_dims
static void parse_rot(const JSON& x, MIXER_CARD& m, int dflt_dims, int most, const std::string& where) {
    m.rot_dims = 0;
    const JSON* t = present(x, "rot");
    if (!t) return;
    m.rot_dims = present(*t, "dims") ? need_int(*t, "dims", where + ".rot") : dflt_dims;
    m.rot_base = need_num(*t, "base", where + ".rot");
    if (const JSON* s = present(*t, "scaling")) {
        const std::string ws = where + ".rot.scaling";
        m.yarn_factor = need_num(*s, "factor", ws), m.yarn_original = need_num(*s, "original", ws);
        m.yarn_fast = need_num(*s, "fast", ws), m.yarn_slow = need_num(*s, "slow", ws);
        if (!(m.yarn_factor > 0.0) || !(m.yarn_original > 0.0) || !(m.yarn_fast > 0.0) || !(m.yarn_slow > 0.0))
            throw std::runtime_error("config: " + ws + ": factor, original, fast, slow must be positive");
    }
    if (m.rot_dims < 0 || m.rot_dims > most || m.rot_dims % 2 || (m.rot_dims > 0 && !(m.rot_base > 0.0)))
        throw std::runtime_error("config: " + where + ".rot: dims must be even and at most " + std::to_string(most) + ", base positive");
}

// config.json: {"architecture": "Fazolorn", "vocab", "width", "norm": {"eps"}, "logit_scale", "loop": {"start", "stop", "times"},
//   "layers": [{"type": "mingru", "mixer": {"width"}} |
//              {"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}, "rot": {"base", "dims"}}} |
//              {"type": "latent_attention", "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot": {..., "scaling"}}},
//              each with "mlp": null | {"kind": "dense", "ff", "limit"} |
//                               {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale", "groups": {"count", "keep"}}}]}
// Keys that may be left out or null: loop (every layer runs once), logit_scale (1), kv_heads (= heads), vdim of "attention" (= dim), scale
// (1 / sqrt of the query size), mask (every earlier position), rot (no rotation), rot.dims, rot.scaling, router.scale (1), router.groups (one).
static void ParseFazolorn(const JSON& h, MODEL_CARD& c) {
    c.vocab        = need_int(h, "vocab", "config");
    c.n_embd       = need_int(h, "width", "config");
    c.norm_rms_eps = (float)need_num(h.at("norm"), "eps", "norm");
    c.norm_groups  = 1;
    if (const JSON* s = present(h, "logit_scale")) c.logit_scale = (float)s->as_double(1.0);
    const JSON& ls = h.at("layers");
    if (!ls.is_array() || ls.arr.empty()) throw std::runtime_error("config: layers must be a non-empty list");
    const JSON* shapes = h.find("tensor_shapes");
    for (size_t i = 0; i < ls.arr.size(); i++) {
        const JSON& l = ls.arr[i];
        const std::string where = "layers[" + std::to_string(i) + "]", wm = where + ".mixer";
        LAYER_CARD lc;
        MIXER_CARD& m = lc.mixer;
        m.type        = l.at("type").as_string();
        const JSON& x = l.at("mixer");
        if (m.type == "mingru") {
            m.width = need_int(x, "width", wm);
            if (m.width < 1) throw std::runtime_error("config: " + wm + ".width must be positive");
        } else if (m.type == "attention") {
            m.heads = need_int(x, "heads", wm), m.kv_heads = present(x, "kv_heads") ? need_int(x, "kv_heads", wm) : m.heads;
            m.dim = need_int(x, "dim", wm), m.vdim = present(x, "vdim") ? need_int(x, "vdim", wm) : m.dim;
            m.scale = present(x, "scale") ? (float)need_num(x, "scale", wm) : 1.0f / std::sqrt((float)m.dim);
            if (const JSON* k = present(x, "mask")) m.block = need_int(*k, "size", wm + ".mask");
            if (m.heads < 1 || m.kv_heads < 1 || m.heads % m.kv_heads || m.dim < 1 || m.dim > 512 || m.block < 0)
                throw std::runtime_error("config: " + wm + ": kv_heads must divide heads, 1 <= dim <= 512, mask.size >= 0");
            if (m.vdim != m.dim) throw std::runtime_error("config: " + wm + ": v is the un-rotated k, so vdim must equal dim");
            parse_rot(x, m, m.dim, m.dim, wm);
        } else if (m.type == "latent_attention") {
            m.heads = need_int(x, "heads", wm), m.dim = need_int(x, "dim", wm), m.rot_dim = need_int(x, "rot_dim", wm);
            m.vdim = need_int(x, "vdim", wm), m.kv_rank = need_int(x, "kv_rank", wm);
            if (present(x, "q_rank")) m.q_rank = need_int(x, "q_rank", wm);
            else if (shapes)  // the latent's size from the checkpoint's tensor shapes
                if (const JSON* t = shapes->find("l" + std::to_string(i) + ".mix.dq"))
                    if (t->is_array() && !t->arr.empty()) m.q_rank = t->arr[0].as_int();
            m.scale = present(x, "scale") ? (float)need_num(x, "scale", wm) : 1.0f / std::sqrt((float)(m.dim + m.rot_dim));
            if (m.heads < 1 || m.dim < 1 || m.rot_dim < 0 || m.vdim < 1 || m.kv_rank < 1 || m.q_rank < 1 || m.kv_rank + m.rot_dim > 640)
                throw std::runtime_error("config: " + wm + ": heads, dim, vdim, kv_rank, q_rank must be positive and kv_rank + rot_dim <= 640");
            parse_rot(x, m, m.rot_dim, m.rot_dim, wm);
        } else {
            throw std::runtime_error("config: " + where + ": unknown mixer type '" + m.type + "'");
        }
        if (const JSON* f = present(l, "mlp")) {
            const std::string kind = f->at("kind").as_string(), wf = where + ".mlp";
            MOE_CARD& e = lc.mlp;
            e.present = true;
            if (kind == "dense") {
                e.dense = true, e.ff = need_int(*f, "ff", wf), e.limit = (float)need_num(*f, "limit", wf);
                if (e.ff < 1 || !(e.limit > 0.f)) throw std::runtime_error("config: " + wf + ": ff and limit must be positive");
            } else if (kind == "moe") {
                const JSON& r = f->at("router");
                e.sigmoid_route = true;
                e.experts = need_int(r, "experts", wf + ".router"), e.top = need_int(r, "top", wf + ".router");
                e.ff = need_int(f->at("expert"), "ff", wf + ".expert");
                e.route_scale = present(r, "scale") ? (float)need_num(r, "scale", wf + ".router") : 1.f;
                if (const JSON* g = present(r, "groups"))
                    e.groups = need_int(*g, "count", wf + ".router.groups"), e.keep = need_int(*g, "keep", wf + ".router.groups");
                if (e.experts < 1 || e.ff < 1 || e.groups < 1 || e.groups > 32 || e.experts % e.groups || e.keep < 1 || e.keep > e.groups || e.top < 1 ||
                    e.top > e.keep * (e.experts / e.groups))
                    throw std::runtime_error("config: " + wf + ".router: groups.count (<= 32) must divide experts, 1 <= keep <= count, 1 <= top <= keep * experts / count");
            } else {
                throw std::runtime_error("config: " + wf + ".kind '" + kind + "' is not built");
            }
        }
        c.layers.push_back(lc);
    }
    c.n_layers = (int)c.layers.size();
    c.loop_start = c.loop_stop = 0, c.loop_times = 1;
    if (const JSON* lp = present(h, "loop")) {
        c.loop_start = need_int(*lp, "start", "loop"), c.loop_stop = need_int(*lp, "stop", "loop"), c.loop_times = need_int(*lp, "times", "loop");
        if (c.loop_start < 0 || c.loop_stop <= c.loop_start || c.loop_stop > c.n_layers || c.loop_times < 1)
            throw std::runtime_error("config: loop: 0 <= start < stop <= layers, times >= 1");
    }
    if (c.vocab < 1 || c.n_embd < 1) throw std::runtime_error("config: vocab, width must be positive");
    c.n_head = c.n_head_kv = 1, c.head_dim = c.n_embd, c.n_ff = 0, c.tie_word_embeddings = false;
}

std::vector<LayerRun> LayerRuns(const MODEL_CARD& c) {
    std::vector<LayerRun> r;
    const int L = (int)c.layers.size();
    const bool loop = c.loop_stop > c.loop_start;
    for (int i = 0; i < (loop ? c.loop_start : L); i++) r.push_back({i, (int)r.size(), -1});
    if (loop) {
        for (int t = 0; t < c.loop_times; t++)
            for (int i = c.loop_start; i < c.loop_stop; i++) r.push_back({i, (int)r.size(), i == c.loop_start ? t : -1});
        for (int i = c.loop_stop; i < L; i++) r.push_back({i, (int)r.size(), -1});
    }
    return r;
}

// ------------------------------------------------------------------------------------------------------------ build
namespace {
struct Builder {
    Fish& f;
    int next_id = 0;
    void Tensor(const std::string& name, int rows, int cols, hGTensor& out) {
        out = std::make_shared<GTensor>(f.ctx, name, rows, cols);  // bf16 as stored
        f.tensors[name]    = out;
        f.tensor_ids[name] = next_id++;
    }
    template <typename T>
    int Buf(T** p, size_t bytes) {
        void* d = nullptr;
        int rc  = kf_malloc(f.ctx, std::max<size_t>(bytes, 16), &d);
        if (rc) return rc;
        f.owned.push_back(d);
        *p = (T*)d;
        return KF_OK;
    }
};
struct FzlExtra : GeNeuron {  // tensors of the model that belong to no layer
    hGTensor step;            // [loop_times][width]: added before every pass of the repeated layers
};
}  // namespace

static int BuildFazolorn(Fish& f) {
    std::string* hFishErr = &f.error;
    const MODEL_CARD& c   = f.config;
    if (f.tp_world != 1) {
        f.error = "the Fazolorn stack runs on one GPU (no tensor-parallel shard plan)";
        return KF_ERR_UNSUPPORTED;
    }
    Builder b{f};
    const int E = c.n_embd, L = (int)c.layers.size();
    const bool f32   = c.compute_f32;
    const size_t asz = f32 ? 4 : 2;
    f.embed.hFish = &f, f.embed.name = "embed";
    b.Tensor("embed", c.vocab, E, f.embed.w);
    f.cls.hFish = &f, f.cls.name = "head";
    f.cls.norm.hFish = &f, f.cls.norm.rms_eps = c.norm_rms_eps;
    b.Tensor("final.norm", 1, E, f.cls.norm.w);
    f.cls.proj.hFish = &f, f.cls.proj.nIn = E, f.cls.proj.nOut = c.vocab;
    b.Tensor("head", c.vocab, E, f.cls.proj.w);

    f.max_tokens = std::max(std::max(64, c.max_batch), c.max_prefill);
    f.logit_rows = c.logit_rows_cfg > 0 ? std::min(c.logit_rows_cfg, f.max_tokens) : std::max(64, c.max_batch);
    const size_t T = f.max_tokens;
    auto hs    = std::make_shared<HybridScratch>();
    f.hscratch = hs;
    size_t maxU = 1, maxV = 1, maxY = 1, maxL = 1, maxA = 1, maxMid = 1, maxE = 1, maxTop = 1, maxFF = 1, maxH1 = 1;
    for (int i = 0; i < L; i++) {
        const LAYER_CARD& lc = c.layers[i];
        const MIXER_CARD& m  = lc.mixer;
        const std::string p = "l" + std::to_string(i) + ".", mp = p + "mix.";
        auto blk   = std::make_unique<FzlBlock>();
        blk->hFish = &f, blk->name = p, blk->layer = i;
        blk->norm1.hFish = &f, blk->norm1.eps = c.norm_rms_eps;
        b.Tensor(p + "norm1", 1, E, blk->norm1.w);
        if (lc.mlp.present) {
            blk->norm2.hFish = &f, blk->norm2.eps = c.norm_rms_eps;
            b.Tensor(p + "norm2", 1, E, blk->norm2.w);
        }
        if (m.type == "mingru") {
            auto g = std::make_unique<MinGRU>();
            g->hFish = &f, g->name = mp, g->card = m;
            b.Tensor(mp + "z", m.width, E, g->z), b.Tensor(mp + "z.b", 1, m.width, g->z_b);
            b.Tensor(mp + "x", m.width, E, g->x), b.Tensor(mp + "x.b", 1, m.width, g->x_b);
            b.Tensor(mp + "g", m.width, E, g->g), b.Tensor(mp + "o", E, m.width, g->o);
            blk->cat.Plan({g->z, g->x, g->g});
            maxA = std::max<size_t>(maxA, m.width);
            blk->gru = std::move(g);
        } else if (m.type == "attention") {
            auto a = std::make_unique<BlockAttention>();
            a->hFish = &f, a->name = mp, a->card = m;
            const int nq = m.heads * m.dim, nk = m.kv_heads * m.dim;
            b.Tensor(mp + "q", nq, E, a->q), b.Tensor(mp + "q.b", 1, nq, a->q_b);
            b.Tensor(mp + "k", nk, E, a->k), b.Tensor(mp + "k.b", 1, nk, a->k_b);
            b.Tensor(mp + "pb", 1, m.heads, a->pb);
            b.Tensor(mp + "o", E, nq, a->o);
            if (m.rot_dims > 0) {
                const std::vector<double> fr = StretchedFrequencies(m.rot_dims, m.rot_base, m.yarn_factor, m.yarn_original, m.yarn_fast, m.yarn_slow, &a->amp);
                KF_TRY(b.Buf(&a->inv_freq, fr.size() * sizeof(double)));
                KF_TRY(kf_h2d(f.ctx, a->inv_freq, fr.data(), fr.size() * sizeof(double)));
                KF_TRY(kf_ctx_sync(f.ctx));  // fr leaves scope
            }
            blk->cat.Plan({a->q, a->k});
            maxA = std::max<size_t>(maxA, nq), maxY = std::max<size_t>(maxY, nq / 2 + 1);  // maxY: the bf16 query of the panel kernel
            blk->attn = std::move(a);
        } else {
            auto a = std::make_unique<LatentAttention>();
            a->hFish = &f, a->name = mp, a->card = m, a->layer = i, a->layout = 1;
            const int nq = m.heads * (m.dim + m.rot_dim), W = m.kv_rank + m.rot_dim;
            b.Tensor(mp + "dq", m.q_rank, E, a->dq), b.Tensor(mp + "dq.norm", 1, m.q_rank, a->dq_norm);
            b.Tensor(mp + "uq", nq, m.q_rank, a->uq);
            b.Tensor(mp + "dkv", W, E, a->dkv), b.Tensor(mp + "dkv.norm", 1, m.kv_rank, a->dkv_norm);
            b.Tensor(mp + "uk", m.heads * m.dim, m.kv_rank, a->uk), b.Tensor(mp + "uv", m.heads * m.vdim, m.kv_rank, a->uv);
            b.Tensor(mp + "o", E, m.heads * m.vdim, a->o);
            const std::vector<double> fr = m.rot_dims > 0 ? StretchedFrequencies(m.rot_dims, m.rot_base, m.yarn_factor, m.yarn_original, m.yarn_fast, m.yarn_slow, &a->amp)
                                                          : std::vector<double>(1, 0.0);
            KF_TRY(b.Buf(&a->inv_freq, fr.size() * sizeof(double)));
            KF_TRY(kf_h2d(f.ctx, a->inv_freq, fr.data(), fr.size() * sizeof(double)));
            KF_TRY(kf_ctx_sync(f.ctx));
            blk->cat.Plan({a->dq, a->dkv});
            maxV = std::max<size_t>(maxV, nq), maxY = std::max<size_t>(maxY, (size_t)m.heads * W), maxL = std::max<size_t>(maxL, (size_t)m.heads * m.kv_rank);
            maxA = std::max<size_t>(maxA, (size_t)m.heads * m.vdim), maxMid = std::max<size_t>(maxMid, m.q_rank);
            blk->lat = std::move(a);
        }
        KF_TRY(b.Buf((char**)&blk->cat.w, (size_t)blk->cat.rows * E * 2));
        KF_TRY(kf_memset(f.ctx, blk->cat.w, 0, (size_t)blk->cat.rows * E * 2));
        maxU = std::max<size_t>(maxU, blk->cat.rows);
        if (lc.mlp.present && lc.mlp.dense) {
            auto e = std::make_unique<ClampedFF>();
            e->hFish = &f, e->name = p + "mlp", e->card = lc.mlp;
            b.Tensor(p + "mlp.gate", lc.mlp.ff, E, e->gate), b.Tensor(p + "mlp.up", lc.mlp.ff, E, e->up), b.Tensor(p + "mlp.down", E, lc.mlp.ff, e->down);
            e->cat.Plan({e->gate, e->up});
            KF_TRY(b.Buf((char**)&e->cat.w, (size_t)e->cat.rows * E * 2));
            KF_TRY(kf_memset(f.ctx, e->cat.w, 0, (size_t)e->cat.rows * E * 2));
            maxU = std::max<size_t>(maxU, e->cat.rows), maxH1 = std::max<size_t>(maxH1, lc.mlp.ff);
            blk->dense = std::move(e);
        } else if (lc.mlp.present) {
            const MOE_CARD& mc = lc.mlp;
            auto e = std::make_unique<MoE>();
            e->hFish = &f, e->name = p + "mlp", e->card = mc;
            b.Tensor(p + "mlp.router", mc.experts, E, e->router);
            b.Tensor(p + "mlp.correction", 1, mc.experts, e->router_b);
            e->gate.resize(mc.experts), e->up.resize(mc.experts), e->down.resize(mc.experts);
            for (int k = 0; k < mc.experts; k++) {
                const std::string ep = p + "mlp.e" + std::to_string(k) + ".";
                b.Tensor(ep + "gate", mc.ff, E, e->gate[k]), b.Tensor(ep + "up", mc.ff, E, e->up[k]), b.Tensor(ep + "down", E, mc.ff, e->down[k]);
            }
            KF_TRY(b.Buf(&e->tables, (size_t)3 * mc.experts * sizeof(void*)));
            maxE = std::max<size_t>(maxE, mc.experts), maxTop = std::max<size_t>(maxTop, mc.top), maxFF = std::max<size_t>(maxFF, mc.ff);
            maxU = std::max<size_t>(maxU, mc.experts);
            blk->moe = std::move(e);
        }
        f.blocks.push_back(std::move(blk));
    }
    if (c.loop_stop > c.loop_start) {  // kept behind the layers' blocks: the model's tensors that belong to no layer
        auto x = std::make_unique<FzlExtra>();
        x->hFish = &f, x->name = "loop";
        b.Tensor("loop.step", c.loop_times, E, x->step);
        f.blocks.push_back(std::move(x));
    }
    // cache and state: one entry per RUN of a layer, so every pass of the repeated layers has its own
    const std::vector<LayerRun> runs = LayerRuns(c);
    f.states.layers.resize(runs.size());
    f.states.max_seq = c.max_seq_len, f.states.f32 = f32;
    for (const LayerRun& r : runs) {
        const MIXER_CARD& m      = c.layers[r.layer].mixer;
        SeqStateCache::Layer& sl = f.states.layers[r.cache];
        if (m.type == "mingru") {
            sl.state_stride = (size_t)m.width;
            KF_TRY(b.Buf(&sl.state, (size_t)c.max_batch * sl.state_stride * 4));
            f.states.total_bytes += (size_t)c.max_batch * sl.state_stride * 4;
            continue;
        }
        if (m.type == "attention") {
            // a ring of rows: every query of a step of up to max_tokens tokens still finds its block behind it after the step's rows are in
            sl.ring    = m.block > 0 ? (int)std::min<long long>(c.max_seq_len, (long long)m.block + (long long)T - 1) : c.max_seq_len;
            sl.row_dim = 2 * m.kv_heads * m.dim, sl.row_stride = (size_t)sl.ring * sl.row_dim;
        } else {
            sl.row_dim = m.kv_rank + m.rot_dim, sl.row_stride = (size_t)c.max_seq_len * sl.row_dim;
        }
        // zeroed once: a reader may load rows of positions that the sequence has not written (masked, but they must hold numbers)
        KF_TRY(b.Buf((char**)&sl.rows, (size_t)c.max_batch * sl.row_stride * asz));
        KF_TRY(kf_memset(f.ctx, sl.rows, 0, (size_t)c.max_batch * sl.row_stride * asz));
        f.states.total_bytes += (size_t)c.max_batch * sl.row_stride * asz;
    }
    // activations: fp32 residual stream; matmul inputs in the activation type
    KF_TRY(kf_malloc(f.ctx, T * E * 4, &f.x));
    KF_TRY(b.Buf((char**)&hs->hact, T * E * asz));
    KF_TRY(b.Buf(&hs->sub, T * E * 4));
    KF_TRY(b.Buf(&hs->u, T * maxU * 4));
    KF_TRY(b.Buf(&hs->v, T * maxV * 4));
    KF_TRY(b.Buf(&hs->y, T * maxY * 4));
    KF_TRY(b.Buf(&hs->lat, T * maxL * 4));
    KF_TRY(b.Buf((char**)&hs->act, T * maxA * asz));
    KF_TRY(b.Buf((char**)&hs->mid, T * maxMid * asz));
    KF_TRY(b.Buf(&hs->hist, T * E * 4));  // the embedding output, added again before every later pass of the repeated layers
    const size_t TT = T * maxTop;
    KF_TRY(b.Buf(&hs->idx, TT * 4));
    KF_TRY(b.Buf(&hs->wgt, TT * 4));
    KF_TRY(b.Buf(&hs->offsets, (maxE + 1) * 4));
    KF_TRY(b.Buf(&hs->entry_slot, TT * 4));
    KF_TRY(b.Buf(&hs->slot_row, TT * 4));
    KF_TRY(b.Buf(&hs->slot_group, TT * 4));
    KF_TRY(b.Buf(&hs->work, (2 * TT + maxE) * 4));
    KF_TRY(b.Buf((char**)&hs->h1, std::max(TT * maxFF, T * maxH1) * asz));
    KF_TRY(b.Buf(&hs->yslots, TT * E * 4));
    KF_TRY(b.Buf((char**)&hs->head_in, (size_t)f.logit_rows * E * asz));
    KF_TRY(kf_malloc(f.ctx, (size_t)f.logit_rows * c.vocab * 2, &f.logits));
    KF_TRY(kf_malloc(f.ctx, (size_t)f.logit_rows * c.vocab * 4, (void**)&f.logits_f32));
    KF_TRY(kf_malloc(f.ctx, T * 4, (void**)&f.d_tokens));
    KF_TRY(kf_malloc(f.ctx, T * 4, (void**)&f.d_pos));
    KF_TRY(kf_malloc(f.ctx, T * 4, (void**)&f.d_next));
    KF_TRY(kf_malloc(f.ctx, T * 4, (void**)&f.d_slot));
    KF_TRY(kf_malloc(f.ctx, T * 4, (void**)&f.d_sel));
    KF_TRY(kf_host_alloc(T * 4 * 5, (void**)&f.h_stage));
    KF_TRY(kf_host_alloc((size_t)f.logit_rows * c.vocab * 2, (void**)&f.h_logits));
    KF_TRY(kf_host_alloc((size_t)f.logit_rows * c.vocab * 4, (void**)&f.h_logits_f32));
    KF_TRY(kf_ctx_sync(f.ctx));
    f.attn_hint = c.max_seq_len - 1;
    return KF_OK;
}

static int PrepareFazolorn(Fish& f) {
    for (int i = 0; i < f.config.n_layers; i++) {
        FzlBlock* b = static_cast<FzlBlock*>(f.blocks[i].get());
        int rc = b->cat.Fill(f.ctx);
        if (!rc && b->dense) rc = b->dense->cat.Fill(f.ctx);
        if (!rc && b->moe) rc = b->moe->Prepare();
        if (rc) return rc;
    }
    return KF_OK;
}

// ------------------------------------------------------------------------------------------------------------ step
static int Lin(Fish& f, float* y, int ldy, const hGTensor& w, const void* x, int ldx, int M) {
    kf_tensor_desc d = w->Desc();
    return kf_linear_g(f.ctx, y, ldy, &d, x, f.config.compute_f32 ? 1 : 0, ldx, M);
}
static int LinStacked(Fish& f, float* y, const StackedLinear& s, const void* x, int M) {
    kf_tensor_desc d = {};
    d.data_dev = s.w, d.rows = s.rows, d.cols = s.cols, d.type = KF_T_BF16, d.group = 128;
    return kf_linear_g(f.ctx, y, s.rows, &d, x, f.config.compute_f32 ? 1 : 0, s.cols, M);
}

int MinGRU::cuInfer(int M, const float* u, int ldu, const int* off, int cache) {
    Fish& f = *hFish;
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const int ak = f.config.compute_f32 ? 1 : 0, Wd = card.width;
    const int nseq = f.seq_mode ? M : 1, T = f.seq_mode ? 1 : M;
    SeqStateCache::Layer& sl = f.states.layers[cache];
    KF_TRY(kf_mingru(f.ctx, s.act, ak, Wd, u + off[0], ldu, z_b->data, u + off[1], ldu, x_b->data, u + off[2], ldu, sl.state, sl.state_stride, f.d_pos, f.d_slot,
                     nseq, T, Wd));
    KF_TRY(Lin(f, s.sub, f.config.n_embd, o, s.act, Wd, M));
    return KF_OK;
}

int BlockAttention::cuInfer(int M, float* u, int ldu, int off, int cache) {
    Fish& f = *hFish;
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const MIXER_CARD& m = card;
    const MODEL_CARD& c = f.config;
    const int ak = c.compute_f32 ? 1 : 0;
    const int nq = m.heads * m.dim, nk = m.kv_heads * m.dim;
    SeqStateCache::Layer& sl = f.states.layers[cache];
    // a block longer than the ring means the ring was cut to max_seq rows: every position lies in block 0 and none is ever masked
    const int blk = m.block <= sl.ring ? m.block : 0;
    // biases, rotation of q (in place) and k; the row [rotated k | un-rotated k] joins the ring: the second half serves as v
    // panels of one sequence with head sizes the tensor-core kernel takes go there; everything else (decode, other sizes, 32-bit) to the general kernel
    const bool tile = !ak && f.panel_consecutive && f.seq_mode == 0 && M >= 16 && (m.dim == 64 || m.dim == 128);
    KF_TRY(kf_qk_prepare_ex(f.ctx, u + off, ldu, nq, nk, nk, m.dim, q_b->data, k_b->data, 1, nullptr, nullptr, c.norm_rms_eps, m.rot_dims, inv_freq, amp, 1, sl.rows,
                            ak, sl.row_stride, sl.ring, tile ? s.y : nullptr, f.d_pos, f.d_slot, M));
    if (tile)
        KF_TRY(kf_attn_sigmoid_prefill(f.ctx, s.act, nq, s.y, sl.rows, sl.row_stride, sl.ring, pb->data, f.d_pos, f.d_slot, M, m.heads, m.kv_heads, m.dim, m.scale,
                                       blk, 1.f));
    else
        KF_TRY(kf_attn_sigmoid(f.ctx, s.act, ak, nq, u + off, ldu, sl.rows, ak, sl.row_stride, sl.ring, pb->data, f.d_pos, f.d_slot, M, m.heads, m.kv_heads, m.dim,
                               m.dim, m.scale, blk, 0, f.attn_hint + 1, 1.f));
    KF_TRY(Lin(f, s.sub, c.n_embd, o, s.act, nq, M));
    return KF_OK;
}

int ClampedFF::cuInfer(int M) {
    Fish& f = *hFish;
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const int ak = f.config.compute_f32 ? 1 : 0, F = card.ff;
    KF_TRY(LinStacked(f, s.u, cat, s.hact, M));
    KF_TRY(kf_glu_clamped(f.ctx, s.h1, ak, F, s.u + cat.off[0], cat.rows, s.u + cat.off[1], cat.rows, M, F, card.limit, kAlpha, 1.f));
    KF_TRY(Lin(f, s.sub, f.config.n_embd, down, s.h1, F, M));
    return KF_OK;
}

int FzlBlock::cuInfer(int M, int cache, const float** pending) {
    Fish& f = *hFish;
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const MODEL_CARD& c = f.config;
    const int E = c.n_embd, ak = c.compute_f32 ? 1 : 0;
    float* x = (float*)f.x;
    // one matmul for everything in the mixer that reads norm1(x)
    KF_TRY(LinStacked(f, s.u, cat, s.hact, M));
    if (gru) KF_TRY(gru->cuInfer(M, s.u, cat.rows, cat.off.data(), cache));
    else if (attn) KF_TRY(attn->cuInfer(M, s.u, cat.rows, cat.off[0], cache));
    else KF_TRY(lat->cuInfer(M, s.u, cat.rows, cat.off[0], cat.off[1], -1, cache));
    *pending = s.sub;
    if (!dense && !moe) return KF_OK;
    // x += mixer; hact = norm2(x)
    KF_TRY(kf_residual_prenorm(f.ctx, x, s.hact, ak, s.sub, E, nullptr, 0, nullptr, norm2.w->data, M, E, norm2.eps));
    if (dense) {
        KF_TRY(dense->cuInfer(M));
        return KF_OK;  // *pending = sub: the next norm adds it
    }
    KF_TRY(Lin(f, s.u, moe->card.experts, moe->router, s.hact, E, M));
    KF_TRY(moe->cuInfer(M, s.u, moe->card.experts, 0, 0, x));  // the experts' weighted sum goes straight into the residual
    *pending = nullptr;
    return KF_OK;
}

static int ForwardFazolorn(Fish& f, int M, bool want_logits) {
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const MODEL_CARD& c = f.config;
    const int E = c.n_embd, ak = c.compute_f32 ? 1 : 0;
    float* x = (float*)f.x;
    const bool loop = c.loop_stop > c.loop_start;
    const uint16_t* step = loop ? (const uint16_t*)static_cast<FzlExtra*>(f.blocks[c.n_layers].get())->step->data : nullptr;
    kf_tensor_desc de = f.embed.w->Desc();
    KF_TRY(kf_embed_f32_scaled(f.ctx, x, loop && c.loop_times > 1 ? s.hist : nullptr, &de, f.d_tokens, M, 1.f));
    const float* pending = nullptr;  // a sublayer result that the next norm still has to add to x
    for (const LayerRun& r : LayerRuns(c)) {
        FzlBlock* blk = static_cast<FzlBlock*>(f.blocks[r.layer].get());
        // x += pending (+ the embedding output before a later pass) (+ this pass's step vector); hact = norm1(x) -- one launch
        KF_TRY(kf_residual_prenorm(f.ctx, x, s.hact, ak, pending, E, r.pass > 0 ? s.hist : nullptr, E, r.pass >= 0 ? step + (size_t)r.pass * E : nullptr,
                                   blk->norm1.w->data, M, E, blk->norm1.eps));
        KF_TRY(blk->cuInfer(M, r.cache, &pending));
    }
    if (want_logits && f.n_rows > 0) {
        const int R = f.n_rows;
        if (pending) KF_TRY(kf_residual_prenorm(f.ctx, x, nullptr, ak, pending, E, nullptr, 0, nullptr, nullptr, M, E, c.norm_rms_eps));
        KF_TRY(kf_group_rmsnorm(f.ctx, s.head_in, ak, E, nullptr, 0.f, x, E, nullptr, 0, nullptr, 0, f.cls.norm.w->data, f.d_sel, R, E, 1, c.norm_rms_eps));
        KF_TRY(Lin(f, f.logits_f32, c.vocab, f.cls.proj.w, s.head_in, E, R));
        KF_TRY(kf_scale_f32(f.ctx, f.logits_f32, (size_t)R * c.vocab, c.logit_scale));
        KF_TRY(kf_f32_to_bf16(f.ctx, f.logits, f.logits_f32, (size_t)R * c.vocab));
    }
    return KF_OK;
}

const ARCH_ENTRY* FazolornArch() {
    static const ARCH_ENTRY e = {"FAZOLORN", ParseFazolorn, BuildFazolorn, ForwardFazolorn, PrepareFazolorn};
    return &e;
}

}  // namespace koifish
