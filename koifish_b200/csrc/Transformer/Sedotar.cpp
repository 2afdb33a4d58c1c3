// Sedotar.cpp -- config parsing, construction and the per-layer step of the Sedotar stack (see Sedotar.hpp).
#include "Sedotar.hpp"

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

std::vector<double> StretchedFrequencies(int dims, double base, double factor, double original, double fast, double slow, float* amp) {
    const int half = dims / 2;
    std::vector<double> f((size_t)half);
    for (int i = 0; i < half; i++) f[i] = std::pow(base, -2.0 * i / dims);
    *amp = 1.f;
    if (factor > 0.0) {
        const double PI = 3.14159265358979323846;
        auto at = [&](double turns) { return dims * std::log(original / (2.0 * PI * turns)) / (2.0 * std::log(base)); };
        const double lo = std::max(std::floor(at(fast)), 0.0), hi = std::min(std::ceil(at(slow)), (double)dims - 1.0);
        for (int i = 0; i < half; i++) {
            const double ramp = std::min(1.0, std::max(0.0, (i - lo) / std::max(hi - lo, 0.001)));
            f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp);
        }
        *amp = (float)(0.1 * std::log(factor) + 1.0);
    }
    return f;
}

// config.json: {"architecture": "Sedotar", "vocab", "width", "embedding": {"scale"}, "norm": {"eps"},
//   "layers": [{"type": "parallel", "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "conv", "scale", "softcap", "mask": {"size"},
//               "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}}, "left_scale",
//               "right": {"heads", "kv_heads", "dim", "vdim", "conv"}, "right_scale"}, "mlp": {"kind": "dense", "ff"} | null}]}
// Keys that may be left out or null: kv_heads (= heads), scale (dim^-1/2), softcap (not capped), mask (all keys), rot (no rotation),
// rot.scaling (plain frequencies), the two branch scales (1), embedding (scale 1).
static void ParseSedotar(const JSON& h, MODEL_CARD& c) {
    c.vocab  = need_int(h, "vocab", "config");
    c.n_embd = need_int(h, "width", "config");
    if (const JSON* e = present(h, "embedding"))
        if (const JSON* s = present(*e, "scale")) c.embed_scale = (float)s->as_double(1.0);
    c.norm_rms_eps = (float)need_num(h.at("norm"), "eps", "norm");
    c.norm_groups  = 1;
    const JSON& ls = h.at("layers");
    if (!ls.is_array() || ls.arr.empty()) throw std::runtime_error("config: layers must be a non-empty list");
    const JSON* shapes = h.find("tensor_shapes");
    for (size_t i = 0; i < ls.arr.size(); i++) {
        const JSON& l = ls.arr[i];
        const std::string where = "layers[" + std::to_string(i) + "]";
        LAYER_CARD lc;
        MIXER_CARD& m = lc.mixer;
        m.type        = l.at("type").as_string();
        if (m.type != "parallel") throw std::runtime_error("config: " + where + ": unknown mixer type '" + m.type + "'");
        const JSON& x = l.at("mixer");
        const JSON& a = x.at("left");
        const JSON& r = x.at("right");
        const std::string wl = where + ".mixer.left", wr = where + ".mixer.right";
        m.heads = need_int(a, "heads", wl), m.kv_heads = present(a, "kv_heads") ? need_int(a, "kv_heads", wl) : m.heads;
        m.dim = need_int(a, "dim", wl), m.vdim = need_int(a, "vdim", wl), m.conv = present(a, "conv") ? need_int(a, "conv", wl) : 1;
        m.scale   = present(a, "scale") ? (float)need_num(a, "scale", wl) : 1.0f / std::sqrt((float)m.dim);
        m.softcap = present(a, "softcap") ? (float)need_num(a, "softcap", wl) : 0.f;
        if (const JSON* k = present(a, "mask")) m.window = need_int(*k, "size", wl + ".mask");
        if (const JSON* t = present(a, "rot")) {
            m.rot_dims = need_int(*t, "dims", wl + ".rot"), m.rot_base = need_num(*t, "base", wl + ".rot");
            if (const JSON* s = present(*t, "scaling")) {
                const std::string ws = wl + ".rot.scaling";
                m.yarn_factor = need_num(*s, "factor", ws), m.yarn_original = need_num(*s, "original", ws);
                m.yarn_fast = need_num(*s, "fast", ws), m.yarn_slow = need_num(*s, "slow", ws);
                if (!(m.yarn_factor > 0.0) || !(m.yarn_original > 0.0) || !(m.yarn_fast > 0.0) || !(m.yarn_slow > 0.0))
                    throw std::runtime_error("config: " + ws + ": factor, original, fast, slow must be positive");
            }
        }
        // the sink is a tensor, not a key: present unless the checkpoint's shapes are known and lack it
        m.sink = !shapes || shapes->find("l" + std::to_string(i) + ".mix.left.sink") != nullptr;
        if (m.heads < 1 || m.kv_heads < 1 || m.heads % m.kv_heads || m.dim < 1 || m.vdim < 1 || m.vdim > 512 || m.conv < 1 || m.window < 0 || m.rot_dims < 0 ||
            m.rot_dims > m.dim || m.rot_dims % 2 || (m.rot_dims > 0 && !(m.rot_base > 0.0)) || m.softcap < 0.f)
            throw std::runtime_error("config: " + wl + ": kv_heads must divide heads, vdim <= 512, rot.dims even and <= dim, conv >= 1");
        auto rc = std::make_shared<MIXER_CARD>();
        rc->type  = "scalar_delta";
        rc->heads = need_int(r, "heads", wr), rc->kv_heads = present(r, "kv_heads") ? need_int(r, "kv_heads", wr) : rc->heads;
        rc->dim = need_int(r, "dim", wr), rc->vdim = need_int(r, "vdim", wr), rc->conv = present(r, "conv") ? need_int(r, "conv", wr) : 1;
        if (rc->heads < 1 || rc->kv_heads < 1 || rc->heads % rc->kv_heads || rc->dim < 1 || rc->dim > 512 || rc->vdim < 1 || rc->conv < 1)
            throw std::runtime_error("config: " + wr + ": kv_heads must divide heads; 1 <= dim <= 512, conv >= 1");
        m.right       = rc;
        m.left_scale  = present(x, "left_scale") ? (float)need_num(x, "left_scale", where + ".mixer") : 1.f;
        m.right_scale = present(x, "right_scale") ? (float)need_num(x, "right_scale", where + ".mixer") : 1.f;
        if (const JSON* f = present(l, "mlp")) {
            const std::string kind = f->at("kind").as_string();
            if (kind != "dense") throw std::runtime_error("config: " + where + ".mlp.kind '" + kind + "' is not built");
            lc.mlp.present = true, lc.mlp.dense = true, lc.mlp.ff = need_int(*f, "ff", where + ".mlp");
            if (lc.mlp.ff < 1) throw std::runtime_error("config: " + where + ".mlp: ff must be positive");
        }
        c.layers.push_back(lc);
    }
    c.n_layers = (int)c.layers.size();
    if (c.vocab < 1 || c.n_embd < 1) throw std::runtime_error("config: vocab, width must be positive");
    c.n_head = c.n_head_kv = 1, c.head_dim = c.n_embd, c.n_ff = 0, c.tie_word_embeddings = true;
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
}  // namespace

static int BuildSedotar(Fish& f) {
    std::string* hFishErr = &f.error;
    const MODEL_CARD& c   = f.config;
    if (f.tp_world != 1) {
        f.error = "the Sedotar stack runs on one GPU (no tensor-parallel shard plan)";
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
    f.cls.proj.w = f.embed.w;  // the head is the embedding table itself

    f.max_tokens = std::max(std::max(64, c.max_batch), c.max_prefill);
    f.logit_rows = c.logit_rows_cfg > 0 ? std::min(c.logit_rows_cfg, f.max_tokens) : std::max(64, c.max_batch);
    const size_t T = f.max_tokens;
    auto hs    = std::make_shared<HybridScratch>();
    f.hscratch = hs;
    size_t maxU = 1, maxV = 1, maxY = 1, maxL = 1, maxA = 1, maxH1 = 1;
    f.states.layers.resize(L);
    f.states.max_seq = c.max_seq_len, f.states.f32 = f32;
    for (int i = 0; i < L; i++) {
        const LAYER_CARD& lc = c.layers[i];
        const MIXER_CARD& m  = lc.mixer;
        const MIXER_CARD& r  = *m.right;
        const std::string p = "l" + std::to_string(i) + ".", lp = p + "mix.left.", rp = p + "mix.right.";
        auto blk   = std::make_unique<SedotarBlock>();
        blk->hFish = &f, blk->name = p, blk->layer = i;
        blk->norm1.hFish = &f, blk->norm1.eps = c.norm_rms_eps;
        b.Tensor(p + "norm1", 1, E, blk->norm1.w);
        SeqStateCache::Layer& sl = f.states.layers[i];
        // left: rotated sliding-window attention
        auto a = std::make_unique<WindowAttention>();
        a->hFish = &f, a->name = lp, a->card = m, a->layer = i;
        const int nq = m.heads * m.dim, nk = m.kv_heads * m.dim, nv = m.kv_heads * m.vdim, no = m.heads * m.vdim, Cl = nq + nk + nv;
        b.Tensor(lp + "q", nq, E, a->q), b.Tensor(lp + "k", nk, E, a->k), b.Tensor(lp + "v", nv, E, a->v);
        b.Tensor(lp + "q.norm", 1, nq, a->qn), b.Tensor(lp + "k.norm", 1, nk, a->kn);
        b.Tensor(lp + "q.conv", nq, m.conv, a->qc), b.Tensor(lp + "k.conv", nk, m.conv, a->kc), b.Tensor(lp + "v.conv", nv, m.conv, a->vc);
        if (m.sink) b.Tensor(lp + "sink", 1, m.heads, a->sink);
        b.Tensor(lp + "o", E, no, a->o);
        a->convs.Plan({a->qc, a->kc, a->vc});
        KF_TRY(b.Buf((char**)&a->convs.w, (size_t)a->convs.rows * m.conv * 2));
        if (m.rot_dims > 0) {
            const std::vector<double> fr = StretchedFrequencies(m.rot_dims, m.rot_base, m.yarn_factor, m.yarn_original, m.yarn_fast, m.yarn_slow, &a->amp);
            KF_TRY(b.Buf(&a->inv_freq, fr.size() * sizeof(double)));
            KF_TRY(kf_h2d(f.ctx, a->inv_freq, fr.data(), fr.size() * sizeof(double)));
            KF_TRY(kf_ctx_sync(f.ctx));  // fr leaves scope
        }
        // a ring of rows: every query of a step of up to max_tokens tokens still finds the window behind it after the step's rows are in
        sl.ring    = m.window > 0 ? (int)std::min<long long>(c.max_seq_len, (long long)m.window + (long long)T - 1) : c.max_seq_len;
        sl.row_dim = nk + nv, sl.row_stride = (size_t)sl.ring * sl.row_dim;
        // right: the gated delta rule with one decay per head
        auto d = std::make_unique<ScalarDeltaMixer>();
        d->hFish = &f, d->name = rp, d->card = r, d->layer = i;
        const int rq = r.kv_heads * r.dim, rv = r.heads * r.vdim, Cr = 2 * rq + rv;
        b.Tensor(rp + "q", rq, E, d->q), b.Tensor(rp + "q.conv", rq, r.conv, d->qc);
        b.Tensor(rp + "k", rq, E, d->k), b.Tensor(rp + "k.conv", rq, r.conv, d->kc);
        b.Tensor(rp + "v", rv, E, d->v), b.Tensor(rp + "v.conv", rv, r.conv, d->vc);
        b.Tensor(rp + "b", r.heads, E, d->b), b.Tensor(rp + "a", r.heads, E, d->a);
        b.Tensor(rp + "A_log", 1, r.heads, d->A_log), b.Tensor(rp + "dt_bias", 1, r.heads, d->dt_bias);
        b.Tensor(rp + "norm", 1, r.vdim, d->norm);
        b.Tensor(rp + "g", rv, E, d->g), b.Tensor(rp + "o", E, rv, d->o);
        d->convs.Plan({d->qc, d->kc, d->vc});
        KF_TRY(b.Buf((char**)&d->convs.w, (size_t)d->convs.rows * r.conv * 2));
        sl.state_stride = (size_t)r.heads * r.dim * r.vdim;
        a->tail_off = 0, d->tail_off = (size_t)std::max(1, m.conv - 1) * Cl;
        sl.tail_stride = d->tail_off + (size_t)std::max(1, r.conv - 1) * Cr;
        // zeroed once: a reader may load rows of positions that the sequence has not written (masked, but they must hold numbers)
        KF_TRY(b.Buf((char**)&sl.rows, (size_t)c.max_batch * sl.row_stride * asz));
        KF_TRY(kf_memset(f.ctx, sl.rows, 0, (size_t)c.max_batch * sl.row_stride * asz));
        KF_TRY(b.Buf(&sl.state, (size_t)c.max_batch * sl.state_stride * 4));
        KF_TRY(b.Buf(&sl.tail, (size_t)c.max_batch * sl.tail_stride * 4));
        f.states.total_bytes += (size_t)c.max_batch * (sl.row_stride * asz + (sl.state_stride + sl.tail_stride) * 4);
        blk->cat.Plan({a->q, a->k, a->v, d->q, d->k, d->v, d->b, d->a, d->g});
        blk->off = blk->cat.off;
        KF_TRY(b.Buf((char**)&blk->cat.w, (size_t)blk->cat.rows * E * 2));
        KF_TRY(kf_memset(f.ctx, blk->cat.w, 0, (size_t)blk->cat.rows * E * 2));
        maxU = std::max<size_t>(maxU, blk->cat.rows);
        maxV = std::max<size_t>(maxV, Cl), maxL = std::max<size_t>(maxL, Cr), maxY = std::max<size_t>(maxY, std::max(rv, nq / 2 + 1));  // scan read-out; the bf16 query of the panel kernel
        blk->out.Plan({a->o, d->o});
        KF_TRY(b.Buf((char**)&blk->out.w, (size_t)E * blk->out.cols * 2));
        maxA = std::max<size_t>(maxA, blk->out.cols);
        blk->left = std::move(a), blk->right = std::move(d);
        if (lc.mlp.present) {
            auto e = std::make_unique<GatedFF>();
            e->hFish = &f, e->name = p + "mlp", e->card = lc.mlp;
            blk->norm2.hFish = &f, blk->norm2.eps = c.norm_rms_eps;
            b.Tensor(p + "norm2", 1, E, blk->norm2.w);
            b.Tensor(p + "mlp.gate", lc.mlp.ff, E, e->gate), b.Tensor(p + "mlp.up", lc.mlp.ff, E, e->up), b.Tensor(p + "mlp.down", E, lc.mlp.ff, e->down);
            e->cat.Plan({e->gate, e->up});
            KF_TRY(b.Buf((char**)&e->cat.w, (size_t)e->cat.rows * E * 2));
            KF_TRY(kf_memset(f.ctx, e->cat.w, 0, (size_t)e->cat.rows * E * 2));
            maxU  = std::max<size_t>(maxU, e->cat.rows);
            maxH1 = std::max<size_t>(maxH1, lc.mlp.ff);
            blk->ff = std::move(e);
        }
        f.blocks.push_back(std::move(blk));
    }
    // activations: fp32 residual stream; matmul inputs in the activation type
    KF_TRY(kf_malloc(f.ctx, T * E * 4, &f.x));
    KF_TRY(b.Buf((char**)&hs->hact, T * E * asz));
    KF_TRY(b.Buf(&hs->sub, T * E * 4));
    KF_TRY(b.Buf(&hs->u, T * maxU * 4));
    KF_TRY(b.Buf(&hs->v, T * maxV * 4));
    KF_TRY(b.Buf(&hs->lat, T * maxL * 4));
    KF_TRY(b.Buf(&hs->y, T * maxY * 4));
    KF_TRY(b.Buf((char**)&hs->act, T * maxA * asz));
    KF_TRY(b.Buf((char**)&hs->h1, T * maxH1 * asz));
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

void SummedLinear::Plan(const std::vector<hGTensor>& tensors) {
    parts = tensors, off.clear(), cols = 0, rows = tensors[0]->ne[0];
    for (auto& t : parts) off.push_back(cols), cols += t->ne[1];
}
int SummedLinear::Fill(kf_ctx* ctx) const {
    for (size_t i = 0; i < parts.size(); i++) {
        int rc = kf_d2d_2d(ctx, (char*)w + (size_t)off[i] * 2, (size_t)cols * 2, parts[i]->data, (size_t)parts[i]->ne[1] * 2, (size_t)parts[i]->ne[1] * 2, (size_t)rows);
        if (rc) return rc;
    }
    return KF_OK;
}
static int PrepareSedotar(Fish& f) {
    for (auto& n : f.blocks) {
        SedotarBlock* b = static_cast<SedotarBlock*>(n.get());
        int rc = b->cat.Fill(f.ctx);
        if (!rc) rc = b->out.Fill(f.ctx);
        if (!rc) rc = b->left->convs.Fill(f.ctx);
        if (!rc) rc = b->right->convs.Fill(f.ctx);
        if (!rc && b->ff) rc = b->ff->cat.Fill(f.ctx);
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

int WindowAttention::cuInfer(int M, const float* u, int ldu, int off, void* out, int ldo, float out_scale) {
    Fish& f = *hFish;
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const MIXER_CARD& m = card;
    const MODEL_CARD& c = f.config;
    const int ak = c.compute_f32 ? 1 : 0;
    const int nq = m.heads * m.dim, nk = m.kv_heads * m.dim, nv = m.kv_heads * m.vdim, C = nq + nk + nv;
    const int nseq = f.seq_mode ? M : 1, T = f.seq_mode ? 1 : M;
    SeqStateCache::Layer& sl = f.states.layers[layer];
    // q | k | v through their short convolutions (no activation); whole-row norms, rotation; this step's keys and values join the ring
    KF_TRY(kf_conv1d(f.ctx, s.v, u, ldu, off, convs.w, nullptr, sl.tail + tail_off, sl.tail_stride, f.d_pos, f.d_slot, nseq, T, C, m.conv, 0));
    // panels of one sequence with head sizes the tensor-core kernel takes go there; everything else (decode, other sizes, 32-bit) to the general kernel
    const bool tile = !ak && f.panel_consecutive && f.seq_mode == 0 && M >= 16 && m.dim == m.vdim && (m.dim == 64 || m.dim == 128) && ldo % 2 == 0;
    const void* snk = sink ? sink->data : nullptr;
    // a window longer than the ring means the ring was cut to max_seq rows: every position is below it and none is ever masked
    const int win = m.window <= sl.ring ? m.window : 0;
    KF_TRY(kf_qk_prepare(f.ctx, s.v, C, nq, nk, nv, m.dim, qn->data, kn->data, c.norm_rms_eps, m.rot_dims, inv_freq, amp, 0, sl.rows, ak, sl.row_stride, sl.ring,
                         tile ? s.y : nullptr, f.d_pos, f.d_slot, M));
    if (tile)
        KF_TRY(kf_attn_window_prefill(f.ctx, out, ldo, s.y, sl.rows, sl.row_stride, sl.ring, snk, f.d_pos, f.d_slot, M, m.heads, m.kv_heads, m.dim, m.scale,
                                      m.softcap, win, out_scale));
    else
        KF_TRY(kf_attn_window(f.ctx, out, ak, ldo, s.v, C, sl.rows, ak, sl.row_stride, sl.ring, snk, f.d_pos, f.d_slot, M, m.heads, m.kv_heads, m.dim, m.vdim,
                              m.scale, m.softcap, win, f.attn_hint + 1, out_scale));
    return KF_OK;
}

int ScalarDeltaMixer::cuInfer(int M, const float* u, int ldu, const int* off, void* out, int ldo, float out_scale) {
    Fish& f = *hFish;
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const MIXER_CARD& m = card;
    const MODEL_CARD& c = f.config;
    const int ak = c.compute_f32 ? 1 : 0;
    const int nq = m.kv_heads * m.dim, nv = m.heads * m.vdim, C = 2 * nq + nv;
    const int nseq = f.seq_mode ? M : 1, T = f.seq_mode ? 1 : M;
    SeqStateCache::Layer& sl = f.states.layers[layer];
    KF_TRY(kf_conv1d(f.ctx, s.lat, u, ldu, off[0], convs.w, nullptr, sl.tail + tail_off, sl.tail_stride, f.d_pos, f.d_slot, nseq, T, C, m.conv, 1));
    KF_TRY(kf_gated_scan_ex(f.ctx, s.y, nv, s.lat, C, s.lat + nq, C, s.lat + 2 * nq, C, u + off[2], ldu, dt_bias->data, A_log->data, u + off[1], ldu, sl.state,
                            sl.state_stride, f.d_pos, f.d_slot, nseq, T, m.heads, m.kv_heads, m.dim, m.vdim, 1, 1, 1.f, 1, 1e-6f, 1.0f / std::sqrt((float)m.dim), 1));
    // per-head RMS norm of the read-out (weight shared by the heads) times silu(gate)
    KF_TRY(kf_group_rmsnorm_wadd(f.ctx, out, ak, ldo, nullptr, 0.f, s.y, nv, u + off[3], ldu, nullptr, 4, norm->data, 1, 0.f, out_scale, nullptr, M, nv, m.heads,
                                 c.norm_rms_eps));
    return KF_OK;
}

int SedotarBlock::cuInfer(int M) {
    Fish& f = *hFish;
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const MODEL_CARD& c = f.config;
    const MIXER_CARD& m = c.layers[layer].mixer;
    const int E = c.n_embd, ak = c.compute_f32 ? 1 : 0;
    float* x = (float*)f.x;
    // hact holds x in the activation type (written by whoever updated x last).  One matmul for everything in the mixer that reads it.
    KF_TRY(LinStacked(f, s.u, cat, s.hact, M));
    // each branch leaves (its scale) x (its result) in its columns of `act`; one matmul over [W_o left | W_o right] then forms
    // left_scale * W_l y_l + right_scale * W_r y_r
    const size_t asz = ak ? 4 : 2;
    KF_TRY(left->cuInfer(M, s.u, cat.rows, off[0], s.act, out.cols, m.left_scale));
    const int roff[4] = {off[3], off[6], off[7], off[8]};
    KF_TRY(right->cuInfer(M, s.u, cat.rows, roff, (char*)s.act + (size_t)out.off[1] * asz, out.cols, m.right_scale));
    kf_tensor_desc dw = {};
    dw.data_dev = out.w, dw.rows = out.rows, dw.cols = out.cols, dw.type = KF_T_BF16, dw.group = 128;
    KF_TRY(kf_linear_g(f.ctx, s.sub, E, &dw, s.act, ak, out.cols, M));
    // x += norm1(mixer); hact = the new x
    KF_TRY(kf_postnorm_residual(f.ctx, x, s.hact, ak, s.sub, E, 1.f, nullptr, 0, 0.f, norm1.w->data, 1.f, M, E, norm1.eps));
    if (ff) {
        const int F = ff->card.ff;
        KF_TRY(LinStacked(f, s.u, ff->cat, s.hact, M));
        KF_TRY(kf_bias_act(f.ctx, s.h1, ak ? 1 : 0, F, s.u, ff->cat.rows, nullptr, 4, s.u + F, ff->cat.rows, M, F));  // relu(gate) * up
        KF_TRY(Lin(f, s.sub, E, ff->down, s.h1, F, M));
        KF_TRY(kf_postnorm_residual(f.ctx, x, s.hact, ak, s.sub, E, 1.f, nullptr, 0, 0.f, norm2.w->data, 1.f, M, E, norm2.eps));
    }
    return KF_OK;
}

static int ForwardSedotar(Fish& f, int M, bool want_logits) {
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const MODEL_CARD& c = f.config;
    const int E = c.n_embd, ak = c.compute_f32 ? 1 : 0;
    kf_tensor_desc de = f.embed.w->Desc();
    KF_TRY(kf_embed_f32_scaled(f.ctx, (float*)f.x, nullptr, &de, f.d_tokens, M, c.embed_scale));
    KF_TRY(kf_bias_act(f.ctx, s.hact, ak ? 1 : 0, E, (const float*)f.x, E, nullptr, 0, nullptr, 0, M, E));
    for (auto& n : f.blocks) KF_TRY(static_cast<SedotarBlock*>(n.get())->cuInfer(M));
    if (want_logits && f.n_rows > 0) {
        const int R = f.n_rows;
        KF_TRY(kf_group_rmsnorm_wadd(f.ctx, s.head_in, ak, E, nullptr, 0.f, (float*)f.x, E, nullptr, 0, nullptr, 0, f.cls.norm.w->data, 0, 1.f, 1.f, f.d_sel, R,
                                     E, 1, c.norm_rms_eps));
        KF_TRY(Lin(f, f.logits_f32, c.vocab, f.cls.proj.w, s.head_in, E, R));
        KF_TRY(kf_f32_to_bf16(f.ctx, f.logits, f.logits_f32, (size_t)R * c.vocab));
    }
    return KF_OK;
}

const ARCH_ENTRY* SedotarArch() {
    static const ARCH_ENTRY e = {"SEDOTAR", ParseSedotar, BuildSedotar, ForwardSedotar, PrepareSedotar};
    return &e;
}

}  // namespace koifish
