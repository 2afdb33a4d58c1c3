// Sipazen.cpp -- config parsing, construction and the per-layer step of the Sipazen hybrid stack (see Sipazen.hpp).
#include "Sipazen.hpp"

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
// config.json: {"architecture": "Sipazen", "vocab", "width", "residual_mult", "norm": {"eps", "groups"}, "layers": [{"type", "mixer", "mlp"}]}
static void ParseSipazen(const JSON& h, MODEL_CARD& c) {
    c.vocab         = need_int(h, "vocab", "config");
    c.n_embd        = need_int(h, "width", "config");
    if (const JSON* r = h.find("residual_mult")) c.residual_mult = (float)r->as_double(1.0);
    const JSON& nm  = h.at("norm");
    c.norm_rms_eps  = (float)nm.at("eps").as_double(1e-5);
    c.norm_groups   = nm.contains("groups") ? need_int(nm, "groups", "norm") : 1;
    const JSON& ls  = h.at("layers");
    if (!ls.is_array() || ls.arr.empty()) throw std::runtime_error("config: layers must be a non-empty list");
    for (size_t i = 0; i < ls.arr.size(); i++) {
        const JSON& l = ls.arr[i];
        const std::string where = "layers[" + std::to_string(i) + "]";
        LAYER_CARD lc;
        MIXER_CARD& m = lc.mixer;
        m.type        = l.at("type").as_string();
        const JSON& x = l.at("mixer");
        if (m.type == "mamba2") {
            m.heads = need_int(x, "heads", where), m.vdim = need_int(x, "vdim", where), m.state = need_int(x, "state", where);
            m.groups = x.contains("groups") ? need_int(x, "groups", where) : 1;
            m.norm_groups = x.contains("norm_groups") ? need_int(x, "norm_groups", where) : 1;
            m.conv = need_int(x, "conv", where);
            if (m.heads < 1 || m.vdim < 1 || m.state < 1 || m.groups < 1 || m.heads % m.groups || m.conv < 1 || m.norm_groups < 1 ||
                (m.heads * m.vdim) % m.norm_groups)
                throw std::runtime_error("config: " + where + ": groups must divide heads, norm_groups must divide heads * vdim");
        } else if (m.type == "latent_attention") {
            m.heads = need_int(x, "heads", where), m.dim = need_int(x, "dim", where), m.rot_dim = need_int(x, "rot_dim", where);
            m.vdim = need_int(x, "vdim", where), m.kv_rank = need_int(x, "kv_rank", where);
            m.scale = x.contains("scale") ? (float)x.at("scale").as_double(1.0) : 1.0f / std::sqrt((float)(m.dim + m.rot_dim));
            m.rot_dims = m.rot_dim;
            if (const JSON* r = x.find("rot")) {
                if (r->contains("base")) m.rot_base = r->at("base").as_double(10000.0);
                if (r->contains("dims")) m.rot_dims = need_int(*r, "dims", where + ".rot");
            }
            if (m.heads < 1 || m.dim < 1 || m.rot_dim < 0 || m.vdim < 1 || m.kv_rank < 1 || m.rot_dims < 0 || m.rot_dims > m.rot_dim || m.rot_dims % 2)
                throw std::runtime_error("config: " + where + ": rot.dims must be even and at most rot_dim");
        } else {
            throw std::runtime_error("config: " + where + ": unknown mixer type '" + m.type + "'");
        }
        const JSON* f = l.find("mlp");
        if (f && !f->is_null()) {
            const std::string kind = f->at("kind").as_string();
            if (kind != "moe") throw std::runtime_error("config: " + where + ".mlp.kind '" + kind + "' is not built");
            lc.mlp.present = true;
            lc.mlp.experts = need_int(f->at("router"), "experts", where + ".mlp.router");
            lc.mlp.top     = need_int(f->at("router"), "top", where + ".mlp.router");
            lc.mlp.ff      = need_int(f->at("expert"), "ff", where + ".mlp.expert");
            const JSON* sh = f->find("shared");
            if (sh && !sh->is_null()) lc.mlp.shared_ff = need_int(*sh, "ff", where + ".mlp.shared");
            if (lc.mlp.experts < 1 || lc.mlp.top < 1 || lc.mlp.top > lc.mlp.experts || lc.mlp.ff < 1)
                throw std::runtime_error("config: " + where + ".mlp: 1 <= top <= experts");
        }
        c.layers.push_back(lc);
    }
    c.n_layers = (int)c.layers.size();
    if (c.vocab < 1 || c.n_embd < 1 || c.norm_groups < 1 || c.n_embd % c.norm_groups) throw std::runtime_error("config: norm.groups must divide width");
    // fields of the dense card that generic code reads
    c.n_head = c.n_head_kv = 1, c.head_dim = c.n_embd, c.n_ff = 0, c.tie_word_embeddings = false;
}

// ------------------------------------------------------------------------------------------------------------ build
namespace {
struct Builder {
    Fish& f;
    std::string* hFishErr;
    int next_id = 0;
    int Tensor(const std::string& name, int rows, int cols, hGTensor& out) {
        out = std::make_shared<GTensor>(f.ctx, name, rows, cols);  // bf16 as stored; this stack has no quantised storage
        f.tensors[name]    = out;
        f.tensor_ids[name] = next_id++;
        return KF_OK;
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

static int BuildSipazen(Fish& f) {
    std::string* hFishErr = &f.error;
    const MODEL_CARD& c   = f.config;
    if (f.tp_world != 1) {
        f.error = "the Sipazen stack runs on one GPU (no tensor-parallel shard plan)";
        return KF_ERR_UNSUPPORTED;
    }
    Builder b{f, hFishErr};
    const int E = c.n_embd;
    const bool f32 = c.compute_f32;
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
    auto hs = std::make_shared<HybridScratch>();
    f.hscratch = hs;
    size_t maxU = 1, maxV = 1, maxY = 1, maxL = 1, maxA = 1, maxE = 1, maxTop = 1, maxFF = 1, maxSF = 1;
    f.states.layers.resize(c.layers.size());
    f.states.max_seq = c.max_seq_len, f.states.f32 = f32;
    for (size_t i = 0; i < c.layers.size(); i++) {
        const LAYER_CARD& lc = c.layers[i];
        const MIXER_CARD& m  = lc.mixer;
        const std::string p  = "l" + std::to_string(i) + ".";
        auto blk   = std::make_unique<HybridBlock>();
        blk->hFish = &f, blk->name = p, blk->layer = (int)i;
        GroupNorm* norms[4]  = {&blk->norm1, &blk->norm1b, &blk->norm2, &blk->norm2b};
        const char* nname[4] = {"norm1", "norm1b", "norm2", "norm2b"};
        for (int k = 0; k < 4; k++) {
            if (k >= 2 && !lc.mlp.present) break;
            norms[k]->hFish = &f, norms[k]->groups = c.norm_groups, norms[k]->eps = c.norm_rms_eps;
            b.Tensor(p + nname[k], 1, E, norms[k]->w);
        }
        b.Tensor(p + "rg1", E, E, blk->rg1);
        b.Tensor(p + "rg1.b", 1, E, blk->rg1_b);
        SeqStateCache::Layer& sl = f.states.layers[i];
        if (m.type == "mamba2") {
            auto s = std::make_unique<SSMixer>();
            s->hFish = &f, s->name = p + "mix", s->card = m, s->layer = (int)i;
            const int inner = m.heads * m.vdim, C = inner + 2 * m.groups * m.state, rows = 2 * inner + 2 * m.groups * m.state + m.heads;
            b.Tensor(p + "mix.in", rows, E, s->in);
            b.Tensor(p + "mix.conv", C, m.conv, s->conv);
            b.Tensor(p + "mix.conv.b", 1, C, s->conv_b);
            b.Tensor(p + "mix.dt_bias", 1, m.heads, s->dt_bias);
            b.Tensor(p + "mix.A_log", 1, m.heads, s->A_log);
            b.Tensor(p + "mix.D", 1, m.heads, s->D);
            b.Tensor(p + "mix.norm", 1, inner, s->norm);
            b.Tensor(p + "mix.o", E, inner, s->o);
            sl.state_stride = (size_t)inner * m.state;
            sl.tail_stride  = (size_t)std::max(1, m.conv - 1) * C;
            KF_TRY(b.Buf(&sl.state, (size_t)c.max_batch * sl.state_stride * 4));
            KF_TRY(b.Buf(&sl.tail, (size_t)c.max_batch * sl.tail_stride * 4));
            f.states.total_bytes += (size_t)c.max_batch * (sl.state_stride + sl.tail_stride) * 4;
            maxV = std::max<size_t>(maxV, C), maxY = std::max<size_t>(maxY, inner), maxA = std::max<size_t>(maxA, inner);
            blk->ssm = std::move(s);
        } else {
            auto a = std::make_unique<LatentAttention>();
            a->hFish = &f, a->name = p + "mix", a->card = m, a->layer = (int)i;
            const int qd = m.heads * (m.dim + m.rot_dim), W = m.kv_rank + m.rot_dim;
            b.Tensor(p + "mix.q", qd, E, a->q);
            b.Tensor(p + "mix.dkv", W, E, a->dkv);
            b.Tensor(p + "mix.dkv.norm", 1, m.kv_rank, a->dkv_norm);
            b.Tensor(p + "mix.uk", m.heads * m.dim, m.kv_rank, a->uk);
            b.Tensor(p + "mix.uv", m.heads * m.vdim, m.kv_rank, a->uv);
            b.Tensor(p + "mix.sink", 1, m.heads, a->sink);
            b.Tensor(p + "mix.g", m.heads * m.vdim, E, a->g);
            b.Tensor(p + "mix.o", E, m.heads * m.vdim, a->o);
            // rotation frequencies base^(-2i/dims) in double: the angle pos * f_i and its sine / cosine are formed in double on the device
            std::vector<double> fr((size_t)std::max(1, m.rot_dims / 2));
            for (int k = 0; k < m.rot_dims / 2; k++) fr[k] = std::pow(m.rot_base, -2.0 * k / (double)m.rot_dims);
            KF_TRY(b.Buf(&a->inv_freq, fr.size() * 8));
            KF_TRY(kf_h2d(f.ctx, a->inv_freq, fr.data(), fr.size() * 8));
            KF_TRY(kf_ctx_sync(f.ctx));
            sl.row_dim = W, sl.row_stride = (size_t)c.max_seq_len * W;
            KF_TRY(b.Buf((char**)&sl.rows, (size_t)c.max_batch * sl.row_stride * asz));
            f.states.total_bytes += (size_t)c.max_batch * sl.row_stride * asz;
            maxV = std::max<size_t>(maxV, W), maxY = std::max<size_t>(maxY, (size_t)m.heads * W);
            maxL = std::max<size_t>(maxL, (size_t)m.heads * m.kv_rank);
            maxA = std::max<size_t>(maxA, (size_t)m.heads * m.vdim);
            blk->attn = std::move(a);
        }
        if (lc.mlp.present) {
            const MOE_CARD& mc = lc.mlp;
            b.Tensor(p + "rg2", E, E, blk->rg2);
            b.Tensor(p + "rg2.b", 1, E, blk->rg2_b);
            auto e = std::make_unique<MoE>();
            e->hFish = &f, e->name = p + "mlp", e->card = mc;
            b.Tensor(p + "mlp.router", mc.experts, E, e->router);
            b.Tensor(p + "mlp.router.b", 1, mc.experts, e->router_b);
            e->gate.resize(mc.experts), e->up.resize(mc.experts), e->down.resize(mc.experts);
            for (int k = 0; k < mc.experts; k++) {
                const std::string ep = p + "mlp.e" + std::to_string(k) + ".";
                b.Tensor(ep + "gate", mc.ff, E, e->gate[k]);
                b.Tensor(ep + "up", mc.ff, E, e->up[k]);
                b.Tensor(ep + "down", E, mc.ff, e->down[k]);
            }
            if (mc.shared_ff > 0) {
                b.Tensor(p + "mlp.shared.gate", mc.shared_ff, E, e->sh_gate);
                b.Tensor(p + "mlp.shared.up", mc.shared_ff, E, e->sh_up);
                b.Tensor(p + "mlp.shared.down", E, mc.shared_ff, e->sh_down);
                b.Tensor(p + "mlp.shared.sg", 1, E, e->sh_sg);
            }
            KF_TRY(b.Buf(&e->tables, (size_t)3 * mc.experts * sizeof(void*)));
            maxE = std::max<size_t>(maxE, mc.experts), maxTop = std::max<size_t>(maxTop, mc.top), maxFF = std::max<size_t>(maxFF, mc.ff);
            maxSF = std::max<size_t>(maxSF, mc.shared_ff);
            blk->moe = std::move(e);
        }
        // stacked first projections of each sublayer
        std::vector<hGTensor> c1 = {blk->rg1};
        if (blk->ssm) c1.push_back(blk->ssm->in);
        else c1.insert(c1.end(), {blk->attn->q, blk->attn->dkv, blk->attn->g});
        blk->cat1.Plan(c1);
        KF_TRY(b.Buf((char**)&blk->cat1.w, (size_t)blk->cat1.rows * E * 2));
        KF_TRY(kf_memset(f.ctx, blk->cat1.w, 0, (size_t)blk->cat1.rows * E * 2));
        maxU = std::max<size_t>(maxU, blk->cat1.rows);
        if (blk->moe) {
            std::vector<hGTensor> c2 = {blk->rg2, blk->moe->router};
            if (blk->moe->sh_sg) c2.push_back(blk->moe->sh_sg);
            blk->cat2.Plan(c2);
            KF_TRY(b.Buf((char**)&blk->cat2.w, (size_t)blk->cat2.rows * E * 2));
            KF_TRY(kf_memset(f.ctx, blk->cat2.w, 0, (size_t)blk->cat2.rows * E * 2));
            maxU = std::max<size_t>(maxU, blk->cat2.rows);
        }
        f.blocks.push_back(std::move(blk));
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
    const size_t TT = T * maxTop;
    KF_TRY(b.Buf(&hs->idx, TT * 4));
    KF_TRY(b.Buf(&hs->wgt, TT * 4));
    KF_TRY(b.Buf(&hs->offsets, (maxE + 1) * 4));
    KF_TRY(b.Buf(&hs->entry_slot, TT * 4));
    KF_TRY(b.Buf(&hs->slot_row, TT * 4));
    KF_TRY(b.Buf(&hs->slot_group, TT * 4));
    KF_TRY(b.Buf(&hs->work, (2 * TT + maxE) * 4));
    KF_TRY(b.Buf((char**)&hs->h1, TT * maxFF * asz));
    KF_TRY(b.Buf(&hs->yslots, TT * E * 4));
    KF_TRY(b.Buf((char**)&hs->hs, T * maxSF * asz));
    KF_TRY(b.Buf(&hs->shared, T * E * 4));
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
    f.attn_hint = c.max_seq_len - 1;
    return KF_OK;
}

void StackedLinear::Plan(const std::vector<hGTensor>& tensors) {
    parts = tensors, off.clear(), rows = 0, cols = tensors[0]->ne[1];
    for (auto& t : parts) off.push_back(rows), rows += t->ne[0];
    rows = (rows + 15) / 16 * 16;
}
int StackedLinear::Fill(kf_ctx* ctx) const {
    for (size_t i = 0; i < parts.size(); i++) {
        int rc = kf_d2d(ctx, (char*)w + (size_t)off[i] * cols * 2, parts[i]->data, (size_t)parts[i]->ne[0] * cols * 2);
        if (rc) return rc;
    }
    return KF_OK;
}
// device pointer tables of the experts, once every tensor has its data
int MoE::Prepare() {
    Fish& f = *hFish;
    std::vector<const void*> t((size_t)3 * card.experts);
    for (int k = 0; k < card.experts; k++) t[k] = gate[k]->data, t[card.experts + k] = up[k]->data, t[2 * card.experts + k] = down[k]->data;
    int rc = kf_h2d(f.ctx, tables, t.data(), t.size() * sizeof(void*));
    if (!rc) rc = kf_ctx_sync(f.ctx);
    return rc;
}
static int PrepareSipazen(Fish& f) {
    for (auto& n : f.blocks) {
        HybridBlock* b = static_cast<HybridBlock*>(n.get());
        int rc = b->cat1.Fill(f.ctx);
        if (!rc && b->moe) rc = b->cat2.Fill(f.ctx);
        if (!rc && b->moe) rc = b->moe->Prepare();
        if (rc) return rc;
    }
    return KF_OK;
}

// ------------------------------------------------------------------------------------------------------------ step
static int Lin(Fish& f, float* y, const hGTensor& w, const void* x, int M) {
    kf_tensor_desc d = w->Desc();
    return kf_linear_g(f.ctx, y, d.rows, &d, x, f.config.compute_f32 ? 1 : 0, d.cols, M);
}

int SSMixer::cuInfer(int M, const float* u, int ldu, int off_in) {
    Fish& f = *hFish;
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const MIXER_CARD& m = card;
    const int inner = m.heads * m.vdim, C = inner + 2 * m.groups * m.state;
    const float* ui = u + off_in;  // [z | x | B | C | dt] of every token, row stride ldu
    const int nseq = f.seq_mode ? M : 1, T = f.seq_mode ? 1 : M;
    const int ak = f.config.compute_f32 ? 1 : 0;
    SeqStateCache::Layer& sl = f.states.layers[layer];
    KF_TRY(kf_conv_silu(f.ctx, s.v, ui, ldu, inner, conv->data, conv_b->data, sl.tail, sl.tail_stride, f.d_pos, f.d_slot, nseq, T, C, m.conv));
    KF_TRY(kf_ssm_scan(f.ctx, s.y, inner, s.v, ui, ldu, 2 * inner + 2 * m.groups * m.state, dt_bias->data, A_log->data, D->data, sl.state, sl.state_stride,
                       f.d_pos, f.d_slot, nseq, T, m.heads, m.vdim, m.state, m.groups));
    // y * silu(z), then RMS norm in norm_groups parts
    KF_TRY(kf_group_rmsnorm(f.ctx, s.act, ak, inner, nullptr, 0.f, s.y, inner, ui, ldu, nullptr, 2, norm->data, nullptr, M, inner, m.norm_groups,
                            f.config.norm_rms_eps));
    KF_TRY(Lin(f, s.sub, o, s.act, M));
    return KF_OK;
}

int LatentAttention::cuInfer(int M, const float* u, int ldu, int off_q, int off_dkv, int off_g, int cache_layer) {
    Fish& f = *hFish;
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const MIXER_CARD& m = card;
    const int ak = f.config.compute_f32 ? 1 : 0;
    SeqStateCache::Layer& sl = f.states.layers[cache_layer < 0 ? layer : cache_layer];
    const float* qv = u + off_q;
    int ldq = ldu;
    if (dq) {  // queries through their latent: RMS norm of the down-projection, then the up-projection
        const int nq = m.heads * (m.dim + m.rot_dim);
        KF_TRY(kf_group_rmsnorm(f.ctx, s.mid, ak, m.q_rank, nullptr, 0.f, u + off_q, ldu, nullptr, 0, nullptr, 0, dq_norm->data, nullptr, M, m.q_rank, 1,
                                f.config.norm_rms_eps));
        kf_tensor_desc d = uq->Desc();
        KF_TRY(kf_linear_g(f.ctx, s.v, nq, &d, s.mid, ak, m.q_rank, M));
        qv = s.v, ldq = nq;
    }
    KF_TRY(kf_latent_append_ex(f.ctx, sl.rows, ak, sl.row_stride, u + off_dkv, ldu, dkv_norm->data, inv_freq, f.d_pos, f.d_slot, M, m.kv_rank, m.rot_dim,
                               m.rot_dims, f.config.norm_rms_eps, layout, amp));
    KF_TRY(kf_latent_attention_ex(f.ctx, s.lat, s.y, qv, ldq, uk->data, sink ? sink->data : nullptr, sl.rows, ak, sl.row_stride, inv_freq, f.d_pos, f.d_slot, M,
                                  m.heads, m.dim, m.rot_dim, m.rot_dims, m.kv_rank, m.scale, f.attn_hint, layout, amp));
    KF_TRY(kf_latent_expand(f.ctx, s.act, ak, s.lat, uv->data, off_g >= 0 ? u + off_g : nullptr, ldu, M, m.heads, m.vdim, m.kv_rank));
    KF_TRY(Lin(f, s.sub, o, s.act, M));
    return KF_OK;
}

int MoE::cuInfer(int M, const float* u, int ldu, int off_router, int off_sg, float* into_residual) {
    Fish& f = *hFish;
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const int E = f.config.n_embd, X = card.experts, top = card.top;
    const int ak = f.config.compute_f32 ? 1 : 0;
    const void* rb = router_b ? router_b->data : nullptr;
    if (card.sigmoid_route)
        KF_TRY(kf_moe_route_grouped(f.ctx, s.idx, s.wgt, s.offsets, s.entry_slot, s.slot_row, s.slot_group, s.work, u + off_router, ldu, rb, M, X, top, card.groups,
                                    card.keep, card.route_scale));
    else
        KF_TRY(kf_moe_route(f.ctx, s.idx, s.wgt, s.offsets, s.entry_slot, s.slot_row, s.slot_group, s.work, u + off_router, ldu, rb, M, X, top));
    const void* const* tb = (const void* const*)tables;
    KF_TRY(kf_linear_grouped(f.ctx, s.h1, card.ff, tb, tb + X, X, card.ff, E, s.hact, ak, E, s.offsets, s.slot_group, s.slot_row, M * top));
    KF_TRY(kf_linear_grouped(f.ctx, s.yslots, E, tb + 2 * X, nullptr, X, E, card.ff, s.h1, ak, card.ff, s.offsets, s.slot_group, nullptr, M * top));
    const bool sh = card.shared_ff > 0;
    if (sh) {
        kf_tensor_desc dg = sh_gate->Desc(), du = sh_up->Desc();
        KF_TRY(kf_linear_g_swiglu(f.ctx, s.hs, card.shared_ff, &dg, &du, s.hact, ak, E, M));
        KF_TRY(Lin(f, s.shared, sh_down, s.hs, M));
    }
    KF_TRY(kf_moe_combine_ex(f.ctx, into_residual ? into_residual : s.sub, s.yslots, s.entry_slot, s.wgt, sh ? s.shared : nullptr, sh ? u + off_sg : nullptr, ldu,
                             M, E, top, into_residual ? 1 : 0));
    return KF_OK;
}

int HybridBlock::cuInfer(int M) {
    Fish& f = *hFish;
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const MODEL_CARD& c = f.config;
    const int E = c.n_embd, ak = c.compute_f32 ? 1 : 0;
    float* x = (float*)f.x;
    // h = norm1(x); sub = mixer(h); x += m * norm1b(sub * sigmoid(rg1 h + b))
    KF_TRY(kf_group_rmsnorm(f.ctx, s.hact, ak, E, nullptr, 0.f, x, E, nullptr, 0, nullptr, 0, norm1.w->data, nullptr, M, E, norm1.groups, norm1.eps));
    // one matmul for everything that reads h: the residual gate's logits (columns 0 .. E) and the mixer's first projections
    kf_tensor_desc d1 = {};
    d1.data_dev = cat1.w, d1.rows = cat1.rows, d1.cols = cat1.cols, d1.type = KF_T_BF16, d1.group = 128;
    KF_TRY(kf_linear_g(f.ctx, s.u, cat1.rows, &d1, s.hact, ak, E, M));
    KF_TRY(ssm ? ssm->cuInfer(M, s.u, cat1.rows, cat1.off[1]) : attn->cuInfer(M, s.u, cat1.rows, cat1.off[1], cat1.off[2], cat1.off[3]));
    KF_TRY(kf_group_rmsnorm(f.ctx, nullptr, 2, E, x, c.residual_mult, s.sub, E, s.u, cat1.rows, rg1_b->data, 1, norm1b.w->data, nullptr, M, E, norm1b.groups,
                            norm1b.eps));
    if (moe) {
        KF_TRY(kf_group_rmsnorm(f.ctx, s.hact, ak, E, nullptr, 0.f, x, E, nullptr, 0, nullptr, 0, norm2.w->data, nullptr, M, E, norm2.groups, norm2.eps));
        kf_tensor_desc d2 = {};
        d2.data_dev = cat2.w, d2.rows = cat2.rows, d2.cols = cat2.cols, d2.type = KF_T_BF16, d2.group = 128;
        KF_TRY(kf_linear_g(f.ctx, s.u, cat2.rows, &d2, s.hact, ak, E, M));
        KF_TRY(moe->cuInfer(M, s.u, cat2.rows, cat2.off[1], cat2.off.size() > 2 ? cat2.off[2] : 0));
        KF_TRY(kf_group_rmsnorm(f.ctx, nullptr, 2, E, x, c.residual_mult, s.sub, E, s.u, cat2.rows, rg2_b->data, 1, norm2b.w->data, nullptr, M, E,
                                norm2b.groups, norm2b.eps));
    }
    return KF_OK;
}

static int ForwardSipazen(Fish& f, int M, bool want_logits) {
    std::string* hFishErr = &f.error;
    HybridScratch& s = *f.hscratch;
    const MODEL_CARD& c = f.config;
    kf_tensor_desc de = f.embed.w->Desc();
    KF_TRY(kf_embed_f32(f.ctx, (float*)f.x, &de, f.d_tokens, M));
    for (auto& n : f.blocks) KF_TRY(static_cast<HybridBlock*>(n.get())->cuInfer(M));
    if (want_logits && f.n_rows > 0) {  // final norm of the selected rows, then the head; a bf16 copy feeds the sampler
        const int R = f.n_rows, ak = c.compute_f32 ? 1 : 0;
        KF_TRY(kf_group_rmsnorm(f.ctx, s.head_in, ak, c.n_embd, nullptr, 0.f, (float*)f.x, c.n_embd, nullptr, 0, nullptr, 0, f.cls.norm.w->data, f.d_sel, R,
                                c.n_embd, c.norm_groups, c.norm_rms_eps));
        KF_TRY(Lin(f, f.logits_f32, f.cls.proj.w, s.head_in, R));
        KF_TRY(kf_f32_to_bf16(f.ctx, f.logits, f.logits_f32, (size_t)R * c.vocab));
    }
    return KF_OK;
}

const ARCH_ENTRY* SipazenArch() {
    static const ARCH_ENTRY e = {"SIPAZEN", ParseSipazen, BuildSipazen, ForwardSipazen, PrepareSipazen};
    return &e;
}

}  // namespace koifish
