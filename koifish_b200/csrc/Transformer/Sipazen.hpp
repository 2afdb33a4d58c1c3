// Sipazen.hpp -- neurons of the Sipazen hybrid stack: every layer is  x += m * norm_b(gate(h) * mixer(h)),  h = norm(x),  followed by
// the same arrangement around a mixture-of-experts feed-forward; the mixer is either a state-space recurrence (SSMixer) or attention
// over a compressed latent with a softmax sink (LatentAttention).  The residual stream x, the norms, the router, the recurrence and
// the attention scores are fp32; what feeds a matmul is written in the activation type (bf16, or float when the whole model runs in
// 32-bit).  The neurons use the model's shared scratch (HybridScratch) and its SeqStateCache; the step function, CUDA-graph replay,
// sampler and generation loop are Fish's own.  The reference has no counterpart (its inference path is the Qwen3 block, QWen.cpp:16-145).
#pragma once
#include "QWen3.hpp"

namespace koifish {

struct HybridScratch {  // device buffers shared by all layers, sized for max_tokens
    void* hact = nullptr;        // normed input of a sublayer, activation type [T][E]
    float* sub = nullptr;        // sublayer result [T][E]
    float* u = nullptr;          // result of a sublayer's stacked first projections [T][widest stack]: gate logits | in-projection or q | dkv | g ...
    float* v = nullptr;          // convolution output / latent down-projection
    float* y = nullptr;          // scan output / absorbed queries
    float* lat = nullptr;        // attended latent [T][H][rank]
    void* act = nullptr;         // input of the output projection, activation type
    // mixture of experts
    int32_t *idx = nullptr, *offsets = nullptr, *entry_slot = nullptr, *slot_row = nullptr, *slot_group = nullptr, *work = nullptr;
    float* wgt = nullptr;
    void* h1 = nullptr;          // [T * top][ff] activation type
    float* yslots = nullptr;     // [T * top][E]
    void* hs = nullptr;          // shared expert hidden, activation type
    float* shared = nullptr;     // [T][E]
    void* head_in = nullptr;     // final norm of the selected rows, activation type
    // stacks with low-rank projections, a per-layer token input, a depth-weighted residual, a gated LRU
    void* mid = nullptr;         // second-stage matmul inputs (low-rank middles, token-gated side input), activation type
    float* hist = nullptr;       // [layers + 1][T][E] results of the embedding and of every layer
    float* lru_work = nullptr;   // [2][T][widest LRU]: decay and input term of every token
};

// Several weights that read the same normed input, stacked row-wise into ONE matrix at load (rows padded to a multiple of 16 so that the
// tuned kernels take it): one launch instead of one per weight; consumers read their columns of the result at off[i] with stride `rows`.
struct StackedLinear {
    void* w = nullptr;  // device bf16 [rows][cols]
    int rows = 0, cols = 0;
    std::vector<hGTensor> parts;
    std::vector<int> off;
    void Plan(const std::vector<hGTensor>& tensors);  // sizes only
    int Fill(kf_ctx* ctx) const;                      // copy the parts' rows (after every tensor has data)
};
struct GroupNorm : GeNeuron {
    hGTensor w;
    int groups = 1;
    float eps = 1e-5f;
};
struct SSMixer : GeNeuron {
    MIXER_CARD card;
    int layer = 0;
    hGTensor in, conv, conv_b, dt_bias, A_log, D, norm, o;
    int cuInfer(int M, const float* u, int ldu, int off_in);  // u: stacked first projections; in-projection at column off_in; -> sub
};
struct LatentAttention : GeNeuron {
    MIXER_CARD card;
    int layer = 0;
    hGTensor q, dkv, dkv_norm, uk, uv, sink, g, o;  // sink, g may be absent: plain softmax, no output gate
    hGTensor dq, dq_norm, uq;    // queries through a latent (card.q_rank > 0): q = uq . rmsnorm(dq h); then `q` is absent
    double* inv_freq = nullptr;  // device [rot_dims / 2]
    int layout = 0;              // rotation pairs: 0 (i, i + dims/2), 1 (2i, 2i + 1)
    float amp = 1.f;             // multiplies cosine and sine
    // u: the stacked first projections; off_q: the query projection (or, with a query latent, its down-projection); off_g < 0: no gate;
    // cache_layer: which entry of the model's SeqStateCache holds this run's rows (-1: `layer`)
    int cuInfer(int M, const float* u, int ldu, int off_q, int off_dkv, int off_g, int cache_layer = -1);
};
struct MoE : GeNeuron {
    MOE_CARD card;
    hGTensor router, router_b;  // router_b: bias of the softmax routing, or the selection correction of the sigmoid routing
    std::vector<hGTensor> gate, up, down;
    hGTensor sh_gate, sh_up, sh_down, sh_sg;
    void** tables = nullptr;  // device: [3][experts] weight pointers (gate | up | down)
    int Prepare();
    // into_residual: the weighted sum of the experts is added to that buffer instead of being written to the sublayer result
    int cuInfer(int M, const float* u, int ldu, int off_router, int off_sg, float* into_residual = nullptr);
};
struct HybridBlock : GeNeuron {
    int layer = 0;
    GroupNorm norm1, norm1b, norm2, norm2b;
    hGTensor rg1, rg1_b, rg2, rg2_b;
    StackedLinear cat1, cat2;  // [rg1 | the mixer's first projections], [rg2 | router | shared-expert gate]
    std::unique_ptr<SSMixer> ssm;
    std::unique_ptr<LatentAttention> attn;
    std::unique_ptr<MoE> moe;
    int cuInfer(int M);
};

}  // namespace koifish
