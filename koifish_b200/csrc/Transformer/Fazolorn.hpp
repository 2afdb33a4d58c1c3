// Fazolorn.hpp -- neurons of the Fazolorn stack.  Pre-norm layers,
//     x += mixer(norm1(x)),   x += ff(norm2(x)),      norm(y) = y / sqrt(mean(y^2) + eps) * w,
// of which a range [loop_start, loop_stop) runs loop_times times in a row on the same weights -- every pass with a cache / state of its
// own -- and, before pass t, x += [t > 0] (the embedding output) + step[t].  Mixers:
//   MinGRU              z = sigmoid(W_z h + b_z), u = W_x h + b_x, c = u + 1/2 (u >= 0) | sigmoid(u);  s <- (1 - z) s + z c per channel;
//                       W_o (s * silu(W_g h)).  State [width] fp32 per sequence slot.
//   BlockAttention      grouped-query attention with biased q, k projections, v = the un-rotated k (there is no value
//                       projection), rotation in halves, weights sigmoid(scale q.k + b_h) -- no softmax, not normalised -- over the keys
//                       of the query's own block of `block` positions, aligned to position 0.  Cache: a ring of block + (step) - 1 rows
//                       [rotated k | unrotated k] per slot.
//   LatentAttention     (Sipazen.hpp) with the queries through a latent, stretched frequencies, neighbouring rotation pairs, no sink / gate.
// Feed-forward: dense, clamped -- g = min(W_g h, L), u = clamp(W_u h, +-L), W_d (g sigmoid(alpha g) (u + 1)) -- or routed experts (MoE,
// Sipazen.hpp) chosen from sigmoid scores inside the best groups of experts.  The head's result is multiplied by logit_scale.
// The residual, norms, router, recurrence, rotation angles and attention scores are fp32; matmul inputs are written in the activation type.
// The neurons use the model's HybridScratch and SeqStateCache (Sipazen.hpp, QWen3.hpp); step function, graphs, sampler and generation loop
// are Fish's own.  The reference has no counterpart (its inference path is the Qwen3 block, QWen.cpp:16-145).
#pragma once
#include "Sedotar.hpp"

namespace koifish {

struct MinGRU : GeNeuron {
    MIXER_CARD card;
    hGTensor z, z_b, x, x_b, g, o;
    // u: stacked first projections, z | x | g at columns off[0..2]; cache: entry of the SeqStateCache that holds this run's state -> sub
    int cuInfer(int M, const float* u, int ldu, const int* off, int cache);
};
struct BlockAttention : GeNeuron {
    MIXER_CARD card;
    hGTensor q, q_b, k, k_b, pb, o;
    double* inv_freq = nullptr;  // device [rot_dims / 2]
    float amp = 1.f;
    // u: stacked first projections, q | k consecutive from column off -> sub
    int cuInfer(int M, float* u, int ldu, int off, int cache);
};
struct ClampedFF : GeNeuron {  // W_down (g sigmoid(alpha g) (u + 1)), g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit)
    MOE_CARD card;
    hGTensor gate, up, down;
    StackedLinear cat;  // gate | up
    static constexpr float kAlpha = 1.702f;
    int cuInfer(int M);  // reads hact -> sub
};
struct FzlBlock : GeNeuron {
    int layer = 0;
    GroupNorm norm1, norm2;
    StackedLinear cat;  // everything in the mixer that reads norm1(x)
    std::unique_ptr<MinGRU> gru;
    std::unique_ptr<BlockAttention> attn;
    std::unique_ptr<LatentAttention> lat;
    std::unique_ptr<ClampedFF> dense;
    std::unique_ptr<MoE> moe;
    // One run of the layer.  On entry hact = norm1(x); on return *pending is the sublayer result that is still to be added to x (nullptr:
    // x is complete).  cache: entry of the SeqStateCache for this run.
    int cuInfer(int M, int cache, const float** pending);
};

// the order in which the layers run: (layer, cache entry, pass number at the first layer of a repeated pass or -1)
struct LayerRun {
    int layer, cache, pass;
};
std::vector<LayerRun> LayerRuns(const MODEL_CARD& c);

}  // namespace koifish
