// Sedotar.hpp -- neurons of the Sedotar stack.  A layer normalises what a sublayer RETURNS, not what it reads:
//     x += norm1(mixer(x)),   x += norm2(ff(x)),      norm(y) = y / rms(y) * (1 + w)
// so the sublayers read the residual stream itself (written in the activation type by the step that updated it).  The mixer is a pair
// that reads the same input:  left_scale * WindowAttention(x) + right_scale * ScalarDeltaMixer(x).
//   WindowAttention    q, k, v projections, a short causal convolution on each, RMS norm over the WHOLE q row and the whole k row,
//                      rotation of the first rot_dims entries of every head (interleaved pairs, frequencies stretched between two
//                      wavelengths), scores capped by tanh, the last `window` keys only, a sink term per head in the softmax.  Its keys
//                      and values live in a ring of window + (step size) - 1 rows per sequence slot.
//   ScalarDeltaMixer   the gated delta rule with ONE decay per head and token, exp(-e^A softplus(W_a x + dt_bias)), short convolutions
//                      with SiLU on q, k, v, unit q / k, write strength sigmoid(W_b x); per-head RMS norm of the read-out times
//                      silu(W_g x).  Its state [heads][vdim][dim] is fp32 per sequence slot.
// The feed-forward is W_down(relu(W_gate x) * (W_up x)).  The head is the embedding table itself.  The residual, norms, decays, the
// recurrence, rotation angles, scores and the softmax are fp32; matmul inputs are written in the activation type.  The neurons use the
// model's HybridScratch and SeqStateCache (Sipazen.hpp, QWen3.hpp); step function, graphs, sampler and generation loop are Fish's own.
// The reference has no counterpart (its inference path is the Qwen3 block, QWen.cpp:16-145).
#pragma once
#include "Sipazen.hpp"

namespace koifish {

struct WindowAttention : GeNeuron {
    MIXER_CARD card;
    int layer = 0;
    hGTensor q, k, v, qn, kn, qc, kc, vc, sink, o;
    StackedLinear convs;          // q.conv | k.conv | v.conv as one [channels][taps] table
    double* inv_freq = nullptr;   // device [rot_dims / 2], stretched frequencies
    float amp = 1.f;              // multiplies cosine and sine
    size_t tail_off = 0;          // where this mixer's convolution inputs start inside the layer's tail region
    // u: the stacked first projections, q | k | v at column off; out_scale * (attended values) go to out [M][ldo] in the activation type
    int cuInfer(int M, const float* u, int ldu, int off, void* out, int ldo, float out_scale);
};
struct ScalarDeltaMixer : GeNeuron {
    MIXER_CARD card;
    int layer = 0;
    hGTensor q, k, v, qc, kc, vc, b, a, A_log, dt_bias, norm, g, o;
    StackedLinear convs;
    size_t tail_off = 0;
    // off: columns of q (k, v follow), b, a, g in u; out_scale * (gated, normed read-out) goes to out [M][ldo] in the activation type
    int cuInfer(int M, const float* u, int ldu, const int* off, void* out, int ldo, float out_scale);
};
struct GatedFF : GeNeuron {  // down(act(gate x) * (up x)), act = relu
    MOE_CARD card;
    hGTensor gate, up, down;
    StackedLinear cat;  // gate | up
};
// Several weights whose results are ADDED, stacked column-wise into ONE matrix at load: y = [W_a | W_b] [x_a ; x_b] = W_a x_a + W_b x_b in
// one launch; the producers write x_a and x_b side by side at off[i] of a row of `cols` entries.
struct SummedLinear {
    void* w = nullptr;  // device bf16 [rows][cols]
    int rows = 0, cols = 0;
    std::vector<hGTensor> parts;
    std::vector<int> off;
    void Plan(const std::vector<hGTensor>& tensors);
    int Fill(kf_ctx* ctx) const;
};
struct SedotarBlock : GeNeuron {
    int layer = 0;
    GroupNorm norm1, norm2;
    StackedLinear cat;  // everything that reads x in the mixer: left q k v, right q k v b a g
    SummedLinear out;   // left o | right o: the branch scales ride on the branches' outputs, so one matmul forms a_l W_l y_l + a_r W_r y_r
    std::vector<int> off;
    std::unique_ptr<WindowAttention> left;
    std::unique_ptr<ScalarDeltaMixer> right;
    std::unique_ptr<GatedFF> ff;
    int cuInfer(int M);
};

// frequencies of a rotation over `dims` entries with base `base`, stretched by `factor` beyond the wavelength original / slow and left alone
// below original / fast, a linear ramp between (factor <= 0: plain base^(-2i/dims)); *amp = 0.1 ln(factor) + 1 (1 when not stretched)
std::vector<double> StretchedFrequencies(int dims, double base, double factor, double original, double fast, double slow, float* amp);

}  // namespace koifish
