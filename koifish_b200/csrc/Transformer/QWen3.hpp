// QWen3.hpp -- host-side mirror of the reference's operator surface for Qwen3 decode / prefill:
//   MODEL_CARD / CLI_params keys   (src/CLI_params.hpp:263-385, src/Utils/CLI_params.cpp:1480-1545, 2224-2300)
//   neurons  SLP, LayerNormal, ROPE, SelfAttention, FFN, TokenEmbed, Head4Token (src/Manifold/Neuron.hpp:363-802) with the
//            cuInfer / Forw / cuFlow entry points of src/Device/CUDA/QKV.cu:617-706, NeuronFuse.cu:176-207, 305-381, 615-656,
//            842-862, T.cu:569-573, kernel/rope.cu:645-672
//   KVCache  (src/Utils/Cache.hpp:22-53, Cache.cpp:14-60)
//   QWen3 / Fish  (src/Transformer/QWen.cpp:16-145, src/Manifold/Fish.cpp:13-95, GoPT.cpp:1111-1235 Chat loop)
// plus what the reference does not have: tensor-parallel sharding (one process per GPU) and CUDA-graph replay of a token.
#pragma once
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "../Tensor/GTensor.hpp"

namespace koifish {

// ---- config -------------------------------------------------------------------------------------------------------------
// One layer of a hybrid stack (config "layers": [{"type", "mixer": {...}, "mlp": {...} | null}, ...]): which sequence mixer it has, with
// that mixer's sizes, and its feed-forward.  Layers of one model may differ in every size.
struct MIXER_CARD {
    std::string type;  // "mamba2" (state-space) | "latent_attention" | "channel_delta" | "gla" | "parallel" (attention beside a gated LRU) |
                       // "mingru" (channel-wise gated recurrence) | "attention" (sigmoid-weighted, inside blocks of positions)
    // state-space mixer: heads x vdim inner channels, state rows per head, B/C groups, gated-norm groups, convolution taps
    int heads = 0, vdim = 0, state = 0, groups = 1, norm_groups = 1, conv = 1;
    // latent attention: per head `dim` plain + `rot_dim` rotated query/key entries, values of vdim, latent rank; rotation on the first
    // rot_dims entries of the rotated part with frequencies rot_base^(-2i/rot_dims); score scale
    int dim = 0, rot_dim = 0, kv_rank = 0, rot_dims = 0;
    double rot_base = 10000.0;
    float scale = 1.f;
    // matrix-state recurrences (gated delta rule, gated linear attention): heads x vdim values, kv_heads x dim queries / keys, decay
    // temperature tau (gla), low ranks of the decay and gate projections (read from the tensors' shapes)
    int kv_heads = 0, rank_a = 0, rank_g = 0;
    float tau = 1.f;
    // attention with a logarithmic distance penalty and a query temperature t = 1 + coef * ln(floor((pos + 1) / every) + 1) (every 0: none)
    float qt_coef = 0.f;
    int qt_every  = 0;
    // real-gated linear recurrent unit beside the attention of a "parallel" mixer
    int lru_width = 0, lru_blocks = 1, lru_conv = 1;
    // rotated sliding-window attention: keys of the last `window` positions (0: all), scores capped by softcap * tanh(s / softcap) (0: not),
    // a sink term per head in the softmax, frequencies stretched between two wavelengths (yarn_factor 0: plain rot_base^(-2i/rot_dims))
    int window = 0;
    float softcap = 0.f;
    bool sink = false;
    double yarn_factor = 0.0, yarn_original = 0.0, yarn_fast = 0.0, yarn_slow = 0.0;
    // latent attention whose queries pass a latent of q_rank entries (RMS-normed) before their up-projection (0: projected directly)
    int q_rank = 0;
    // sigmoid-weighted attention: a query sees the keys of its own block of `block` consecutive positions, aligned to position 0 (0: all)
    int block = 0;
    // channel-wise gated recurrence (minGRU): channels of the state
    int width = 0;
    // two mixers side by side that read the same input (Sedotar's "parallel"): this card is the left one, `right` the other; the result is
    // left_scale * left + right_scale * right
    std::shared_ptr<MIXER_CARD> right;
    float left_scale = 1.f, right_scale = 1.f;
};
struct MOE_CARD {
    bool present = false;
    bool dense   = false;  // one feed-forward of width ff with biases instead of routed experts
    int experts = 0, top = 0, ff = 0;
    int shared_ff = 0;  // 0: no shared expert
    float limit = 0.f;  // dense, clamped form: gate <= limit, |up| <= limit (0: the feed-forward is not of that form)
    // routing from sigmoid scores: selection over score + a learned correction inside the `keep` best of `groups` groups of neighbouring
    // experts, weights route_scale * score, not renormalised (sigmoid_route false: softmax routing)
    bool sigmoid_route = false;
    int groups = 1, keep = 1;
    float route_scale = 1.f;
};
struct LAYER_CARD {
    MIXER_CARD mixer;
    MOE_CARD mlp;
};

struct MODEL_CARD {
    std::string arch = "QWEN3";
    int n_layers = 0, n_embd = 0, n_ff = 0, n_head = 0, n_head_kv = 0, head_dim = 128;
    int vocab = 151936;  // pad_vocab_size, CLI_params.hpp:327
    int max_pos_embeddings = 32768, n_ctx = 1024;
    int max_seq_len  = 1024;  // chat_sampler.seq_len default, CLI_params.hpp:697 ; JSON gpt.max_seq_len
    float rope_theta = 10000.f;  // random-init default (Neuron.cpp:612-620); HF card: config.json rope_theta
    float norm_rms_eps = 1e-6f;  // QWen.cpp:16-58
    bool tie_word_embeddings = false;
    bool isQKNormal = true, isSeparateQKV = true;  // QWen3 flags (QWen.cpp:16-58)
    JSON jQuant;                                    // the "quantizer" block
    int seed = 42;
    float init_sigma = 0.02f, norm_sigma = 0.0f;  // huTensor.cu:204 ; norms FIX_1
    int max_batch = 1;                            // independent sequences (batched decode)
    int max_prefill = 64;                         // tokens per prefill panel (gpt.max_prefill): sizes the activation buffers
    int awq_repack  = 0;                          // gpt.awq_repack: vendor AWQ tensors re-laid-out at load into PackedQ 4-bit storage (fast kernels)
    // hybrid stacks (arch SIPAZEN): per-layer cards, grouped RMS norm, residual multiplier; fp32 residual stream
    std::vector<LAYER_CARD> layers;
    int norm_groups     = 1;
    float residual_mult = 1.f;
    bool compute_f32    = false;  // gpt.compute_dtype = "float32": activations, caches and matmuls in true 32-bit (hybrid stacks only)
    int logit_rows_cfg  = 0;      // gpt.logit_rows: rows of the logits buffers (default max(64, max_batch))
    float embed_scale   = 1.f;    // the embedding row is multiplied by this
    int side_dim        = 0;      // per-layer token input: entries of the side embedding that each layer reads (0: none)
    // layers loop_start .. loop_stop - 1 run loop_times times in a row on the same weights, each pass with a cache / state of its own
    int loop_start = 0, loop_stop = 0, loop_times = 1;
    float logit_scale = 1.f;      // the head's result is multiplied by this
    bool IsHybrid() const { return !layers.empty(); }

    // accepts a Koifish JSON (cases/qwen3/*.json layout) or an HF config.json, optionally wrapped as {"hf_config": {...}}
    static MODEL_CARD FromJSON(const JSON& j);
    int q_dim() const { return n_head * head_dim; }
    int kv_dim() const { return n_head_kv * head_dim; }
};

struct Fish;
struct HybridScratch;  // Sipazen.hpp
bool ShardPlan(const MODEL_CARD& c, const std::string& name, int rank, int world, int* rows_g, int* cols_g, int* rows_l, int* cols_l, int* row0,
               int* col0);

size_t AwqRepackBytes(int OCl, int ICl);
void AwqRepackWindow(const void* qweight, const void* qzeros, const void* scales, int IC, int OC, int r0, int OCl, int c0, int ICl, uint8_t* out_blob);
void AwqShardWindow(const void* qweight, const void* qzeros, const void* scales, int IC, int OC, int r0, int OCl, int c0, int ICl, uint8_t* out_blob);

// ---- neurons --------------------------------------------------------------------------------------------------------------
struct GeNeuron {
    std::string name;
    Fish* hFish = nullptr;
    virtual ~GeNeuron() {}
};
// SLP: linear neuron, y = x W^T (src/Manifold/Neuron.hpp:404; SLP::Forw NeuronFuse.cu:305-381)
struct SLP : GeNeuron {
    hGTensor w;
    int nIn = 0, nOut = 0;
    bool Empty() const { return !w; }
    // rhs[M][nOut] = lhs[M][nIn] . W^T ; epilogue: KF_EPI_*; returns KF status
    int Forw(void* rhs, const void* lhs, int M, int epilogue = KF_EPI_NONE, const void* residual = nullptr);
};
struct LayerNormal : GeNeuron {
    hGTensor w;
    float rms_eps = 1e-6f;
    int cuFlow(void* out, const void* inp, int rows);  // chat branch -> CU_rms_infer (T.cu:569-573)
};
struct SelfAttention;
struct ROPE : GeNeuron {
    hGTensor q_norm, k_norm;  // hnQ / hnK
    void* table = nullptr;    // (cos, sin)[max_seq][hd/2]
    float theta = 10000.f;
    int cuInfer(SelfAttention* hQKV, int M);  // rope.cu:645-672
};
struct SelfAttention : GeNeuron {
    int layid = 0;  // 1-based like the reference (QKV.cu:630 uses layid - 1)
    LayerNormal norm;
    SLP Q, K, V, proj_cat;
    ROPE rope;
    int n_head = 0, n_head_kv = 0, head_dim = 0;  // LOCAL (per tensor-parallel rank) head counts
    int cuInfer(void* inpL /* x in/out [M][E] */, int M);  // QKV.cu:617-706
};
struct FFN : GeNeuron {
    int layid = 0;
    LayerNormal norm;
    SLP gate, up, down;
    int latent = 0;  // LOCAL ffn width
    int cuInfer(void* inpL, int M);  // NeuronFuse.cu:615-656
};
struct TokenEmbed : GeNeuron {
    hGTensor w;
    int cuInfer(void* out, int M);  // NeuronFuse.cu:176-207
};
struct Head4Token : GeNeuron {
    LayerNormal norm;  // the final model.norm (a separate LayerNormal neuron in the reference graph)
    SLP proj;
    int cuInfer_1(void* logits, const void* inp, int M);  // NeuronFuse.cu:842-862
};
// KVCache: two bf16 tensors [nLayer][max_batch][max_seq][kv_dim_local] (Cache.cpp:14-27 has no batch dimension)
struct KVCache {
    void *key = nullptr, *value = nullptr;
    int n_layer = 0, max_batch = 1, max_seq = 0, kv_dim = 0;
    enum CTYPE { KV_KEY, KV_VAL };
    void* Get(CTYPE t, int layer, int pos = 0, int seq = 0) const;  // Cache.cpp:43-58
    size_t seq_stride() const { return (size_t)max_seq * kv_dim; }
    size_t bytes() const { return (size_t)2 * n_layer * max_batch * max_seq * kv_dim * 2; }
};

// Cache and state of a hybrid stack, per layer and per sequence slot: an attention layer keeps one row per position (latent + shared
// rotated key, in the activation type), a state-space layer a fixed-size fp32 state (heads x vdim x state) plus the last conv - 1 inputs
// of its convolution.  Slots are handed out and taken back by Acquire / Release; a slot is not cleared on reuse: its first token has
// position 0 and the kernels start from zero there.
struct SeqStateCache {
    struct Layer {
        void* rows = nullptr;      // [max_batch][max_seq][row_dim]
        size_t row_stride = 0;     // elements per slot
        int row_dim = 0;
        float* state = nullptr;    // [max_batch][state_stride]
        size_t state_stride = 0;
        float* tail = nullptr;     // [max_batch][tail_stride]
        size_t tail_stride = 0;
        int ring = 0;              // > 0: the rows of a slot are a ring of this many positions (position p in row p % ring), not max_seq rows
    };
    std::vector<Layer> layers;
    int max_batch = 1, max_seq = 0;
    bool f32 = false;
    size_t total_bytes = 0;
    std::vector<int> free_slots;  // LIFO: the slot released last is handed out next
    void InitSlots(int n);
    int Acquire();             // -1: none free
    bool Release(int slot);    // false: not a slot in use
};

// ---- model registry: one entry per architecture name (config "architecture" / model.arch) -----------------------------------------
struct ARCH_ENTRY {
    const char* name;                                    // upper case
    void (*parse)(const JSON& hf_or_root, MODEL_CARD& card);  // fills the card from the config (nullptr: the Qwen3 keys)
    int (*build)(Fish& f);                               // tensors, neurons, caches, activation buffers
    int (*forward)(Fish& f, int M, bool want_logits);    // one step over the staged tokens
    int (*prepare)(Fish& f);                             // after every tensor has data (device pointer tables); may be nullptr
};
const ARCH_ENTRY* FindArch(const std::string& name);
const ARCH_ENTRY* SipazenArch();  // Sipazen.cpp
const ARCH_ENTRY* KivoraxArch();  // Kivorax.cpp
const ARCH_ENTRY* SedotarArch();  // Sedotar.cpp
const ARCH_ENTRY* FazolornArch(); // Fazolorn.cpp

// ---- the model ------------------------------------------------------------------------------------------------------------
struct Fish {
    kf_ctx* ctx = nullptr;
    MODEL_CARD config;
    int tp_rank = 0, tp_world = 1;
    TokenEmbed embed;
    std::vector<std::unique_ptr<SelfAttention>> attn;
    std::vector<std::unique_ptr<FFN>> ffn;
    Head4Token cls;
    KVCache cache;
    const ARCH_ENTRY* arch = nullptr;
    std::vector<std::unique_ptr<GeNeuron>> blocks;  // hybrid stacks: one block neuron per layer
    SeqStateCache states;                           // ... and their cache / state manager
    std::shared_ptr<HybridScratch> hscratch;        // ... and their shared activation buffers
    std::vector<void*> owned;                       // device buffers of the architecture's own (freed with the model)
    int32_t *d_slot = nullptr, *d_sel = nullptr;    // per token: sequence slot; per logits row: the token it is taken from
    float* logits_f32 = nullptr;                    // hybrid stacks: fp32 logits [logit_rows][vocab]
    float* h_logits_f32 = nullptr;                  // pinned
    int n_rows = 0;                                 // logits rows of the current step
    bool tables_ready = false;                      // arch->prepare ran since the last tensor change
    std::map<std::string, hGTensor> tensors;  // by HF name (NN2NAME, QWen.cpp:61-145)
    std::map<std::string, int> tensor_ids;    // synthetic-weight seed ids (shared definition with the test oracle)

    // activations (views into one scratch allocation, like gBUFF; huTensor.cu:922-1003)
    int max_tokens = 0;
    void *x = nullptr, *xb = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *hb = nullptr, *logits = nullptr;
    float* part_f32 = nullptr;
    int32_t *d_tokens = nullptr, *d_pos = nullptr, *d_next = nullptr;
    // CHAT_SAMPLER (CLI_params.hpp:663-719): temperature 0 = greedy; d_rng = one xorshift64* state per sequence row
    float samp_temperature = 0.f, samp_top_p = 0.95f;
    int samp_top_k = 50, samp_selection = 0;
    uint64_t* d_rng = nullptr;
    int SetSampler(float temperature, int top_k, float top_p, uint64_t seed, int selection);
    int PickNext(int rows);  // d_next[r] = argmax or a sample of logits row r
    int32_t* h_stage  = nullptr;  // pinned staging: tokens | pos | next
    uint16_t* h_logits = nullptr; // pinned
    int seq_mode = 0;             // 0: the M tokens of a forward are one sequence (prefill) ; 1: M independent sequences
    int gqa_min_batch = 0;        // > 0: batched decode from this many sequences uses kf_attn_decode_gqa (env KF_GQA_MIN_BATCH, sweeps); 0: rule in cuInfer
    int logit_rows = 0;           // rows of the logits buffers (max(64, max_batch)); bigger panels report the last token only
    bool panel_consecutive = false;  // prefill panel at positions pos[0] .. pos[0] + M - 1 -> tensor-core flash attention
    bool last_only = false;       // mode 2: logits / argmax of the last token of the panel only
    bool tp_fuse = false;         // this forward runs the exchange as the epilogue of O / down (tensor parallel, <= 8 tokens, peer buffers)
    int attn_hint = 0;            // upper bound of the positions of the current forward (power-of-two bucket - 1): sizes the attention split
    int CtxBucket() const;        // log2 of that bucket; part of the graph key, so graphs are re-captured as the context grows
    std::map<uint64_t, kf_graph*> graphs;  // per (M, mode) replayable token graphs
    std::set<uint64_t> warm;               // signatures that already ran eagerly once (workspaces sized) -> next call captures
    bool use_graphs = true;
    void* rope_table_shared = nullptr;
    int staged_pos_max = 0;
    int staged_M       = 0;      // tokens / positions staged on the device by the last Forward() (0: nothing staged yet)
    uint64_t graph_gen = 0;      // kf_scratch_generation() the captured graphs were recorded under
    void SyncGraphGeneration();  // drop the graphs when a context scratch buffer they point to has been re-allocated since
    std::string error;
    size_t weight_bytes = 0;
    bool weights_dirty  = true;  // weight_bytes must be recounted (set by ResetGraphs, which every tensor-changing path calls)

    Fish(kf_ctx* ctx, const MODEL_CARD& card, int tp_rank, int tp_world);
    ~Fish();
    int BuildQwen3();
    int ForwardQwen3(int M, bool want_logits);
    int Build();                 // allocate tensors + buffers (Fish::MakeInstance -> Build, Fish.cpp:13-95)
    int InitParamRandom();       // huTensor::InitParam random path + quantise at load
    int SetTensor(const std::string& hf_name, const void* host_bf16, int rows, int cols);  // SERIALIZE path: full (unsharded) tensor
    // vendor AWQ arrays of one linear (full shape), cut to this rank's window and kept in the vendor layout (GeQuant::ExTensor, GeQuant.cpp:144-200)
    int SetTensorAWQ(const std::string& hf_name, const void* qweight_i32, const void* qzeros_i32, const void* scales_f16, int in_features, int out_features);
    bool all_resident = false;  // every tensor has device data (checked once by Forward)
    hGTensor GetTensor(const std::string& hf_name) const;
    // one forward over M tokens already staged in d_tokens / d_pos (ForwardOnRLS, gLLM.cpp:755-769); logits for all M rows
    int ForwardOnRLS(int M, bool want_logits);
    // public step: host tokens/pos in, logits (optional) + greedy next tokens (optional) out.  H2D/D2H inside.
    int Forward(const int32_t* tokens, const int32_t* pos, int M, int seq_mode, uint16_t* logits_out, int32_t* next_out);
    // the same step with a sequence slot (modes 0 / 2; mode 1 uses slots 0 .. M-1), an optional choice of logits rows (sel: indices into
    // the M tokens, n_sel <= logit_rows) and fp32 logits (hybrid stacks).  Forward() is ForwardEx(slot 0, all rows).
    int ForwardEx(const int32_t* tokens, const int32_t* pos, int M, int seq_mode, int slot, const int32_t* sel, int n_sel, uint16_t* logits_out,
                  float* logits_f32_out, int32_t* next_out);
    // the resident tensors exactly as they sit in HBM (data || gama per tensor): SerialGamaData, reference huTensor.cu:413-458
    int SaveBlobs(const std::string& path);
    int LoadBlobs(const std::string& path);
    // the reference's own container (fish.kun, CKP_KOIFISH): the same payloads behind a safetensors header with szData / szGama per tensor
    int SaveKun(const std::string& path, const std::string& config_json);
    int LoadKun(const std::string& path, int* n_loaded, int* n_skipped);
    // Fish::Chat's generation loop (GoPT.cpp:1111-1235): prefill, then sample / stop on eos or a full window / feed back.  stop_reason: 1 eos,
    // 2 max_new tokens produced, 3 context window full
    int Generate(const int32_t* prompt, int n_prompt, int pos0, int max_new, int eos_id, int32_t* out, int* n_out, int* stop_reason);
    // device-resident greedy loop: n_steps graph replays feeding argmax back as the next token (no host round trip)
    int DecodeLoop(int n_steps, int M);
    uint64_t UseGraph(int M, bool want_logits);
    void ResetGraphs();
    int AllocTensor(const std::string& name, int rows, int cols, int id, hGTensor& out);
};

}  // namespace koifish
