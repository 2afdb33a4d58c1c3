// linrec.cu -- linear-recurrence sequence mixers beside the selective scan of seqmix.cu:
//   (1) matrix-state recurrences with a decay per key channel: per head an fp32 state S [dk x dv] and, per token,
//           S <- diag(g_t) S ;  then either   S <- S + k_t v_t^T                                   (gated linear attention)
//                                     or      u = beta_t (v_t - S^T k_t),  S <- S + k_t u^T        (gated delta rule)
//       and o_t = S^T q_t, taken after the write of token t.  The decay is formed in fp32 from a logit z while the
//       token is staged: g = sigmoid(z + b)^(1/tau), or g = exp(-exp(A_h) softplus(z + b)).  q and k may be made unit vectors per head.
//   (2) a real-gated linear recurrent unit over channels: block-diagonal gate matmuls r, i = sigmoid(W u_b + b), decay
//       a = exp(-c r softplus(lam)), state s <- a s + sqrt(1 - a^2) i u, output s * y.
// State lives in fp32 per (sequence slot, layer) and persists between calls; a slot whose first staged token has position 0 starts
// from zero without a clearing pass.  Tokens are nseq sequences of T consecutive tokens (prefill panel 1 x M, batched decode M x 1).
// No reference equivalent (the reference's inference path is the Qwen3 attention block only).
#include <math.h>

#include <algorithm>

#include "kf_common.cuh"

namespace {
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float log_sigmoid_f(float z) { return z >= 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) { return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }

struct ScanArgs {
    float* y;          // [M][ldy] heads x dv
    int ldy;
    const float *q, *k, *v, *z, *beta;  // fp32 rows; q / k: kv-head major [G][dk]; v: [H][dv]; z: [H][dk]; beta logits [H] (delta only)
    int ldq, ldk, ldv, ldz, ldb;
    const uint16_t* zbias;   // bf16 [H * dk]
    const uint16_t* A_log;   // bf16 [H] (decay kind 1)
    float* state;            // [slot][H][dv][dk]
    size_t state_stride;
    const int32_t *pos, *slot;
    int T, H, G, dk, dv;
    int R, PB, TB, dkp;      // dkp: padded length of a staged row
    int delta;               // 1: delta-rule write, 0: plain outer-product write
    int decay_kind;          // 0: sigmoid(z + b)^(1/tau) ; 1: exp(-exp(A_h) softplus(z + b))
    int unit_qk;             // q, k divided by sqrt(sum x^2 + unit_eps) per head
    int z_head;              // 1: one decay per head and token (z: [H], zbias: [H]) shared by the head's key channels
    float inv_tau, q_scale, unit_eps;
};

// grid (heads, sequences, column chunks).  Thread (pl, r) keeps the NPT (16 or 8) consecutive rows n = r * NPT + i of state column p0 + pl in
// registers; the R lanes of a column are adjacent and reduce with shuffles.  TB tokens are staged in shared memory per pass: k, q
// (normalised there), the decay (formed there), v, beta.  FULL (dk == R * NPT): a thread's slice of k, q and the decay is NPT / 4 16-byte
// shared loads each and nothing is bounds-checked; otherwise rows beyond dk read k = q = 0 and leave their (zero) state alone.
constexpr int NPT_MAX = 16;
template <bool DELTA, bool FULL, int NPT>
__global__ void __launch_bounds__(256) kf_gated_scan_kernel(ScanArgs a) {
    extern __shared__ __align__(16) float sm[];
    // staged rows are padded by 4 floats after every 16: the R lanes of a column read slices 20 floats apart, which fall into different
    // banks (slices exactly 16 apart would collide two by two)
    const int dk = a.dk, TB = a.TB, PB = a.PB, R = a.R, dkp = a.dkp;
    auto ix = [](int n) { return n + ((n >> 4) << 2); };
    float* sK = sm;                  // [TB][dkp]
    float* sQ = sK + TB * dkp;       // [TB][dkp]
    float* sG = sQ + TB * dkp;       // [TB][dkp]
    float* sV = sG + TB * dkp;       // [TB][PB]
    float* sB = sV + TB * PB;        // [TB]
    float* sKQ = sB + TB;            // [TB] k . q of the staged (normalised, scaled) rows: the delta rule's read-out needs it
    const int h = blockIdx.x, seq = blockIdx.y, p0 = blockIdx.z * PB;
    const int kh = h / (a.H / a.G);
    const int tid = threadIdx.x, pl = tid / R, r = tid - pl * R, p = p0 + pl;
    const bool live = pl < PB && p < a.dv;
    const int m0 = seq * a.T, n0 = r * NPT;
    float* st = a.state + (size_t)a.slot[m0] * a.state_stride + ((size_t)h * a.dv + (live ? p : 0)) * dk;
    const bool fresh = a.pos[m0] == 0;
    float S[NPT];
#pragma unroll
    for (int i = 0; i < NPT; i++) S[i] = (live && n0 + i < dk && !fresh) ? st[n0 + i] : 0.f;
    const float Aexp = a.decay_kind == 1 ? expf(bf16_bits_to_f32(a.A_log[h])) : 0.f;
    const bool zh = a.z_head != 0;  // one decay per head and token: formed once per staged token (sG[tt]), not per key channel
    const int warp = tid >> 5, lane = tid & 31, nwarp = blockDim.x >> 5;
    for (int t0 = 0; t0 < a.T; t0 += TB) {
        const int nt = min(TB, a.T - t0);
        __syncthreads();
        // four elements per thread and step: their global loads are issued together, then the decays are formed
        for (int i0 = tid; i0 < nt * dk; i0 += 4 * blockDim.x) {
            float kv[4], qv[4], zv[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = i0 + e * blockDim.x;
                if (i < nt * dk) {
                    const int tt = i / dk, n = i - tt * dk;
                    const size_t m = (size_t)(m0 + t0 + tt);
                    kv[e] = a.k[m * a.ldk + kh * dk + n], qv[e] = a.q[m * a.ldq + kh * dk + n];
                    if (!zh) zv[e] = a.z[m * a.ldz + h * dk + n] + (a.zbias ? bf16_bits_to_f32(a.zbias[h * dk + n]) : 0.f);
                }
            }
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = i0 + e * blockDim.x;
                if (i < nt * dk) {
                    const int tt = i / dk, o = tt * dkp + ix(i - tt * dk);
                    sK[o] = kv[e], sQ[o] = qv[e];
                    if (!zh) sG[o] = a.decay_kind == 1 ? expf(-Aexp * softplus_f(zv[e])) : expf(log_sigmoid_f(zv[e]) * a.inv_tau);
                }
            }
        }
        if (zh)
            for (int i = tid; i < nt; i += blockDim.x) {
                const float z = a.z[(size_t)(m0 + t0 + i) * a.ldz + h] + (a.zbias ? bf16_bits_to_f32(a.zbias[h]) : 0.f);
                sG[i] = a.decay_kind == 1 ? expf(-Aexp * softplus_f(z)) : expf(log_sigmoid_f(z) * a.inv_tau);
            }
        for (int i0 = tid; i0 < nt * PB; i0 += 4 * blockDim.x) {
            float vv[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int i = i0 + e * blockDim.x, tt = i / PB, c = i - tt * PB;
                vv[e] = (i < nt * PB && p0 + c < a.dv) ? a.v[(size_t)(m0 + t0 + tt) * a.ldv + h * a.dv + p0 + c] : 0.f;
            }
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (i0 + e * blockDim.x < nt * PB) sV[i0 + e * blockDim.x] = vv[e];
        }
        if (DELTA)
            for (int i = tid; i < nt; i += blockDim.x) sB[i] = sigmoid_f(a.beta[(size_t)(m0 + t0 + i) * a.ldb + h]);
        __syncthreads();
        // unit vectors / query scale: one warp per staged token
        for (int tt = warp; tt < nt; tt += nwarp) {
            float sq = 0.f, sk = 0.f;
            if (a.unit_qk) {
                for (int n = lane; n < dk; n += 32) sq = fmaf(sQ[tt * dkp + ix(n)], sQ[tt * dkp + ix(n)], sq), sk = fmaf(sK[tt * dkp + ix(n)], sK[tt * dkp + ix(n)], sk);
                sq = warp_sum(sq), sk = warp_sum(sk);
            }
            const float fq = a.unit_qk ? a.q_scale / sqrtf(sq + a.unit_eps) : a.q_scale;
            const float fk = a.unit_qk ? 1.f / sqrtf(sk + a.unit_eps) : 1.f;
            float kq = 0.f;
            for (int n = lane; n < dk; n += 32) {
                const float qn = sQ[tt * dkp + ix(n)] * fq, kn = sK[tt * dkp + ix(n)] * fk;
                sQ[tt * dkp + ix(n)] = qn;
                if (a.unit_qk) sK[tt * dkp + ix(n)] = kn;
                kq = fmaf(kn, qn, kq);
            }
            if (DELTA) {
                kq = warp_sum(kq);
                if (lane == 0) sKQ[tt] = kq;
            }
        }
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {
            float kk[NPT], qq[NPT], gg[NPT];
            if (FULL) {
                const float4* k4 = reinterpret_cast<const float4*>(sK + tt * dkp + ix(n0));
                const float4* q4 = reinterpret_cast<const float4*>(sQ + tt * dkp + ix(n0));
                const float4* g4 = reinterpret_cast<const float4*>(sG + tt * dkp + ix(n0));
#pragma unroll
                for (int j = 0; j < NPT / 4; j++) {
                    const float4 kv = k4[j], qv = q4[j];
                    kk[4 * j] = kv.x, kk[4 * j + 1] = kv.y, kk[4 * j + 2] = kv.z, kk[4 * j + 3] = kv.w;
                    qq[4 * j] = qv.x, qq[4 * j + 1] = qv.y, qq[4 * j + 2] = qv.z, qq[4 * j + 3] = qv.w;
                }
                if (zh) {
                    const float gh = sG[tt];
#pragma unroll
                    for (int i = 0; i < NPT; i++) gg[i] = gh;
                } else {
#pragma unroll
                    for (int j = 0; j < NPT / 4; j++) {
                        const float4 gv = g4[j];
                        gg[4 * j] = gv.x, gg[4 * j + 1] = gv.y, gg[4 * j + 2] = gv.z, gg[4 * j + 3] = gv.w;
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < NPT; i++) {
                    const bool in = n0 + i < dk;
                    const int o = tt * dkp + ix(n0 + i);
                    kk[i] = in ? sK[o] : 0.f, qq[i] = in ? sQ[o] : 0.f, gg[i] = in ? sG[zh ? tt : o] : 1.f;
                }
            }
            const float vv = sV[tt * PB + (pl < PB ? pl : 0)];
            float w = vv;
            if (DELTA) {
                // With D = diag(g) S the write is S' = D + k w^T, so the read-out S'^T q = D^T q + (k . q) w: both sums run over D in ONE pass
                // (two independent chains, their cross-lane sums interleaved) instead of a second pass over S' that waits for w.
                float d[4] = {0.f, 0.f, 0.f, 0.f}, e[4] = {0.f, 0.f, 0.f, 0.f};  // four partial sums each: the chains are 4 deep, not 16
#pragma unroll
                for (int i = 0; i < NPT; i++) {
                    S[i] *= gg[i];
                    d[i & 3] = fmaf(S[i], kk[i], d[i & 3]);
                    e[i & 3] = fmaf(S[i], qq[i], e[i & 3]);
                }
                float dot = (d[0] + d[1]) + (d[2] + d[3]), rd = (e[0] + e[1]) + (e[2] + e[3]);
                for (int o = R >> 1; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o), rd += __shfl_xor_sync(0xffffffffu, rd, o);
                w = sB[tt] * (vv - dot);
#pragma unroll
                for (int i = 0; i < NPT; i++) S[i] = fmaf(kk[i], w, S[i]);
                if (live && r == 0) a.y[(size_t)(m0 + t0 + tt) * a.ldy + h * a.dv + p] = fmaf(sKQ[tt], w, rd);
                continue;
            }
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < NPT; i++) {
                S[i]     = fmaf(gg[i], S[i], kk[i] * w);
                c[i & 3] = fmaf(S[i], qq[i], c[i & 3]);
            }
            float acc = (c[0] + c[1]) + (c[2] + c[3]);
            for (int o = R >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (live && r == 0) a.y[(size_t)(m0 + t0 + tt) * a.ldy + h * a.dv + p] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NPT; i++)
            if (n0 + i < dk) st[n0 + i] = S[i];
    }
}

// ------------------------------------------------------------------------------------------------------------ real-gated LRU
// Gates of TT tokens x 128 output channels of one block b:  r = sigmoid(Wr[b] u_b + br), i = sigmoid(Wi[b] u_b + bi), fp32 FMAs over
// the bf16 weights (staged transposed through shared memory so that every weight is read once per TT tokens); then
//   a = exp(-c r softplus(lam)),  A[m][ch] = a,  Bv[m][ch] = sqrt(1 - a^2) i u.
constexpr int GT = 8;
__global__ void __launch_bounds__(128) kf_rglru_gates_kernel(float* __restrict__ A, float* __restrict__ Bv, const float* __restrict__ u, int ldu,
                                                             const uint16_t* __restrict__ Wr, const uint16_t* __restrict__ br, const uint16_t* __restrict__ Wi,
                                                             const uint16_t* __restrict__ bi, const uint16_t* __restrict__ lam, int M, int width, int bs,
                                                             float c) {
    __shared__ float su[GT][32];
    __shared__ float swr[32][129], swi[32][129];
    const int m0 = blockIdx.x * GT, b = blockIdx.y, o0 = blockIdx.z * 128, o = o0 + threadIdx.x;
    const int nt = min(GT, M - m0);
    const uint16_t* wr = Wr + (size_t)b * bs * bs;
    const uint16_t* wi = Wi + (size_t)b * bs * bs;
    float ar[GT], ai[GT];
#pragma unroll
    for (int t = 0; t < GT; t++) ar[t] = ai[t] = 0.f;
    for (int i0 = 0; i0 < bs; i0 += 32) {
        __syncthreads();
        for (int e = threadIdx.x; e < 128 * 32; e += 128) {
            const int oo = e >> 5, ii = e & 31;
            const bool ok = o0 + oo < bs && i0 + ii < bs;
            swr[ii][oo] = ok ? bf16_bits_to_f32(wr[(size_t)(o0 + oo) * bs + i0 + ii]) : 0.f;
            swi[ii][oo] = ok ? bf16_bits_to_f32(wi[(size_t)(o0 + oo) * bs + i0 + ii]) : 0.f;
        }
        for (int e = threadIdx.x; e < GT * 32; e += 128) {
            const int t = e >> 5, ii = e & 31;
            su[t][ii] = (t < nt && i0 + ii < bs) ? u[(size_t)(m0 + t) * ldu + b * bs + i0 + ii] : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int ii = 0; ii < 32; ii++) {
            const float w1 = swr[ii][threadIdx.x], w2 = swi[ii][threadIdx.x];
#pragma unroll
            for (int t = 0; t < GT; t++) ar[t] = fmaf(w1, su[t][ii], ar[t]), ai[t] = fmaf(w2, su[t][ii], ai[t]);
        }
    }
    if (o >= bs) return;
    const int ch = b * bs + o;
    const float sp = softplus_f(bf16_bits_to_f32(lam[ch])), b1 = bf16_bits_to_f32(br[ch]), b2 = bf16_bits_to_f32(bi[ch]);
#pragma unroll
    for (int t = 0; t < GT; t++) {
        if (t >= nt) break;
        const float rg = sigmoid_f(ar[t] + b1), ig = sigmoid_f(ai[t] + b2);
        const float la = -c * rg * sp;
        const size_t m = (size_t)(m0 + t);
        A[m * width + ch]  = expf(la);
        Bv[m * width + ch] = sqrtf(-expm1f(2.f * la)) * ig * u[m * ldu + ch];
    }
}
// s <- A s + Bv along the T tokens of a sequence, out = s * gelu_tanh(y + yb) in the activation type.  A CTA owns 32 channels (one per
// lane) and its W warps each a run of consecutive tokens: a first pass reduces every run to one affine map s -> P s + B, the maps of the
// earlier runs give a warp its incoming state, a second pass replays the run and writes.  Loads are 128-byte rows across the lanes.
constexpr int LRU_W = 16;
template <typename TO>
__global__ void __launch_bounds__(32 * LRU_W) kf_rglru_scan_kernel(TO* __restrict__ out, int ldo, const float* __restrict__ A, const float* __restrict__ Bv,
                                                                   const float* __restrict__ y, int ldy, const uint16_t* __restrict__ yb,
                                                                   float* __restrict__ state, size_t state_stride, const int32_t* __restrict__ pos,
                                                                   const int32_t* __restrict__ slot, int T, int width) {
    __shared__ float sP[LRU_W][32], sB[LRU_W][32];
    const int seq = blockIdx.y, lane = threadIdx.x & 31, w = threadIdx.x >> 5, W = blockDim.x >> 5;
    const int ch = blockIdx.x * 32 + lane, m0 = seq * T;
    const bool live = ch < width;
    const int run = (T + W - 1) / W, t_lo = min(T, w * run), t_hi = min(T, t_lo + run);
    float* st = state + (size_t)slot[m0] * state_stride + (live ? ch : 0);
    float s = (pos[m0] == 0 || !live) ? 0.f : *st;
    float P = 1.f, B = 0.f;
    if (W > 1 && live) {
#pragma unroll 4
        for (int t = t_lo; t < t_hi; t++) {
            const size_t m = (size_t)(m0 + t);
            const float av = A[m * width + ch];
            B = fmaf(av, B, Bv[m * width + ch]);
            P *= av;
        }
    }
    sP[w][lane] = P, sB[w][lane] = B;
    __syncthreads();
    for (int q = 0; q < w; q++) s = fmaf(sP[q][lane], s, sB[q][lane]);
    if (!live) return;
    const float bias = yb ? bf16_bits_to_f32(yb[ch]) : 0.f;
#pragma unroll 4
    for (int t = t_lo; t < t_hi; t++) {
        const size_t m = (size_t)(m0 + t);
        s = fmaf(A[m * width + ch], s, Bv[m * width + ch]);
        const float o = s * gelu_tanh_f(y[m * ldy + ch] + bias);
        if (sizeof(TO) == 2) ((uint16_t*)out)[m * ldo + ch] = f32_to_bf16_bits(o);
        else ((float*)out)[m * ldo + ch] = o;
    }
    if (w == W - 1) *st = s;  // the last run ends at token T - 1 (runs may be empty only at the end when T < W, which the launch rules out)
}
// minGRU: per channel a gated recurrence; update gate and candidate are functions of the same position's input alone,
//     z = sigmoid(zl + zb),   u = xl + xb,   c = u + 1/2 (u >= 0) | sigmoid(u) (u < 0),   s <- (1 - z) s + z c,   out = s * silu(gl)
// with 1 - z formed as sigmoid(-(zl + zb)), not by subtraction.  Same launch shape as kf_rglru_scan_kernel: a CTA owns 32 channels, its warps runs of consecutive
// tokens; a first pass reduces every run to one affine map, a second replays it from the run's incoming state.  STASH: a run has at most
// MINGRU_RUN tokens and the first pass leaves (1 - z, z c) of each in registers -- all its loads are independent and in flight together --
// so the second pass reads only gl; otherwise the gates are recomputed in the second pass.  Both forms do the same fp32 operations in the
// same order.
constexpr int MINGRU_RUN = 32;
template <typename TO, bool STASH>
__global__ void __launch_bounds__(32 * LRU_W) kf_mingru_kernel(TO* __restrict__ out, int ldo, const float* __restrict__ zl, int ldz, const uint16_t* __restrict__ zb,
                                                               const float* __restrict__ xl, int ldx, const uint16_t* __restrict__ xb,
                                                               const float* __restrict__ gl, int ldg, float* __restrict__ state, size_t state_stride,
                                                               const int32_t* __restrict__ pos, const int32_t* __restrict__ slot, int T, int width) {
    __shared__ float sP[LRU_W][32], sB[LRU_W][32];
    const int seq = blockIdx.y, lane = threadIdx.x & 31, w = threadIdx.x >> 5, W = blockDim.x >> 5;
    const int ch = blockIdx.x * 32 + lane, m0 = seq * T;
    const bool live = ch < width;
    const int run = (T + W - 1) / W, t_lo = min(T, w * run), t_hi = min(T, t_lo + run);
    float* st = state + (size_t)slot[m0] * state_stride + (live ? ch : 0);
    float s = (pos[m0] == 0 || !live) ? 0.f : *st;
    const float bz = (live && zb) ? bf16_bits_to_f32(zb[ch]) : 0.f, bx = (live && xb) ? bf16_bits_to_f32(xb[ch]) : 0.f;
    // (1 - z, z c) from the two logits; z and 1 - z share one exponential: e = exp(-|zv|), the larger of the two is 1 / (1 + e), the smaller
    // e / (1 + e), either accurate to fp32 rounding however large |zv| is
    auto mix = [&](float zv, float u, float& keep, float& add) {
        const float e = expf(-fabsf(zv)), big = 1.f / (1.f + e), small = e * big;
        keep = zv >= 0.f ? small : big;
        add  = (zv >= 0.f ? big : small) * (u >= 0.f ? u + 0.5f : sigmoid_f(u));
    };
    auto gates = [&](size_t m, float& keep, float& add) { mix(zl[m * ldz + ch] + bz, xl[m * ldx + ch] + bx, keep, add); };
    auto emit = [&](size_t m, float sv) {
        const float g = gl[m * ldg + ch];
        const float o = sv * g * sigmoid_f(g);
        if (sizeof(TO) == 2) ((uint16_t*)out)[m * ldo + ch] = f32_to_bf16_bits(o);
        else ((float*)out)[m * ldo + ch] = o;
    };
    float P = 1.f, B = 0.f;
    if (STASH) {
        // loads first, all of them independent and in flight together, the arithmetic after them; a token past the run's end is not read
        // and contributes the identity map
        float kp[MINGRU_RUN], ad[MINGRU_RUN];
        const int nrun = live ? t_hi - t_lo : 0;
        const float* zp = zl + (size_t)(m0 + t_lo) * ldz + ch;
        const float* xp = xl + (size_t)(m0 + t_lo) * ldx + ch;
#pragma unroll
        for (int i = 0; i < MINGRU_RUN; i++) {
            kp[i] = i < nrun ? zp[(size_t)i * ldz] : 0.f;
            ad[i] = i < nrun ? xp[(size_t)i * ldx] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < MINGRU_RUN; i++) {
            float keep, add;
            mix(kp[i] + bz, ad[i] + bx, keep, add);
            kp[i] = i < nrun ? keep : 1.f;
            ad[i] = i < nrun ? add : 0.f;
            B = fmaf(kp[i], B, ad[i]), P *= kp[i];
        }
        sP[w][lane] = P, sB[w][lane] = B;
        __syncthreads();
        for (int q = 0; q < w; q++) s = fmaf(sP[q][lane], s, sB[q][lane]);
        if (!live) return;
        const float* gp = gl + (size_t)(m0 + t_lo) * ldg + ch;
        TO* op = out + (size_t)(m0 + t_lo) * ldo + ch;
#pragma unroll
        for (int i0 = 0; i0 < MINGRU_RUN; i0 += 8) {
            float g[8];
#pragma unroll
            for (int j = 0; j < 8; j++) g[j] = i0 + j < nrun ? gp[(size_t)(i0 + j) * ldg] : 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                if (i0 + j < nrun) {
                    s = fmaf(kp[i0 + j], s, ad[i0 + j]);
                    const float o = s * g[j] * sigmoid_f(g[j]);
                    if (sizeof(TO) == 2) op[(size_t)(i0 + j) * ldo] = (TO)f32_to_bf16_bits(o);
                    else op[(size_t)(i0 + j) * ldo] = (TO)o;
                }
            }
        }
    } else {
        if (W > 1 && live) {
#pragma unroll 4
            for (int t = t_lo; t < t_hi; t++) {
                float keep, add;
                gates((size_t)(m0 + t), keep, add);
                B = fmaf(keep, B, add);
                P *= keep;
            }
        }
        sP[w][lane] = P, sB[w][lane] = B;
        __syncthreads();
        for (int q = 0; q < w; q++) s = fmaf(sP[q][lane], s, sB[q][lane]);
        if (!live) return;
#pragma unroll 4
        for (int t = t_lo; t < t_hi; t++) {
            float keep, add;
            gates((size_t)(m0 + t), keep, add);
            s = fmaf(keep, s, add);
            emit((size_t)(m0 + t), s);
        }
    }
    if (t_hi == T && t_lo < T) *st = s;  // the run that ends at the last token leaves the state
}
}  // namespace

// minGRU over nseq x T tokens: z_logit, x_logit, g_logit float rows [M][ld*] of `width` channels (bf16 biases of the first two, or NULL);
// out [M][ldo] = s * silu(g) in the activation type; state: float [slot][width], started from zero at position 0.
extern "C" int kf_mingru(kf_ctx* ctx, void* out, int out_f32, int ldo, const float* z_logit, int ldz, const void* z_bias_bf16, const float* x_logit, int ldx,
                         const void* x_bias_bf16, const float* g_logit, int ldg, float* state, size_t state_stride, const int32_t* pos_dev,
                         const int32_t* slot_dev, int nseq, int T, int width) {
    if (!ctx || !out || !z_logit || !x_logit || !g_logit || !state || !pos_dev || !slot_dev) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, nseq >= 1 && T >= 1 && width >= 1 && state_stride >= (size_t)width, "shape");
    dim3 grid((width + 31) / 32, nseq);
    const int warps = std::max(1, std::min(LRU_W, T / 8)), threads = 32 * warps;  // runs of at least 8 tokens; one warp when decoding
    const bool stash = warps > 1 && (T + warps - 1) / warps <= MINGRU_RUN;  // one warp (decoding): the short form, less code to fetch
#define KF_MINGRU_LAUNCH(TO, ST)                                                                                                              \
    kf_mingru_kernel<TO, ST><<<grid, threads, 0, ctx->stream>>>((TO*)out, ldo, z_logit, ldz, (const uint16_t*)z_bias_bf16, x_logit, ldx,      \
                                                                (const uint16_t*)x_bias_bf16, g_logit, ldg, state, state_stride, pos_dev, slot_dev, T, width)
    if (out_f32) {
        if (stash) KF_MINGRU_LAUNCH(float, true);
        else KF_MINGRU_LAUNCH(float, false);
    } else {
        if (stash) KF_MINGRU_LAUNCH(uint16_t, true);
        else KF_MINGRU_LAUNCH(uint16_t, false);
    }
#undef KF_MINGRU_LAUNCH
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}

// Matrix-state recurrence over nseq x T tokens (see the head of this file).  q, k: float rows with G kv heads of dk entries at row strides
// ldq / ldk; v: H heads of dv entries; z: decay logits H x dk (+ bf16 bias zbias or NULL); beta_logit: H per token (delta rule only).
// decay_kind 0: g = sigmoid(z + b)^(1/tau); 1: g = exp(-exp(A_log[h]) softplus(z + b)).  state: float [slot][H][dv][dk].
// decay_per_head 1: z holds ONE logit per head and token ([H] at row stride ldz, zbias [H]); every key channel of the head decays alike.
extern "C" int kf_gated_scan_ex(kf_ctx* ctx, float* y, int ldy, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* z,
                             int ldz, const void* zbias_bf16, const void* A_log_bf16, const float* beta_logit, int ldb, float* state, size_t state_stride,
                             const int32_t* pos_dev, const int32_t* slot_dev, int nseq, int T, int H, int G, int dk, int dv, int delta, int decay_kind,
                             float tau, int unit_qk, float unit_eps, float q_scale, int decay_per_head) {
    if (!ctx || !y || !q || !k || !v || !z || !state || !pos_dev || !slot_dev) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, nseq >= 1 && T >= 1 && H >= 1 && G >= 1 && H % G == 0 && dk >= 1 && dv >= 1 && dk <= 32 * NPT_MAX, "key size <= 512, kv heads divide heads");
    KF_REQUIRE(ctx, (!delta || beta_logit) && (decay_kind == 0 ? tau > 0.f : A_log_bf16 != nullptr) && state_stride >= (size_t)H * dk * dv, "arguments");
    ScanArgs a = {};
    a.y = y, a.ldy = ldy, a.q = q, a.k = k, a.v = v, a.z = z, a.beta = beta_logit, a.ldq = ldq, a.ldk = ldk, a.ldv = ldv, a.ldz = ldz, a.ldb = ldb;
    a.zbias = (const uint16_t*)zbias_bf16, a.A_log = (const uint16_t*)A_log_bf16, a.state = state, a.state_stride = state_stride;
    a.pos = pos_dev, a.slot = slot_dev, a.T = T, a.H = H, a.G = G, a.dk = dk, a.dv = dv, a.delta = delta, a.decay_kind = decay_kind;
    a.unit_qk = unit_qk, a.inv_tau = decay_kind == 0 ? 1.f / tau : 0.f, a.q_scale = q_scale, a.unit_eps = unit_eps, a.z_head = decay_per_head ? 1 : 0;
    // rows of a state column per lane: 16, or 8 for keys of up to 128 entries (a shorter dependent chain per token, twice the lanes per column)
    const int NPT = (dk <= 128 && dk % 8 == 0 && dk >= 16) ? 8 : 16;
    int R = 1;
    while (R * NPT < dk) R <<= 1;
    // up to 256 threads per CTA: the per-token chain of a warp is latency-bound and as long whatever the grid, while the staging of a pass (and
    // the decay's exponentials, formed once per CTA) is shared by the CTA's columns -- so columns are NOT spread over more, thinner CTAs
    const int PB = std::max(1, std::min(dv, 256 / R));
    const int threads = std::max(32, ((PB * R + 31) / 32) * 32);
    const int dkp = ((dk + 15) / 16) * 20;
    int TB = (int)std::min<size_t>(32, (44 * 1024 / sizeof(float)) / (size_t)(3 * dkp + PB + 2));
    TB = std::max(1, std::min(TB, T));
    const size_t smem = (size_t)(3 * TB * dkp + TB * PB + 2 * TB) * sizeof(float);
    KF_REQUIRE(ctx, smem <= 48 * 1024, "staging area");
    a.R = R, a.PB = PB, a.TB = TB, a.dkp = dkp;
    const dim3 grid(H, nseq, (dv + PB - 1) / PB);
    const bool full = dk == R * NPT;
#define KF_SCAN(D, F, N) kf_gated_scan_kernel<D, F, N><<<grid, threads, smem, ctx->stream>>>(a)
#define KF_SCAN_N(D, F) (NPT == 8 ? KF_SCAN(D, F, 8) : KF_SCAN(D, F, 16))
    if (delta) {
        if (full) KF_SCAN_N(true, true);
        else KF_SCAN_N(true, false);
    } else {
        if (full) KF_SCAN_N(false, true);
        else KF_SCAN_N(false, false);
    }
#undef KF_SCAN_N
#undef KF_SCAN
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}

extern "C" int kf_gated_scan(kf_ctx* ctx, float* y, int ldy, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* z,
                             int ldz, const void* zbias_bf16, const void* A_log_bf16, const float* beta_logit, int ldb, float* state, size_t state_stride,
                             const int32_t* pos_dev, const int32_t* slot_dev, int nseq, int T, int H, int G, int dk, int dv, int delta, int decay_kind,
                             float tau, int unit_qk, float unit_eps, float q_scale) {
    return kf_gated_scan_ex(ctx, y, ldy, q, ldq, k, ldk, v, ldv, z, ldz, zbias_bf16, A_log_bf16, beta_logit, ldb, state, state_stride, pos_dev, slot_dev, nseq, T, H,
                            G, dk, dv, delta, decay_kind, tau, unit_qk, unit_eps, q_scale, 0);
}

// Real-gated linear recurrent unit over `width` channels in `blocks` equal parts.  u: float [M][ldu] (the convolved branch); gate weights
// bf16 [blocks][bs][bs] ([out][in]) with biases [width]; lam bf16 [width]; y_logit: float [M][ldy] (+ bf16 bias), the other branch before
// its gelu.  out [M][ldo] = s * gelu_tanh(y) in the activation type.  work: float scratch [2][M][width].  state: float [slot][width].
extern "C" int kf_rglru(kf_ctx* ctx, void* out, int out_f32, int ldo, float* work, const float* u, int ldu, const void* w_r_bf16, const void* b_r_bf16,
                        const void* w_i_bf16, const void* b_i_bf16, const void* lam_bf16, float decay_c, const float* y_logit, int ldy,
                        const void* y_bias_bf16, float* state, size_t state_stride, const int32_t* pos_dev, const int32_t* slot_dev, int nseq, int T,
                        int width, int blocks) {
    if (!ctx || !out || !work || !u || !w_r_bf16 || !b_r_bf16 || !w_i_bf16 || !b_i_bf16 || !lam_bf16 || !y_logit || !state || !pos_dev || !slot_dev)
        return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, nseq >= 1 && T >= 1 && width >= 1 && blocks >= 1 && width % blocks == 0 && state_stride >= (size_t)width, "blocks must divide width");
    const int M = nseq * T, bs = width / blocks;
    float *A = work, *Bv = work + (size_t)M * width;
    kf_rglru_gates_kernel<<<dim3((M + GT - 1) / GT, blocks, (bs + 127) / 128), 128, 0, ctx->stream>>>(
        A, Bv, u, ldu, (const uint16_t*)w_r_bf16, (const uint16_t*)b_r_bf16, (const uint16_t*)w_i_bf16, (const uint16_t*)b_i_bf16, (const uint16_t*)lam_bf16, M,
        width, bs, decay_c);
    KF_LAUNCH_CHECK(ctx);
    dim3 grid((width + 31) / 32, nseq);
    const int warps = std::max(1, std::min(LRU_W, T / 8)), threads = 32 * warps;  // runs of at least 8 tokens; one warp when decoding
    if (out_f32)
        kf_rglru_scan_kernel<float><<<grid, threads, 0, ctx->stream>>>((float*)out, ldo, A, Bv, y_logit, ldy, (const uint16_t*)y_bias_bf16, state, state_stride, pos_dev,
                                                                 slot_dev, T, width);
    else
        kf_rglru_scan_kernel<uint16_t><<<grid, threads, 0, ctx->stream>>>((uint16_t*)out, ldo, A, Bv, y_logit, ldy, (const uint16_t*)y_bias_bf16, state, state_stride,
                                                                    pos_dev, slot_dev, T, width);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
