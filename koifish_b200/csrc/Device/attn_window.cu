// attn_window.cu -- causal grouped-query softmax attention over a SLIDING WINDOW of rotated keys:
//     s_ij = cap * tanh((q_i . k_j) * scale / cap)      (cap <= 0: no capping),      i - window < j <= i      (window <= 0: all keys),
//     o_i  = sum_j e^{s_ij} v_j / (e^{sink_h} + sum_j e^{s_ij})                      (sink NULL: no extra term),
// for any per-head key size dk and value size dv.  Two steps:
//   kf_qk_prepare   RMS norm of the WHOLE query row and of the whole key row (one mean over all heads; weight of the row's size), then the
//                   rotation of the first rot_dims entries of every head by pos * f_i (pairs (2i, 2i+1) or (i, i + rot_dims/2); the table
//                   of f_i is the caller's, so any frequency scaling is a matter of the table; cosine and sine are multiplied by `amp`);
//                   the query is rewritten in place (fp32), the key and the value go to the sequence slot's cache.
//   kf_attn_window  scores, softmax and the weighted sum in fp32 over the cached rows of the window.
// The cache of a slot is a RING of `ring` rows [k (G x dk) | v (G x dv)] in the activation type (bf16 bits or float): position p sits in
// row p % ring.  With ring >= window + (tokens per step) - 1 a whole step can be appended before its queries are answered; memory does
// not grow with the sequence.  A slot is never cleared: a sequence that starts at position 0 reads only rows that it wrote.
// One kernel serves prompts (M tokens of one slot) and decoding (one token of each of M slots): a CTA per (token, head, key split), a
// lane per key for the scores, lanes over the value entries for the sum, online softmax per warp, warps merged at the end.
// Beside kf_attn_bias (attn_bias.cu: distance penalty, no rotation) and kf_attn_* (attention.cu: Qwen3's path).  No reference equivalent.
#include <math.h>

#include <algorithm>

#include "kf_common.cuh"

namespace {
template <typename TC>
__device__ __forceinline__ float ldc(const TC* p);
template <>
__device__ __forceinline__ float ldc<uint16_t>(const uint16_t* p) { return bf16_bits_to_f32(*p); }
template <>
__device__ __forceinline__ float ldc<float>(const float* p) { return *p; }

struct PrepArgs {
    float* x;  // [M][ldx]: q (nq) | k (nk) | v (nv), consecutive
    uint16_t* qb;  // optional bf16 copy of the finished q, [M][nq] (what the tensor-core panel kernel reads)
    int ldx, nq, nk, nv, hd;
    const uint16_t *qw, *kw;  // bf16 [nq], [nk] or NULL (that row is not normed)
    const uint16_t *qb_add, *kb_add;  // bf16 [nq], [nk] or NULL: biases added to q and k before anything else
    int v_from_k;             // 1: v is a copy of k taken ahead of the rotation (x holds no v; nv == nk)
    float eps, amp;
    int rot_dims, layout;     // layout 0: pairs (2i, 2i+1); 1: pairs (i, i + rot_dims / 2)
    const double* inv_freq;   // [rot_dims / 2]
    void* cache;
    size_t slot_stride;
    int ring;
    const int32_t *pos, *slot;
};

template <typename TC>
__global__ void __launch_bounds__(256) kf_qk_prepare_kernel(PrepArgs a) {
    extern __shared__ float sm[];
    __shared__ float red[32];
    const int m = blockIdx.x, n = a.nq + a.nk, half = a.rot_dims >> 1;
    float* sx = sm;          // [nq + nk] normed, not yet rotated
    float* sc = sx + n;      // [half] cos * amp
    float* ss = sc + half;   // [half] sin * amp
    float* row = a.x + (size_t)m * a.ldx;
    const int p = a.pos[m];
    float q2 = 0.f, k2 = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = row[i];
        if (i < a.nq) {
            if (a.qb_add) v += bf16_bits_to_f32(a.qb_add[i]);
        } else if (a.kb_add) {
            v += bf16_bits_to_f32(a.kb_add[i - a.nq]);
        }
        sx[i] = v;
        if (i < a.nq) q2 = fmaf(v, v, q2);
        else k2 = fmaf(v, v, k2);
    }
    // the angle pos * f_i is formed and brought into [-pi, pi] in double (a few double operations), its cosine and sine in float: the
    // reduced angle is exact to 2e-7, which is more than 32-bit angles keep at positions in the thousands
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const double ang = (double)p * a.inv_freq[i];
        const float r = (float)(ang - 6.283185307179586 * rint(ang * 0.15915494309189535));
        float s, c;
        sincosf(r, &s, &c);
        sc[i] = c * a.amp, ss[i] = s * a.amp;
    }
    q2 = block_sum(q2, red);
    k2 = block_sum(k2, red);
    const float fq = a.qw ? 1.0f / sqrtf(q2 / (float)a.nq + a.eps) : 1.f;
    const float fk = a.kw ? 1.0f / sqrtf(k2 / (float)a.nk + a.eps) : 1.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        if (i < a.nq) {
            if (a.qw) sx[i] *= fq * bf16_bits_to_f32(a.qw[i]);
        } else if (a.kw) {
            sx[i] *= fk * bf16_bits_to_f32(a.kw[i - a.nq]);
        }
    }
    __syncthreads();
    const int W = a.nk + a.nv;
    TC* crow = (TC*)a.cache + (size_t)a.slot[m] * a.slot_stride + (size_t)(p % a.ring) * W;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int d = (i < a.nq ? i : i - a.nq) % a.hd;
        float v = sx[i];
        if (d < a.rot_dims) {
            int f, partner;
            bool first;
            if (a.layout == 0) f = d >> 1, first = !(d & 1), partner = i ^ 1;
            else first = d < half, f = first ? d : d - half, partner = first ? i + half : i - half;
            const float o = sx[partner];
            v = first ? v * sc[f] - o * ss[f] : v * sc[f] + o * ss[f];
        }
        if (i < a.nq) {
            row[i] = v;
            if (a.qb) a.qb[(size_t)m * a.nq + i] = f32_to_bf16_bits(v);
        } else if (sizeof(TC) == 2) ((uint16_t*)crow)[i - a.nq] = f32_to_bf16_bits(v);
        else ((float*)crow)[i - a.nq] = v;
    }
    for (int i = threadIdx.x; i < a.nv; i += blockDim.x) {
        const float v = a.v_from_k ? sx[a.nq + i] : row[n + i];
        if (sizeof(TC) == 2) ((uint16_t*)crow)[a.nk + i] = f32_to_bf16_bits(v);
        else ((float*)crow)[a.nk + i] = v;
    }
}

struct WinArgs {
    void* out;  // [M][ldo] activation type, heads x dv
    int ldo, out_f32;
    const float* q;  // [M][ldq] heads x dk, normed and rotated
    int ldq;
    const void* cache;
    size_t slot_stride;
    int ring, window;
    const uint16_t* sink;  // bf16 [H] or NULL
    const int32_t *pos, *slot;
    int H, G, dk, dv;
    float scale, softcap, out_scale;
    int nsplit;  // the keys of a token are dealt to nsplit CTAs (blockIdx.z); > 1: partial (max, sum, weighted values) go to ws
    float* ws;   // [M][H][nsplit][dv + 2]
    // sigmoid-weighted attention (kf_attn_sigmoid): keys of the query's own block of `block` positions only (0: no blocks), a bias per
    // head inside the sigmoid (bf16 [H] or NULL)
    int block;
    const uint16_t* pbias;
};

__device__ __forceinline__ void win_store(const WinArgs& a, int m, int h, int d, float o) {
    o *= a.out_scale;
    if (a.out_f32) ((float*)a.out)[(size_t)m * a.ldo + h * a.dv + d] = o;
    else ((uint16_t*)a.out)[(size_t)m * a.ldo + h * a.dv + d] = f32_to_bf16_bits(o);
}

constexpr int AW = 4;  // warps per CTA
template <typename TC, int VPL>
__global__ void __launch_bounds__(AW * 32) kf_attn_window_kernel(WinArgs a) {
    extern __shared__ float sm[];
    float* sq   = sm;                // [dk]
    float* sacc = sq + a.dk;         // [AW][dv]
    float* sml  = sacc + AW * a.dv;  // [AW][2]
    const int m = blockIdx.x, h = blockIdx.y, kh = h / (a.H / a.G);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p = a.pos[m], W = a.G * (a.dk + a.dv);
    const TC* base = (const TC*)a.cache + (size_t)a.slot[m] * a.slot_stride;
    for (int d = threadIdx.x; d < a.dk; d += blockDim.x) sq[d] = a.q[(size_t)m * a.ldq + h * a.dk + d] * a.scale;
    __syncthreads();
    float mx = -INFINITY, l = 0.f, acc[VPL];
#pragma unroll
    for (int i = 0; i < VPL; i++) acc[i] = 0.f;
    const bool vec = sizeof(TC) == 2 && a.dk % 8 == 0 && W % 8 == 0 && (a.slot_stride % 8) == 0 && (((uintptr_t)a.cache & 15) == 0);
    const float inv_cap = a.softcap > 0.f ? 1.f / a.softcap : 0.f;
    // the visible keys are lo .. p; this CTA's share: [j_lo, j_hi), whole 32-key steps per split
    const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0, nkeys = p - lo + 1;
    const int chunk = a.nsplit > 1 ? (((nkeys + a.nsplit - 1) / a.nsplit + 31) & ~31) : nkeys;
    const int j_lo = lo + blockIdx.z * chunk, j_hi = min(p + 1, j_lo + chunk);
    for (int j0 = j_lo + warp * 32; j0 < j_hi; j0 += AW * 32) {
        const int j = j0 + lane;
        float s = -INFINITY;
        if (j < j_hi) {
            const TC* kr = base + (size_t)(j % a.ring) * W + kh * a.dk;
            float d0 = 0.f, d1 = 0.f;
            if (vec) {
                for (int d = 0; d < a.dk; d += 8) {
                    const uint4 kv = *reinterpret_cast<const uint4*>((const uint16_t*)kr + d);
                    d0 = fmaf(bf16lo(kv.x), sq[d], d0), d1 = fmaf(bf16hi(kv.x), sq[d + 1], d1);
                    d0 = fmaf(bf16lo(kv.y), sq[d + 2], d0), d1 = fmaf(bf16hi(kv.y), sq[d + 3], d1);
                    d0 = fmaf(bf16lo(kv.z), sq[d + 4], d0), d1 = fmaf(bf16hi(kv.z), sq[d + 5], d1);
                    d0 = fmaf(bf16lo(kv.w), sq[d + 6], d0), d1 = fmaf(bf16hi(kv.w), sq[d + 7], d1);
                }
            } else {
                for (int d = 0; d < a.dk; d++) d0 = fmaf(ldc<TC>(kr + d), sq[d], d0);
            }
            s = d0 + d1;
            if (a.softcap > 0.f) s = a.softcap * tanhf(s * inv_cap);
        }
        const float bm = warp_max(s), nm = fmaxf(mx, bm);
        const float corr = expf(mx - nm), pj = j < j_hi ? expf(s - nm) : 0.f;  // mx = -inf on the first pass: corr = 0
        l = l * corr + warp_sum(pj);
#pragma unroll
        for (int i = 0; i < VPL; i++) acc[i] *= corr;
        mx = nm;
        const int nk = min(32, j_hi - j0);
        constexpr int U = VPL <= 4 ? 4 : (VPL <= 8 ? 2 : 1);  // keys per step: their value loads are issued together
        for (int t = 0; t < nk; t += U) {
            float pt[U], x[U][VPL];
#pragma unroll
            for (int e = 0; e < U; e++) {
                pt[e] = __shfl_sync(0xffffffffu, pj, (t + e) & 31);
                const TC* vr = base + (size_t)(min(j0 + t + e, j_hi - 1) % a.ring) * W + a.G * a.dk + kh * a.dv;
#pragma unroll
                for (int i = 0; i < VPL; i++) {
                    const int d = i * 32 + lane;
                    x[e][i] = d < a.dv ? ldc<TC>(vr + d) : 0.f;
                }
            }
#pragma unroll
            for (int e = 0; e < U; e++)
#pragma unroll
                for (int i = 0; i < VPL; i++) acc[i] = fmaf(t + e < nk ? pt[e] : 0.f, x[e][i], acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < VPL; i++) {
        const int d = i * 32 + lane;
        if (d < a.dv) sacc[warp * a.dv + d] = acc[i];
    }
    if (lane == 0) sml[warp * 2] = mx, sml[warp * 2 + 1] = l;
    __syncthreads();
    const bool last = a.nsplit == 1;
    const float snk = (a.sink && last) ? bf16_bits_to_f32(a.sink[h]) : -INFINITY;
    float Mx = snk;
    for (int w = 0; w < AW; w++) Mx = fmaxf(Mx, sml[w * 2]);
    float L = snk == -INFINITY ? 0.f : expf(snk - Mx), f[AW];  // the sink counts once in the denominator and carries no value
    for (int w = 0; w < AW; w++) f[w] = sml[w * 2] == -INFINITY ? 0.f : expf(sml[w * 2] - Mx), L += f[w] * sml[w * 2 + 1];
    if (!last) {  // partial result of this split; kf_attn_window_merge_kernel finishes
        float* part = a.ws + (((size_t)m * a.H + h) * a.nsplit + blockIdx.z) * (a.dv + 2);
        if (threadIdx.x == 0) part[0] = Mx, part[1] = L;
        for (int d = threadIdx.x; d < a.dv; d += blockDim.x) {
            float o = 0.f;
            for (int w = 0; w < AW; w++) o = fmaf(f[w], sacc[w * a.dv + d], o);
            part[2 + d] = o;
        }
        return;
    }
    for (int d = threadIdx.x; d < a.dv; d += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < AW; w++) o = fmaf(f[w], sacc[w * a.dv + d], o);
        win_store(a, m, h, d, o / L);
    }
}
// the splits of one (token, head) merged in split order with the sink, written in the activation type
__global__ void kf_attn_window_merge_kernel(WinArgs a) {
    const int m = blockIdx.x, h = blockIdx.y;
    const float* part = a.ws + ((size_t)m * a.H + h) * a.nsplit * (a.dv + 2);
    const float snk = a.sink ? bf16_bits_to_f32(a.sink[h]) : -INFINITY;
    float Mx = snk;
    for (int z = 0; z < a.nsplit; z++) Mx = fmaxf(Mx, part[(size_t)z * (a.dv + 2)]);
    float L = snk == -INFINITY ? 0.f : expf(snk - Mx);
    for (int z = 0; z < a.nsplit; z++) {
        const float mz = part[(size_t)z * (a.dv + 2)];
        if (mz != -INFINITY) L += expf(mz - Mx) * part[(size_t)z * (a.dv + 2) + 1];
    }
    for (int d = threadIdx.x; d < a.dv; d += blockDim.x) {
        float o = 0.f;
        for (int z = 0; z < a.nsplit; z++) {
            const float mz = part[(size_t)z * (a.dv + 2)];
            if (mz != -INFINITY) o = fmaf(expf(mz - Mx), part[(size_t)z * (a.dv + 2) + 2 + d], o);
        }
        win_store(a, m, h, d, o / L);
    }
}
// ---- sigmoid-weighted attention: o_i = sum_j sigmoid(scale q_i . k_j + b_h) v_j over the visible keys, NOT normalised over the keys.
// Visible: j <= i, j in the block of `block` positions that holds i (blocks aligned to position 0; block 0: none), and inside the window
// when one is given.  Same work split as kf_attn_window_kernel (CTA per (token, head, key split), a lane per key for the scores, lanes over
// the value entries for the sum); the splits' partial sums are added in split order.
__device__ __forceinline__ float sig_f(float z) { return 1.f / (1.f + expf(-z)); }
template <typename TC, int VPL>
__global__ void __launch_bounds__(AW * 32) kf_attn_sigmoid_kernel(WinArgs a) {
    extern __shared__ float sm[];
    float* sq   = sm;         // [dk]
    float* sacc = sq + a.dk;  // [AW][dv]
    const int m = blockIdx.x, h = blockIdx.y, kh = h / (a.H / a.G);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p = a.pos[m], W = a.G * (a.dk + a.dv);
    const TC* base = (const TC*)a.cache + (size_t)a.slot[m] * a.slot_stride;
    for (int d = threadIdx.x; d < a.dk; d += blockDim.x) sq[d] = a.q[(size_t)m * a.ldq + h * a.dk + d] * a.scale;
    __syncthreads();
    float acc[VPL];
#pragma unroll
    for (int i = 0; i < VPL; i++) acc[i] = 0.f;
    const bool vec = sizeof(TC) == 2 && a.dk % 8 == 0 && W % 8 == 0 && (a.slot_stride % 8) == 0 && (((uintptr_t)a.cache & 15) == 0);
    const float hb = a.pbias ? bf16_bits_to_f32(a.pbias[h]) : 0.f;
    int lo = a.block > 0 ? (p / a.block) * a.block : 0;
    if (a.window > 0) lo = max(lo, p - a.window + 1);
    const int nkeys = p - lo + 1;
    const int chunk = a.nsplit > 1 ? (((nkeys + a.nsplit - 1) / a.nsplit + 31) & ~31) : nkeys;
    const int j_lo = lo + blockIdx.z * chunk, j_hi = min(p + 1, j_lo + chunk);
    for (int j0 = j_lo + warp * 32; j0 < j_hi; j0 += AW * 32) {
        const int j = j0 + lane;
        float pj = 0.f;
        if (j < j_hi) {
            const TC* kr = base + (size_t)(j % a.ring) * W + kh * a.dk;
            float d0 = 0.f, d1 = 0.f;
            if (vec) {
                for (int d = 0; d < a.dk; d += 8) {
                    const uint4 kv = *reinterpret_cast<const uint4*>((const uint16_t*)kr + d);
                    d0 = fmaf(bf16lo(kv.x), sq[d], d0), d1 = fmaf(bf16hi(kv.x), sq[d + 1], d1);
                    d0 = fmaf(bf16lo(kv.y), sq[d + 2], d0), d1 = fmaf(bf16hi(kv.y), sq[d + 3], d1);
                    d0 = fmaf(bf16lo(kv.z), sq[d + 4], d0), d1 = fmaf(bf16hi(kv.z), sq[d + 5], d1);
                    d0 = fmaf(bf16lo(kv.w), sq[d + 6], d0), d1 = fmaf(bf16hi(kv.w), sq[d + 7], d1);
                }
            } else {
                for (int d = 0; d < a.dk; d++) d0 = fmaf(ldc<TC>(kr + d), sq[d], d0);
            }
            pj = sig_f(d0 + d1 + hb);
        }
        const int nk = min(32, j_hi - j0);
        constexpr int U = VPL <= 4 ? 4 : (VPL <= 8 ? 2 : 1);  // keys per step: their value loads are issued together
        for (int t = 0; t < nk; t += U) {
            float pt[U], x[U][VPL];
#pragma unroll
            for (int e = 0; e < U; e++) {
                pt[e] = __shfl_sync(0xffffffffu, pj, (t + e) & 31);
                const TC* vr = base + (size_t)(min(j0 + t + e, j_hi - 1) % a.ring) * W + a.G * a.dk + kh * a.dv;
#pragma unroll
                for (int i = 0; i < VPL; i++) {
                    const int d = i * 32 + lane;
                    x[e][i] = d < a.dv ? ldc<TC>(vr + d) : 0.f;
                }
            }
#pragma unroll
            for (int e = 0; e < U; e++)
#pragma unroll
                for (int i = 0; i < VPL; i++) acc[i] = fmaf(t + e < nk ? pt[e] : 0.f, x[e][i], acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < VPL; i++) {
        const int d = i * 32 + lane;
        if (d < a.dv) sacc[warp * a.dv + d] = acc[i];
    }
    __syncthreads();
    for (int d = threadIdx.x; d < a.dv; d += blockDim.x) {
        float o = 0.f;
        for (int w = 0; w < AW; w++) o += sacc[w * a.dv + d];
        if (a.nsplit == 1) win_store(a, m, h, d, o);
        else a.ws[(((size_t)m * a.H + h) * a.nsplit + blockIdx.z) * a.dv + d] = o;
    }
}
__global__ void kf_attn_sigmoid_merge_kernel(WinArgs a) {
    const int m = blockIdx.x, h = blockIdx.y;
    const float* part = a.ws + ((size_t)m * a.H + h) * a.nsplit * a.dv;
    for (int d = threadIdx.x; d < a.dv; d += blockDim.x) {
        float o = 0.f;
        for (int z = 0; z < a.nsplit; z++) o += part[(size_t)z * a.dv + d];
        win_store(a, m, h, d, o);
    }
}
}  // namespace

// x[m] = [q (nq) | k (nk) | v (nv)] floats at row stride ldx.  q and k: RMS norm over the whole row part (weights bf16 [nq] / [nk]; NULL:
// none), then the rotation of the first rot_dims entries of each head of size head_dim by pos[m] * inv_freq[i] with cos and sin times amp
// (layout 0: pairs (2i, 2i+1); 1: pairs (i, i + rot_dims/2); rot_dims 0: none).  q is rewritten in place; k | v become row pos[m] % ring of
// the slot's cache [slot][ring][nk + nv] in the cache's type.  q_bf16_out (optional): a bf16 copy of the finished q, [M][nq].
extern "C" int kf_qk_prepare(kf_ctx* ctx, float* x, int ldx, int nq, int nk, int nv, int head_dim, const void* q_norm_bf16, const void* k_norm_bf16, float eps,
                             int rot_dims, const double* inv_freq_dev, float amp, int layout, void* cache, int cache_f32, size_t slot_stride, int ring,
                             void* q_bf16_out, const int32_t* pos_dev, const int32_t* slot_dev, int M) {
    return kf_qk_prepare_ex(ctx, x, ldx, nq, nk, nv, head_dim, nullptr, nullptr, 0, q_norm_bf16, k_norm_bf16, eps, rot_dims, inv_freq_dev, amp, layout, cache,
                            cache_f32, slot_stride, ring, q_bf16_out, pos_dev, slot_dev, M);
}
// kf_qk_prepare with biases on q and k (bf16 [nq] / [nk] or NULL, added first) and, with v_from_k = 1, values that ARE the keys as they
// stand before the rotation: x[m] = [q | k] only, nv must equal nk, and the cache row is [rotated k | unrotated k].
extern "C" int kf_qk_prepare_ex(kf_ctx* ctx, float* x, int ldx, int nq, int nk, int nv, int head_dim, const void* q_bias_bf16, const void* k_bias_bf16,
                                int v_from_k, const void* q_norm_bf16, const void* k_norm_bf16, float eps, int rot_dims, const double* inv_freq_dev, float amp,
                                int layout, void* cache, int cache_f32, size_t slot_stride, int ring, void* q_bf16_out, const int32_t* pos_dev,
                                const int32_t* slot_dev, int M) {
    if (!ctx || !x || !cache || !pos_dev || !slot_dev) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, M >= 1 && nq >= 1 && nk >= 1 && nv >= 1 && head_dim >= 1 && nq % head_dim == 0 && nk % head_dim == 0 && ring >= 1, "shape");
    KF_REQUIRE(ctx, !v_from_k || nv == nk, "values taken from the keys have the keys' size");
    KF_REQUIRE(ctx, rot_dims >= 0 && rot_dims <= head_dim && rot_dims % 2 == 0 && (rot_dims == 0 || inv_freq_dev) && (layout == 0 || layout == 1), "rotation");
    KF_REQUIRE(ctx, slot_stride >= (size_t)ring * (nk + nv), "slot stride");
    PrepArgs a = {};
    a.x = x, a.ldx = ldx, a.nq = nq, a.nk = nk, a.nv = nv, a.hd = head_dim, a.qw = (const uint16_t*)q_norm_bf16, a.kw = (const uint16_t*)k_norm_bf16;
    a.eps = eps, a.amp = amp, a.rot_dims = rot_dims, a.layout = layout, a.inv_freq = inv_freq_dev, a.cache = cache, a.slot_stride = slot_stride, a.ring = ring;
    a.pos = pos_dev, a.slot = slot_dev, a.qb = (uint16_t*)q_bf16_out;
    a.qb_add = (const uint16_t*)q_bias_bf16, a.kb_add = (const uint16_t*)k_bias_bf16, a.v_from_k = v_from_k ? 1 : 0;
    const size_t smem = (size_t)(nq + nk + rot_dims) * sizeof(float);
    KF_REQUIRE(ctx, smem <= 48 * 1024, "query + key row");
    if (cache_f32) kf_qk_prepare_kernel<float><<<M, 256, smem, ctx->stream>>>(a);
    else kf_qk_prepare_kernel<uint16_t><<<M, 256, smem, ctx->stream>>>(a);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}

// out [M][ldo] (heads x dv, activation type) = attention of token m over the rows of positions max(0, pos[m] - window + 1) .. pos[m] of its
// slot's ring (its own row appended before).  window <= 0: every position from 0; softcap <= 0: scores are not capped; sink: bf16 [H] or
// NULL.  ring must cover the window (and, for window <= 0, every position).  max_keys_hint: an upper bound of the keys a token sees (sizes
// the split of the keys over CTAs; the result does not depend on it beyond rounding).  out_scale multiplies the result before it is rounded.
extern "C" int kf_attn_window(kf_ctx* ctx, void* out, int out_f32, int ldo, const float* q, int ldq, const void* cache, int cache_f32, size_t slot_stride,
                              int ring, const void* sink_bf16, const int32_t* pos_dev, const int32_t* slot_dev, int M, int H, int G, int dk, int dv, float scale,
                              float softcap, int window, int max_keys_hint, float out_scale) {
    if (!ctx || !out || !q || !cache || !pos_dev || !slot_dev) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, M >= 1 && H >= 1 && G >= 1 && H % G == 0 && dk >= 1 && dv >= 1 && dv <= 512 && ring >= 1 && (window <= 0 || ring >= window),
               "value size <= 512, kv heads divide heads, the ring covers the window");
    WinArgs a = {};
    a.out = out, a.ldo = ldo, a.out_f32 = out_f32, a.q = q, a.ldq = ldq, a.cache = cache, a.slot_stride = slot_stride, a.ring = ring, a.window = window;
    a.sink = (const uint16_t*)sink_bf16, a.pos = pos_dev, a.slot = slot_dev, a.H = H, a.G = G, a.dk = dk, a.dv = dv, a.scale = scale, a.softcap = softcap, a.out_scale = out_scale;
    const size_t smem = (size_t)(dk + AW * dv + AW * 2) * sizeof(float);
    KF_REQUIRE(ctx, smem <= 48 * 1024, "key size");
    if (window > 0) max_keys_hint = std::min(max_keys_hint, window);
    int nsplit = 1;  // few (token, head) pairs and many keys (decoding): the keys are dealt to several CTAs so that the SMs are busy
    if (M * H < 2 * ctx->sm_count && max_keys_hint >= 4 * AW * 32)
        nsplit = std::max(1, std::min(std::min(64, (2 * ctx->sm_count) / (M * H)), max_keys_hint / (2 * AW * 32)));
    if (nsplit > 1) {
        KF_REQUIRE(ctx, kf_ensure_attn_ws(ctx, (size_t)M * H * nsplit * (dv + 2) * sizeof(float)) == KF_OK, "attention workspace");
        a.ws = ctx->attn_ws;
    }
    a.nsplit = nsplit;
    dim3 grid(M, H, nsplit);
    const int vpl = (dv + 31) / 32;
#define KF_AWK(TC, V) kf_attn_window_kernel<TC, V><<<grid, AW * 32, smem, ctx->stream>>>(a)
    if (cache_f32) {
        if (vpl <= 2) KF_AWK(float, 2);
        else if (vpl <= 4) KF_AWK(float, 4);
        else if (vpl <= 8) KF_AWK(float, 8);
        else KF_AWK(float, 16);
    } else {
        if (vpl <= 2) KF_AWK(uint16_t, 2);
        else if (vpl <= 4) KF_AWK(uint16_t, 4);
        else if (vpl <= 8) KF_AWK(uint16_t, 8);
        else KF_AWK(uint16_t, 16);
    }
#undef KF_AWK
    KF_LAUNCH_CHECK(ctx);
    if (nsplit > 1) {
        kf_attn_window_merge_kernel<<<dim3(M, H), 128, 0, ctx->stream>>>(a);
        KF_LAUNCH_CHECK(ctx);
    }
    return KF_OK;
}

// out [M][ldo] (heads x dv, activation type) = sum over the visible keys j of sigmoid(scale q . k_j + head_bias[h]) v_j -- no softmax, the
// weights are not normalised.  Visible: positions <= pos[m] inside the block of `block` consecutive positions (aligned to position 0) that
// holds pos[m] (block <= 0: every earlier position), and inside the last `window` positions when window > 0.  Cache rows as in
// kf_attn_window ([k | v] per position in a ring); the ring must cover a block (and every position when there are no blocks and no window).
extern "C" int kf_attn_sigmoid(kf_ctx* ctx, void* out, int out_f32, int ldo, const float* q, int ldq, const void* cache, int cache_f32, size_t slot_stride,
                               int ring, const void* head_bias_bf16, const int32_t* pos_dev, const int32_t* slot_dev, int M, int H, int G, int dk, int dv,
                               float scale, int block, int window, int max_keys_hint, float out_scale) {
    if (!ctx || !out || !q || !cache || !pos_dev || !slot_dev) return KF_ERR_BAD_ARG;
    const int span = (block > 0 && window > 0) ? std::min(block, window) : block > 0 ? block : window > 0 ? window : 0;  // most keys a query sees (0: all)
    KF_REQUIRE(ctx, M >= 1 && H >= 1 && G >= 1 && H % G == 0 && dk >= 1 && dv >= 1 && dv <= 512 && ring >= 1 && ring >= span,
               "value size <= 512, kv heads divide heads, the ring covers a block or the window");
    WinArgs a = {};
    a.out = out, a.ldo = ldo, a.out_f32 = out_f32, a.q = q, a.ldq = ldq, a.cache = cache, a.slot_stride = slot_stride, a.ring = ring, a.window = window;
    a.pos = pos_dev, a.slot = slot_dev, a.H = H, a.G = G, a.dk = dk, a.dv = dv, a.scale = scale, a.out_scale = out_scale;
    a.block = block > 0 ? block : 0, a.pbias = (const uint16_t*)head_bias_bf16;
    const size_t smem = (size_t)(dk + AW * dv) * sizeof(float);
    KF_REQUIRE(ctx, smem <= 48 * 1024, "key size");
    if (window > 0) max_keys_hint = std::min(max_keys_hint, window);
    if (block > 0) max_keys_hint = std::min(max_keys_hint, block);
    int nsplit = 1;
    if (M * H < 2 * ctx->sm_count && max_keys_hint >= 4 * AW * 32)
        nsplit = std::max(1, std::min(std::min(64, (2 * ctx->sm_count) / (M * H)), max_keys_hint / (2 * AW * 32)));
    if (nsplit > 1) {
        KF_REQUIRE(ctx, kf_ensure_attn_ws(ctx, (size_t)M * H * nsplit * dv * sizeof(float)) == KF_OK, "attention workspace");
        a.ws = ctx->attn_ws;
    }
    a.nsplit = nsplit;
    dim3 grid(M, H, nsplit);
    const int vpl = (dv + 31) / 32;
#define KF_ASK(TC, V) kf_attn_sigmoid_kernel<TC, V><<<grid, AW * 32, smem, ctx->stream>>>(a)
    if (cache_f32) {
        if (vpl <= 2) KF_ASK(float, 2);
        else if (vpl <= 4) KF_ASK(float, 4);
        else if (vpl <= 8) KF_ASK(float, 8);
        else KF_ASK(float, 16);
    } else {
        if (vpl <= 2) KF_ASK(uint16_t, 2);
        else if (vpl <= 4) KF_ASK(uint16_t, 4);
        else if (vpl <= 8) KF_ASK(uint16_t, 8);
        else KF_ASK(uint16_t, 16);
    }
#undef KF_ASK
    KF_LAUNCH_CHECK(ctx);
    if (nsplit > 1) {
        kf_attn_sigmoid_merge_kernel<<<dim3(M, H), 128, 0, ctx->stream>>>(a);
        KF_LAUNCH_CHECK(ctx);
    }
    return KF_OK;
}
