// ops_f32.cu -- the small ops of models whose residual stream, norms and routers are kept in 32-bit floats: embedding rows widened to
// fp32, grouped RMS norm (optionally of a gated input, optionally accumulated into the residual), and the router / dispatch / combine
// steps of a mixture of experts.  Outputs that feed a matmul are written in the activation type: bf16 bits, or float for a model that
// runs entirely in 32-bit.  No reference equivalent (the reference's norms are CU_rms_infer over bf16 rows, layernorm.cuh:801-859, and
// it has no expert routing on the inference path).
#include <math.h>

#include <algorithm>

#include "kf_common.cuh"

namespace {
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

__device__ __forceinline__ float gelu_tanh_f(float z) { return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }

__global__ void kf_embed_f32_kernel(float* __restrict__ out, float* __restrict__ out2, const uint16_t* __restrict__ table, const int32_t* __restrict__ tokens,
                                    int dim, float scale) {
    const uint16_t* row = table + (size_t)tokens[blockIdx.x] * dim;
    float* o            = out + (size_t)blockIdx.x * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = bf16_bits_to_f32(row[i]) * scale;
        o[i] = v;
        if (out2) out2[(size_t)blockIdx.x * dim + i] = v;
    }
}

// out[r][c] = act(in[r][c] + bias[c]) (* mul[r][c]) ; ACT 0: identity, 1: gelu (tanh form), 2: relu squared, 3: silu, 4: relu.
// OUT 0: bf16 bits, 1: float, 2: out (float) += result.
template <int ACT, int OUT>
__global__ void kf_bias_act_kernel(void* __restrict__ out, int ldo, const float* __restrict__ in, int ldi, const uint16_t* __restrict__ bias,
                                   const float* __restrict__ mul, int ldm, int cols) {
    const int r = blockIdx.y;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x) {
        float v = in[(size_t)r * ldi + c] + (bias ? bf16_bits_to_f32(bias[c]) : 0.f);
        if (ACT == 1) v = gelu_tanh_f(v);
        if (ACT == 2) v = v > 0.f ? v * v : 0.f;
        if (ACT == 3) v = v * sigmoid_f(v);
        if (ACT == 4) v = fmaxf(v, 0.f);
        if (mul) v *= mul[(size_t)r * ldm + c];
        if (OUT == 0) ((uint16_t*)out)[(size_t)r * ldo + c] = f32_to_bf16_bits(v);
        else if (OUT == 1) ((float*)out)[(size_t)r * ldo + c] = v;
        else ((float*)out)[(size_t)r * ldo + c] += v;
    }
}
// out[r][c] = gelu_tanh(in[r][c]) * table[token[r]][c0 + c]   (a per-token embedding slice gating a projection), activation type out
template <typename TO>
__global__ void kf_token_gate_kernel(TO* __restrict__ out, int ldo, const float* __restrict__ in, int ldi, const uint16_t* __restrict__ table, int ldt, int c0,
                                     const int32_t* __restrict__ tokens, int cols) {
    const int r = blockIdx.x;
    const uint16_t* e = table + (size_t)tokens[r] * ldt + c0;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = gelu_tanh_f(in[(size_t)r * ldi + c]) * bf16_bits_to_f32(e[c]);
        if (sizeof(TO) == 2) ((uint16_t*)out)[(size_t)r * ldo + c] = f32_to_bf16_bits(v);
        else ((float*)out)[(size_t)r * ldo + c] = v;
    }
}
// Weighted sum over the depth of a stack: hist[n_prev] = x (this layer's result) ; x = sum_{j < n_prev} w[j] * hist[j] + w[n_prev] * x.
// hist: [n_prev + 1][hist_stride] floats; n = rows * dim elements.
__global__ void kf_depth_mix_kernel(float* __restrict__ x, float* __restrict__ hist, size_t hist_stride, const uint16_t* __restrict__ w, int n_prev, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float cur = x[i];
    hist[(size_t)n_prev * hist_stride + i] = cur;
    float s = 0.f;
    for (int j = 0; j < n_prev; j++) s = fmaf(bf16_bits_to_f32(w[j]), hist[(size_t)j * hist_stride + i], s);
    x[i] = fmaf(bf16_bits_to_f32(w[n_prev]), cur, s);
}

// One block per (row, group).  v = x * gatefn(g) (GATE 0: none, 1: sigmoid(g + gate_bias), 2: silu(g));  r = v / sqrt(mean_group(v^2) + eps) * w;
// GATE 3 / 4: the gate multiplies the normed result instead, r *= sigmoid(g) / silu(g).  w_shared: one weight of group size for all groups.
// ACC: res[row] += mult * r (fp32 residual stream)  else  out[row] = r in the activation type.  w_add is added to every weight in
// fp32 (1 for weights that are stored around zero).
template <int GATE, bool ACC, typename TO>
__global__ void __launch_bounds__(256) kf_group_norm_kernel(TO* __restrict__ out, int ldo, float* __restrict__ res, const float* __restrict__ x, int ldx,
                                                            const float* __restrict__ gate, int ldg, const uint16_t* __restrict__ gate_bias,
                                                            const uint16_t* __restrict__ w, const int32_t* __restrict__ row_idx, int dim, int groups,
                                                            float eps, float mult, int w_shared, float w_add, float out_mult) {
    __shared__ float red[32];
    const int r = blockIdx.x, grp = blockIdx.y, gs = dim / groups;
    const int src = row_idx ? row_idx[r] : r;
    const float* xr = x + (size_t)src * ldx + grp * gs;
    const float* gr = GATE ? gate + (size_t)src * ldg + grp * gs : nullptr;
    auto val = [&](int i) -> float {
        float v = xr[i];
        if (GATE == 1) v *= sigmoid_f(gr[i] + (gate_bias ? bf16_bits_to_f32(gate_bias[grp * gs + i]) : 0.f));
        if (GATE == 2) {
            const float z = gr[i];
            v *= z * sigmoid_f(z);
        }
        return v;
    };
    float ss = 0.f;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        const float v = val(i);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)gs + eps);
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        float o = val(i) * s * (w_add + bf16_bits_to_f32(w[w_shared ? i : grp * gs + i]));
        if (GATE == 3) o *= sigmoid_f(gr[i]);
        if (GATE == 4) {
            const float z = gr[i];
            o *= z * sigmoid_f(z);
        }
        if (ACC) {
            float* p = res + (size_t)r * dim + grp * gs + i;
            *p       = *p + mult * o;
        } else if (sizeof(TO) == 2) {
            ((uint16_t*)out)[(size_t)r * ldo + grp * gs + i] = f32_to_bf16_bits(o * out_mult);
        } else {
            ((float*)out)[(size_t)r * ldo + grp * gs + i] = o * out_mult;
        }
    }
}

// Post-norm residual step of one row:  v = sa * a + sb * b (b optional);  res += v / sqrt(mean(v^2) + eps) * (w_add + w);  the new
// residual row is also written in the activation type (what the next sublayer's matmul reads) when act_out is given.
template <typename TO>
__global__ void __launch_bounds__(256) kf_postnorm_residual_kernel(float* __restrict__ res, TO* __restrict__ act_out, const float* __restrict__ a, int lda, float sa,
                                                                   const float* __restrict__ b, int ldb, float sb, const uint16_t* __restrict__ w, float w_add,
                                                                   int dim, float eps) {
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float* ar = a + (size_t)r * lda;
    const float* br = b ? b + (size_t)r * ldb : nullptr;
    auto val = [&](int i) -> float { return br ? fmaf(sb, br[i], sa * ar[i]) : sa * ar[i]; };
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = val(i);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)dim + eps);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float* p = res + (size_t)r * dim + i;
        const float x = *p + val(i) * s * (w_add + bf16_bits_to_f32(w[i]));
        *p = x;
        if (act_out) {
            if (sizeof(TO) == 2) ((uint16_t*)act_out)[(size_t)r * dim + i] = f32_to_bf16_bits(x);
            else ((float*)act_out)[(size_t)r * dim + i] = x;
        }
    }
}

// Pre-norm residual step of one row:  res += a + b + vec (each optional);  act_out = res / sqrt(mean(res^2) + eps) * w in the activation
// type (what the next sublayer's matmul reads; w NULL: only the sum).
template <typename TO>
__global__ void __launch_bounds__(256) kf_residual_prenorm_kernel(float* __restrict__ res, TO* __restrict__ act_out, const float* __restrict__ a, int lda,
                                                                  const float* __restrict__ b, int ldb, const uint16_t* __restrict__ vec,
                                                                  const uint16_t* __restrict__ w, int dim, float eps) {
    __shared__ float red[32];
    const int r = blockIdx.x;
    float* xr = res + (size_t)r * dim;
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = xr[i];
        if (a) v += a[(size_t)r * lda + i];
        if (b) v += b[(size_t)r * ldb + i];
        if (vec) v += bf16_bits_to_f32(vec[i]);
        if (a || b || vec) xr[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (!w) return;
    ss = block_sum(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)dim + eps);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {  // a thread re-reads what it wrote itself
        const float v = xr[i] * s * bf16_bits_to_f32(w[i]);
        if (sizeof(TO) == 2) ((uint16_t*)act_out)[(size_t)r * dim + i] = f32_to_bf16_bits(v);
        else ((float*)act_out)[(size_t)r * dim + i] = v;
    }
}
// out = g' * sigmoid(alpha * g') * (u' + shift),  g' = min(g, limit), u' = clamp(u, -limit, limit)  (limit <= 0: not clamped)
template <typename TO>
__global__ void kf_glu_clamped_kernel(TO* __restrict__ out, int ldo, const float* __restrict__ g, int ldg, const float* __restrict__ u, int ldu, int cols,
                                      float limit, float alpha, float shift) {
    const int r = blockIdx.y;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x) {
        float gv = g[(size_t)r * ldg + c], uv = u[(size_t)r * ldu + c];
        if (limit > 0.f) gv = fminf(gv, limit), uv = fminf(fmaxf(uv, -limit), limit);
        const float v = gv * sigmoid_f(alpha * gv) * (uv + shift);
        if (sizeof(TO) == 2) ((uint16_t*)out)[(size_t)r * ldo + c] = f32_to_bf16_bits(v);
        else ((float*)out)[(size_t)r * ldo + c] = v;
    }
}
__global__ void kf_scale_f32_kernel(float* __restrict__ x, size_t n, float s) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] *= s;
}

__global__ void kf_f32_to_bf16_kernel(uint16_t* __restrict__ out, const float* __restrict__ in, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f32_to_bf16_bits(in[i]);
}

// ---- mixture of experts ---------------------------------------------------------------------------------------------------
// How a token's experts are chosen and weighted.  kind 0: arg-max over logits (+ bias), weights from a softmax (the kernels' `full` flag).
// kind 1: scores s = sigmoid(logit); the choice runs over s + bias; the experts form `groups` equal contiguous groups, a group is ranked
// by the sum of its top-2 choice values and only the `keep` best groups can be chosen from; weights = scale * s of the chosen, not
// renormalised.
struct RouteMode {
    int kind, groups, keep;
    float scale;
};
// one warp routes one token in kind 1.  taken: the token's chosen experts so far (shared or global memory, written by lane 0).
__device__ __forceinline__ void route_grouped_warp(int* taken, int32_t* idx, float* __restrict__ wgt, const float* __restrict__ lg,
                                                   const uint16_t* __restrict__ bias, int E, int top, const RouteMode md, int lane) {
    const int per = E / md.groups;
    // lane g keeps the rank value of group g (groups <= 32): the top-2 choice values of the group, found by all lanes together
    float gscore = -INFINITY;
    for (int g = 0; g < md.groups; g++) {
        float a = -INFINITY, b = -INFINITY;  // largest, second largest of this lane's share
        for (int e = g * per + lane; e < (g + 1) * per; e += 32) {
            const float v = sigmoid_f(lg[e]) + (bias ? bf16_bits_to_f32(bias[e]) : 0.f);
            if (v > a) b = a, a = v;
            else if (v > b) b = v;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float oa = __shfl_xor_sync(0xffffffffu, a, o), ob = __shfl_xor_sync(0xffffffffu, b, o);
            const float hi = fmaxf(a, oa), lo = fmaxf(fminf(a, oa), fmaxf(b, ob));
            a = hi, b = lo;
        }
        if (lane == g) gscore = per > 1 ? a + b : a;
    }
    unsigned kept = 0;
    for (int r = 0; r < md.keep; r++) {
        float best = (lane < md.groups && !((kept >> lane) & 1u)) ? gscore : -INFINITY;
        int bi     = (lane < md.groups && !((kept >> lane) & 1u)) ? lane : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi   = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi))) best = ob, bi = oi;
        }
        if (bi != 0x7fffffff) kept |= 1u << bi;
    }
    for (int j = 0; j < top; j++) {
        float best = -INFINITY;
        int bi     = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            if (!((kept >> (e / per)) & 1u)) continue;
            bool was = false;
            for (int q = 0; q < j; q++) was = was || taken[q] == e;
            if (was) continue;
            const float v = sigmoid_f(lg[e]) + (bias ? bf16_bits_to_f32(bias[e]) : 0.f);
            if (bi == 0x7fffffff || v > best || (v == best && e < bi)) best = v, bi = e;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi   = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ob > best || (ob == best && oi < bi))) best = ob, bi = oi;
        }
        if (lane == 0) taken[j] = bi, idx[j] = bi, wgt[j] = md.scale * sigmoid_f(lg[bi]);
        __syncwarp();
    }
}
// one warp per token: `top` rounds of arg-max over the E router logits (+ bias), ties to the lower index; weights = softmax over the
// chosen logits only, or (full) the chosen entries of the softmax over ALL experts, not renormalised.  All in fp32.
__global__ void __launch_bounds__(128) kf_moe_route_kernel(int32_t* __restrict__ idx, float* __restrict__ wgt, const float* __restrict__ logits, int ldl,
                                                           const uint16_t* __restrict__ bias, int M, int E, int top, int full, const RouteMode md) {
    const int m = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (m >= M) return;
    const float* lg = logits + (size_t)m * ldl;
    if (md.kind == 1) {
        route_grouped_warp(idx + (size_t)m * top, idx + (size_t)m * top, wgt + (size_t)m * top, lg, bias, E, top, md, lane);
        return;
    }
    float first = 0.f, den = 0.f;
    for (int j = 0; j < top; j++) {
        float best = -INFINITY;
        int bi     = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            bool taken = false;
            for (int q = 0; q < j; q++) taken = taken || idx[(size_t)m * top + q] == e;
            if (taken) continue;
            const float v = lg[e] + (bias ? bf16_bits_to_f32(bias[e]) : 0.f);
            if (v > best || (v == best && e < bi)) best = v, bi = e;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi   = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) best = ob, bi = oi;
        }
        if (j == 0) first = best;
        const float p = expf(best - first);
        den += p;
        if (lane == 0) idx[(size_t)m * top + j] = bi, wgt[(size_t)m * top + j] = p;
        __syncwarp();
    }
    if (full) {  // the denominator runs over every expert (first = the largest logit)
        float d = 0.f;
        for (int e = lane; e < E; e += 32) d += expf(lg[e] + (bias ? bf16_bits_to_f32(bias[e]) : 0.f) - first);
        den = warp_sum(d);
    }
    if (lane < top) {
        for (int j = lane; j < top; j += 32) wgt[(size_t)m * top + j] /= den;
    }
}
// few tokens (decode): routing and the dispatch tables in ONE block -- warps route the tokens, then thread i ranks entry i among the
// earlier entries of its expert, the lanes of warp 0 count one expert each and scan the counts
constexpr int kRouteSmall = 256;
__global__ void __launch_bounds__(256) kf_moe_route_small_kernel(int32_t* __restrict__ idx, float* __restrict__ wgt, int32_t* __restrict__ offsets,
                                                                 int32_t* __restrict__ entry_slot, int32_t* __restrict__ slot_row,
                                                                 int32_t* __restrict__ slot_group, const float* __restrict__ logits, int ldl,
                                                                 const uint16_t* __restrict__ bias, int M, int E, int top, int full, const RouteMode md) {
    __shared__ int sidx[kRouteSmall];
    __shared__ int srank[kRouteSmall];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n = M * top;
    for (int m = warp; m < M; m += 8) {
        const float* lg = logits + (size_t)m * ldl;
        if (md.kind == 1) {
            route_grouped_warp(sidx + m * top, idx + (size_t)m * top, wgt + (size_t)m * top, lg, bias, E, top, md, lane);
            continue;
        }
        float first = 0.f, den = 0.f;
        for (int j = 0; j < top; j++) {
            float best = -INFINITY;
            int bi     = 0x7fffffff;
            for (int e = lane; e < E; e += 32) {
                bool taken = false;
                for (int q = 0; q < j; q++) taken = taken || sidx[m * top + q] == e;
                if (taken) continue;
                const float v = lg[e] + (bias ? bf16_bits_to_f32(bias[e]) : 0.f);
                if (v > best || (v == best && e < bi)) best = v, bi = e;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi   = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ob > best || (ob == best && oi < bi)) best = ob, bi = oi;
            }
            if (j == 0) first = best;
            const float p = expf(best - first);
            den += p;
            if (lane == 0) sidx[m * top + j] = bi, idx[(size_t)m * top + j] = bi, wgt[(size_t)m * top + j] = p;
            __syncwarp();
        }
        if (full) {
            float d = 0.f;
            for (int e = lane; e < E; e += 32) d += expf(lg[e] + (bias ? bf16_bits_to_f32(bias[e]) : 0.f) - first);
            den = warp_sum(d);
        }
        for (int j = lane; j < top; j += 32) wgt[(size_t)m * top + j] /= den;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        int r = 0;
        for (int j = 0; j < i; j++) r += sidx[j] == sidx[i];
        srank[i] = r;
    }
    __syncthreads();
    if (warp == 0) {  // offsets: lane l counts the entries of expert e0 + l, a scan over the lanes places them behind the experts before
        int base = 0;
        for (int e0 = 0; e0 < E; e0 += 32) {
            const int e = e0 + lane;
            int c = 0;
            for (int j = 0; j < n; j++) c += sidx[j] == e;  // e >= E matches nothing
            int incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            if (e < E) offsets[e] = base + incl - c;
            base += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) offsets[E] = base;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int e = sidx[i], sl = offsets[e] + srank[i];
        entry_slot[i] = sl, slot_row[sl] = i / top, slot_group[sl] = e;
    }
}
// one block per expert: the entries (token, choice) routed to it, ranked in entry order (ballot + popc compaction)
__global__ void __launch_bounds__(256) kf_moe_rank_kernel(int32_t* __restrict__ rank, int32_t* __restrict__ count, const int32_t* __restrict__ idx, int n) {
    __shared__ int wsum[8];
    __shared__ int base;
    const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) base = 0;
    __syncthreads();
    for (int i0 = 0; i0 < n; i0 += 256) {
        const int i    = i0 + threadIdx.x;
        const bool hit = i < n && idx[i] == e;
        const unsigned b = __ballot_sync(0xffffffffu, hit);
        if (lane == 0) wsum[warp] = __popc(b);
        __syncthreads();
        int before = base;
        for (int q = 0; q < warp; q++) before += wsum[q];
        if (hit) rank[i] = before + __popc(b & ((1u << lane) - 1));
        __syncthreads();
        if (threadIdx.x == 0) {
            int t = 0;
            for (int q = 0; q < 8; q++) t += wsum[q];
            base += t;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) count[e] = base;
}
// offsets = exclusive scan of the counts (one thread: E is small); then each entry learns its slot
__global__ void kf_moe_offsets_kernel(int32_t* __restrict__ offsets, const int32_t* __restrict__ count, int E) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int s = 0;
        for (int e = 0; e < E; e++) offsets[e] = s, s += count[e];
        offsets[E] = s;
    }
}
__global__ void kf_moe_slots_kernel(int32_t* __restrict__ entry_slot, int32_t* __restrict__ slot_row, int32_t* __restrict__ slot_group,
                                    const int32_t* __restrict__ idx, const int32_t* __restrict__ rank, const int32_t* __restrict__ offsets, int n, int top) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int e = idx[i], s = offsets[e] + rank[i];
    entry_slot[i] = s, slot_row[s] = i / top, slot_group[s] = e;
}
// out[m] = sum_j wgt[m][j] * y[slot(m, j)]  (+ sigmoid(sg[m]) * shared[m]), choices added in their routing order
__global__ void kf_moe_combine_kernel(float* __restrict__ out, const float* __restrict__ y, const int32_t* __restrict__ entry_slot,
                                      const float* __restrict__ wgt, const float* __restrict__ shared, const float* __restrict__ sg, int ldsg, int dim, int top,
                                      int accumulate) {
    const int m = blockIdx.x;
    const float gate = shared ? (sg ? sigmoid_f(sg[(size_t)m * ldsg]) : 1.f) : 0.f;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float s = 0.f;
        for (int j = 0; j < top; j++) s = fmaf(wgt[(size_t)m * top + j], y[(size_t)entry_slot[(size_t)m * top + j] * dim + d], s);
        if (shared) s = fmaf(gate, shared[(size_t)m * dim + d], s);
        out[(size_t)m * dim + d] = accumulate ? out[(size_t)m * dim + d] + s : s;
    }
}
}  // namespace

// out[m] = scale * W[token[m]] as floats; out2 (optional) receives a second copy
extern "C" int kf_embed_f32_scaled(kf_ctx* ctx, float* out, float* out2, const kf_tensor_desc* w, const int32_t* tokens_dev, int M, float scale) {
    if (!ctx || !out || !w || !tokens_dev) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, w->type == KF_T_BF16 && M >= 1, "bf16 table");
    kf_embed_f32_kernel<<<M, 256, 0, ctx->stream>>>(out, out2, (const uint16_t*)w->data_dev, tokens_dev, w->cols, scale);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
extern "C" int kf_embed_f32(kf_ctx* ctx, float* out, const kf_tensor_desc* w, const int32_t* tokens_dev, int M) {
    return kf_embed_f32_scaled(ctx, out, nullptr, w, tokens_dev, M, 1.f);
}
// out[rows][ldo] = act(in[rows][ldi] + bias) (* mul); act 0: none, 1: gelu (tanh form), 2: relu squared, 3: silu, 4: relu; out_kind 0: bf16 bits,
// 1: float, 2: float out += result.  bias: bf16 [cols] or NULL; mul: float [rows][ldm] or NULL.
extern "C" int kf_bias_act(kf_ctx* ctx, void* out, int out_kind, int ldo, const float* in, int ldi, const void* bias_bf16, int act, const float* mul, int ldm,
                           int rows, int cols) {
    if (!ctx || !out || !in) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, rows >= 1 && cols >= 1 && act >= 0 && act <= 4 && out_kind >= 0 && out_kind <= 2, "act / out kind");
    dim3 grid(std::min(64, (cols + 255) / 256), rows);
    const uint16_t* b = (const uint16_t*)bias_bf16;
#define KF_BA(A, O) kf_bias_act_kernel<A, O><<<grid, 256, 0, ctx->stream>>>(out, ldo, in, ldi, b, mul, ldm, cols)
#define KF_BA_O(A) (out_kind == 0 ? KF_BA(A, 0) : out_kind == 1 ? KF_BA(A, 1) : KF_BA(A, 2))
    if (act == 0) KF_BA_O(0);
    else if (act == 1) KF_BA_O(1);
    else if (act == 2) KF_BA_O(2);
    else if (act == 3) KF_BA_O(3);
    else KF_BA_O(4);
#undef KF_BA_O
#undef KF_BA
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
extern "C" int kf_token_gate(kf_ctx* ctx, void* out, int out_f32, int ldo, const float* in, int ldi, const void* table_bf16, int ldt, int c0,
                             const int32_t* tokens_dev, int rows, int cols) {
    if (!ctx || !out || !in || !table_bf16 || !tokens_dev) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, rows >= 1 && cols >= 1 && c0 >= 0 && c0 + cols <= ldt, "slice inside the table row");
    if (out_f32) kf_token_gate_kernel<float><<<rows, 128, 0, ctx->stream>>>((float*)out, ldo, in, ldi, (const uint16_t*)table_bf16, ldt, c0, tokens_dev, cols);
    else kf_token_gate_kernel<uint16_t><<<rows, 128, 0, ctx->stream>>>((uint16_t*)out, ldo, in, ldi, (const uint16_t*)table_bf16, ldt, c0, tokens_dev, cols);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
extern "C" int kf_depth_mix(kf_ctx* ctx, float* x, float* hist, size_t hist_stride, const void* w_bf16, int n_prev, size_t n) {
    if (!ctx || !x || !hist || !w_bf16) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, n_prev >= 0 && n >= 1 && hist_stride >= n, "history stride");
    kf_depth_mix_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(x, hist, hist_stride, (const uint16_t*)w_bf16, n_prev, n);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}

// gate_kind 0: none; 1: x * sigmoid(gate + gate_bias); 2: x * silu(gate).  out_kind 0: bf16 bits [rows][ldo]; 1: float [rows][ldo];
// 2: res[rows][dim] += mult * result (out is ignored).  row_idx (device, optional): source row of each output row.
// gate_kind 3 / 4: sigmoid(gate) / silu(gate) multiply the normed result; w_shared: the weight has dim / groups entries, used by every group.
// w_add: added to every weight in fp32 (1 for weights stored around zero, 0 for plain weights).  out_mult: factor on the rows written to
// out (out_kind 0 / 1), applied in fp32 before the rounding.
extern "C" int kf_group_rmsnorm_wadd(kf_ctx* ctx, void* out, int out_kind, int ldo, float* res, float mult, const float* x, int ldx, const float* gate, int ldg,
                                     const void* gate_bias_bf16, int gate_kind, const void* w_bf16, int w_shared, float w_add, float out_mult,
                                     const int32_t* row_idx, int rows, int dim, int groups, float eps) {
    if (!ctx || !x || !w_bf16) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, rows >= 1 && dim >= 1 && groups >= 1 && dim % groups == 0, "groups must divide dim");
    KF_REQUIRE(ctx, gate_kind >= 0 && gate_kind <= 4 && (gate_kind == 0 || gate) && out_kind >= 0 && out_kind <= 2 && (out_kind == 2 ? res != nullptr : out != nullptr),
               "gate / out kind");
    dim3 grid(rows, groups);
    const uint16_t *gb = (const uint16_t*)gate_bias_bf16, *w = (const uint16_t*)w_bf16;
#define KF_GN(G, A, T) kf_group_norm_kernel<G, A, T><<<grid, 256, 0, ctx->stream>>>((T*)out, ldo, res, x, ldx, gate, ldg, gb, w, row_idx, dim, groups, eps, mult, w_shared, w_add, out_mult)
    if (out_kind == 2) {
        if (gate_kind == 0) KF_GN(0, true, float);
        else if (gate_kind == 1) KF_GN(1, true, float);
        else if (gate_kind == 2) KF_GN(2, true, float);
        else if (gate_kind == 3) KF_GN(3, true, float);
        else KF_GN(4, true, float);
    } else if (out_kind == 1) {
        if (gate_kind == 0) KF_GN(0, false, float);
        else if (gate_kind == 1) KF_GN(1, false, float);
        else if (gate_kind == 2) KF_GN(2, false, float);
        else if (gate_kind == 3) KF_GN(3, false, float);
        else KF_GN(4, false, float);
    } else {
        if (gate_kind == 0) KF_GN(0, false, uint16_t);
        else if (gate_kind == 1) KF_GN(1, false, uint16_t);
        else if (gate_kind == 2) KF_GN(2, false, uint16_t);
        else if (gate_kind == 3) KF_GN(3, false, uint16_t);
        else KF_GN(4, false, uint16_t);
    }
#undef KF_GN
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
extern "C" int kf_group_rmsnorm_ex(kf_ctx* ctx, void* out, int out_kind, int ldo, float* res, float mult, const float* x, int ldx, const float* gate, int ldg,
                                   const void* gate_bias_bf16, int gate_kind, const void* w_bf16, int w_shared, const int32_t* row_idx, int rows, int dim,
                                   int groups, float eps) {
    return kf_group_rmsnorm_wadd(ctx, out, out_kind, ldo, res, mult, x, ldx, gate, ldg, gate_bias_bf16, gate_kind, w_bf16, w_shared, 0.f, 1.f, row_idx, rows,
                                 dim, groups, eps);
}
extern "C" int kf_group_rmsnorm(kf_ctx* ctx, void* out, int out_kind, int ldo, float* res, float mult, const float* x, int ldx, const float* gate, int ldg,
                                const void* gate_bias_bf16, int gate_kind, const void* w_bf16, const int32_t* row_idx, int rows, int dim, int groups,
                                float eps) {
    if (gate_kind > 2) return KF_ERR_BAD_ARG;
    return kf_group_rmsnorm_ex(ctx, out, out_kind, ldo, res, mult, x, ldx, gate, ldg, gate_bias_bf16, gate_kind, w_bf16, 0, row_idx, rows, dim, groups, eps);
}
// res[rows][dim] += rmsnorm(sa * a + sb * b) * (w_add + w);  act_out (optional, [rows][dim] in the activation type) = the new res.
// b may be NULL (one branch).  The norm runs over the whole row.
extern "C" int kf_postnorm_residual(kf_ctx* ctx, float* res, void* act_out, int act_f32, const float* a, int lda, float sa, const float* b, int ldb, float sb,
                                    const void* w_bf16, float w_add, int rows, int dim, float eps) {
    if (!ctx || !res || !a || !w_bf16) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, rows >= 1 && dim >= 1, "shape");
    if (act_f32)
        kf_postnorm_residual_kernel<float><<<rows, 256, 0, ctx->stream>>>(res, (float*)act_out, a, lda, sa, b, ldb, sb, (const uint16_t*)w_bf16, w_add, dim, eps);
    else
        kf_postnorm_residual_kernel<uint16_t><<<rows, 256, 0, ctx->stream>>>(res, (uint16_t*)act_out, a, lda, sa, b, ldb, sb, (const uint16_t*)w_bf16, w_add, dim, eps);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
// res[rows][dim] += a + b + vec (a, b: float rows or NULL; vec: bf16 [dim] or NULL); act_out (with w_bf16) = rmsnorm(res) * w in the
// activation type.  w_bf16 NULL: the sum only.
extern "C" int kf_residual_prenorm(kf_ctx* ctx, float* res, void* act_out, int act_f32, const float* a, int lda, const float* b, int ldb, const void* vec_bf16,
                                   const void* w_bf16, int rows, int dim, float eps) {
    if (!ctx || !res || (w_bf16 && !act_out)) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, rows >= 1 && dim >= 1, "shape");
    if (!w_bf16 && !a && !b && !vec_bf16) return KF_OK;
    if (act_f32)
        kf_residual_prenorm_kernel<float><<<rows, 256, 0, ctx->stream>>>(res, (float*)act_out, a, lda, b, ldb, (const uint16_t*)vec_bf16, (const uint16_t*)w_bf16, dim, eps);
    else
        kf_residual_prenorm_kernel<uint16_t><<<rows, 256, 0, ctx->stream>>>(res, (uint16_t*)act_out, a, lda, b, ldb, (const uint16_t*)vec_bf16, (const uint16_t*)w_bf16, dim, eps);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
// out[rows][ldo] (activation type) = g' * sigmoid(alpha * g') * (u' + shift) with g' = min(gate, limit), u' = clamp(up, -limit, limit); limit <= 0: no clamp
extern "C" int kf_glu_clamped(kf_ctx* ctx, void* out, int out_f32, int ldo, const float* gate, int ldg, const float* up, int ldu, int rows, int cols, float limit,
                              float alpha, float shift) {
    if (!ctx || !out || !gate || !up) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, rows >= 1 && cols >= 1, "shape");
    dim3 grid(std::min(64, (cols + 255) / 256), rows);
    if (out_f32) kf_glu_clamped_kernel<float><<<grid, 256, 0, ctx->stream>>>((float*)out, ldo, gate, ldg, up, ldu, cols, limit, alpha, shift);
    else kf_glu_clamped_kernel<uint16_t><<<grid, 256, 0, ctx->stream>>>((uint16_t*)out, ldo, gate, ldg, up, ldu, cols, limit, alpha, shift);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
extern "C" int kf_scale_f32(kf_ctx* ctx, float* x, size_t n, float s) {
    if (!ctx || !x) return KF_ERR_BAD_ARG;
    if (!n || s == 1.f) return KF_OK;
    kf_scale_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(x, n, s);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
extern "C" int kf_f32_to_bf16(kf_ctx* ctx, void* out_bf16, const float* in, size_t n) {
    if (!ctx || !out_bf16 || !in) return KF_ERR_BAD_ARG;
    if (!n) return KF_OK;
    kf_f32_to_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>((uint16_t*)out_bf16, in, n);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}

// Router of a mixture of experts over fp32 logits [M][ldl] (+ bf16 bias [E] or NULL): idx / wgt [M][top]; then the dispatch tables:
// offsets [E + 1], entry_slot [M * top] (where each (token, choice) sits among the expert-sorted slots), slot_row / slot_group [M * top].
// work: device int32 scratch of 2 * M * top + E entries.
// full_softmax 0: weights = softmax over the chosen logits; 1: the chosen entries of the softmax over all E experts (not renormalised).
static int moe_route_impl(kf_ctx* ctx, int32_t* idx, float* wgt, int32_t* offsets, int32_t* entry_slot, int32_t* slot_row, int32_t* slot_group,
                          int32_t* work, const float* logits, int ldl, const void* bias_bf16, int M, int E, int top, int full_softmax, const RouteMode md) {
    if (!ctx || !idx || !wgt || !offsets || !entry_slot || !slot_row || !slot_group || !work || !logits) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, M >= 1 && E >= 1 && top >= 1 && top <= E && ldl >= E, "1 <= top <= experts");
    const int n = M * top;
    if (n <= kRouteSmall && (long long)E * n <= 16384) {
        kf_moe_route_small_kernel<<<1, 256, 0, ctx->stream>>>(idx, wgt, offsets, entry_slot, slot_row, slot_group, logits, ldl, (const uint16_t*)bias_bf16, M, E, top, full_softmax, md);
        KF_LAUNCH_CHECK(ctx);
        return KF_OK;
    }
    int32_t *rank = work, *count = work + n;
    kf_moe_route_kernel<<<(M + 3) / 4, 128, 0, ctx->stream>>>(idx, wgt, logits, ldl, (const uint16_t*)bias_bf16, M, E, top, full_softmax, md);
    KF_LAUNCH_CHECK(ctx);
    kf_moe_rank_kernel<<<E, 256, 0, ctx->stream>>>(rank, count, idx, n);
    KF_LAUNCH_CHECK(ctx);
    kf_moe_offsets_kernel<<<1, 32, 0, ctx->stream>>>(offsets, count, E);
    KF_LAUNCH_CHECK(ctx);
    kf_moe_slots_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>(entry_slot, slot_row, slot_group, idx, rank, offsets, n, top);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
extern "C" int kf_moe_route_ex(kf_ctx* ctx, int32_t* idx, float* wgt, int32_t* offsets, int32_t* entry_slot, int32_t* slot_row, int32_t* slot_group,
                               int32_t* work, const float* logits, int ldl, const void* bias_bf16, int M, int E, int top, int full_softmax) {
    const RouteMode md = {0, 1, 1, 1.f};
    return moe_route_impl(ctx, idx, wgt, offsets, entry_slot, slot_row, slot_group, work, logits, ldl, bias_bf16, M, E, top, full_softmax, md);
}
// The same tables from sigmoid scores: the choice runs over sigmoid(logit) + choice_bias (bf16 [E] or NULL) inside the `keep` best of
// `groups` equal contiguous groups of experts (a group ranks by the sum of its top-2 choice values; groups <= 32, groups 1: no
// grouping); weights = scale * sigmoid(logit) of the chosen experts, not renormalised.  top <= keep * (E / groups).
extern "C" int kf_moe_route_grouped(kf_ctx* ctx, int32_t* idx, float* wgt, int32_t* offsets, int32_t* entry_slot, int32_t* slot_row, int32_t* slot_group,
                                    int32_t* work, const float* logits, int ldl, const void* choice_bias_bf16, int M, int E, int top, int groups, int keep,
                                    float scale) {
    if (!ctx) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, groups >= 1 && groups <= 32 && E >= 1 && E % groups == 0 && keep >= 1 && keep <= groups && top >= 1 && top <= keep * (E / groups),
               "groups <= 32 divide the experts; 1 <= keep <= groups; top <= keep * experts / groups");
    const RouteMode md = {1, groups, keep, scale};
    return moe_route_impl(ctx, idx, wgt, offsets, entry_slot, slot_row, slot_group, work, logits, ldl, choice_bias_bf16, M, E, top, 0, md);
}
extern "C" int kf_moe_route(kf_ctx* ctx, int32_t* idx, float* wgt, int32_t* offsets, int32_t* entry_slot, int32_t* slot_row, int32_t* slot_group,
                            int32_t* work, const float* logits, int ldl, const void* bias_bf16, int M, int E, int top) {
    return kf_moe_route_ex(ctx, idx, wgt, offsets, entry_slot, slot_row, slot_group, work, logits, ldl, bias_bf16, M, E, top, 0);
}
// accumulate 1: out += the combination (the residual stream takes the experts' sum directly)
extern "C" int kf_moe_combine_ex(kf_ctx* ctx, float* out, const float* y_slots, const int32_t* entry_slot, const float* wgt, const float* shared,
                                 const float* shared_gate_logit, int ld_gate, int M, int dim, int top, int accumulate) {
    if (!ctx || !out || !y_slots || !entry_slot || !wgt) return KF_ERR_BAD_ARG;
    kf_moe_combine_kernel<<<M, 256, 0, ctx->stream>>>(out, y_slots, entry_slot, wgt, shared, shared_gate_logit, ld_gate, dim, top, accumulate);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
extern "C" int kf_moe_combine(kf_ctx* ctx, float* out, const float* y_slots, const int32_t* entry_slot, const float* wgt, const float* shared,
                              const float* shared_gate_logit, int ld_gate, int M, int dim, int top) {
    return kf_moe_combine_ex(ctx, out, y_slots, entry_slot, wgt, shared, shared_gate_logit, ld_gate, M, dim, top, 0);
}
