// seqmix.cu -- sequence mixers beside the GQA attention of attention.cu:
//   (1) selective state-space mixing (state-space duality form): a short causal convolution per channel with SiLU, then per head the
//       recurrence  S_t = exp(-exp(A) dt_t) S_{t-1} + dt_t B_t x_t^T,  y_t = S_t^T C_t + D x_t  with S an [N x P] fp32 state per
//       (sequence slot, head) that persists between calls, like the K/V rows of the attention cache;
//   (2) attention over a compressed latent: every cached row holds the normalised latent c (rank r) and ONE rotated key part shared by
//       all heads; queries are absorbed into latent space (q' = W_uk^T q), scores and the softmax -- whose denominator also holds a
//       learned per-head sink term -- run in fp32 over the cached rows, and the attended latent is expanded per head by W_uv.
// Everything that enters the recurrence or the softmax is fp32; the cache rows are stored in the activation type (bf16 bits, or float
// for a model run entirely in 32-bit).  A token m carries (pos[m], slot[m]); a slot whose first token has position 0 starts from a
// zero state without any clearing pass.  Tokens are laid out as nseq sequences of T consecutive tokens each (prefill panel: 1 x M;
// batched decode: M x 1).  No reference equivalent (the reference has neither mixer on its inference path).
#include <math.h>

#include <algorithm>

#include "kf_common.cuh"

namespace {
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ------------------------------------------------------------------------------------------------------------ causal convolution
// out[m][c] = silu(b[c] + sum_j w[c][j] * in(t - (K-1-j))), in(t') = u[t'] inside the panel, the slot's stored tail before it, 0 before
// the start of the sequence.  tail: [slot][K-1][C], oldest first.
__global__ void kf_conv_silu_kernel(float* __restrict__ out, const float* __restrict__ u, int ldu, const uint16_t* __restrict__ w, const uint16_t* __restrict__ b,
                                    const float* __restrict__ tail, size_t tail_stride, const int32_t* __restrict__ pos, const int32_t* __restrict__ slot,
                                    int T, int C, int K, int act) {
    const int m = blockIdx.x, seq = m / T, t = m - seq * T;
    const int p = pos[m];
    const float* tl = tail + (size_t)slot[m] * tail_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float s = b ? bf16_bits_to_f32(b[c]) : 0.f;
        for (int j = 0; j < K; j++) {
            const int back = K - 1 - j;
            if (p - back < 0) continue;  // before the sequence started
            float v;
            if (t - back >= 0) v = u[(size_t)(m - back) * ldu + c];
            else v = tl[(size_t)(K - 1 + (t - back)) * C + c];  // t - back in [-(K-1), -1]
            s = fmaf(bf16_bits_to_f32(w[(size_t)c * K + j]), v, s);
        }
        out[(size_t)m * C + c] = act ? s * sigmoid_f(s) : s;
    }
}
// the new tail of each sequence: its last K-1 inputs (a thread owns a channel and walks oldest -> newest, so the in-place shift is safe)
__global__ void kf_conv_tail_kernel(float* __restrict__ tail, size_t tail_stride, const float* __restrict__ u, int ldu, const int32_t* __restrict__ pos,
                                    const int32_t* __restrict__ slot, int T, int C, int K) {
    const int seq = blockIdx.x, m0 = seq * T;
    float* tl = tail + (size_t)slot[m0] * tail_stride;
    const int p0 = pos[m0];
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        for (int i = 0; i < K - 1; i++) {
            const int t = T - (K - 1) + i;  // panel-relative index of the input that lands in tail[i]
            float v;
            if (t >= 0) v = u[(size_t)(m0 + t) * ldu + c];
            else v = (p0 + t >= 0) ? tl[(size_t)(K - 1 + t) * C + c] : 0.f;
            tl[(size_t)i * C + c] = v;
        }
    }
}

// One token per sequence (decoding): the convolution and the advance of the tail in ONE launch.  A thread owns a channel of a sequence: it
// reads the channel's stored inputs, forms the output with the same sum as kf_conv_silu_kernel, then shifts the tail by one.
__global__ void kf_conv_step_kernel(float* __restrict__ out, const float* __restrict__ u, int ldu, const uint16_t* __restrict__ w, const uint16_t* __restrict__ b,
                                    float* __restrict__ tail, size_t tail_stride, const int32_t* __restrict__ pos, const int32_t* __restrict__ slot, int C, int K,
                                    int act) {
    const int m = blockIdx.x, p = pos[m];
    float* tl = tail + (size_t)slot[m] * tail_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        const float cur = u[(size_t)m * ldu + c];
        float s = b ? bf16_bits_to_f32(b[c]) : 0.f;
        for (int j = 0; j < K; j++) {
            const int back = K - 1 - j;
            if (p - back < 0) continue;  // before the sequence started
            const float v = back == 0 ? cur : tl[(size_t)(K - 1 - back) * C + c];
            s = fmaf(bf16_bits_to_f32(w[(size_t)c * K + j]), v, s);
        }
        out[(size_t)m * C + c] = act ? s * sigmoid_f(s) : s;
        for (int i = 0; i + 1 < K - 1; i++) tl[(size_t)i * C + c] = (p - (K - 2 - i) >= 0) ? tl[(size_t)(i + 1) * C + c] : 0.f;
        if (K > 1) tl[(size_t)(K - 2) * C + c] = cur;
    }
}

// ------------------------------------------------------------------------------------------------------------ selective scan
// grid (heads, sequences, p-chunks).  Thread (p, r) keeps NPT consecutive state rows n of column p in registers; the R threads of a
// column are adjacent lanes and reduce y with shuffles.  Tokens are staged through shared memory TB at a time.
constexpr int NPT = 16;
__global__ void __launch_bounds__(1024) kf_ssm_scan_kernel(float* __restrict__ y, int ldy, const float* __restrict__ xbc, int C, const float* __restrict__ u,
                                                           int ldu, int z_unused, int dt_off, const uint16_t* __restrict__ dt_bias,
                                                           const uint16_t* __restrict__ A_log, const uint16_t* __restrict__ Dw, float* __restrict__ state,
                                                           size_t state_stride, const int32_t* __restrict__ pos, const int32_t* __restrict__ slot, int T,
                                                           int H, int P, int N, int G, int R, int PB, int TB) {
    extern __shared__ float sm[];
    float* sB  = sm;                 // [TB][N]
    float* sC  = sB + TB * N;        // [TB][N]
    float* sX  = sC + TB * N;        // [TB][PB]
    float* sDt = sX + TB * PB;       // [TB]
    float* sA  = sDt + TB;           // [TB]
    const int h = blockIdx.x, seq = blockIdx.y, p0 = blockIdx.z * PB;
    const int g = h / (H / G), inner = H * P;
    const int tid = threadIdx.x, pl = tid / R, r = tid - pl * R, p = p0 + pl;
    const bool live = pl < PB && p < P;
    const int m0 = seq * T;
    float* st = state + (size_t)slot[m0] * state_stride + ((size_t)h * P + (live ? p : 0)) * N;
    float S[NPT];
    const bool fresh = pos[m0] == 0;
    // state row held in S[i]: the rows are dealt to the R lanes of a column four at a time, n = ((i / 4) * R + r) * 4 + i % 4, so that the
    // lanes' 16-byte loads of B and C are consecutive in shared memory
#define KF_SSM_ROW(i) ((((i) >> 2) * R + r) * 4 + ((i) & 3))
#pragma unroll
    for (int i = 0; i < NPT; i++) {
        const int n = KF_SSM_ROW(i);
        S[i] = (live && n < N && !fresh) ? st[n] : 0.f;
    }
    const bool vec4 = (N & 3) == 0;
    const float Aneg = -expf(bf16_bits_to_f32(A_log[h])), Dh = bf16_bits_to_f32(Dw[h]), dtb = bf16_bits_to_f32(dt_bias[h]);
    for (int t0 = 0; t0 < T; t0 += TB) {
        const int nt = min(TB, T - t0);
        __syncthreads();
        for (int i = tid; i < nt * N; i += blockDim.x) {
            const int tt = i / N, n = i - tt * N;
            const float* row = xbc + (size_t)(m0 + t0 + tt) * C;
            sB[tt * N + n] = row[inner + g * N + n];
            sC[tt * N + n] = row[inner + G * N + g * N + n];
        }
        for (int i = tid; i < nt * PB; i += blockDim.x) {
            const int tt = i / PB, q = i - tt * PB;
            sX[tt * PB + q] = (p0 + q < P) ? xbc[(size_t)(m0 + t0 + tt) * C + h * P + p0 + q] : 0.f;
        }
        for (int i = tid; i < nt; i += blockDim.x) {
            const float dtv = softplus_f(u[(size_t)(m0 + t0 + i) * ldu + dt_off + h] + dtb);
            sDt[i] = dtv, sA[i] = expf(Aneg * dtv);
        }
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {
            const float dtv = sDt[tt], av = sA[tt], xv = sX[tt * PB + (pl < PB ? pl : 0)];
            const float dx = dtv * xv;
            float acc = 0.f;
            if (vec4) {  // this thread's 16 rows as four 16-byte loads each of B and C
                const float4* b4 = reinterpret_cast<const float4*>(sB + tt * N);
                const float4* c4 = reinterpret_cast<const float4*>(sC + tt * N);
#pragma unroll
                for (int i = 0; i < NPT / 4; i++) {
                    const int q = i * R + r;
                    if (q * 4 >= N) continue;
                    const float4 bv = b4[q], cv = c4[q];
                    S[4 * i + 0] = fmaf(av, S[4 * i + 0], dx * bv.x), acc = fmaf(S[4 * i + 0], cv.x, acc);
                    S[4 * i + 1] = fmaf(av, S[4 * i + 1], dx * bv.y), acc = fmaf(S[4 * i + 1], cv.y, acc);
                    S[4 * i + 2] = fmaf(av, S[4 * i + 2], dx * bv.z), acc = fmaf(S[4 * i + 2], cv.z, acc);
                    S[4 * i + 3] = fmaf(av, S[4 * i + 3], dx * bv.w), acc = fmaf(S[4 * i + 3], cv.w, acc);
                }
            } else {
#pragma unroll
                for (int i = 0; i < NPT; i++) {
                    const int n = KF_SSM_ROW(i);
                    if (n < N) {
                        S[i] = fmaf(av, S[i], dx * sB[tt * N + n]);
                        acc  = fmaf(S[i], sC[tt * N + n], acc);
                    }
                }
            }
            for (int o = R >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (live && r == 0) y[(size_t)(m0 + t0 + tt) * ldy + h * P + p] = fmaf(Dh, xv, acc);
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NPT; i++) {
            const int n = KF_SSM_ROW(i);
            if (n < N) st[n] = S[i];
        }
    }
#undef KF_SSM_ROW
}

// ------------------------------------------------------------------------------------------------------------ latent attention
// cache row = [c (rank) | rotated shared key (rot_dim)].  One block per token: RMS norm of the first `rank` entries of the down
// projection times w; rotate-half on the first `dims` entries of the rest (pair i <-> i + dims/2, angle pos * inv_freq[i] formed in double,
// sine / cosine evaluated in double).
template <typename TC>
__global__ void __launch_bounds__(256) kf_latent_append_kernel(TC* __restrict__ cache, size_t slot_stride, const float* __restrict__ ckr, int ldc,
                                                               const uint16_t* __restrict__ w, const double* __restrict__ inv_freq,
                                                               const int32_t* __restrict__ pos, const int32_t* __restrict__ slot, int rank, int rot_dim,
                                                               int dims, float eps, int pairs, float amp) {
    __shared__ float red[32];
    const int m = blockIdx.x, W = rank + rot_dim;
    const float* in = ckr + (size_t)m * ldc;
    TC* row = cache + (size_t)slot[m] * slot_stride + (size_t)pos[m] * W;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) ss = fmaf(in[i], in[i], ss);
    ss = block_sum(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)rank + eps);
    auto put = [&](int i, float v) {
        if (sizeof(TC) == 2) ((uint16_t*)row)[i] = f32_to_bf16_bits(v);
        else ((float*)row)[i] = v;
    };
    for (int i = threadIdx.x; i < rank; i += blockDim.x) put(i, in[i] * s * bf16_bits_to_f32(w[i]));
    const int half = dims / 2;
    const float fp = (float)pos[m];
    for (int i = threadIdx.x; i < rot_dim; i += blockDim.x) {
        float v = in[rank + i];
        if (i < dims) {
            // pairs 0: entry j turns with entry j + dims/2; 1: entry 2j with entry 2j + 1.  first: this entry is the first of its pair
            const bool first = pairs ? !(i & 1) : i < half;
            const int j = pairs ? i >> 1 : (first ? i : i - half);
            double sn, cs;
            sincos((double)fp * inv_freq[j], &sn, &cs);  // angle, sine and cosine in double
            const float a = in[rank + (pairs ? 2 * j : j)], b = in[rank + (pairs ? 2 * j + 1 : j + half)];
            v = (first ? a * (float)cs - b * (float)sn : b * (float)cs + a * (float)sn) * amp;
        }
        put(rank + i, v);
    }
}
// q' [M][H][rank + rot_dim] = scale * [ W_uk[h]^T q_plain[h]  |  rotate(q_rot[h]) ]; one block per (QT tokens, head): a weight element
// read once serves QT tokens
constexpr int QT = 8;
__global__ void __launch_bounds__(128) kf_latent_query_kernel(float* __restrict__ qa, const float* __restrict__ q, int ldq, const uint16_t* __restrict__ Wuk,
                                                              const double* __restrict__ inv_freq, const int32_t* __restrict__ pos, int M, int H, int dn,
                                                              int rot_dim, int dims, int rank, float scale, int pairs, float amp) {
    extern __shared__ float sq[];  // [QT][dn + rot_dim]
    const int m0 = blockIdx.x * QT, h = blockIdx.y, D = dn + rot_dim, W = rank + rot_dim;
    const int nt = min(QT, M - m0);
    for (int i = threadIdx.x; i < nt * D; i += blockDim.x) {
        const int t = i / D, d = i - t * D;
        sq[t * D + d] = q[(size_t)(m0 + t) * ldq + (size_t)h * D + d];
    }
    __syncthreads();
    for (int c = blockIdx.z * blockDim.x + threadIdx.x; c < rank; c += gridDim.z * blockDim.x) {
        float s[QT];
#pragma unroll
        for (int t = 0; t < QT; t++) s[t] = 0.f;
#pragma unroll 8
        for (int d = 0; d < dn; d++) {
            const float w = bf16_bits_to_f32(Wuk[((size_t)h * dn + d) * rank + c]);
#pragma unroll
            for (int t = 0; t < QT; t++) s[t] = fmaf(sq[(t < nt ? t : 0) * D + d], w, s[t]);
        }
#pragma unroll
        for (int t = 0; t < QT; t++)
            if (t < nt) qa[((size_t)(m0 + t) * H + h) * W + c] = s[t] * scale;
    }
    const int half = dims / 2;
    for (int i = blockIdx.z * blockDim.x + threadIdx.x; i < nt * rot_dim; i += gridDim.z * blockDim.x) {
        const int t = i / rot_dim, e = i - t * rot_dim;
        const float* sr = sq + t * D + dn;
        float v = sr[e];
        if (e < dims) {
            const bool first = pairs ? !(e & 1) : e < half;
            const int j = pairs ? e >> 1 : (first ? e : e - half);
            double sn, cs;
            sincos((double)pos[m0 + t] * inv_freq[j], &sn, &cs);
            const float a = sr[pairs ? 2 * j : j], b = sr[pairs ? 2 * j + 1 : j + half];
            v = (first ? a * (float)cs - b * (float)sn : b * (float)cs + a * (float)sn) * amp;
        }
        qa[((size_t)(m0 + t) * H + h) * W + rank + e] = v * scale;
    }
}
// One block (4 warps) per (token, head): warp w takes keys w, w + 4, ...; a lane owns elements lane, lane + 32, ... of a row.  Online
// softmax per warp, merged in shared memory; the sink joins the denominator once: den += exp(sink - max).  out = sum_j p_j c_j / den.
constexpr int LMAX = 20;  // elements per lane: rank + rot_dim <= 640
template <typename TC>
__global__ void __launch_bounds__(128) kf_latent_attn_kernel(float* __restrict__ out, const float* __restrict__ qa, const TC* __restrict__ cache,
                                                             size_t slot_stride, const uint16_t* __restrict__ sink, const int32_t* __restrict__ pos,
                                                             const int32_t* __restrict__ slot, int H, int rank, int rot_dim) {
    extern __shared__ float sm[];  // [4][rank] accumulators + [4] max + [4] sum
    const int m = blockIdx.x, h = blockIdx.y, W = rank + rot_dim;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* q = qa + ((size_t)m * H + h) * W;
    float qr[LMAX], acc[LMAX];
#pragma unroll
    for (int i = 0; i < LMAX; i++) {
        const int e = lane + 32 * i;
        qr[i] = e < W ? q[e] : 0.f, acc[i] = 0.f;
    }
    const TC* base = cache + (size_t)slot[m] * slot_stride;
    const int last = pos[m];
    float mx = -INFINITY, sum = 0.f;
    for (int j = warp; j <= last; j += 4) {
        const TC* row = base + (size_t)j * W;
        float kv[LMAX], s = 0.f;
#pragma unroll
        for (int i = 0; i < LMAX; i++) {
            const int e = lane + 32 * i;
            float v = 0.f;
            if (e < W) v = sizeof(TC) == 2 ? bf16_bits_to_f32(((const uint16_t*)row)[e]) : ((const float*)row)[e];
            kv[i] = v;
            s     = fmaf(qr[i], v, s);
        }
        s = warp_sum(s);
        const float nm = fmaxf(mx, s), corr = expf(mx - nm), pj = expf(s - nm);
        sum = sum * corr + pj;
#pragma unroll
        for (int i = 0; i < LMAX; i++) acc[i] = acc[i] * corr + pj * kv[i];
        mx = nm;
    }
    float* sacc = sm;
    float* smx  = sm + 4 * rank;
    float* ssum = smx + 4;
#pragma unroll
    for (int i = 0; i < LMAX; i++) {
        const int e = lane + 32 * i;
        if (e < rank) sacc[warp * rank + e] = acc[i];
    }
    if (lane == 0) smx[warp] = mx, ssum[warp] = sum;
    __syncthreads();
    const float sk = sink ? bf16_bits_to_f32(sink[h]) : -INFINITY;  // no sink: no extra term in the denominator
    float M4 = sk;
    for (int w = 0; w < 4; w++) M4 = fmaxf(M4, smx[w]);
    float den = sink ? expf(sk - M4) : 0.f, f[4];
    for (int w = 0; w < 4; w++) f[w] = smx[w] == -INFINITY ? 0.f : expf(smx[w] - M4), den += ssum[w] * f[w];
    float* o = out + ((size_t)m * H + h) * rank;
    for (int e = threadIdx.x; e < rank; e += blockDim.x) {
        float v = 0.f;
        for (int w = 0; w < 4; w++) v += sacc[w * rank + e] * f[w];
        o[e] = v / den;
    }
}
// ---- the same attention on tensor cores (bf16 cache rows; rank and rank + rot_dim multiples of 8) --------------------------------------
// One CTA (4 warps) per (token, group of 16 heads, key split).  The 16 heads of a token are the 16 rows of an m16n8k16 tile and share
// every cached row, so a row is fetched once per 16 heads.  Per block of 16 keys, staged in shared memory with cp.async (two buffers):
//   scores  S[16 x 16] = Q'[16 x W] C^T : the W/16 k-steps are dealt round-robin to the 4 warps, partial tiles summed through shared memory;
//   softmax online in fp32, every warp alike (rows gr and gr + 8 of a lane's fragment, quad shuffles);
//   values  O[16 x rank] += P C[:, :rank] : warp w owns a quarter of the rank; the fp32 weights P enter the bf16 tensor-core product as
//           hi + lo (two mma per tile), which keeps 16 bits of each weight.
// Splits write (O, max, sum) to a workspace; kf_latent_merge_kernel combines them and adds the sink term to the denominator.
constexpr int KSW = 10;   // k-steps of 16 per warp: W <= 640
constexpr int NTW = 16;   // value n-tiles of 8 per warp: rank <= 512
__device__ __forceinline__ void ldsm_x4(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory"); }

__global__ void __launch_bounds__(128) kf_latent_attn_mma_kernel(float* __restrict__ part_o, float* __restrict__ part_ml, const float* __restrict__ qa,
                                                                 const uint16_t* __restrict__ cache, size_t slot_stride, const int32_t* __restrict__ pos,
                                                                 const int32_t* __restrict__ slot, int H, int HG, int rank, int rot_dim, int S) {
    extern __shared__ __align__(16) unsigned char smraw[];
    const int W = rank + rot_dim, W16 = (W + 15) & ~15, LD = W16 + 8;  // row pitch in bf16 elements (16-byte multiple, 4-bank skew)
    uint16_t* sQ  = (uint16_t*)smraw;                 // [16][LD]
    uint16_t* sK0 = sQ + 16 * LD;                     // two key tiles [16][LD]
    float* sS     = (float*)(sK0 + 2 * 16 * LD);      // [4 warps][2 n-tiles][32 lanes][4]
    const int m = blockIdx.x, hg = blockIdx.y, sp = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gr = lane >> 2, tg = lane & 3;
    const int last = pos[m];
    const int nblk = (last + 16) / 16;                 // key blocks covering 0 .. last
    const int per  = (nblk + S - 1) / S;
    const int b_lo = sp * per, b_hi = min(nblk, b_lo + per);
    const uint16_t* base = cache + (size_t)slot[m] * slot_stride;
    // queries of this head group as bf16, zero rows beyond H and zero columns beyond W; zero the pad columns of both key tiles
    for (int i = tid; i < 16 * W16; i += 128) {
        const int r = i / W16, c = i - r * W16, h = hg * 16 + r;
        sQ[r * LD + c] = (h < H && c < W) ? f32_to_bf16_bits(qa[((size_t)m * H + h) * W + c]) : (uint16_t)0;
    }
    for (int i = tid; i < 2 * 16 * (W16 - W); i += 128) {
        const int r = i / (W16 - W), c = W + i - r * (W16 - W);
        sK0[r * LD + c] = 0;
    }
    const int chunks = W / 8;  // 16-byte pieces per row
    auto stage = [&](int blk, int buf) {
        uint16_t* dst = sK0 + buf * 16 * LD;
        for (int i = tid; i < 16 * chunks; i += 128) {
            const int r = i / chunks, c = (i - r * chunks) * 8, j = blk * 16 + r;
            if (j <= last) cp_async16(dst + r * LD + c, base + (size_t)j * W + c);
            else *reinterpret_cast<uint4*>(dst + r * LD + c) = make_uint4(0, 0, 0, 0);  // rows past the query: never written to the cache yet
        }
    };
    if (b_lo < b_hi) stage(b_lo, 0);
    __syncthreads();
    // this warp's query fragments: k-steps warp, warp + 4, ...
    const int nks = W16 / 16;
    uint32_t af[KSW][4];
#pragma unroll
    for (int i = 0; i < KSW; i++) {
        const int ks = warp + 4 * i;
        if (ks < nks) ldsm_x4(af[i], sQ + (lane & 15) * LD + ks * 16 + (lane >> 4) * 8);
        else af[i][0] = af[i][1] = af[i][2] = af[i][3] = 0;
    }
    const int ntw = (rank / 8 + 3) / 4;  // n-tiles per warp
    const int nt0 = warp * ntw;          // first n-tile of this warp
    float acc[NTW][4];
#pragma unroll
    for (int i = 0; i < NTW; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float mx0 = -INFINITY, mx1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    for (int blk = b_lo; blk < b_hi; blk++) {
        const int buf = (blk - b_lo) & 1;
        cp_async_wait_all();
        __syncthreads();  // tile `blk` is in place; every warp is done with the other buffer and with sS
        if (blk + 1 < b_hi) stage(blk + 1, buf ^ 1);
        const uint16_t* sK = sK0 + buf * 16 * LD;
        float sp4[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int i = 0; i < KSW; i++) {
            const int ks = warp + 4 * i;
            if (ks < nks) {
                uint32_t b[4];  // (keys 0-7, k lo) (keys 0-7, k hi) (keys 8-15, k lo) (keys 8-15, k hi)
                ldsm_x4(b, sK + ((lane & 7) + (lane >> 4) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
                mma16816(sp4[0], af[i], b[0], b[1]);
                mma16816(sp4[1], af[i], b[2], b[3]);
            }
        }
        float4* sS4 = reinterpret_cast<float4*>(sS);
        sS4[(warp * 2 + 0) * 32 + lane] = make_float4(sp4[0][0], sp4[0][1], sp4[0][2], sp4[0][3]);
        sS4[(warp * 2 + 1) * 32 + lane] = make_float4(sp4[1][0], sp4[1][1], sp4[1][2], sp4[1][3]);
        __syncthreads();
        float sc[2][4];
#pragma unroll
        for (int t = 0; t < 2; t++) {
            sc[t][0] = sc[t][1] = sc[t][2] = sc[t][3] = 0.f;
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const float4 v = sS4[(w * 2 + t) * 32 + lane];
                sc[t][0] += v.x, sc[t][1] += v.y, sc[t][2] += v.z, sc[t][3] += v.w;
            }
        }
        // causal mask: key index of fragment entry (t, e) is blk*16 + t*8 + tg*2 + (e & 1); rows: e < 2 -> gr, else gr + 8
        const int j0 = blk * 16 + tg * 2;
#pragma unroll
        for (int t = 0; t < 2; t++)
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (j0 + t * 8 + (e & 1) > last) sc[t][e] = -INFINITY;
        float r0 = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
        float r1 = fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3]));
        r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, 1)), r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, 2));
        r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, 1)), r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, 2));
        const float n0 = fmaxf(mx0, r0), n1 = fmaxf(mx1, r1);  // finite: key blk*16 <= last is never masked
        const float c0 = expf(mx0 - n0), c1 = expf(mx1 - n1);
        float p[2][4];
#pragma unroll
        for (int t = 0; t < 2; t++) {
            p[t][0] = expf(sc[t][0] - n0), p[t][1] = expf(sc[t][1] - n0);
            p[t][2] = expf(sc[t][2] - n1), p[t][3] = expf(sc[t][3] - n1);
        }
        float s0 = p[0][0] + p[0][1] + p[1][0] + p[1][1], s1 = p[0][2] + p[0][3] + p[1][2] + p[1][3];
        s0 += __shfl_xor_sync(0xffffffffu, s0, 1), s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 1), s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
        l0 = l0 * c0 + s0, l1 = l1 * c1 + s1, mx0 = n0, mx1 = n1;
        // P as A fragments, hi and lo parts: a0 (gr, k 0-7) a1 (gr+8, k 0-7) a2 (gr, k 8-15) a3 (gr+8, k 8-15)
        uint32_t ph[4], pl[4];
        auto split = [&](float a, float b, uint32_t& hi, uint32_t& lo) {
            const __nv_bfloat16 ah = __float2bfloat16_rn(a), bh = __float2bfloat16_rn(b);
            hi = pack_bf16x2(__bfloat162float(ah), __bfloat162float(bh));
            lo = pack_bf16x2(a - __bfloat162float(ah), b - __bfloat162float(bh));
        };
        split(p[0][0], p[0][1], ph[0], pl[0]);
        split(p[0][2], p[0][3], ph[1], pl[1]);
        split(p[1][0], p[1][1], ph[2], pl[2]);
        split(p[1][2], p[1][3], ph[3], pl[3]);
#pragma unroll
        for (int i = 0; i < NTW; i += 2) {
            if (i < ntw) {
#pragma unroll
                for (int e = 0; e < 4; e++) acc[i][e] *= (e < 2 ? c0 : c1), acc[i + 1][e] *= (e < 2 ? c0 : c1);
                const int nt = nt0 + i;  // two n-tiles per ldmatrix: (keys 0-7, n) (keys 8-15, n) (keys 0-7, n + 8) (keys 8-15, n + 8)
                if (nt * 8 < rank) {
                    uint32_t b[4];
                    int col = nt * 8 + (lane >> 4) * 8;
                    if (col >= W16) col = nt * 8;  // the second tile lies past the row: fetch the first again, its result is dropped
                    ldsm_x4_t(b, sK + (lane & 15) * LD + col);
                    mma16816(acc[i], ph, b[0], b[1]);
                    mma16816(acc[i], pl, b[0], b[1]);
                    if (i + 1 < ntw && (nt + 1) * 8 < rank) {
                        mma16816(acc[i + 1], ph, b[2], b[3]);
                        mma16816(acc[i + 1], pl, b[2], b[3]);
                    }
                }
            }
        }
    }
    // partial results of this split: rows gr and gr + 8 of the head group
    const int h0 = hg * 16 + gr, h1 = h0 + 8;
    float* po0 = part_o + (((size_t)m * HG * 16 + h0) * S + sp) * rank;
    float* po1 = part_o + (((size_t)m * HG * 16 + h1) * S + sp) * rank;
#pragma unroll
    for (int i = 0; i < NTW; i++) {
        const int c = (nt0 + i) * 8 + tg * 2;
        if (i < ntw && c < rank) {
            *reinterpret_cast<float2*>(po0 + c) = make_float2(acc[i][0], acc[i][1]);
            *reinterpret_cast<float2*>(po1 + c) = make_float2(acc[i][2], acc[i][3]);
        }
    }
    if (warp == 0 && tg == 0) {
        float* ml0 = part_ml + (((size_t)m * HG * 16 + h0) * S + sp) * 2;
        float* ml1 = part_ml + (((size_t)m * HG * 16 + h1) * S + sp) * 2;
        ml0[0] = mx0, ml0[1] = l0, ml1[0] = mx1, ml1[1] = l1;
    }
}
// out[m][h] = sum_s O_s exp(m_s - M) / (exp(sink_h - M) + sum_s l_s exp(m_s - M)),  M = max(sink_h, m_s)
__global__ void __launch_bounds__(128) kf_latent_merge_kernel(float* __restrict__ out, const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                              const uint16_t* __restrict__ sink, int H, int HG, int rank, int S) {
    const int m = blockIdx.x, h = blockIdx.y;
    const float* ml = part_ml + ((size_t)m * HG * 16 + h) * S * 2;
    const float* po = part_o + ((size_t)m * HG * 16 + h) * S * rank;
    __shared__ float fac[64];  // exp(m_s - M) per split (S <= 64), 0 for an empty split
    const float sk = sink ? bf16_bits_to_f32(sink[h]) : -INFINITY;
    float M = sk;
    for (int s = 0; s < S; s++) M = fmaxf(M, ml[2 * s]);
    if ((int)threadIdx.x < S) fac[threadIdx.x] = ml[2 * threadIdx.x] == -INFINITY ? 0.f : expf(ml[2 * threadIdx.x] - M);
    __syncthreads();
    float den = sink ? expf(sk - M) : 0.f;
    for (int s = 0; s < S; s++) den += ml[2 * s + 1] * fac[s];
    float* o = out + ((size_t)m * H + h) * rank;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        float v = 0.f;
#pragma unroll 4
        for (int s = 0; s < S; s++) v = fmaf(po[(size_t)s * rank + c], fac[s], v);
        o[c] = v / den;
    }
}
// head outputs: o[m][h*dv + e] = (W_uv[h*dv + e] . lat[m][h]) * sigmoid(gate[m][h*dv + e]) in the activation type; warp per output
template <typename TO>
__global__ void __launch_bounds__(256) kf_latent_expand_kernel(TO* __restrict__ o, const float* __restrict__ lat, const uint16_t* __restrict__ Wuv,
                                                               const float* __restrict__ gate, int ldg, int H, int dv, int rank) {
    const int m = blockIdx.x, h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* l = lat + ((size_t)m * H + h) * rank;
    for (int e = warp; e < dv; e += 8) {
        const uint16_t* w = Wuv + ((size_t)h * dv + e) * rank;
        float s = 0.f;
#pragma unroll 8
        for (int c = lane; c < rank; c += 32) s = fmaf(l[c], bf16_bits_to_f32(w[c]), s);
        s = warp_sum(s);
        if (lane == 0) {
            const size_t idx = (size_t)m * H * dv + (size_t)h * dv + e;
            const float v    = gate ? s * sigmoid_f(gate[(size_t)m * ldg + h * dv + e]) : s;
            if (sizeof(TO) == 2) ((uint16_t*)o)[idx] = f32_to_bf16_bits(v);
            else ((float*)o)[idx] = v;
        }
    }
}
}  // namespace

// xbc_out [M][C] = silu(conv(u[:, c0 : c0 + C])) per channel; then the slot's tail is advanced.  u: float [M][ldu]; w bf16 [C][K]; b bf16 [C].
// act 0: no activation, 1: SiLU.  tail may be shared by several convolutions of one layer: pass each its own region of the slot's tail.
extern "C" int kf_conv1d(kf_ctx* ctx, float* xbc_out, const float* u, int ldu, int c0, const void* w_bf16, const void* b_bf16, float* tail,
                         size_t tail_stride, const int32_t* pos_dev, const int32_t* slot_dev, int nseq, int T, int C, int K, int act) {
    if (!ctx || !xbc_out || !u || !w_bf16 || !tail || !pos_dev || !slot_dev) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, nseq >= 1 && T >= 1 && C >= 1 && K >= 1 && tail_stride >= (size_t)(K - 1) * C, "shape");
    if (T == 1) {  // decoding: output and tail in one launch
        kf_conv_step_kernel<<<dim3(nseq, (C + 255) / 256), 256, 0, ctx->stream>>>(xbc_out, u + c0, ldu, (const uint16_t*)w_bf16, (const uint16_t*)b_bf16, tail,
                                                                                tail_stride, pos_dev, slot_dev, C, K, act);
        KF_LAUNCH_CHECK(ctx);
        return KF_OK;
    }
    kf_conv_silu_kernel<<<dim3(nseq * T, (C + 255) / 256), 256, 0, ctx->stream>>>(xbc_out, u + c0, ldu, (const uint16_t*)w_bf16, (const uint16_t*)b_bf16, tail, tail_stride, pos_dev,
                                                           slot_dev, T, C, K, act);
    KF_LAUNCH_CHECK(ctx);
    if (K > 1) {
        kf_conv_tail_kernel<<<dim3(nseq, (C + 255) / 256), 256, 0, ctx->stream>>>(tail, tail_stride, u + c0, ldu, pos_dev, slot_dev, T, C, K);
        KF_LAUNCH_CHECK(ctx);
    }
    return KF_OK;
}
extern "C" int kf_conv_silu(kf_ctx* ctx, float* xbc_out, const float* u, int ldu, int c0, const void* w_bf16, const void* b_bf16, float* tail,
                            size_t tail_stride, const int32_t* pos_dev, const int32_t* slot_dev, int nseq, int T, int C, int K) {
    return kf_conv1d(ctx, xbc_out, u, ldu, c0, w_bf16, b_bf16, tail, tail_stride, pos_dev, slot_dev, nseq, T, C, K, 1);
}
// y [M][ldy] (heads x P) from xbc [M][C = H*P + 2*G*N] (x | B | C after the convolution) and the step logits u[:, dt_off + h];
// state: float [slot][H][P][N] with state_stride floats per slot.
extern "C" int kf_ssm_scan(kf_ctx* ctx, float* y, int ldy, const float* xbc, const float* u, int ldu, int dt_off, const void* dt_bias_bf16,
                           const void* A_log_bf16, const void* D_bf16, float* state, size_t state_stride, const int32_t* pos_dev, const int32_t* slot_dev,
                           int nseq, int T, int H, int P, int N, int G) {
    if (!ctx || !y || !xbc || !u || !dt_bias_bf16 || !A_log_bf16 || !D_bf16 || !state || !pos_dev || !slot_dev) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, nseq >= 1 && T >= 1 && H >= 1 && P >= 1 && N >= 1 && G >= 1 && H % G == 0 && N <= 32 * NPT, "state size <= 512, groups divide heads");
    KF_REQUIRE(ctx, state_stride >= (size_t)H * P * N, "state stride");
    int R = 1;
    while (R * NPT < N) R <<= 1;
    int PB = std::min(P, 1024 / R);
    while (PB > 16 && (long long)H * nseq * ((P + PB - 1) / PB) < ctx->sm_count) PB = (PB + 1) / 2;  // fewer heads than SMs: split the columns
    const int threads = ((PB * R + 31) / 32) * 32;
    // tokens staged per pass: as many as fit 40 KB (each pass exposes one global-memory round trip), at most 64
    int TB = (int)std::min<size_t>(64, (40 * 1024 / sizeof(float)) / (size_t)(2 * N + PB + 2));
    TB = std::max(4, std::min(TB, T));
    const size_t smem = (size_t)(2 * TB * N + TB * PB + 2 * TB) * sizeof(float);
    KF_REQUIRE(ctx, smem <= 48 * 1024, "state too large for the staging area");
    dim3 grid(H, nseq, (P + PB - 1) / PB);
    kf_ssm_scan_kernel<<<grid, threads, smem, ctx->stream>>>(y, ldy, xbc, H * P + 2 * G * N, u, ldu, 0, dt_off, (const uint16_t*)dt_bias_bf16,
                                                            (const uint16_t*)A_log_bf16, (const uint16_t*)D_bf16, state, state_stride, pos_dev, slot_dev, T,
                                                            H, P, N, G, R, PB, TB);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}

extern "C" int kf_latent_append(kf_ctx* ctx, void* cache, int cache_f32, size_t slot_stride, const float* ckr, int ldc, const void* norm_w_bf16,
                                const double* inv_freq_dev, const int32_t* pos_dev, const int32_t* slot_dev, int M, int rank, int rot_dim, int rot_dims,
                                float eps) {
    return kf_latent_append_ex(ctx, cache, cache_f32, slot_stride, ckr, ldc, norm_w_bf16, inv_freq_dev, pos_dev, slot_dev, M, rank, rot_dim, rot_dims, eps, 0, 1.f);
}
// the same with the pair layout of the rotation (0: entry i with i + rot_dims/2; 1: entry 2i with 2i + 1) and a factor `amp` on cosine and sine
extern "C" int kf_latent_append_ex(kf_ctx* ctx, void* cache, int cache_f32, size_t slot_stride, const float* ckr, int ldc, const void* norm_w_bf16,
                                   const double* inv_freq_dev, const int32_t* pos_dev, const int32_t* slot_dev, int M, int rank, int rot_dim, int rot_dims,
                                   float eps, int layout, float amp) {
    if (!ctx || !cache || !ckr || !norm_w_bf16 || !inv_freq_dev || !pos_dev || !slot_dev) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, M >= 1 && rank >= 1 && rot_dim >= 0 && rot_dims >= 0 && rot_dims <= rot_dim && rot_dims % 2 == 0 && (layout == 0 || layout == 1),
               "rotated dims: even, <= rot_dim");
    if (cache_f32)
        kf_latent_append_kernel<float><<<M, 256, 0, ctx->stream>>>((float*)cache, slot_stride, ckr, ldc, (const uint16_t*)norm_w_bf16, inv_freq_dev, pos_dev,
                                                                  slot_dev, rank, rot_dim, rot_dims, eps, layout, amp);
    else
        kf_latent_append_kernel<uint16_t><<<M, 256, 0, ctx->stream>>>((uint16_t*)cache, slot_stride, ckr, ldc, (const uint16_t*)norm_w_bf16, inv_freq_dev,
                                                                     pos_dev, slot_dev, rank, rot_dim, rot_dims, eps, layout, amp);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
// lat_out [M][H][rank]: attention of every (token, head) over the rows 0 .. pos[m] of its slot.  q: float [M][ldq], heads laid out as
// [dn plain | rot_dim rotated]; w_uk bf16 [H*dn][rank]; sink bf16 [H]; qa_work: float scratch [M][H][rank + rot_dim].
extern "C" int kf_latent_attention(kf_ctx* ctx, float* lat_out, float* qa_work, const float* q, int ldq, const void* w_uk_bf16, const void* sink_bf16,
                                   const void* cache, int cache_f32, size_t slot_stride, const double* inv_freq_dev, const int32_t* pos_dev,
                                   const int32_t* slot_dev, int M, int H, int dn, int rot_dim, int rot_dims, int rank, float scale, int max_pos_hint) {
    if (!sink_bf16) return KF_ERR_BAD_ARG;
    return kf_latent_attention_ex(ctx, lat_out, qa_work, q, ldq, w_uk_bf16, sink_bf16, cache, cache_f32, slot_stride, inv_freq_dev, pos_dev, slot_dev, M, H, dn,
                                  rot_dim, rot_dims, rank, scale, max_pos_hint, 0, 1.f);
}
// the same with an optional sink (NULL: a plain softmax over the keys), the pair layout of the rotation and the factor on cosine and sine
// as in kf_latent_append_ex
extern "C" int kf_latent_attention_ex(kf_ctx* ctx, float* lat_out, float* qa_work, const float* q, int ldq, const void* w_uk_bf16, const void* sink_bf16,
                                      const void* cache, int cache_f32, size_t slot_stride, const double* inv_freq_dev, const int32_t* pos_dev,
                                      const int32_t* slot_dev, int M, int H, int dn, int rot_dim, int rot_dims, int rank, float scale, int max_pos_hint,
                                      int layout, float amp) {
    if (!ctx || !lat_out || !qa_work || !q || !w_uk_bf16 || !cache || !inv_freq_dev || !pos_dev || !slot_dev) return KF_ERR_BAD_ARG;
    KF_REQUIRE(ctx, M >= 1 && H >= 1 && dn >= 1 && rank >= 1 && rank + rot_dim <= 32 * LMAX && rot_dims <= rot_dim && rot_dims % 2 == 0 &&
                        (layout == 0 || layout == 1), "rank + rot_dim <= 640");
    dim3 grid(M, H), qgrid((M + QT - 1) / QT, H, (rank + 127) / 128);
    kf_latent_query_kernel<<<qgrid, 128, (size_t)QT * (dn + rot_dim) * 4, ctx->stream>>>(qa_work, q, ldq, (const uint16_t*)w_uk_bf16, inv_freq_dev, pos_dev, M,
                                                                                       H, dn, rot_dim, rot_dims, rank, scale, layout, amp);
    KF_LAUNCH_CHECK(ctx);
    if (!cache_f32 && rank % 8 == 0 && (rank + rot_dim) % 8 == 0 && rank <= NTW * 32 && rank + rot_dim <= KSW * 64 && (slot_stride * 2) % 16 == 0 &&
        ((uintptr_t)cache & 15) == 0) {
        // tensor-core path: 16 heads per CTA; keys split over CTAs when tokens x head groups alone would leave SMs idle
        const int HG = (H + 15) / 16, W16 = (rank + rot_dim + 15) & ~15, LD = W16 + 8;
        const int nblk = (std::max(0, max_pos_hint) + 16) / 16;
        int S = std::max(1, std::min((2 * ctx->sm_count) / std::max(1, M * HG), (nblk + 3) / 4));
        S = std::min(S, 64);
        const size_t rows = (size_t)M * HG * 16 * S;
        KF_REQUIRE(ctx, kf_ensure_attn_ws(ctx, rows * (rank + 2) * sizeof(float)) == KF_OK, "attention workspace");
        float* part_o  = ctx->attn_ws;
        float* part_ml = part_o + rows * rank;
        const size_t smem = (size_t)3 * 16 * LD * 2 + 4 * 2 * 32 * 16;
        static bool attr_set = false;
        if (!attr_set) {
            KF_CUDA(ctx, cudaFuncSetAttribute(kf_latent_attn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
            attr_set = true;
        }
        KF_REQUIRE(ctx, smem <= 96 * 1024, "row too wide for the staging area");
        kf_latent_attn_mma_kernel<<<dim3(M, HG, S), 128, smem, ctx->stream>>>(part_o, part_ml, qa_work, (const uint16_t*)cache, slot_stride, pos_dev, slot_dev,
                                                                             H, HG, rank, rot_dim, S);
        KF_LAUNCH_CHECK(ctx);
        kf_latent_merge_kernel<<<grid, 128, 0, ctx->stream>>>(lat_out, part_o, part_ml, (const uint16_t*)sink_bf16, H, HG, rank, S);
        KF_LAUNCH_CHECK(ctx);
        return KF_OK;
    }
    const size_t smem = (size_t)(4 * rank + 8) * 4;
    if (cache_f32)
        kf_latent_attn_kernel<float><<<grid, 128, smem, ctx->stream>>>(lat_out, qa_work, (const float*)cache, slot_stride, (const uint16_t*)sink_bf16, pos_dev,
                                                                      slot_dev, H, rank, rot_dim);
    else
        kf_latent_attn_kernel<uint16_t><<<grid, 128, smem, ctx->stream>>>(lat_out, qa_work, (const uint16_t*)cache, slot_stride, (const uint16_t*)sink_bf16,
                                                                         pos_dev, slot_dev, H, rank, rot_dim);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
extern "C" int kf_latent_expand(kf_ctx* ctx, void* out, int out_f32, const float* lat, const void* w_uv_bf16, const float* gate_logit, int ldg, int M, int H,
                                int dv, int rank) {
    if (!ctx || !out || !lat || !w_uv_bf16) return KF_ERR_BAD_ARG;
    dim3 grid(M, H);
    if (out_f32)
        kf_latent_expand_kernel<float><<<grid, 256, 0, ctx->stream>>>((float*)out, lat, (const uint16_t*)w_uv_bf16, gate_logit, ldg, H, dv, rank);
    else
        kf_latent_expand_kernel<uint16_t><<<grid, 256, 0, ctx->stream>>>((uint16_t*)out, lat, (const uint16_t*)w_uv_bf16, gate_logit, ldg, H, dv, rank);
    KF_LAUNCH_CHECK(ctx);
    return KF_OK;
}
