// Gated delta rule: a linear-attention recurrence whose per-head state S [dim x vd] is decayed, corrected
// towards the new value along the new key, and read with the query, token after token:
//
//   S <- g_t S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//
// (the read-out sees the token's own write). Three kernels:
//
//   delta_prep    q, k -> unit vectors per head, x / sqrt(sum(x^2) + 1e-6), q also times dim^(-1/2);
//                 beta = sigmoid(b_raw);  g = exp(-exp(A_log_h) * softplus(a_raw + dt_bias_h))       (fp32 out)
//   delta_rule    the recurrence. The columns of S are independent given k, q, g and beta, so a CTA takes a
//                 tile of columns of one head of one sequence; a column's dim values are spread over L adjacent
//                 lanes (about 16 values a lane, in registers) that add their parts of the two dot products
//                 by shuffles in a fixed order. Half of the CTA's threads compute; the other half stage the next
//                 sixteen tokens' keys, queries, values, decays and betas in shared memory (two buffers) and
//                 write the last sixteen outputs, so that the chain from token to token waits on no load from
//                 global memory. S is fp32 [n_slots + 1][H][dim][vd], carried per slot.
//   gated_rmsnorm out = o / rms(o over the head's vd) * w[d] * act(gate),  act = silu or sigmoid
//
// The decay is one number a head, or one a head and key channel (g then has H * dim values a row and multiplies
// the rows of S: S <- diag(g_t) S); the recurrence kernel stages such a decay like a key.
//
// All arithmetic is fp32. A sequence's rows are walked in order, so a prompt run whole, in pieces or token by
// token performs the same operations in the same order.
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

struct DeltaPrepArgs {
    int H, G, dim, ldc, ldab;
    float q_scale;
};

// one CTA a row; a warp a head of q or k
template <typename T>
__global__ void __launch_bounds__(128)
delta_prep_kernel(const T* __restrict__ qk, const T* __restrict__ a_raw, const T* __restrict__ b_raw,
                  VecRef A_log, VecRef dt_bias, float* __restrict__ qn, float* __restrict__ kn,
                  float* __restrict__ g_out, float* __restrict__ beta_out, DeltaPrepArgs a,
                  const float* __restrict__ a_ch, int lda) {
    griddep_launch_small();
    griddep_wait();
    const int row = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* src = qk + (size_t)row * a.ldc;
    for (int hh = warp; hh < 2 * a.G; hh += 4) {
        const T* v = src + (size_t)hh * a.dim;                  // q heads, then k heads
        float ss = 0.f;
        for (int d = lane; d < a.dim; d += 32) {
            const float f = to_f32(v[d]);
            ss = fmaf(f, f, ss);
        }
        const float r = (1.0f / sqrtf(warp_sum(ss) + 1e-6f)) * (hh < a.G ? a.q_scale : 1.0f);
        float* dst = hh < a.G ? qn + ((size_t)row * a.G + hh) * a.dim : kn + ((size_t)row * a.G + (hh - a.G)) * a.dim;
        for (int d = lane; d < a.dim; d += 32) dst[d] = to_f32(v[d]) * r;
    }
    for (int h = threadIdx.x; h < a.H; h += blockDim.x) {
        const float bv = to_f32(b_raw[(size_t)row * a.ldab + h]);
        if (a_ch == nullptr) {
            const float av = to_f32(a_raw[(size_t)row * a.ldab + h]);
            g_out[(size_t)row * a.H + h] = expf(-expf(A_log.at(h)) * softplus_f(av + dt_bias.at(h)));
        }
        beta_out[(size_t)row * a.H + h] = 1.0f / (1.0f + expf(-bv));
    }
    if (a_ch != nullptr) {                                      // one decay a head and key channel
        const int n = a.H * a.dim;
        for (int i = threadIdx.x; i < n; i += blockDim.x)
            g_out[(size_t)row * n + i] = expf(-expf(A_log.at(i / a.dim)) * softplus_f(a_ch[(size_t)row * lda + i] + dt_bias.at(i)));
    }
}

constexpr int DELTA_THREADS = 128;
constexpr int DELTA_TB = 16;                // tokens staged in shared memory at a time (8 where 16 do not fit)

struct DeltaArgs {
    int B, H, G, dim, vd, n_slots, ldv;
    int L;                                   // lanes a column (a power of two)
    int per;                                 // key values a lane: ceil(dim / L) rounded up to a multiple of 4
    int vec;                                 // 1: keys and queries can be fetched four values at a time
};

// Keys and queries of a staged token lie in shared memory lane chunk by lane chunk: `per` values, then zeros up to
// RMAX (what a lane reads), then 4 unused floats, so that the L lanes of a column read their chunks (as 16-byte
// vectors) from different banks.
__device__ __forceinline__ int kq_slot(int i, int per, int stride) { return (i / per) * stride + i % per; }

template <typename T, int RMAX, bool CH, int TB>
__global__ void __launch_bounds__(2 * DELTA_THREADS)
delta_rule_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const T* __restrict__ v,
                  const float* __restrict__ g, const float* __restrict__ beta, float* __restrict__ state,
                  float* __restrict__ o, const int* __restrict__ cu_q, const int* __restrict__ slots, DeltaArgs a) {
    extern __shared__ float sm[];
    griddep_wait();
    const int b = blockIdx.z, h = blockIdx.y;
    const int slot = slots[b];
    const int q0 = cu_q[b], q1 = cu_q[b + 1];
    if (slot < 0 || slot >= a.n_slots || q1 <= q0) return;
    const int L = a.L, per = a.per;
    const int JT = DELTA_THREADS / L;                            // columns of this CTA
    const bool stager = threadIdx.x >= DELTA_THREADS;            // the second half of the CTA stages, the first computes
    const int tid = threadIdx.x % DELTA_THREADS;
    const int l = tid % L, jl = tid / L;
    const int j = blockIdx.x * JT + jl;
    const bool on = j < a.vd;
    const int jj = on ? j : a.vd - 1;
    const int kvh = h / (a.H / a.G);
    constexpr int CS = RMAX + 4;                                 // floats of a lane's chunk
    const int row = CS * L;                                      // floats of a staged key (or query)
    const int nk = TB * row, nv = TB * JT;
    float* ks = sm;                                              // [2][TB][row]
    float* qs = ks + 2 * nk;                                     // [2][TB][row]
    float* vs = qs + 2 * nk;                                     // [2][TB][JT]
    float* os = vs + 2 * nv;                                     // [2][TB][JT]
    float* gs = os + 2 * nv;                                     // [2][2][TB]: decay, beta
    float* gv = gs + 4 * TB;                               // [2][TB][row]: a decay per key channel (CH)
    for (int i = threadIdx.x; i < 4 * nk; i += 2 * DELTA_THREADS) ks[i] = 0.f;      // the unused slots stay zero
    if (CH)
        for (int i = threadIdx.x; i < 2 * nk; i += 2 * DELTA_THREADS) gv[i] = 0.f;
    __syncthreads();

    auto stage = [&](int k) {                                    // block k of the sequence's rows -> buffer k & 1
        const int t0 = q0 + k * TB, nt = min(TB, q1 - t0), buf = k & 1;
        if (a.vec) {
            // four consecutive values a load, four loads of k and of q a thread issued before the first is used
            const int d4 = a.dim / 4, total = nt * d4;
            for (int base = tid; base < total; base += 4 * DELTA_THREADS) {
                float4 kk[4], qq[4], gg[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int idx = base + e * DELTA_THREADS;
                    if (idx < total) {
                        const size_t src = ((size_t)(t0 + idx / d4) * a.G + kvh) * a.dim + (size_t)(idx % d4) * 4;
                        kk[e] = *reinterpret_cast<const float4*>(kn + src);
                        qq[e] = *reinterpret_cast<const float4*>(qn + src);
                        if (CH) gg[e] = *reinterpret_cast<const float4*>(g + ((size_t)(t0 + idx / d4) * a.H + h) * a.dim + (size_t)(idx % d4) * 4);
                    }
                }
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int idx = base + e * DELTA_THREADS;
                    if (idx < total) {
                        const int at = buf * nk + (idx / d4) * row + kq_slot((idx % d4) * 4, per, CS);
                        *reinterpret_cast<float4*>(ks + at) = kk[e];
                        *reinterpret_cast<float4*>(qs + at) = qq[e];
                        if (CH) *reinterpret_cast<float4*>(gv + at) = gg[e];
                    }
                }
            }
        }
#pragma unroll 4
        for (int idx = tid; idx < (a.vec ? 0 : nt * a.dim); idx += DELTA_THREADS) {
            const int tt = idx / a.dim, i = idx % a.dim;
            const size_t src = ((size_t)(t0 + tt) * a.G + kvh) * a.dim + i;
            const int at = buf * nk + tt * row + kq_slot(i, per, CS);
            ks[at] = kn[src];
            qs[at] = qn[src];
            if (CH) gv[at] = g[((size_t)(t0 + tt) * a.H + h) * a.dim + i];
        }
        for (int idx = tid; idx < nt * JT; idx += DELTA_THREADS) {
            const int tt = idx / JT, col = blockIdx.x * JT + idx % JT;
            vs[buf * nv + idx] = col < a.vd ? to_f32(v[(size_t)(t0 + tt) * a.ldv + (size_t)h * a.vd + col]) : 0.f;
        }
        if (tid < nt) {
            gs[buf * 2 * TB + tid] = CH ? 1.0f : g[(size_t)(t0 + tid) * a.H + h];
            gs[buf * 2 * TB + TB + tid] = beta[(size_t)(t0 + tid) * a.H + h];
        }
    };
    auto write_out = [&](int k) {
        const int t0 = q0 + k * TB, nt = min(TB, q1 - t0), buf = k & 1;
        for (int idx = tid; idx < nt * JT; idx += DELTA_THREADS) {
            const int tt = idx / JT, col = blockIdx.x * JT + idx % JT;
            if (col < a.vd) o[(size_t)(t0 + tt) * a.H * a.vd + (size_t)h * a.vd + col] = os[buf * nv + idx];
        }
    };

    float S[RMAX];
    float* st = state + (((size_t)slot * a.H + h) * a.dim) * a.vd + jj;
    const int i0 = l * per;
    if (!stager) {
#pragma unroll
        for (int r = 0; r < RMAX; r++) S[r] = (r < per && i0 + r < a.dim) ? st[(size_t)(i0 + r) * a.vd] : 0.f;
    } else {
        stage(0);
    }
    __syncthreads();
    const int n_blocks = (q1 - q0 + TB - 1) / TB;
    for (int k = 0; k < n_blocks; k++) {
        if (stager) {
            if (k + 1 < n_blocks) stage(k + 1);
            if (k > 0) write_out(k - 1);
        } else {
            const int nt = min(TB, q1 - q0 - k * TB), buf = k & 1;
            for (int tt = 0; tt < nt; tt++) {
                const float gt = gs[buf * 2 * TB + tt], bt = gs[buf * 2 * TB + TB + tt];
                const float4* k4 = reinterpret_cast<const float4*>(ks + buf * nk + tt * row + l * CS);
                const float4* q4 = reinterpret_cast<const float4*>(qs + buf * nk + tt * row + l * CS);
                float kr[RMAX];
                float d4[4] = {0.f, 0.f, 0.f, 0.f};             // four partial sums: four short chains instead of a long one
#pragma unroll
                for (int r = 0; r < RMAX; r += 4) {
                    const float4 kk = k4[r >> 2];
                    kr[r] = kk.x; kr[r + 1] = kk.y; kr[r + 2] = kk.z; kr[r + 3] = kk.w;
                }
                if (CH) {
                    const float4* g4 = reinterpret_cast<const float4*>(gv + buf * nk + tt * row + l * CS);
#pragma unroll
                    for (int r = 0; r < RMAX; r += 4) {
                        const float4 gg = g4[r >> 2];
                        S[r] *= gg.x; S[r + 1] *= gg.y; S[r + 2] *= gg.z; S[r + 3] *= gg.w;
                    }
                }
#pragma unroll
                for (int r = 0; r < RMAX; r++) {
                    if (!CH) S[r] *= gt;
                    d4[r & 3] = fmaf(S[r], kr[r], d4[r & 3]);
                }
                float dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
                for (int s = L >> 1; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
                const float u = bt * (vs[buf * nv + tt * JT + jl] - dot);
                float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int r = 0; r < RMAX; r += 4) {
                    const float4 qq = q4[r >> 2];
                    S[r] = fmaf(kr[r], u, S[r]);
                    S[r + 1] = fmaf(kr[r + 1], u, S[r + 1]);
                    S[r + 2] = fmaf(kr[r + 2], u, S[r + 2]);
                    S[r + 3] = fmaf(kr[r + 3], u, S[r + 3]);
                    o4[0] = fmaf(S[r], qq.x, o4[0]);
                    o4[1] = fmaf(S[r + 1], qq.y, o4[1]);
                    o4[2] = fmaf(S[r + 2], qq.z, o4[2]);
                    o4[3] = fmaf(S[r + 3], qq.w, o4[3]);
                }
                float out = (o4[0] + o4[1]) + (o4[2] + o4[3]);
                for (int s = L >> 1; s > 0; s >>= 1) out += __shfl_xor_sync(0xffffffffu, out, s);
                if (l == 0) os[buf * nv + tt * JT + jl] = out;
            }
        }
        __syncthreads();
    }
    if (stager) {
        write_out(n_blocks - 1);
    } else if (on) {
#pragma unroll
        for (int r = 0; r < RMAX; r++)
            if (r < per && i0 + r < a.dim) st[(size_t)(i0 + r) * a.vd] = S[r];
    }
}

// a warp a (row, head)
template <typename T>
__global__ void __launch_bounds__(128)
gated_rmsnorm_kernel(const float* __restrict__ o, const T* __restrict__ gate, int ldg, VecRef w, T* __restrict__ out,
                     int n_heads_total, int H, int vd, float eps, int gate_sigmoid) {
    griddep_launch_small();
    griddep_wait();
    const int idx = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (idx >= n_heads_total) return;
    const int lane = threadIdx.x & 31;
    const int row = idx / H, h = idx % H;
    const float* src = o + ((size_t)row * H + h) * vd;
    float ss = 0.f;
    for (int d = lane; d < vd; d += 32) ss = fmaf(src[d], src[d], ss);
    const float r = 1.0f / sqrtf(warp_sum(ss) / (float)vd + eps);
    const T* gt = gate + (size_t)row * ldg + (size_t)h * vd;
    T* dst = out + ((size_t)row * H + h) * vd;
    for (int d = lane; d < vd; d += 32) {
        const float z = to_f32(gt[d]);
        const float sg = 1.0f / (1.0f + expf(-z));
        dst[d] = from_f32<T>(src[d] * r * w.at(d) * (gate_sigmoid ? sg : z * sg));
    }
}

}  // namespace

// qk [T, ldc]: G*dim query then G*dim key values a row (after their convolution and activation); a_raw, b_raw
// [T, ldab] with H values a row; all in dtype. A_log, dt_bias [H] in w_dtype. Outputs fp32: qn, kn [T, G*dim],
// g, beta [T, H].
// a_ch, when given (fp32 [T, lda], H*dim values a row), makes the decay one a head and key channel: dt_bias then has
// H*dim values, g [T, H*dim], and a_raw is not read.
MYNAH_API int mynah_delta_prep(const void* qk, int ldc, const void* a_raw, const void* b_raw, int ldab, int dtype,
                               const void* A_log, const void* dt_bias, int w_dtype,
                               float* qn, float* kn, float* g, float* beta,
                               int T, int H, int G, int dim, const float* a_ch, int lda, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && H > 0 && G > 0 && dim > 0 && H % G == 0, "delta_prep: bad sizes T=%d H=%d G=%d dim=%d", T, H, G, dim);
    const DeltaPrepArgs a{H, G, dim, ldc, ldab, 1.0f / sqrtf((float)dim)};
    const VecRef al{A_log, w_dtype}, db{dt_bias, w_dtype};
    if (dtype == MYNAH_F32)
        mynah_launch(delta_prep_kernel<float>, dim3(T), dim3(128), 0, stream, (const float*)qk, (const float*)a_raw,
                     (const float*)b_raw, al, db, qn, kn, g, beta, a, a_ch, lda);
    else if (dtype == MYNAH_BF16)
        mynah_launch(delta_prep_kernel<bf16>, dim3(T), dim3(128), 0, stream, (const bf16*)qk, (const bf16*)a_raw,
                     (const bf16*)b_raw, al, db, qn, kn, g, beta, a, a_ch, lda);
    else
        return mynah_fail("delta_prep: unsupported dtype %d", dtype);
    return mynah_check_launch("delta_prep");
}

// v [T, ldv] in dtype with head h at h*vd; state fp32 [n_slots + 1, H, dim, vd]; o fp32 [T, H*vd]. g fp32 [T, H], or
// [T, H*dim] with channel_decay.
MYNAH_API int mynah_delta_rule(const float* qn, const float* kn, const void* v, int ldv, int dtype,
                               const float* g, const float* beta, float* state, int n_slots, float* o,
                               const int* cu_q, const int* slots, int B, int H, int G, int dim, int vd,
                               int channel_decay, cudaStream_t stream) {
    if (B == 0) return 0;
    MYNAH_REQUIRE(B > 0 && H > 0 && G > 0 && dim > 0 && vd > 0 && H % G == 0, "delta_rule: bad sizes B=%d H=%d G=%d dim=%d vd=%d", B, H, G, dim, vd);
    MYNAH_REQUIRE(dim <= 1024, "delta_rule: a key of %d values exceeds 1024", dim);
    MYNAH_REQUIRE(B <= 65535 && H <= 65535, "delta_rule: B=%d or H=%d exceeds one launch", B, H);
    int L = 1;
    while (L * 16 < dim && L < 32) L <<= 1;                     // about 16 key values a lane
    const int per = (ceil_div(dim, L) + 3) / 4 * 4;
    const int vec = dim % 4 == 0 && ((reinterpret_cast<uintptr_t>(qn) | reinterpret_cast<uintptr_t>(kn) |
                                      (channel_decay ? reinterpret_cast<uintptr_t>(g) : 0)) & 15) == 0;
    const DeltaArgs a{B, H, G, dim, vd, n_slots, ldv, L, per, vec};
    const int JT = DELTA_THREADS / L;
    const dim3 grid(ceil_div(vd, JT), H, B);
    const int rmax = per <= 16 ? 16 : 32;
    auto smem_for = [&](int tb) {
        return sizeof(float) * ((size_t)(channel_decay ? 6 : 4) * tb * (rmax + 4) * L + (size_t)4 * tb * JT + 4 * tb);
    };
    // a decay per channel is staged like a third key: with the longest keys only half as many tokens fit
    const int tb = smem_for(DELTA_TB) <= 200 * 1024 ? DELTA_TB : DELTA_TB / 2;
    const size_t smem = smem_for(tb);
#define DELTA_LAUNCH(T, RMAX, CH)                                                                                      \
    if (tb == DELTA_TB) { DELTA_LAUNCH_TB(T, RMAX, CH, DELTA_TB); }                                                    \
    else { DELTA_LAUNCH_TB(T, RMAX, CH, DELTA_TB / 2); }
#define DELTA_LAUNCH_TB(T, RMAX, CH, TB)                                                                                   \
    if (smem > 48 * 1024 &&                                                                                            \
        cudaFuncSetAttribute(delta_rule_kernel<T, RMAX, CH, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
        return mynah_fail("delta_rule: %zu bytes of shared memory are not to be had", smem);                          \
    mynah_launch(delta_rule_kernel<T, RMAX, CH, TB>, grid, dim3(2 * DELTA_THREADS), smem, stream, qn, kn, (const T*)v, g, beta, state, o, \
                 cu_q, slots, a)
#define DELTA_LAUNCH_R(T, CH)                  \
    if (rmax == 16) { DELTA_LAUNCH(T, 16, CH); } \
    else { DELTA_LAUNCH(T, 32, CH); }
    if (dtype != MYNAH_F32 && dtype != MYNAH_BF16) return mynah_fail("delta_rule: unsupported dtype %d", dtype);
    if (channel_decay) {
        if (dtype == MYNAH_F32) { DELTA_LAUNCH_R(float, true); }
        else { DELTA_LAUNCH_R(bf16, true); }
    } else {
        if (dtype == MYNAH_F32) { DELTA_LAUNCH_R(float, false); }
        else { DELTA_LAUNCH_R(bf16, false); }
    }
#undef DELTA_LAUNCH_R
#undef DELTA_LAUNCH_TB
#undef DELTA_LAUNCH
    return mynah_check_launch("delta_rule");
}

// out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w * act(gate[t, h, :]), act = silu, or sigmoid with gate_sigmoid;
// o fp32 [T, H*vd], gate [T, ldg] and out [T, H*vd] in dtype, w [vd] in w_dtype.
MYNAH_API int mynah_gated_rmsnorm(const float* o, const void* gate, int ldg, int dtype, const void* w, int w_dtype,
                                  void* out, int T, int H, int vd, float eps, int gate_sigmoid, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && H > 0 && vd > 0, "gated_rmsnorm: bad sizes T=%d H=%d vd=%d", T, H, vd);
    const long long total = (long long)T * H;
    MYNAH_REQUIRE(total <= 0x7fffffffLL, "gated_rmsnorm: too many heads");
    const VecRef wv{w, w_dtype};
    const dim3 grid((unsigned)ceil_div_ll(total, 4));
    if (dtype == MYNAH_F32)
        mynah_launch(gated_rmsnorm_kernel<float>, grid, dim3(128), 0, stream, o, (const float*)gate, ldg, wv, (float*)out,
                     (int)total, H, vd, eps, gate_sigmoid);
    else if (dtype == MYNAH_BF16)
        mynah_launch(gated_rmsnorm_kernel<bf16>, grid, dim3(128), 0, stream, o, (const bf16*)gate, ldg, wv, (bf16*)out,
                     (int)total, H, vd, eps, gate_sigmoid);
    else
        return mynah_fail("gated_rmsnorm: unsupported dtype %d", dtype);
    return mynah_check_launch("gated_rmsnorm");
}
