// Real-gated linear recurrent unit (the recurrent block of Griffin, De et al. 2024) between two branches:
//
//   y = gelu_tanh(W_y h + b_y)                      the gate branch
//   u = conv(W_x h + b_x)                           the recurrent branch (the convolution is seq_conv.cu's)
//   per block b of the channels:  r = sigmoid(Ra_b u_b + ba_b),  i = sigmoid(Ri_b u_b + bi_b)
//   log a = -c r softplus(lam),  a = exp(log a),  S_t = a S_(t-1) + sqrt(1 - a^2) (i u),  out = S y
//
// Three kernels:
//   rglru_in      adds the two projections' biases; the gate branch gets its activation (activation type out), the
//                 recurrent branch stays linear and leaves in fp32 for the convolution
//   rglru_gates   the block-diagonal products, the two sigmoids, the decay and the input's factor: writes a and
//                 b = sqrt(1 - a^2) i u, both fp32. A CTA takes one block of channels and a tile of 16 rows; a thread
//                 an output channel, whose two weight rows it streams while the rows' inputs are broadcast from
//                 shared memory.
//   rglru_scan    S <- a S + b along each sequence, one thread a channel, S fp32 per slot; writes S y.
//
// Gates, decays, the recurrence and its state are fp32; products accumulate in fp32 in a fixed order, so a row's
// result does not depend on the step's other rows.
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// p [T, ldp]: width gate columns at y_off, width recurrent columns at x_off
template <typename T>
__global__ void rglru_in_kernel(const T* __restrict__ p, int ldp, int y_off, int x_off, VecRef by, VecRef bx,
                                T* __restrict__ y, float* __restrict__ x, int width, size_t total) {
    griddep_launch_small();
    griddep_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t row = i / width;
    const int c = (int)(i % width);
    const T* src = p + row * ldp;
    // the product's output is rounded to the activation type before the bias, as a product kernel would store it
    y[i] = from_f32<T>(gelu_tanh_f(round_to<T>(to_f32(src[y_off + c]) + by.at(c))));
    x[i] = to_f32(src[x_off + c]) + bx.at(c);
}

constexpr int GT_ROWS = 16;
constexpr int GT_THREADS = 128;

template <typename TW>
__global__ void __launch_bounds__(GT_THREADS)
rglru_gates_kernel(const float* __restrict__ u, const TW* __restrict__ ra, const TW* __restrict__ ri, VecRef ba, VecRef bi,
                   VecRef lam, float decay_scale, float* __restrict__ a_out, float* __restrict__ b_out, int T, int width,
                   int bw, int staged) {
    extern __shared__ float us[];                                // [GT_ROWS][bw], then (staged) both matrices [k][bw + 1]
    griddep_wait();
    const int blk = blockIdx.y, t0 = blockIdx.x * GT_ROWS;
    const int nt = min(GT_ROWS, T - t0);
    for (int i = threadIdx.x; i < GT_ROWS * bw; i += GT_THREADS) {
        const int tt = i / bw, c = i % bw;
        us[i] = tt < nt ? u[(size_t)(t0 + tt) * width + (size_t)blk * bw + c] : 0.f;
    }
    // small blocks: both matrices pass through shared memory, read along their rows (coalesced) and laid down by k, so
    // that a thread finds its output's weight of k beside its neighbours'; the sums keep their order
    const int ldw = bw + 1;
    float* ws1 = us + GT_ROWS * bw;
    float* ws2 = ws1 + bw * ldw;
    if (staged) {
        const TW* m1 = ra + (size_t)blk * bw * bw;
        const TW* m2 = ri + (size_t)blk * bw * bw;
        for (int i = threadIdx.x; i < bw * bw; i += GT_THREADS) {
            const int o = i / bw, k = i % bw;
            ws1[k * ldw + o] = to_f32(m1[i]);
            ws2[k * ldw + o] = to_f32(m2[i]);
        }
    }
    __syncthreads();
    for (int o = threadIdx.x; o < bw; o += GT_THREADS) {
        const TW* wr = ra + ((size_t)blk * bw + o) * bw;
        const TW* wi = ri + ((size_t)blk * bw + o) * bw;
        float ar[GT_ROWS], ai[GT_ROWS];
#pragma unroll
        for (int tt = 0; tt < GT_ROWS; tt++) ar[tt] = ai[tt] = 0.f;
        for (int k = 0; k < bw; k++) {
            const float w1 = staged ? ws1[k * ldw + o] : to_f32(wr[k]), w2 = staged ? ws2[k * ldw + o] : to_f32(wi[k]);
#pragma unroll
            for (int tt = 0; tt < GT_ROWS; tt++) {
                const float uv = us[tt * bw + k];
                ar[tt] = fmaf(w1, uv, ar[tt]);
                ai[tt] = fmaf(w2, uv, ai[tt]);
            }
        }
        const int c = blk * bw + o;
        const float b1 = ba.at(c), b2 = bi.at(c), sp = softplus_f(lam.at(c));
#pragma unroll
        for (int tt = 0; tt < GT_ROWS; tt++) {
            if (tt >= nt) break;
            const float r = 1.0f / (1.0f + expf(-(ar[tt] + b1)));
            const float g = 1.0f / (1.0f + expf(-(ai[tt] + b2)));
            const float la = -decay_scale * r * sp;
            const float av = expf(la);
            // 1 - a^2 = -expm1(2 log a): exact where a is close to 1
            const float mult = sqrtf(fmaxf(-expm1f(2.0f * la), 0.f));
            const size_t at = (size_t)(t0 + tt) * width + c;
            a_out[at] = av;
            b_out[at] = mult * g * us[tt * bw + o];
        }
    }
}

template <typename T>
__global__ void rglru_scan_kernel(const float* __restrict__ a, const float* __restrict__ bx, const T* __restrict__ y,
                                  float* __restrict__ state, int n_slots, T* __restrict__ out,
                                  const int* __restrict__ cu_q, const int* __restrict__ slots, int width) {
    griddep_wait();
    const int b = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int slot = slots[b];
    const int q0 = cu_q[b], q1 = cu_q[b + 1];
    if (c >= width || slot < 0 || slot >= n_slots || q1 <= q0) return;
    float S = state[(size_t)slot * width + c];
#pragma unroll 4
    for (int t = q0; t < q1; t++) {
        const size_t at = (size_t)t * width + c;
        S = fmaf(a[at], S, bx[at]);
        out[at] = from_f32<T>(S * to_f32(y[at]));
    }
    state[(size_t)slot * width + c] = S;
}

// The same along long sequences: a CTA takes 32 channels of a sequence and cuts its rows into SCAN_PIECES pieces, a warp
// each. A piece first runs from zero and keeps the product of its decays, P, and its end value, E (the recurrence is
// linear: with S entering, the piece ends at P S + E); every warp then folds the pieces before its own in their order
// and runs its piece again from the state it found. A sequence of fewer than SCAN_LONG rows is one piece, summed in the
// order of the kernel above; which way a sequence goes depends on its own length alone.
constexpr int SCAN_PIECES = 32;
constexpr int SCAN_LONG = 128;

template <typename T>
__global__ void __launch_bounds__(32 * SCAN_PIECES)
rglru_scan_pieces_kernel(const float* __restrict__ a, const float* __restrict__ bx, const T* __restrict__ y,
                         float* __restrict__ state, int n_slots, T* __restrict__ out,
                         const int* __restrict__ cu_q, const int* __restrict__ slots, int width) {
    __shared__ float Ps[SCAN_PIECES][32], Es[SCAN_PIECES][32];
    griddep_wait();
    const int b = blockIdx.y;
    const int lane = threadIdx.x, w = threadIdx.y;
    const int c = blockIdx.x * 32 + lane;
    const int slot = slots[b];
    const int q0 = cu_q[b], q1 = cu_q[b + 1];
    if (slot < 0 || slot >= n_slots || q1 <= q0) return;
    const int n = q1 - q0;
    const int per = n < SCAN_LONG ? n : (n + SCAN_PIECES - 1) / SCAN_PIECES;
    const int t0 = min(q1, q0 + w * per), t1 = min(q1, t0 + per);
    const bool live = c < width;
    float P = 1.f, E = 0.f;
    if (live && n >= SCAN_LONG) {
#pragma unroll 4
        for (int t = t0; t < t1; t++) {
            const size_t at = (size_t)t * width + c;
            const float av = a[at];
            P *= av;
            E = fmaf(av, E, bx[at]);
        }
    }
    Ps[w][lane] = P;
    Es[w][lane] = E;
    __syncthreads();
    if (!live) return;
    float S = state[(size_t)slot * width + c];
    for (int j = 0; j < w; j++) S = fmaf(Ps[j][lane], S, Es[j][lane]);
#pragma unroll 4
    for (int t = t0; t < t1; t++) {
        const size_t at = (size_t)t * width + c;
        S = fmaf(a[at], S, bx[at]);
        out[at] = from_f32<T>(S * to_f32(y[at]));
    }
    if (w == (n - 1) / per) state[(size_t)slot * width + c] = S;   // the last piece that has rows
}

}  // namespace

MYNAH_API int mynah_rglru_in(const void* p, int ldp, int y_off, int x_off, int dtype, const void* by, const void* bx, int b_dtype,
                             void* y, float* x, int T, int width, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && width > 0, "rglru_in: bad sizes T=%d width=%d", T, width);
    const size_t total = (size_t)T * width;
    const dim3 grid((unsigned)ceil_div_ll((long long)total, 256));
    const VecRef b1{by, b_dtype}, b2{bx, b_dtype};
    if (dtype == MYNAH_F32)
        mynah_launch(rglru_in_kernel<float>, grid, dim3(256), 0, stream, (const float*)p, ldp, y_off, x_off, b1, b2, (float*)y, x, width, total);
    else if (dtype == MYNAH_BF16)
        mynah_launch(rglru_in_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)p, ldp, y_off, x_off, b1, b2, (bf16*)y, x, width, total);
    else
        return mynah_fail("rglru_in: unsupported dtype %d", dtype);
    return mynah_check_launch("rglru_in");
}

// u fp32 [T, width]; ra, ri [blocks, bw, bw] ([out, in]) in w_dtype; ba, bi, lam [width] in v_dtype; a_out, b_out fp32 [T, width].
MYNAH_API int mynah_rglru_gates(const float* u, const void* ra, const void* ri, int w_dtype, const void* ba, const void* bi,
                                const void* lam, int v_dtype, float decay_scale, float* a_out, float* b_out, int T, int width,
                                int blocks, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && width > 0 && blocks > 0 && width % blocks == 0, "rglru_gates: bad sizes T=%d width=%d blocks=%d", T, width, blocks);
    MYNAH_REQUIRE(blocks <= 65535, "rglru_gates: %d blocks exceed one launch", blocks);
    const int bw = width / blocks;
    const size_t with_weights = sizeof(float) * ((size_t)GT_ROWS * bw + 2 * (size_t)bw * (bw + 1));
    const int staged = with_weights <= 96 * 1024 ? 1 : 0;
    const size_t smem = staged ? with_weights : sizeof(float) * GT_ROWS * bw;
    MYNAH_REQUIRE(smem <= 200 * 1024, "rglru_gates: blocks of %d channels exceed shared memory", bw);
    const dim3 grid(ceil_div(T, GT_ROWS), blocks);
    const VecRef b1{ba, v_dtype}, b2{bi, v_dtype}, lm{lam, v_dtype};
#define GATES_LAUNCH(TW)                                                                                                     \
    if (smem > 48 * 1024 && cudaFuncSetAttribute(rglru_gates_kernel<TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
        return mynah_fail("rglru_gates: %zu bytes of shared memory are not to be had", smem);                              \
    mynah_launch(rglru_gates_kernel<TW>, grid, dim3(GT_THREADS), smem, stream, u, (const TW*)ra, (const TW*)ri, b1, b2, lm,    \
                 decay_scale, a_out, b_out, T, width, bw, staged)
    if (w_dtype == MYNAH_F32) { GATES_LAUNCH(float); }
    else if (w_dtype == MYNAH_BF16) { GATES_LAUNCH(bf16); }
    else return mynah_fail("rglru_gates: unsupported dtype %d", w_dtype);
#undef GATES_LAUNCH
    return mynah_check_launch("rglru_gates");
}

// a, bx fp32 [T, width]; y, out [T, width] in dtype; state fp32 [n_slots + 1, width].
MYNAH_API int mynah_rglru_scan(const float* a, const float* bx, const void* y, int dtype, float* state, int n_slots, void* out,
                               const int* cu_q, const int* slots, int B, int width, int max_q_len, cudaStream_t stream) {
    if (B == 0) return 0;
    MYNAH_REQUIRE(B > 0 && B <= 65535 && width > 0, "rglru_scan: bad sizes B=%d width=%d", B, width);
    if (max_q_len >= SCAN_LONG) {                                    // some sequence is long: the kernel that cuts those into pieces
        const dim3 pgrid(ceil_div(width, 32), B), pblock(32, SCAN_PIECES);
        if (dtype == MYNAH_F32)
            mynah_launch(rglru_scan_pieces_kernel<float>, pgrid, pblock, 0, stream, a, bx, (const float*)y, state, n_slots, (float*)out, cu_q, slots, width);
        else if (dtype == MYNAH_BF16)
            mynah_launch(rglru_scan_pieces_kernel<bf16>, pgrid, pblock, 0, stream, a, bx, (const bf16*)y, state, n_slots, (bf16*)out, cu_q, slots, width);
        else
            return mynah_fail("rglru_scan: unsupported dtype %d", dtype);
        return mynah_check_launch("rglru_scan_pieces");
    }
    const int threads = width >= 4096 ? 128 : 64;
    const dim3 grid(ceil_div(width, threads), B);
    if (dtype == MYNAH_F32)
        mynah_launch(rglru_scan_kernel<float>, grid, dim3(threads), 0, stream, a, bx, (const float*)y, state, n_slots, (float*)out, cu_q, slots, width);
    else if (dtype == MYNAH_BF16)
        mynah_launch(rglru_scan_kernel<bf16>, grid, dim3(threads), 0, stream, a, bx, (const bf16*)y, state, n_slots, (bf16*)out, cu_q, slots, width);
    else
        return mynah_fail("rglru_scan: unsupported dtype %d", dtype);
    return mynah_check_launch("rglru_scan");
}
