// RMS norms that stand BEHIND a sublayer:
//
//   rmsnorm_add      x <- x (+ e) + y / sqrt(mean(y^2) + eps) * gain          (x fp32 in place, y fp32)
//                    and, when asked, the norm of the new x in the same pass:
//                    h = x / sqrt(mean(x^2) + eps2) * gain2                     (h fp32)
//                    e, optional, is another fp32 row added on the way (an input fed back in).
//   rms_pair_mean    out = weight * (a / rms(a) * ga + b / rms(b) * gb)        (a, b, out fp32)
//
// All sums are fp32 and run in an order fixed by the thread layout. A CTA takes one row; the row stays in
// registers between its two passes while it has at most 8 values a thread.
#include "common.cuh"

namespace {

constexpr int NP_THREADS = 256;
constexpr int NP_KEEP = 8;

__global__ void __launch_bounds__(NP_THREADS)
rmsnorm_add_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ extra, VecRef gain,
                   float eps, VecRef gain2, float eps2, float* __restrict__ h, int D) {
    __shared__ float red[32];
    griddep_launch_small();
    griddep_wait();
    const size_t row = (size_t)blockIdx.x * D;
    const bool keep = D <= NP_KEEP * NP_THREADS;
    float v[NP_KEEP];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NP_KEEP; i++) {
        const int d = threadIdx.x + i * NP_THREADS;
        v[i] = d < D ? y[row + d] : 0.f;
        ss = fmaf(v[i], v[i], ss);
    }
    if (!keep)
        for (int d = threadIdx.x + NP_KEEP * NP_THREADS; d < D; d += NP_THREADS) ss = fmaf(y[row + d], y[row + d], ss);
    const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)D + eps);
    float s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NP_KEEP; i++) {
        const int d = threadIdx.x + i * NP_THREADS;
        if (d < D) {
            float nx = x[row + d];
            if (extra != nullptr) nx += extra[row + d];
            nx += v[i] * r * gain.at(d);
            x[row + d] = nx;
            v[i] = nx;
            s2 = fmaf(nx, nx, s2);
        }
    }
    if (!keep)
        for (int d = threadIdx.x + NP_KEEP * NP_THREADS; d < D; d += NP_THREADS) {
            float nx = x[row + d];
            if (extra != nullptr) nx += extra[row + d];
            nx += y[row + d] * r * gain.at(d);
            x[row + d] = nx;
            s2 = fmaf(nx, nx, s2);
        }
    if (h == nullptr) return;
    const float r2 = 1.0f / sqrtf(block_sum(s2, red) / (float)D + eps2);
#pragma unroll
    for (int i = 0; i < NP_KEEP; i++) {
        const int d = threadIdx.x + i * NP_THREADS;
        if (d < D) h[row + d] = v[i] * r2 * gain2.at(d);
    }
    if (!keep)
        for (int d = threadIdx.x + NP_KEEP * NP_THREADS; d < D; d += NP_THREADS) h[row + d] = x[row + d] * r2 * gain2.at(d);
}

__global__ void __launch_bounds__(NP_THREADS)
rms_pair_mean_kernel(const float* __restrict__ a, const float* __restrict__ b, VecRef ga, VecRef gb, float eps,
                     float weight, float* __restrict__ out, int D) {
    __shared__ float red[32];
    griddep_launch_small();
    griddep_wait();
    const size_t row = (size_t)blockIdx.x * D;
    float sa = 0.f, sb = 0.f;
    for (int d = threadIdx.x; d < D; d += NP_THREADS) {
        sa = fmaf(a[row + d], a[row + d], sa);
        sb = fmaf(b[row + d], b[row + d], sb);
    }
    const float ra = 1.0f / sqrtf(block_sum(sa, red) / (float)D + eps);
    const float rb = 1.0f / sqrtf(block_sum(sb, red) / (float)D + eps);
    for (int d = threadIdx.x; d < D; d += NP_THREADS)
        out[row + d] = weight * (a[row + d] * ra * ga.at(d) + b[row + d] * rb * gb.at(d));
}

}  // namespace

// x [T, D] fp32 in place; y [T, D] fp32; extra null or [T, D] fp32; gain [D] in g_dtype. h null, or [T, D] fp32 that
// receives the norm of the new x with gain2 [D] (g2_dtype) and eps2.
MYNAH_API int mynah_rmsnorm_add(float* x, const float* y, const float* extra, const void* gain, int g_dtype, float eps,
                                const void* gain2, int g2_dtype, float eps2, float* h, int T, int D, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && D > 0, "rmsnorm_add: bad sizes T=%d D=%d", T, D);
    MYNAH_REQUIRE(h == nullptr || gain2 != nullptr, "rmsnorm_add: a second norm needs its gain");
    mynah_launch(rmsnorm_add_kernel, dim3(T), dim3(NP_THREADS), 0, stream, x, y, extra, VecRef{gain, g_dtype}, eps,
                 VecRef{gain2, g2_dtype}, eps2, h, D);
    return mynah_check_launch("rmsnorm_add");
}

// a, b, out [T, D] fp32; ga, gb [D] in g_dtype.
MYNAH_API int mynah_rms_pair_mean(const float* a, const float* b, const void* ga, const void* gb, int g_dtype, float eps,
                                  float weight, float* out, int T, int D, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && D > 0, "rms_pair_mean: bad sizes T=%d D=%d", T, D);
    mynah_launch(rms_pair_mean_kernel, dim3(T), dim3(NP_THREADS), 0, stream, a, b, VecRef{ga, g_dtype}, VecRef{gb, g_dtype},
                 eps, weight, out, D);
    return mynah_check_launch("rms_pair_mean");
}
