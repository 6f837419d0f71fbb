// Attention over ONE latent vector per position, from which every head's keys and values are linear maps
// (W_uk, W_uv), plus one rotated key part that all heads share:
//
//   score_h(t, s) = (q_u,h(t) . W_uk,h c(s) + q_r,h(t) . k_r(s)) * scale,     value_h(s) = W_uv,h c(s)
//
// Only c and k_r are cached. The maps move to the query side: with q_a,h = W_uk,h^T q_u,h the score is
// [q_a,h | q_r,h] . [c | k_r], and sum_s p(s) value_h(s) = W_uv,h (sum_s p(s) c(s)). So a position's cache row is
// [c | k_r] (one kv head), the attention kernels run as they are with that row as key AND value, and the first
// kv_rank columns of their output go through W_uv,h. This file has the three steps around them:
//
//   rope_table_freqs   cos/sin tables of given per-pair frequencies (made in double on the host: plain, or
//                      interpolated for long contexts), times a constant
//   latent_prep        per token: c = rms_norm(first kv_rank outputs of the down-projection) * w, k_r rotated,
//                      both written to the token's cache row; every head's q_r rotated into the packed query rows.
//                      Pairs are (2i, 2i+1) ("interleaved") or (i, i + dims/2). Norm and rotation in fp32.
//   head_linear        out[t, h, :] = W_h in[t, h, :] for every head: q_u -> q_a, and latent output -> values
//                      (bfloat16 on tensor cores, the 32-bit run on fused multiply-adds)
#include "layout.cuh"
#include "tile_mm.cuh"
#include "tile_mma.cuh"

namespace {

__global__ void rope_table_freqs_kernel(float* __restrict__ cos_t, float* __restrict__ sin_t, int n_pos, int half,
                                        const double* __restrict__ freqs, double mult) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)n_pos * half) return;
    const int p = (int)(idx / half), i = (int)(idx % half);
    const double a = (double)p * freqs[i];
    cos_t[idx] = (float)(cos(a) * mult);
    sin_t[idx] = (float)(sin(a) * mult);
}

struct LatentPrepArgs {
    int H, dim, rd, r, HDp;          // heads; unrotated and rotated query dims; latent size; stored row width
    int ldq, q_off, lddkv, dkv_off;  // row strides and first columns of the q and down projections
    int rot, interleaved, n_pos;     // rotated dims (<= rd), pairing, table rows
    float eps;
};

// partner and sign of element d of a vector whose first `rot` dims are rotated
__device__ __forceinline__ void rot_pair(int d, int rot, int interleaved, int& i, int& other, float& sign) {
    if (interleaved) {
        i = d >> 1;
        other = d ^ 1;
        sign = (d & 1) ? 1.f : -1.f;
    } else {
        const int half = rot >> 1;
        i = d < half ? d : d - half;
        other = d < half ? d + half : d - half;
        sign = d < half ? -1.f : 1.f;
    }
}

// one CTA a token
template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const T* __restrict__ q, const T* __restrict__ dkv, T* __restrict__ q_out, VecRef w,
                   const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                   const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, PageTable pt,
                   T* __restrict__ k_cache, LatentPrepArgs a, int* __restrict__ status) {
    __shared__ float red[32];
    griddep_launch_small();
    griddep_wait();
    const int t = blockIdx.x;
    const int b = tok_seq[t];
    if (b < 0) return;                                    // a padding row
    const int pos = tok_pos[t];
    const bool rotate = a.rot > 0 && cos_t != nullptr;
    if (rotate && (pos < 0 || pos >= a.n_pos)) {
        if (threadIdx.x == 0) atomicOr(status, MYNAH_ST_POS_RANGE);
        return;
    }
    const int half = a.rot >> 1;
    const float* cr = rotate ? cos_t + (size_t)pos * half : nullptr;
    const float* sr = rotate ? sin_t + (size_t)pos * half : nullptr;
    // the heads' rotated query parts -> columns [r, r + rd) of the packed query row; the padding beyond -> 0
    const T* qrow = q + (size_t)t * a.ldq + a.q_off;
    T* qo = q_out + (size_t)t * a.H * a.HDp;
    const int tail = a.HDp - a.r;                          // rd rotated values, then zeros
    for (int idx = threadIdx.x; idx < a.H * tail; idx += blockDim.x) {
        const int h = idx / tail, d = idx % tail;
        float v = 0.f;
        if (d < a.rd) {
            const T* src = qrow + (size_t)h * (a.dim + a.rd) + a.dim;
            v = to_f32(src[d]);
            if (rotate && d < a.rot) {
                int i, other;
                float sign;
                rot_pair(d, a.rot, a.interleaved, i, other, sign);
                v = v * cr[i] + sign * to_f32(src[other]) * sr[i];
            }
        }
        qo[(size_t)h * a.HDp + a.r + d] = from_f32<T>(v);
    }
    if (dkv == nullptr) return;                            // a run that reads another run's cache brings q only
    const int page = page_of(pt, b, pos);
    if (page < 0) {
        if (threadIdx.x == 0) atomicOr(status, MYNAH_ST_PAGE_RANGE);
        return;
    }
    T* dst = k_cache + ((size_t)page * PAGE_TOKENS + pos % PAGE_TOKENS) * a.HDp;
    const T* drow = dkv + (size_t)t * a.lddkv + a.dkv_off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.r; i += blockDim.x) {
        const float v = to_f32(drow[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)a.r + a.eps);
    for (int i = threadIdx.x; i < a.r; i += blockDim.x) dst[i] = from_f32<T>((to_f32(drow[i]) * s) * w.at(i));
    for (int d = threadIdx.x; d < tail; d += blockDim.x) {
        float v = 0.f;
        if (d < a.rd) {
            v = to_f32(drow[a.r + d]);
            if (rotate && d < a.rot) {
                int i, other;
                float sign;
                rot_pair(d, a.rot, a.interleaved, i, other, sign);
                v = v * cr[i] + sign * to_f32(drow[a.r + other]) * sr[i];
            }
        }
        dst[a.r + d] = from_f32<T>(v);
    }
}

struct HeadLinearArgs {
    int T, H, n_in, n_out;
    int ld_in, head_in, in_off;      // input: row stride, distance between heads, first column inside a head
    int ld_out, head_out, out_off;   // output likewise
    const void* gate;                // null, or rows in the activation type: head h's output is multiplied by
    int ld_gate;                     // sigmoid(gate[t * ld_gate + h]) on the accumulator, before it is rounded
};

template <typename T>
__device__ __forceinline__ float head_gate_of(const HeadLinearArgs& a, int t, int h) {
    if (a.gate == nullptr) return 1.0f;
    return 1.0f / (1.0f + expf(-to_f32(static_cast<const T*>(a.gate)[(size_t)t * a.ld_gate + h])));
}

// grid (token tiles, heads, output tiles); W is [H][n_out][n_in]
template <typename T>
__global__ void __launch_bounds__(tilemm::THREADS)
head_linear_kernel(const T* __restrict__ in, const T* __restrict__ W, T* __restrict__ out, HeadLinearArgs a) {
    constexpr int BM = 64, BN = 64;
    __shared__ tilemm::Smem<BM, BN> s;
    griddep_wait();
    const int t0 = blockIdx.x * BM, h = blockIdx.y, c0 = blockIdx.z * BN;
    for (int i = threadIdx.x; i < BM; i += blockDim.x)
        s.rows[i] = t0 + i < a.T ? in + (size_t)(t0 + i) * a.ld_in + (size_t)h * a.head_in + a.in_off : nullptr;
    float acc[BM / 16][BN / 16];
    tilemm::run<T, BM, BN>(s, W + ((size_t)h * a.n_out + c0) * a.n_in, (size_t)a.n_in, a.n_out - c0, a.n_in, acc);
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
#pragma unroll
    for (int i = 0; i < BM / 16; i++) {
        const int t = t0 + ty + 16 * i;
        if (t >= a.T) continue;
        T* o = out + (size_t)t * a.ld_out + (size_t)h * a.head_out + a.out_off;
        const float gt = head_gate_of<T>(a, t, h);
#pragma unroll
        for (int j = 0; j < BN / 16; j++) {
            const int c = c0 + tx + 16 * j;
            if (c < a.n_out) o[c] = from_f32<T>(a.gate != nullptr ? acc[i][j] * gt : acc[i][j]);
        }
    }
}

// The same on tensor cores for bfloat16 rows that can move 16 bytes at a time. grid (token tiles of 16 MT, heads,
// ceil(n_out / (8 warps * 16 columns))).
template <int MT>
__global__ void __launch_bounds__(256)
head_linear_mma_kernel(const bf16* __restrict__ in, const bf16* __restrict__ W, bf16* __restrict__ out, HeadLinearArgs a) {
    constexpr int NT = 2;
    __shared__ __align__(16) bf16 xs[16 * MT][tilemma::MMA_LDS];
    __shared__ int row_s[16 * MT];
    griddep_wait();
    const int t0 = blockIdx.x * 16 * MT, h = blockIdx.y;
    for (int i = threadIdx.x; i < 16 * MT; i += blockDim.x) row_s[i] = t0 + i < a.T ? t0 + i : -1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int c0 = (blockIdx.z * 8 + warp) * (8 * NT);
    if (c0 >= a.n_out) {                                       // the warp has no columns; it still helps to stage the rows
        const bf16* none[1][NT];
#pragma unroll
        for (int j = 0; j < NT; j++) none[0][j] = W + (size_t)h * a.n_out * a.n_in;
        float acc[1][MT][NT][4];
        tilemma::mma_tile<MT, NT, 1>(xs, row_s, in + (size_t)h * a.head_in + a.in_off, (size_t)a.ld_in, 1, none, a.n_in, acc);
        return;
    }
    const bf16* wrow[1][NT];
#pragma unroll
    for (int j = 0; j < NT; j++) wrow[0][j] = W + ((size_t)h * a.n_out + min(c0 + j * 8 + g, a.n_out - 1)) * a.n_in;
    float acc[1][MT][NT][4];
    tilemma::mma_tile<MT, NT, 1>(xs, row_s, in + (size_t)h * a.head_in + a.in_off, (size_t)a.ld_in, 1, wrow, a.n_in, acc);
#pragma unroll
    for (int m = 0; m < MT; m++)
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int r = row_s[m * 16 + g + 8 * half];
            if (r < 0) continue;
            bf16* o = out + (size_t)r * a.ld_out + (size_t)h * a.head_out + a.out_off;
            const float gt = head_gate_of<bf16>(a, r, h);
#pragma unroll
            for (int j = 0; j < NT; j++)
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    const int c = c0 + j * 8 + 2 * t + q;
                    if (c < a.n_out) o[c] = from_f32<bf16>(a.gate != nullptr ? acc[0][m][j][2 * half + q] * gt : acc[0][m][j][2 * half + q]);
                }
        }
}

}  // namespace

// 1: bfloat16 per-head products run on the plain tiled kernel too (the tests compare the two).
static int g_head_linear_plain = 0;
MYNAH_API int mynah_head_linear_plain(int on) {
    const int before = g_head_linear_plain;
    g_head_linear_plain = on;
    return before;
}

MYNAH_API int mynah_rope_table_freqs(float* cos_t, float* sin_t, int n_pos, int half, const double* freqs, double mult,
                                     cudaStream_t stream) {
    MYNAH_REQUIRE(n_pos > 0 && half > 0, "rope_table_freqs: bad sizes positions=%d pairs=%d", n_pos, half);
    const long long n = (long long)n_pos * half;
    rope_table_freqs_kernel<<<(unsigned)ceil_div_ll(n, 256), 256, 0, stream>>>(cos_t, sin_t, n_pos, half, freqs, mult);
    return mynah_check_launch("rope_table_freqs");
}

// q: rows of the query projection (H heads of dim unrotated then rd rotated values, from column q_off); dkv: rows of
// the down-projection (r latent then rd shared key values, from column dkv_off), or null with k_cache null; q_out:
// [T][H][HDp] packed query rows, of which this writes columns [r, HDp); k_cache: [n_pages][64][HDp].
MYNAH_API int mynah_latent_prep(const void* q, int ldq, int q_off, const void* dkv, int lddkv, int dkv_off, int dtype,
                                void* q_out, int T, int H, int dim, int rd, int r, int HDp,
                                const void* w, int w_dtype, float eps,
                                const float* cos_t, const float* sin_t, int rot, int interleaved, int n_pos,
                                const int* tok_seq, const int* tok_pos,
                                const int* page_indptr, const int* page_ids, const int* page_base, int n_pages,
                                void* k_cache, int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && H > 0 && dim >= 0 && rd >= 0 && r > 0 && HDp >= r + rd, "latent_prep: bad sizes");
    MYNAH_REQUIRE(rot % 2 == 0 && rot <= rd, "latent_prep: %d rotated dims do not fit the rotated part of %d", rot, rd);
    MYNAH_REQUIRE((dkv == nullptr) == (k_cache == nullptr), "latent_prep: the down-projection and the cache go together");
    const LatentPrepArgs a{H, dim, rd, r, HDp, ldq, q_off, lddkv, dkv_off, cos_t ? rot : 0, interleaved, n_pos, eps};
    const VecRef wr{w, w_dtype};
    const PageTable pt{page_indptr, page_ids, page_base, n_pages};
    if (dtype == MYNAH_F32)
        mynah_launch(latent_prep_kernel<float>, dim3(T), dim3(128), 0, stream, (const float*)q, (const float*)dkv, (float*)q_out,
                     wr, cos_t, sin_t, tok_seq, tok_pos, pt, (float*)k_cache, a, status);
    else if (dtype == MYNAH_BF16)
        mynah_launch(latent_prep_kernel<bf16>, dim3(T), dim3(128), 0, stream, (const bf16*)q, (const bf16*)dkv, (bf16*)q_out,
                     wr, cos_t, sin_t, tok_seq, tok_pos, pt, (bf16*)k_cache, a, status);
    else
        return mynah_fail("latent_prep: unsupported dtype %d", dtype);
    return mynah_check_launch("latent_prep");
}

MYNAH_API int mynah_head_linear_gated(const void* in, const void* W, void* out, int dtype, int T, int H, int n_in, int n_out,
                                      int ld_in, int head_in, int in_off, int ld_out, int head_out, int out_off,
                                      const void* gate, int ld_gate, cudaStream_t stream);

MYNAH_API int mynah_head_linear(const void* in, const void* W, void* out, int dtype, int T, int H, int n_in, int n_out,
                                int ld_in, int head_in, int in_off, int ld_out, int head_out, int out_off,
                                cudaStream_t stream) {
    return mynah_head_linear_gated(in, W, out, dtype, T, H, n_in, n_out, ld_in, head_in, in_off, ld_out, head_out, out_off,
                                   nullptr, 0, stream);
}

// The same with every head's output multiplied by sigmoid(gate[t][h]) (gate: rows in the activation type, or null).
MYNAH_API int mynah_head_linear_gated(const void* in, const void* W, void* out, int dtype, int T, int H, int n_in, int n_out,
                                      int ld_in, int head_in, int in_off, int ld_out, int head_out, int out_off,
                                      const void* gate, int ld_gate, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && H > 0 && n_in > 0 && n_out > 0, "head_linear: bad sizes");
    MYNAH_REQUIRE(H <= 65535 && ceil_div(n_out, 64) <= 65535, "head_linear: too many heads or outputs for one launch");
    const HeadLinearArgs a{T, H, n_in, n_out, ld_in, head_in, in_off, ld_out, head_out, out_off, gate, ld_gate};
    const bool mma_ok = dtype == MYNAH_BF16 && !g_head_linear_plain && n_in % 8 == 0 && ld_in % 8 == 0 && head_in % 8 == 0 &&
                        in_off % 8 == 0 && (((uintptr_t)in | (uintptr_t)W) & 15) == 0 && ceil_div(n_out, 128) <= 65535;
    if (mma_ok) {
        if (T <= 16)
            mynah_launch(head_linear_mma_kernel<1>, dim3(1, H, ceil_div(n_out, 128)), dim3(256), 0, stream, (const bf16*)in, (const bf16*)W, (bf16*)out, a);
        else
            mynah_launch(head_linear_mma_kernel<4>, dim3(ceil_div(T, 64), H, ceil_div(n_out, 128)), dim3(256), 0, stream, (const bf16*)in, (const bf16*)W, (bf16*)out, a);
        return mynah_check_launch("head_linear");
    }
    const dim3 grid(ceil_div(T, 64), H, ceil_div(n_out, 64));
    if (dtype == MYNAH_F32)
        mynah_launch(head_linear_kernel<float>, grid, dim3(tilemm::THREADS), 0, stream, (const float*)in, (const float*)W, (float*)out, a);
    else if (dtype == MYNAH_BF16)
        mynah_launch(head_linear_kernel<bf16>, grid, dim3(tilemm::THREADS), 0, stream, (const bf16*)in, (const bf16*)W, (bf16*)out, a);
    else
        return mynah_fail("head_linear: unsupported dtype %d", dtype);
    return mynah_check_launch("head_linear");
}
