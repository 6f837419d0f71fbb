// Windowed softmax attention with a sink, heads whose weights are mixed after the softmax, and rotated values:
//
//   score_g(i, j) = scale * q_g(i) . k(j),   0 <= i - j < window   (q, k rotated by their positions)
//   w_g(i, j)     = exp(score_g(i, j)) / (exp(sink_g) + sum_j' exp(score_g(i, j')))       the sink has no key or value
//   m_h(i, j)     = sum_g talk[h, g] w_g(i, j)                                             mixed weights
//   out_h(i)      = R(-i) sum_j m_h(i, j) R(j) v(j)     R(p): pair m of a value head turned by p * f_m
//
// The cache holds rotated keys and rotated values. Two kernels:
//
//   sink_attn_prep   rotates q and k (first rot dimensions of a head; pairs are (2i, 2i+1) or (i, i + rot/2)), rotates
//                    v over all its dimensions, writes k and v to the cache pages and q to its own rows
//   sink_attn        the general kernel (both precisions, any sizes, prompts and single tokens): a CTA takes one
//                    query with all its heads, since the mixing needs every head's weight of a key. Keys go through
//                    shared memory in chunks; with more than one chunk the scores are formed twice (first for each
//                    head's maximum and denominator, then for the weights). All sums fp32, in an order fixed by the
//                    thread layout and the key's position, whatever else is in the step.
#include "layout.cuh"

namespace {

struct SinkPrepArgs {
    int H, G, dim, vd, ld, rot, n_pos, n_pos_v, interleaved;
};

template <typename T>
__global__ void __launch_bounds__(128)
sink_attn_prep_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache,
                      const float* __restrict__ cos_k, const float* __restrict__ sin_k, const float* __restrict__ cos_v,
                      const float* __restrict__ sin_v, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                      PageTable pt, SinkPrepArgs a, int* __restrict__ status) {
    griddep_launch_small();
    griddep_wait();
    const int row = blockIdx.x;
    const int b = tok_seq[row];
    if (b < 0) return;
    const int pos = tok_pos[row];
    if (pos < 0 || pos >= a.n_pos || pos >= a.n_pos_v) {
        if (threadIdx.x == 0) atomicOr(status, MYNAH_ST_POS_RANGE);
        return;
    }
    const T* src = qkv + (size_t)row * a.ld;
    const int half = a.rot / 2, hv = a.vd / 2;
    const float* ck = cos_k + (size_t)pos * half;
    const float* sk = sin_k + (size_t)pos * half;
    // queries
    const int nq = a.H * a.dim;
    for (int i = threadIdx.x; i < a.H * (a.dim - half); i += blockDim.x) {
        const int h = i / (a.dim - half), e = i % (a.dim - half);
        const T* s = src + (size_t)h * a.dim;
        T* d = q_out + (size_t)row * nq + (size_t)h * a.dim;
        if (e < half) {
            const int i0 = a.interleaved ? 2 * e : e, i1 = a.interleaved ? 2 * e + 1 : e + half;
            const float u = to_f32(s[i0]), v = to_f32(s[i1]);
            d[i0] = from_f32<T>(u * ck[e] - v * sk[e]);
            d[i1] = from_f32<T>(v * ck[e] + u * sk[e]);
        } else {
            d[e + half] = s[e + half];
        }
    }
    if (k_cache == nullptr) return;
    const int page = page_of(pt, b, pos);
    if (page < 0) {
        if (threadIdx.x == 0) atomicOr(status, MYNAH_ST_PAGE_RANGE);
        return;
    }
    for (int i = threadIdx.x; i < a.G * (a.dim - half); i += blockDim.x) {
        const int g = i / (a.dim - half), e = i % (a.dim - half);
        const T* s = src + (size_t)nq + (size_t)g * a.dim;
        T* d = k_cache + (((size_t)page * a.G + g) * PAGE_TOKENS + pos % PAGE_TOKENS) * a.dim;
        if (e < half) {
            const int i0 = a.interleaved ? 2 * e : e, i1 = a.interleaved ? 2 * e + 1 : e + half;
            const float u = to_f32(s[i0]), v = to_f32(s[i1]);
            d[i0] = from_f32<T>(u * ck[e] - v * sk[e]);
            d[i1] = from_f32<T>(v * ck[e] + u * sk[e]);
        } else {
            d[e + half] = s[e + half];
        }
    }
    const float* cv = cos_v + (size_t)pos * hv;
    const float* sv = sin_v + (size_t)pos * hv;
    for (int i = threadIdx.x; i < a.G * hv; i += blockDim.x) {
        const int g = i / hv, e = i % hv;
        const T* s = src + (size_t)nq + (size_t)a.G * a.dim + (size_t)g * a.vd;
        T* d = v_cache + (((size_t)page * a.G + g) * PAGE_TOKENS + pos % PAGE_TOKENS) * a.vd;
        const int i0 = a.interleaved ? 2 * e : e, i1 = a.interleaved ? 2 * e + 1 : e + hv;
        const float u = to_f32(s[i0]), v = to_f32(s[i1]);
        d[i0] = from_f32<T>(u * cv[e] - v * sv[e]);
        d[i1] = from_f32<T>(v * cv[e] + u * sv[e]);
    }
}

constexpr int SA_THREADS = 256;
constexpr int SA_WARPS = SA_THREADS / 32;
constexpr int SA_MAXC = 8;                     // a key of at most 32 * SA_MAXC values

struct SinkAttnArgs {
    int H, G, dim, vd, window, KC, n_pos_v, interleaved;
    float scale;
};

template <typename T>
__global__ void __launch_bounds__(SA_THREADS)
sink_attn_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                 VecRef talk, VecRef sink, const float* __restrict__ cos_v, const float* __restrict__ sin_v,
                 const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, PageTable pt, SinkAttnArgs a,
                 int* __restrict__ status) {
    extern __shared__ float sm[];
    griddep_wait();
    const int row = blockIdx.x;
    const int b = tok_seq[row];
    if (b < 0) return;
    const int p = tok_pos[row];
    if (p < 0 || p >= a.n_pos_v) {
        if (threadIdx.x == 0) atomicOr(status, MYNAH_ST_POS_RANGE);
        return;
    }
    const int H = a.H, G = a.G, HD = a.dim, VD = a.vd, KC = a.KC, rep = H / G;
    float* qs = sm;                              // [H][HD]
    float* S = qs + H * HD;                      // [H][KC] scores, then weights
    float* WM = S + H * KC;                      // [H][KC] mixed weights
    float* O = WM + H * KC;                      // [H][VD]
    float* mx = O + H * VD;                      // [H] running maximum
    float* den = mx + H;                         // [H] running denominator
    int* page_s = reinterpret_cast<int*>(den + H);   // [KC / PAGE_TOKENS + 2] pages of the chunk
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
    const int n = p - lo + 1;
    const int n_chunks = (n + KC - 1) / KC;

    for (int i = threadIdx.x; i < H * HD; i += SA_THREADS) qs[i] = to_f32(q[(size_t)row * H * HD + i]);
    for (int i = threadIdx.x; i < H * VD; i += SA_THREADS) O[i] = 0.f;
    for (int i = threadIdx.x; i < H; i += SA_THREADS) {
        mx[i] = -INFINITY;
        den[i] = 0.f;
    }

    bool bad = false;
    // scores of the chunk's keys [c0, c0 + nk) into S; a warp takes a key and a kv head at a time
    auto scores = [&](int c0, int nk) {
        __syncthreads();                                                   // S free, qs written
        const int first_page = c0 / PAGE_TOKENS;
        for (int i = threadIdx.x; i <= (c0 + nk - 1) / PAGE_TOKENS - first_page; i += SA_THREADS)
            page_s[i] = page_of(pt, b, (first_page + i) * PAGE_TOKENS);
        __syncthreads();
        for (int jc = warp; jc < nk * G; jc += SA_WARPS) {
            const int j = jc / G, c = jc % G;
            const int key = c0 + j;
            const int page = page_s[key / PAGE_TOKENS - first_page];
            if (page < 0) {
                bad = true;
                for (int r = 0; r < rep; r++)
                    if (lane == 0) S[(c * rep + r) * KC + j] = -INFINITY;
                continue;
            }
            const T* kr = k_cache + (((size_t)page * G + c) * PAGE_TOKENS + key % PAGE_TOKENS) * HD;
            float kv[SA_MAXC];
#pragma unroll
            for (int e = 0; e < SA_MAXC; e++) {
                const int d = lane + 32 * e;
                kv[e] = d < HD ? to_f32(kr[d]) : 0.f;
            }
            for (int r = 0; r < rep; r++) {
                const float* qr = qs + (c * rep + r) * HD;
                float dot = 0.f;
#pragma unroll
                for (int e = 0; e < SA_MAXC; e++) {
                    const int d = lane + 32 * e;
                    if (d < HD) dot = fmaf(qr[d], kv[e], dot);
                }
                dot = warp_sum(dot);
                if (lane == 0) S[(c * rep + r) * KC + j] = dot * a.scale;
            }
        }
        __syncthreads();
    };
    // fold the chunk's scores into each head's running maximum and denominator; a warp a head
    auto stats = [&](int nk) {
        for (int g = warp; g < H; g += SA_WARPS) {
            float m = -INFINITY;
            for (int j = lane; j < nk; j += 32) m = fmaxf(m, S[g * KC + j]);
            m = fmaxf(warp_max(m), mx[g]);
            float s = 0.f;
            if (m > -INFINITY)
                for (int j = lane; j < nk; j += 32) s += expf(S[g * KC + j] - m);
            s = warp_sum(s);
            if (lane == 0) {
                den[g] = (m > -INFINITY ? den[g] * expf(mx[g] - m) : 0.f) + s;
                mx[g] = m;
            }
        }
        __syncthreads();
    };

    if (n_chunks == 1) {
        scores(lo, n);
        stats(n);
    } else {
        for (int ch = 0; ch < n_chunks; ch++) {
            const int c0 = lo + ch * KC, nk = min(KC, p + 1 - c0);
            scores(c0, nk);
            stats(nk);
        }
    }
    // the sink joins the denominator
    for (int g = threadIdx.x; g < H; g += SA_THREADS) {
        const float sk = sink.at(g);
        const float m = fmaxf(mx[g], sk);
        den[g] = den[g] * expf(mx[g] - m) + expf(sk - m);
        mx[g] = m;
    }
    __syncthreads();

    for (int ch = 0; ch < n_chunks; ch++) {
        const int c0 = lo + ch * KC, nk = min(KC, p + 1 - c0);
        if (n_chunks > 1) scores(c0, nk);
        for (int i = threadIdx.x; i < H * nk; i += SA_THREADS) {
            const int g = i / nk, j = i % nk;
            S[g * KC + j] = expf(S[g * KC + j] - mx[g]) / den[g];
        }
        __syncthreads();
        for (int i = threadIdx.x; i < H * nk; i += SA_THREADS) {
            const int h = i / nk, j = i % nk;
            float acc = 0.f;
            for (int g = 0; g < H; g++) acc = fmaf(talk.at(h * H + g), S[g * KC + j], acc);
            WM[h * KC + j] = acc;
        }
        __syncthreads();
        // values: a thread takes a column of a kv head and up to four of the group's heads at a time
        const int first_page = c0 / PAGE_TOKENS;
        for (int i = threadIdx.x; i < G * VD; i += SA_THREADS) {
            const int c = i / VD, d = i % VD;
            for (int r0 = 0; r0 < rep; r0 += 4) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                const int nr = min(4, rep - r0);
                const float* w0 = WM + (c * rep + r0) * KC;
                for (int j = 0; j < nk; j++) {
                    const int key = c0 + j;
                    const int page = page_s[key / PAGE_TOKENS - first_page];
                    if (page < 0) continue;
                    const float v = to_f32(v_cache[(((size_t)page * G + c) * PAGE_TOKENS + key % PAGE_TOKENS) * VD + d]);
#pragma unroll
                    for (int r = 0; r < 4; r++)
                        if (r < nr) acc[r] = fmaf(w0[r * KC + j], v, acc[r]);
                }
#pragma unroll
                for (int r = 0; r < 4; r++)
                    if (r < nr) O[(c * rep + r0 + r) * VD + d] += acc[r];
            }
        }
    }
    __syncthreads();
    if (bad && lane == 0) atomicOr(status, MYNAH_ST_PAGE_RANGE);
    // turn every head's sum back by the query's position
    const int hv = VD / 2;
    const float* cv = cos_v + (size_t)p * hv;
    const float* sv = sin_v + (size_t)p * hv;
    for (int i = threadIdx.x; i < H * hv; i += SA_THREADS) {
        const int h = i / hv, e = i % hv;
        const int i0 = a.interleaved ? 2 * e : e, i1 = a.interleaved ? 2 * e + 1 : e + hv;
        const float u = O[h * VD + i0], v = O[h * VD + i1];
        T* dst = out + (size_t)row * H * VD + (size_t)h * VD;
        dst[i0] = from_f32<T>(u * cv[e] + v * sv[e]);
        dst[i1] = from_f32<T>(v * cv[e] - u * sv[e]);
    }
}

}  // namespace

// qkv [T, ld] in dtype: H*dim query, G*dim key, G*vd value columns. q_out [T, H*dim]. k_cache, v_cache: the entry's
// pages (null: a run that reads another run's cache brings only queries). cos_k, sin_k fp32 [n_pos, rot/2];
// cos_v, sin_v fp32 [n_pos_v, vd/2].
MYNAH_API int mynah_sink_attn_prep(const void* qkv, int ld, int dtype, void* q_out, void* k_cache, void* v_cache,
                                   const float* cos_k, const float* sin_k, int n_pos, const float* cos_v, const float* sin_v,
                                   int n_pos_v, const int* tok_seq, const int* tok_pos, const int* page_indptr,
                                   const int* page_ids, const int* page_base, int n_pages, int T, int H, int G, int dim,
                                   int vd, int rot, int interleaved, int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && H > 0 && G > 0 && dim > 0 && vd > 0 && H % G == 0, "sink_attn_prep: bad sizes");
    MYNAH_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dim && vd % 2 == 0, "sink_attn_prep: rot=%d of dim=%d, vd=%d: pairs do not fit", rot, dim, vd);
    const SinkPrepArgs a{H, G, dim, vd, ld, rot, rot > 0 ? n_pos : 0x7fffffff, n_pos_v, interleaved};
    const PageTable pt{page_indptr, page_ids, page_base, n_pages};
    if (dtype == MYNAH_F32)
        mynah_launch(sink_attn_prep_kernel<float>, dim3(T), dim3(128), 0, stream, (const float*)qkv, (float*)q_out, (float*)k_cache,
                     (float*)v_cache, cos_k, sin_k, cos_v, sin_v, tok_seq, tok_pos, pt, a, status);
    else if (dtype == MYNAH_BF16)
        mynah_launch(sink_attn_prep_kernel<bf16>, dim3(T), dim3(128), 0, stream, (const bf16*)qkv, (bf16*)q_out, (bf16*)k_cache,
                     (bf16*)v_cache, cos_k, sin_k, cos_v, sin_v, tok_seq, tok_pos, pt, a, status);
    else
        return mynah_fail("sink_attn_prep: unsupported dtype %d", dtype);
    return mynah_check_launch("sink_attn_prep");
}

// Keys of a chunk for H heads (the scores and the mixed weights of a chunk lie in shared memory side by side).
static int sink_attn_chunk(int H, int dim, int vd, int window) {
    const long long fixed = (long long)H * dim + (long long)H * vd + 2 * H + 64;
    long long kc = (160 * 1024 / 4 - fixed) / (2 * H);
    if (kc > 4096) kc = 4096;
    if (window > 0 && kc > window) kc = window;
    return (int)kc;
}

// q [T, H*dim], out [T, H*vd] in dtype; talk [H, H] and sink [H] in g_dtype; window 0: every earlier key.
MYNAH_API int mynah_sink_attn(const void* q, void* out, int dtype, const void* k_cache, const void* v_cache, const void* talk,
                              const void* sink, int g_dtype, const float* cos_v, const float* sin_v, int n_pos_v,
                              const int* tok_seq, const int* tok_pos, const int* page_indptr, const int* page_ids,
                              const int* page_base, int n_pages, int T, int H, int G, int dim, int vd, int window, float scale,
                              int interleaved, int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && H > 0 && G > 0 && dim > 0 && vd > 0 && H % G == 0 && vd % 2 == 0, "sink_attn: bad sizes");
    MYNAH_REQUIRE(dim <= 32 * SA_MAXC, "sink_attn: a key of %d values exceeds %d", dim, 32 * SA_MAXC);
    MYNAH_REQUIRE(window >= 0, "sink_attn: negative window");
    const int KC = sink_attn_chunk(H, dim, vd, window);
    MYNAH_REQUIRE(KC >= 32 || (window > 0 && KC >= window), "sink_attn: %d heads of %d and %d values exceed shared memory", H, dim, vd);
    const SinkAttnArgs a{H, G, dim, vd, window, KC, n_pos_v, interleaved, scale};
    const PageTable pt{page_indptr, page_ids, page_base, n_pages};
    const size_t smem = sizeof(float) * ((size_t)H * dim + 2 * (size_t)H * KC + (size_t)H * vd + 2 * H + KC / PAGE_TOKENS + 4);
    const VecRef tk{talk, g_dtype}, sk{sink, g_dtype};
#define SINK_LAUNCH(T_)                                                                                                      \
    if (smem > 48 * 1024 && cudaFuncSetAttribute(sink_attn_kernel<T_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
        return mynah_fail("sink_attn: %zu bytes of shared memory are not to be had", smem);                                \
    mynah_launch(sink_attn_kernel<T_>, dim3(T), dim3(SA_THREADS), smem, stream, (const T_*)q, (T_*)out, (const T_*)k_cache,   \
                 (const T_*)v_cache, tk, sk, cos_v, sin_v, tok_seq, tok_pos, pt, a, status)
    if (dtype == MYNAH_F32) { SINK_LAUNCH(float); }
    else if (dtype == MYNAH_BF16) { SINK_LAUNCH(bf16); }
    else return mynah_fail("sink_attn: unsupported dtype %d", dtype);
#undef SINK_LAUNCH
    return mynah_check_launch("sink_attn");
}
