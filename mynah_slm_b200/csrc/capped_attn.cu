// The steps around the attention kernels for grouped-query attention whose projections may carry biases, whose
// heads may be normed, whose heads may hold several score maps over the same values ("differential" attention),
// and whose heads' outputs may be gated:
//
//   capped_attn_prep   per token: every unit of `dim` values of the q and k projections (a head, or one map of a
//                      head) gets its bias, an RMS norm with one gain shared by all units, and a rotation of its first
//                      `rot` dimensions (pairs (i, i + rot/2) or (2i, 2i+1)); queries go to packed rows, keys and
//                      (biased) values to the token's place in the paged cache. All of it in fp32.
//                      With M maps a head, query head h = g * R + j (R query heads a kv head) and map m go to
//                      slot (g * M + m) * R + j of the packed row and key (g, m) to kv head g * M + m, so that the
//                      attention kernels' own grouping (slot / R) pairs every query map with its key map, and kv
//                      head g * M + m reads value head g (the kernels' `vdiv` = M).
//   diff_combine       o_h = unit_rms(a_h,0 - lambda a_h,1) * mult over the head's values, from those slots back to
//                      head order
//   head_gate          x[t, h, :] *= sigmoid(gate[t, h])
#include "layout.cuh"

namespace {

constexpr int PREP_WARPS = 4;
constexpr int PREP_MAXC = 8;       // a unit of at most 32 * PREP_MAXC values

struct CappedPrepArgs {
    int Hq, Gk, Gv;        // units of q, of k, heads of v
    int dim, vd, dimp, vdp;
    int ld, ldq;           // row strides of the projection and of the packed queries
    int maps, R;           // score maps a head; query heads a kv head
    int rot, interleaved, n_pos;
    int has_norm;
    float eps;
};

template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32)
capped_attn_prep_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ bias, VecRef q_gain,
                        VecRef k_gain, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                        const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, PageTable pt,
                        T* __restrict__ k_cache, T* __restrict__ v_cache, CappedPrepArgs a, int* __restrict__ status) {
    __shared__ float unit[PREP_WARPS][32 * PREP_MAXC];
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
    const bool writes = k_cache != nullptr;
    int page = -1;
    if (writes) {
        page = page_of(pt, b, pos);
        if (page < 0) {
            if (threadIdx.x == 0) atomicOr(status, MYNAH_ST_PAGE_RANGE);
            return;
        }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = a.rot >> 1;
    const float* cr = rotate ? cos_t + (size_t)pos * half : nullptr;
    const float* sr = rotate ? sin_t + (size_t)pos * half : nullptr;
    const T* row = qkv + (size_t)t * a.ld;
    const int n_units = a.Hq + (writes ? a.Gk + a.Gv : 0);
    float* mine = unit[warp];
    // a warp a unit: blockIdx.y numbers the groups of PREP_WARPS units of the token
    const int u = blockIdx.y * PREP_WARPS + warp;
    if (u >= n_units) return;
    if (u >= a.Hq + a.Gk) {                                // a value head: bias, then the cache
        const int g = u - a.Hq - a.Gk;
        const int col = (a.Hq + a.Gk) * a.dim + g * a.vd;
        T* dst = v_cache + (((size_t)page * a.Gv + g) * PAGE_TOKENS + pos % PAGE_TOKENS) * a.vdp;
        for (int d = lane; d < a.vdp; d += 32) {
            float v = 0.f;
            if (d < a.vd) v = to_f32(row[col + d]) + (bias != nullptr ? bias[col + d] : 0.f);
            dst[d] = from_f32<T>(v);
        }
        return;
    }
    const bool is_q = u < a.Hq;
    const int col = u * a.dim;                             // q units, then k units, side by side
    float ss = 0.f;
    for (int d = lane; d < a.dim; d += 32) {
        const float v = to_f32(row[col + d]) + (bias != nullptr ? bias[col + d] : 0.f);
        mine[d] = v;
        ss = fmaf(v, v, ss);
    }
    if (a.has_norm) {
        ss = warp_sum(ss);
        const float s = 1.0f / sqrtf(ss / (float)a.dim + a.eps);
        const VecRef& gain = is_q ? q_gain : k_gain;
        for (int d = lane; d < a.dim; d += 32) mine[d] = (mine[d] * s) * gain.at(d);
    }
    __syncwarp();
    T* dst;
    if (is_q) {
        const int h = u / a.maps, m = u % a.maps;
        const int slot = ((h / a.R) * a.maps + m) * a.R + h % a.R;
        dst = q_out + (size_t)t * a.ldq + (size_t)slot * a.dimp;
    } else {
        dst = k_cache + (((size_t)page * a.Gk + (u - a.Hq)) * PAGE_TOKENS + pos % PAGE_TOKENS) * a.dimp;
    }
    for (int d = lane; d < a.dimp; d += 32) {
        float v = 0.f;
        if (d < a.dim) {
            v = mine[d];
            if (rotate && d < a.rot) {
                int i, other;
                float sign;
                if (a.interleaved) {
                    i = d >> 1;
                    other = d ^ 1;
                    sign = (d & 1) ? 1.f : -1.f;
                } else {
                    i = d < half ? d : d - half;
                    other = d < half ? d + half : d - half;
                    sign = d < half ? -1.f : 1.f;
                }
                v = v * cr[i] + sign * mine[other] * sr[i];
            }
        }
        dst[d] = from_f32<T>(v);
    }
}

// The same for units that move 16 bytes at a time: `dim` a power of two from 8 to 256 and `vd` a multiple of 8 (no padding
// columns), rotated pairs that lie whole chunks apart (rot a multiple of 16) or side by side (interleaved). A unit lies
// across dim / 8 lanes, eight values a lane; a warp takes 256 / dim units at once; the partner of a rotated value is the
// same register of another lane of the unit. grid (tokens, groups of units); the last group's CTA also copies the values.
template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32)
capped_attn_prep_vec_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ bias, VecRef q_gain,
                            VecRef k_gain, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                            const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, PageTable pt,
                            T* __restrict__ k_cache, T* __restrict__ v_cache, CappedPrepArgs a, int* __restrict__ status) {
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
    const bool writes = k_cache != nullptr;
    int page = -1;
    if (writes) {
        page = page_of(pt, b, pos);
        if (page < 0) {
            if (threadIdx.x == 0) atomicOr(status, MYNAH_ST_PAGE_RANGE);
            return;
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int L = a.dim >> 3, per_warp = 32 / L;           // lanes a unit, units a warp
    const int half = a.rot >> 1;
    const T* row = qkv + (size_t)t * a.ld;
    const int n_qk = a.Hq + (writes ? a.Gk : 0);
    if (writes && blockIdx.y == gridDim.y - 1) {           // the values: bias, then the cache
        const int col0 = (a.Hq + a.Gk) * a.dim, chunks = a.Gv * a.vd / 8, cpv = a.vd / 8;
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
            float v[8];
            load8(row + col0 + c * 8, v);
            if (bias != nullptr) {
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] += bias[col0 + c * 8 + j];
            }
            const int g = c / cpv;
            store8(v_cache + (((size_t)page * a.Gv + g) * PAGE_TOKENS + pos % PAGE_TOKENS) * a.vd + (c % cpv) * 8, v);
        }
    }
    const int u = (blockIdx.y * PREP_WARPS + warp) * per_warp + lane / L;
    const int l = lane % L;
    const bool on = u < n_qk;
    const bool is_q = u < a.Hq;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (on) {
        load8(row + (size_t)u * a.dim + l * 8, v);
        if (bias != nullptr) {
            float bv[8];
            load8(bias + u * a.dim + l * 8, bv);
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] += bv[j];
        }
    }
    if (a.has_norm) {                                       // every lane takes part in the shuffles, units that are off too
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) ss = fmaf(v[j], v[j], ss);
        for (int o = L >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float s = 1.0f / sqrtf(ss / (float)a.dim + a.eps);
        const VecRef& gain = is_q ? q_gain : k_gain;
        float gv[8];
        if (gain.dtype == MYNAH_F32) load8(static_cast<const float*>(gain.p) + l * 8, gv);
        else load8(static_cast<const bf16*>(gain.p) + l * 8, gv);
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = (v[j] * s) * gv[j];
    }
    if (rotate) {
        const float* cr = cos_t + (size_t)pos * half;
        const float* sr = sin_t + (size_t)pos * half;
        if (a.interleaved) {
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                if (l * 8 + j < a.rot) {                    // pairs beyond the rotated dimensions pass
                    const int i = (l * 8 + j) >> 1;
                    const float c = cr[i], sn = sr[i], x = v[j], y = v[j + 1];
                    v[j] = x * c - y * sn;
                    v[j + 1] = y * c + x * sn;
                }
            }
        } else {
            const int hl = half >> 3;                       // lanes between a value and its partner
            const bool low = l < hl, in = l < 2 * hl;
            const int src = (lane - l) + (in ? (low ? l + hl : l - hl) : l);
            const int i0 = (low ? l : l - hl) * 8;
            float cv[8] = {}, sv[8] = {};
            if (in) {
                load8(cr + i0, cv);
                load8(sr + i0, sv);
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float other = __shfl_sync(0xffffffffu, v[j], src);
                if (in) v[j] = v[j] * cv[j] + (low ? -other : other) * sv[j];
            }
        }
    }
    if (!on) return;
    T* dst;
    if (is_q) {
        const int h = u / a.maps, m = u % a.maps;
        const int slot = ((h / a.R) * a.maps + m) * a.R + h % a.R;
        dst = q_out + (size_t)t * a.ldq + (size_t)slot * a.dim;
    } else {
        dst = k_cache + (((size_t)page * a.Gk + (u - a.Hq)) * PAGE_TOKENS + pos % PAGE_TOKENS) * a.dim;
    }
    store8(dst + l * 8, v);
}

struct DiffArgs {
    int H, R, vd, vdp, lda, ldo;
    float lambda, mult, eps;
};

// one warp a (token, head)
template <typename T>
__global__ void __launch_bounds__(128)
diff_combine_kernel(const T* __restrict__ a_in, T* __restrict__ out, const int* __restrict__ tok_seq, int n_tokens, DiffArgs a) {
    griddep_launch_small();
    griddep_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * 4 + warp;
    if (w >= (long long)n_tokens * a.H) return;
    const int t = (int)(w / a.H), h = (int)(w % a.H);
    if (tok_seq[t] < 0) return;
    const int g = h / a.R, j = h % a.R;
    const T* a0 = a_in + (size_t)t * a.lda + (size_t)((g * 2 + 0) * a.R + j) * a.vdp;
    const T* a1 = a_in + (size_t)t * a.lda + (size_t)((g * 2 + 1) * a.R + j) * a.vdp;
    float v[PREP_MAXC];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < PREP_MAXC; c++) {
        const int d = lane + 32 * c;
        v[c] = d < a.vd ? to_f32(a0[d]) - a.lambda * to_f32(a1[d]) : 0.f;
        ss = fmaf(v[c], v[c], ss);
    }
    ss = warp_sum(ss);
    const float s = a.mult / sqrtf(ss / (float)a.vd + a.eps);
    T* o = out + (size_t)t * a.ldo + (size_t)h * a.vd;
#pragma unroll
    for (int c = 0; c < PREP_MAXC; c++) {
        const int d = lane + 32 * c;
        if (d < a.vd) o[d] = from_f32<T>(v[c] * s);
    }
}

// VEC values a thread (8: heads and row strides that are multiples of 8, 16-byte accesses; else 1)
template <typename T, int VEC>
__global__ void head_gate_kernel(T* __restrict__ x, int ldx, const T* __restrict__ gate, int ldg, int H, int vd, long long n) {
    griddep_launch_small();
    griddep_wait();
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (i >= n) return;
    const int per = H * vd;
    const int t = (int)(i / per), c = (int)(i % per);
    const float z = to_f32(gate[(size_t)t * ldg + c / vd]);
    const float g = 1.0f / (1.0f + expf(-z));
    T* p = x + (size_t)t * ldx + c;
    if constexpr (VEC == 8) {
        float v[8];
        load8(p, v);
#pragma unroll
        for (int k = 0; k < 8; k++) v[k] *= g;
        store8(p, v);
    } else {
        *p = from_f32<T>(to_f32(*p) * g);
    }
}

}  // namespace

// qkv: [T][ld] rows of the projection: Hq units of `dim` (q), then, when the caches are given, Gk units of `dim` (k)
// and Gv heads of `vd` (v). bias: fp32 over those columns, or null. q_gain / k_gain: `dim` values each in gain_dtype,
// or null for no norm. q_out: [T][ldq] packed queries of `dimp` values a slot; k_cache [pages][Gk][PAGE][dimp],
// v_cache [pages][Gv][PAGE][vdp] (both null for a run that brings queries only). Padding columns are written as zeros.
MYNAH_API int mynah_capped_attn_prep(const void* qkv, int dtype, int T, int ld, void* q_out, int ldq, int Hq, int Gk, int Gv,
                                     int dim, int vd, int dimp, int vdp, int maps, int R, const float* bias,
                                     const void* q_gain, const void* k_gain, int gain_dtype, float eps, const float* cos_t,
                                     const float* sin_t, int rot, int interleaved, int n_pos, const int* tok_seq,
                                     const int* tok_pos, const int* page_indptr, const int* page_ids, const int* page_base,
                                     int n_pages, void* k_cache, void* v_cache, int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && Hq > 0 && Gk > 0 && Gv > 0 && dim > 0 && vd > 0 && maps > 0 && R > 0, "capped_attn_prep: bad sizes");
    MYNAH_REQUIRE(dim <= 32 * PREP_MAXC && dimp >= dim && vdp >= vd, "capped_attn_prep: a unit of %d values exceeds %d", dim, 32 * PREP_MAXC);
    MYNAH_REQUIRE(Hq % maps == 0 && (Hq / maps) % R == 0, "capped_attn_prep: %d query units do not divide into maps of %d and groups of %d", Hq, maps, R);
    MYNAH_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dim, "capped_attn_prep: %d rotated dimensions do not fit a unit of %d", rot, dim);
    MYNAH_REQUIRE((k_cache == nullptr) == (v_cache == nullptr), "capped_attn_prep: the two caches go together");
    MYNAH_REQUIRE((q_gain == nullptr) == (k_gain == nullptr), "capped_attn_prep: the two gains go together");
    const CappedPrepArgs a{Hq, Gk, Gv, dim, vd, dimp, vdp, ld, ldq, maps, R, cos_t != nullptr ? rot : 0, interleaved, n_pos,
                           q_gain != nullptr ? 1 : 0, eps};
    const PageTable pt{page_indptr, page_ids, page_base, n_pages};
    const VecRef qg{q_gain, gain_dtype}, kg{k_gain, gain_dtype};
    // units that move 16 bytes at a time take the vector form
    const bool pow2 = (dim & (dim - 1)) == 0;
    const bool vec = pow2 && dim >= 8 && dim <= 256 && vd % 8 == 0 && dimp == dim && vdp == vd && ld % 8 == 0 && ldq % 8 == 0 &&
                     (cos_t == nullptr || rot == 0 || interleaved || rot % 16 == 0) &&
                     (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) & (dtype == MYNAH_F32 ? 31 : 15)) == 0 &&
                     (((uintptr_t)bias | (uintptr_t)q_gain | (uintptr_t)k_gain | (uintptr_t)cos_t | (uintptr_t)sin_t) & 31) == 0;
    if (vec) {
        const int per_cta = PREP_WARPS * (256 / dim);
        const int n_qk = Hq + (k_cache != nullptr ? Gk : 0);
        MYNAH_REQUIRE(ceil_div(n_qk, per_cta) <= 65535, "capped_attn_prep: too many heads for one launch");
        const dim3 vgrid(T, ceil_div(n_qk, per_cta));
        if (dtype == MYNAH_F32)
            mynah_launch(capped_attn_prep_vec_kernel<float>, vgrid, dim3(PREP_WARPS * 32), 0, stream, (const float*)qkv, (float*)q_out, bias,
                         qg, kg, cos_t, sin_t, tok_seq, tok_pos, pt, (float*)k_cache, (float*)v_cache, a, status);
        else if (dtype == MYNAH_BF16)
            mynah_launch(capped_attn_prep_vec_kernel<bf16>, vgrid, dim3(PREP_WARPS * 32), 0, stream, (const bf16*)qkv, (bf16*)q_out, bias,
                         qg, kg, cos_t, sin_t, tok_seq, tok_pos, pt, (bf16*)k_cache, (bf16*)v_cache, a, status);
        else
            return mynah_fail("capped_attn_prep: unsupported dtype %d", dtype);
        return mynah_check_launch("capped_attn_prep");
    }
    const int n_units = Hq + (k_cache != nullptr ? Gk + Gv : 0);
    MYNAH_REQUIRE(ceil_div(n_units, PREP_WARPS) <= 65535, "capped_attn_prep: too many heads for one launch");
    const dim3 grid(T, ceil_div(n_units, PREP_WARPS));
    if (dtype == MYNAH_F32)
        mynah_launch(capped_attn_prep_kernel<float>, grid, dim3(PREP_WARPS * 32), 0, stream, (const float*)qkv, (float*)q_out, bias,
                     qg, kg, cos_t, sin_t, tok_seq, tok_pos, pt, (float*)k_cache, (float*)v_cache, a, status);
    else if (dtype == MYNAH_BF16)
        mynah_launch(capped_attn_prep_kernel<bf16>, grid, dim3(PREP_WARPS * 32), 0, stream, (const bf16*)qkv, (bf16*)q_out, bias, qg,
                     kg, cos_t, sin_t, tok_seq, tok_pos, pt, (bf16*)k_cache, (bf16*)v_cache, a, status);
    else
        return mynah_fail("capped_attn_prep: unsupported dtype %d", dtype);
    return mynah_check_launch("capped_attn_prep");
}

// a: [T][lda], slot (g * 2 + m) * R + j of `vdp` values holds map m of head g * R + j; out: [T][ldo], head h at
// columns [h * vd, (h + 1) * vd): unit_rms(a_0 - lambda a_1) * mult.
MYNAH_API int mynah_diff_combine(const void* a_in, int dtype, int T, int lda, void* out, int ldo, int H, int R, int vd, int vdp,
                                 float lambda, float mult, float eps, const int* tok_seq, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && H > 0 && R > 0 && H % R == 0 && vd > 0 && vd <= 32 * PREP_MAXC && vdp >= vd, "diff_combine: bad sizes");
    const DiffArgs a{H, R, vd, vdp, lda, ldo, lambda, mult, eps};
    const unsigned blocks = (unsigned)(((long long)T * H + 3) / 4);
    if (dtype == MYNAH_F32)
        mynah_launch(diff_combine_kernel<float>, dim3(blocks), dim3(128), 0, stream, (const float*)a_in, (float*)out, tok_seq, T, a);
    else if (dtype == MYNAH_BF16)
        mynah_launch(diff_combine_kernel<bf16>, dim3(blocks), dim3(128), 0, stream, (const bf16*)a_in, (bf16*)out, tok_seq, T, a);
    else
        return mynah_fail("diff_combine: unsupported dtype %d", dtype);
    return mynah_check_launch("diff_combine");
}

// x: [T][ldx] with head h at columns [h * vd, (h + 1) * vd); gate: [T][ldg], head h's logit at column h.
MYNAH_API int mynah_head_gate(void* x, int dtype, int T, int ldx, const void* gate, int ldg, int H, int vd, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && H > 0 && vd > 0, "head_gate: bad sizes");
    const long long n = (long long)T * H * vd;
    const bool vec = vd % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 31) == 0;
    const unsigned blocks = (unsigned)((n / (vec ? 8 : 1) + 255) / 256);
    if (dtype == MYNAH_F32 && vec)
        mynah_launch(head_gate_kernel<float, 8>, dim3(blocks), dim3(256), 0, stream, (float*)x, ldx, (const float*)gate, ldg, H, vd, n);
    else if (dtype == MYNAH_F32)
        mynah_launch(head_gate_kernel<float, 1>, dim3(blocks), dim3(256), 0, stream, (float*)x, ldx, (const float*)gate, ldg, H, vd, n);
    else if (dtype == MYNAH_BF16 && vec)
        mynah_launch(head_gate_kernel<bf16, 8>, dim3(blocks), dim3(256), 0, stream, (bf16*)x, ldx, (const bf16*)gate, ldg, H, vd, n);
    else if (dtype == MYNAH_BF16)
        mynah_launch(head_gate_kernel<bf16, 1>, dim3(blocks), dim3(256), 0, stream, (bf16*)x, ldx, (const bf16*)gate, ldg, H, vd, n);
    else
        return mynah_fail("head_gate: unsupported dtype %d", dtype);
    return mynah_check_launch("head_gate");
}
