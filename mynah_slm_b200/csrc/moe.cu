// Feed-forward of several small experts of which every token uses `top`, and the steps around it:
//
//   moe_route     a token's experts come from a table indexed by its token id ([vocab][top]); the step's
//                 (token, choice) pairs are sorted by expert into one list, cut into tiles of rows that share an
//                 expert. One CTA: count, scan, place. The order inside an expert's list is not fixed, and does
//                 not matter: a row's arithmetic does not depend on its place in a tile.
//   (the two products below run on tensor cores for bfloat16 rows, on fused multiply-adds for the 32-bit run)
//   moe_gate_up   for every tile: g = min(W_gate,e h, limit), u = clamp(W_up,e h, -limit, limit),
//                 y = g * sigmoid(alpha g) * (u + 1), written per pair                         (act: clamped)
//   moe_down      for every tile: W_down,e y, written per pair in fp32
//   moe_combine   out[t] = weight * sum over the token's pairs, in the order of its choices
//
// Prompt steps in bfloat16 take another route to the same result: see "prompts in bfloat16" below.
//
// A second way to pick and to compute (the learned-router form):
//   moe_router    logits z = W_r h + b_r in fp32; a token's experts are the `top` largest (the lower index wins a
//                 tie), their weights the softmax over the chosen logits alone. It writes the choices and the
//                 weights; moe_route then sorts by the choices instead of reading a table.
//   act: plain    y = gelu(W_up,e h) (the exact, erf form), one matrix an expert, no gate
//   moe_combine   out[t] = sum over the token's pairs of weight_pair * row
//
// A third way to pick (the group-limited scored router), with the clamped-gate experts:
//   moe_group_router  scores s = sigmoid(W_r h) in fp32; the choice goes by s + correction; the experts form equal groups
//                 of neighbours, a group counts the sum of its two largest choice scores, only experts of the `keep`
//                 best groups can be chosen (the lower index wins every tie); the `top` largest choice scores among
//                 them are the token's experts, and each counts s (without the correction) times a constant.
//
// The grid of the two products covers the most tiles a step can have (pairs / rows-per-tile + experts); CTAs
// beyond the step's tiles leave at once, so a captured step needs no count from the host.
#include "layout.cuh"
#include "tile_mm.cuh"
#include "tile_mma.cuh"

namespace {

constexpr int MOE_ROUTE_THREADS = 1024;
constexpr int MOE_MAX_EXPERTS = 1024;

// tiles: [0] number of tiles, then per tile (expert, first index into perm, rows)
__global__ void __launch_bounds__(MOE_ROUTE_THREADS)
moe_route_kernel(const int* __restrict__ tokens, const int* __restrict__ tok_seq, const int* __restrict__ table,
                 const int* __restrict__ choice, int T, int V, int top, int E, int BM, int* __restrict__ pair_expert,
                 int* __restrict__ perm, int* __restrict__ tiles, int max_tiles, int* __restrict__ status) {
    __shared__ int count[MOE_MAX_EXPERTS], start[MOE_MAX_EXPERTS];
    griddep_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    const int P = T * top;
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int t = p / top;
        int e = -1;
        if (tok_seq[t] >= 0) {
            if (choice != nullptr) {
                e = choice[p];                                    // a router picked it
            } else {
                const int tok = tokens[t];
                if (tok >= 0 && tok < V) e = table[(size_t)tok * top + p % top];
            }
            if (e < 0 || e >= E) {
                atomicOr(status, MYNAH_ST_TOKEN_RANGE);
                e = -1;
            }
        }
        pair_expert[p] = e;
        if (e >= 0) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, nt = 0;
        for (int e = 0; e < E; e++) {
            start[e] = at;
            for (int r = 0; r < count[e] && nt < max_tiles; r += BM, nt++) {
                tiles[1 + 3 * nt] = e;
                tiles[2 + 3 * nt] = at + r;
                tiles[3 + 3 * nt] = min(BM, count[e] - r);
            }
            at += count[e];
        }
        tiles[0] = nt;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = pair_expert[p];
        if (e >= 0) perm[start[e] + atomicAdd(&count[e], 1)] = p;
    }
}

enum MoeAct : int { MOE_ACT_CLAMPED_GATE = 0, MOE_ACT_GELU = 1 };

struct MoeArgs {
    int top, D, F;
    float limit, alpha;
};

__device__ __forceinline__ float gelu_erf_f(float z) { return 0.5f * z * (1.0f + erff(z * 0.7071067811865476f)); }

// grid (tiles, column tiles of F). h: [T][D] rows; w_gu: [E][2][F][D] (gate rows, then up rows); y: [P][F]
template <typename TA, int BM, int ACT>
__global__ void __launch_bounds__(tilemm::THREADS)
moe_gate_up_kernel(const TA* __restrict__ h, const TA* __restrict__ w_gu, TA* __restrict__ y,
                   const int* __restrict__ perm, const int* __restrict__ tiles, MoeArgs a) {
    constexpr int BN = 64;
    __shared__ tilemm::Smem<BM, BN> s;
    __shared__ int pair_s[BM];
    griddep_wait();
    if ((int)blockIdx.x >= tiles[0]) return;
    const int e = tiles[1 + 3 * blockIdx.x], r0 = tiles[2 + 3 * blockIdx.x], nr = tiles[3 + 3 * blockIdx.x];
    const int c0 = blockIdx.y * BN;
    for (int i = threadIdx.x; i < BM; i += blockDim.x) {
        const int p = i < nr ? perm[r0 + i] : -1;
        pair_s[i] = p;
        s.rows[i] = p >= 0 ? h + (size_t)(p / a.top) * a.D : nullptr;
    }
    constexpr int NMAT = ACT == MOE_ACT_CLAMPED_GATE ? 2 : 1;     // matrices an expert: gate and up, or up alone
    const TA* wg = w_gu + ((size_t)e * NMAT * a.F + c0) * a.D;
    float g[BM / 16][BN / 16], u[BM / 16][BN / 16];
    tilemm::run<TA, BM, BN>(s, wg, (size_t)a.D, a.F - c0, a.D, g);
    if (ACT == MOE_ACT_CLAMPED_GATE) tilemm::run<TA, BM, BN>(s, wg + (size_t)a.F * a.D, (size_t)a.D, a.F - c0, a.D, u);
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
#pragma unroll
    for (int i = 0; i < BM / 16; i++) {
        const int p = pair_s[ty + 16 * i];
        if (p < 0) continue;
#pragma unroll
        for (int j = 0; j < BN / 16; j++) {
            const int c = c0 + tx + 16 * j;
            if (c >= a.F) continue;
            // the products are rounded to the activation type first, as a product kernel would store them
            if (ACT == MOE_ACT_GELU) {
                y[(size_t)p * a.F + c] = from_f32<TA>(gelu_erf_f(round_to<TA>(g[i][j])));
                continue;
            }
            const float gv = fminf(round_to<TA>(g[i][j]), a.limit);
            const float uv = fminf(fmaxf(round_to<TA>(u[i][j]), -a.limit), a.limit);
            y[(size_t)p * a.F + c] = from_f32<TA>(gv * (1.0f / (1.0f + expf(-a.alpha * gv))) * (uv + 1.0f));
        }
    }
}

// grid (tiles, column tiles of D). y: [P][F]; w_down: [E][D][F]; o: fp32 [P][D]
template <typename TA, int BM>
__global__ void __launch_bounds__(tilemm::THREADS)
moe_down_kernel(const TA* __restrict__ y, const TA* __restrict__ w_down, float* __restrict__ o,
                const int* __restrict__ perm, const int* __restrict__ tiles, MoeArgs a) {
    constexpr int BN = 64;
    __shared__ tilemm::Smem<BM, BN> s;
    __shared__ int pair_s[BM];
    griddep_wait();
    if ((int)blockIdx.x >= tiles[0]) return;
    const int e = tiles[1 + 3 * blockIdx.x], r0 = tiles[2 + 3 * blockIdx.x], nr = tiles[3 + 3 * blockIdx.x];
    const int c0 = blockIdx.y * BN;
    for (int i = threadIdx.x; i < BM; i += blockDim.x) {
        const int p = i < nr ? perm[r0 + i] : -1;
        pair_s[i] = p;
        s.rows[i] = p >= 0 ? y + (size_t)p * a.F : nullptr;
    }
    float acc[BM / 16][BN / 16];
    tilemm::run<TA, BM, BN>(s, w_down + ((size_t)e * a.D + c0) * a.F, (size_t)a.F, a.D - c0, a.F, acc);
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
#pragma unroll
    for (int i = 0; i < BM / 16; i++) {
        const int p = pair_s[ty + 16 * i];
        if (p < 0) continue;
#pragma unroll
        for (int j = 0; j < BN / 16; j++) {
            const int c = c0 + tx + 16 * j;
            if (c < a.D) o[(size_t)p * a.D + c] = acc[i][j];
        }
    }
}

// row_of_pair null: pair p's row is p. pair_weight null: every pair counts `weight`.
template <typename TA>
__global__ void moe_combine_kernel(const float* __restrict__ o, const int* __restrict__ pair_expert,
                                   const int* __restrict__ row_of_pair, const float* __restrict__ pair_weight,
                                   TA* __restrict__ out, int top, int D, float weight) {
    griddep_launch_small();
    griddep_wait();
    const int t = blockIdx.x;
    if (D % 4 == 0) {                                       // four columns a thread, 16-byte loads; a column's sum runs in the same order
        for (int c = threadIdx.x * 4; c < D; c += blockDim.x * 4) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int k = 0; k < top; k++) {
                const int p = t * top + k;
                if (pair_expert[p] < 0) continue;
                const float4 v = *reinterpret_cast<const float4*>(o + (size_t)(row_of_pair != nullptr ? row_of_pair[p] : p) * D + c);
                const float vv[4] = {v.x, v.y, v.z, v.w};
                const float w = pair_weight != nullptr ? pair_weight[p] : 0.f;
#pragma unroll
                for (int j = 0; j < 4; j++) acc[j] = pair_weight != nullptr ? fmaf(w, vv[j], acc[j]) : acc[j] + vv[j];
            }
#pragma unroll
            for (int j = 0; j < 4; j++) out[(size_t)t * D + c + j] = from_f32<TA>(pair_weight != nullptr ? acc[j] : acc[j] * weight);
        }
        return;
    }
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; k++) {
            const int p = t * top + k;
            if (pair_expert[p] < 0) continue;
            const float v = o[(size_t)(row_of_pair != nullptr ? row_of_pair[p] : p) * D + c];
            acc = pair_weight != nullptr ? fmaf(pair_weight[p], v, acc) : acc + v;
        }
        out[(size_t)t * D + c] = from_f32<TA>(pair_weight != nullptr ? acc : acc * weight);
    }
}

// eight consecutive values (16-byte aligned for bfloat16, 32 for float) as fp32
__device__ __forceinline__ void load8_f32(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8_f32(const bf16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// The learned router: one CTA a token; a warp an expert's logit at a time, then one thread picks.
constexpr int ROUTER_THREADS = 128;
template <typename TA>
__global__ void __launch_bounds__(ROUTER_THREADS)
moe_router_kernel(const TA* __restrict__ h, const TA* __restrict__ w, VecRef bias, const int* __restrict__ tok_seq,
                  int* __restrict__ choice, float* __restrict__ pair_weight, int D, int E, int top) {
    __shared__ float z[MOE_MAX_EXPERTS];
    griddep_wait();
    const int t = blockIdx.x;
    if (tok_seq[t] < 0) {
        for (int k = threadIdx.x; k < top; k += blockDim.x) {
            choice[t * top + k] = -1;
            pair_weight[t * top + k] = 0.f;
        }
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TA* x = h + (size_t)t * D;
    // rows of a multiple of 8 values go 8 values a lane and load (16 or 32 bytes), four experts of a warp in flight
    const int D8 = D % 8 == 0 ? D : 0;
    for (int e = warp; e < E; e += ROUTER_THREADS / 32) {
        const TA* wr = w + (size_t)e * D;
        float acc = 0.f;
#pragma unroll 2
        for (int d = lane * 8; d < D8; d += 256) {
            float xv[8], wv[8];
            load8_f32(x + d, xv);
            load8_f32(wr + d, wv);
#pragma unroll
            for (int i = 0; i < 8; i++) acc = fmaf(xv[i], wv[i], acc);
        }
        for (int d = D8 + lane; d < D; d += 32) acc = fmaf(to_f32(x[d]), to_f32(wr[d]), acc);
        acc = warp_sum(acc);
        if (lane == 0) z[e] = acc + bias.at(e);
    }
    __syncthreads();
    if (warp != 0) return;
    // the largest logit `top` times over; lanes scan strided slices, the lower index wins a tie
    float zmax = 0.f, sum = 0.f;
    for (int k = 0; k < top; k++) {
        float best = -INFINITY;
        int at = E;
        for (int e = lane; e < E; e += 32)
            if (z[e] > best) { best = z[e]; at = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (k == 0) zmax = best;
        const float w_k = expf(best - zmax);
        sum += w_k;
        if (lane == 0) {
            choice[t * top + k] = at < E ? at : -1;
            pair_weight[t * top + k] = w_k;
            if (at < E) z[at] = -INFINITY;
        }
        __syncwarp();
    }
    const float inv = 1.0f / sum;
    for (int k = lane; k < top; k += 32) pair_weight[t * top + k] *= inv;
}

// The group-limited scored router: one CTA a token; a warp an expert's logit at a time, then warp 0 picks.
template <typename TA>
__global__ void __launch_bounds__(ROUTER_THREADS)
moe_group_router_kernel(const TA* __restrict__ h, const TA* __restrict__ w, VecRef correction, const int* __restrict__ tok_seq,
                        int* __restrict__ choice, float* __restrict__ pair_weight, int D, int E, int top, int groups, int keep,
                        float weight_scale) {
    __shared__ float sc[MOE_MAX_EXPERTS], ch[MOE_MAX_EXPERTS], gs[MOE_MAX_EXPERTS];
    griddep_wait();
    const int t = blockIdx.x;
    if (tok_seq[t] < 0) {
        for (int k = threadIdx.x; k < top; k += blockDim.x) {
            choice[t * top + k] = -1;
            pair_weight[t * top + k] = 0.f;
        }
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TA* x = h + (size_t)t * D;
    const int D8 = D % 8 == 0 ? D : 0;
    for (int e = warp; e < E; e += ROUTER_THREADS / 32) {
        const TA* wr = w + (size_t)e * D;
        float acc = 0.f;
#pragma unroll 2
        for (int d = lane * 8; d < D8; d += 256) {
            float xv[8], wv[8];
            load8_f32(x + d, xv);
            load8_f32(wr + d, wv);
#pragma unroll
            for (int i = 0; i < 8; i++) acc = fmaf(xv[i], wv[i], acc);
        }
        for (int d = D8 + lane; d < D; d += 32) acc = fmaf(to_f32(x[d]), to_f32(wr[d]), acc);
        acc = warp_sum(acc);
        if (lane == 0) {
            const float s = 1.0f / (1.0f + expf(-acc));
            sc[e] = s;
            ch[e] = s + correction.at(e);
        }
    }
    __syncthreads();
    if (warp != 0) return;
    if (keep < groups) {
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float m1 = -INFINITY, m2 = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; e++) {
                const float v = ch[e];
                if (v > m1) { m2 = m1; m1 = v; }
                else if (v > m2) m2 = v;
            }
            gs[g] = per > 1 ? m1 + m2 : m1;
        }
        __syncwarp();
        // the best `keep` groups are marked by +inf in gs; the others' experts leave the choice
        for (int k = 0; k < keep; k++) {
            float best = -INFINITY;
            int at = groups;
            for (int g = lane; g < groups; g += 32)
                if (gs[g] != INFINITY && gs[g] > best) { best = gs[g]; at = g; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
            }
            if (lane == 0 && at < groups) gs[at] = INFINITY;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] != INFINITY) ch[e] = -INFINITY;
        __syncwarp();
    }
    for (int k = 0; k < top; k++) {
        float best = -INFINITY;
        int at = E;
        for (int e = lane; e < E; e += 32)
            if (ch[e] > best) { best = ch[e]; at = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (lane == 0) {
            choice[t * top + k] = at < E ? at : -1;
            pair_weight[t * top + k] = at < E ? sc[at] * weight_scale : 0.f;
            if (at < E) ch[at] = -INFINITY;
        }
        __syncwarp();
    }
}

// ---- the bfloat16 products on tensor cores (the core is in tile_mma.cuh) ----
// A row's bits do not depend on whether the step was a prompt (64-row tiles) or a decode step (16-row tiles).
constexpr int MMA_WARPS = 8;

// grid (tiles, ceil(F / (8 warps * 8 NT columns))). A warp takes 8 NT columns of the gate and the same of the up matrix.
// Decode steps (16-row tiles, mostly one row) take narrow warps, so that many CTAs stream the weights.
template <int MT, int NT, int ACT>
__global__ void __launch_bounds__(MMA_WARPS * 32, 2)
moe_gate_up_mma_kernel(const bf16* __restrict__ h, const bf16* __restrict__ w_gu, bf16* __restrict__ y,
                       const int* __restrict__ perm, const int* __restrict__ tiles, MoeArgs a) {
    __shared__ __align__(16) bf16 xs[16 * MT][tilemma::MMA_LDS];
    __shared__ int pair_s[16 * MT];
    griddep_wait();
    if ((int)blockIdx.x >= tiles[0]) return;
    const int e = tiles[1 + 3 * blockIdx.x], r0 = tiles[2 + 3 * blockIdx.x], nr = tiles[3 + 3 * blockIdx.x];
    for (int i = threadIdx.x; i < 16 * MT; i += blockDim.x) pair_s[i] = i < nr ? perm[r0 + i] : -1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int c0 = (blockIdx.y * MMA_WARPS + warp) * (8 * NT);
    constexpr int NMAT = ACT == MOE_ACT_CLAMPED_GATE ? 2 : 1;     // matrices an expert: gate and up, or up alone
    const bf16* wrow[NMAT][NT];
#pragma unroll
    for (int j = 0; j < NT; j++) {
        const int c = min(c0 + j * 8 + g, a.F - 1);               // columns beyond F read the last row and are not stored
        wrow[0][j] = w_gu + ((size_t)e * NMAT * a.F + c) * a.D;
        if (NMAT == 2) wrow[NMAT - 1][j] = wrow[0][j] + (size_t)a.F * a.D;
    }
    float acc[NMAT][MT][NT][4];
    tilemma::mma_tile<MT, NT, NMAT>(xs, pair_s, h, (size_t)a.D, a.top, wrow, a.D, acc);
#pragma unroll
    for (int m = 0; m < MT; m++)
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int p = pair_s[m * 16 + g + 8 * half];
            if (p < 0) continue;
#pragma unroll
            for (int j = 0; j < NT; j++)
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    const int c = c0 + j * 8 + 2 * t + q;
                    if (c >= a.F) continue;
                    if (ACT == MOE_ACT_GELU) {
                        y[(size_t)p * a.F + c] = from_f32<bf16>(gelu_erf_f(round_to<bf16>(acc[0][m][j][2 * half + q])));
                        continue;
                    }
                    const float gv = fminf(round_to<bf16>(acc[0][m][j][2 * half + q]), a.limit);
                    const float uv = fminf(fmaxf(round_to<bf16>(acc[NMAT - 1][m][j][2 * half + q]), -a.limit), a.limit);
                    y[(size_t)p * a.F + c] = from_f32<bf16>(gv * (1.0f / (1.0f + expf(-a.alpha * gv))) * (uv + 1.0f));
                }
        }
}

// grid (tiles, ceil(D / (8 warps * 8 NT columns)))
template <int MT, int NT>
__global__ void __launch_bounds__(MMA_WARPS * 32, 2)
moe_down_mma_kernel(const bf16* __restrict__ y, const bf16* __restrict__ w_down, float* __restrict__ o,
                    const int* __restrict__ perm, const int* __restrict__ tiles, MoeArgs a) {
    __shared__ __align__(16) bf16 xs[16 * MT][tilemma::MMA_LDS];
    __shared__ int pair_s[16 * MT];
    griddep_wait();
    if ((int)blockIdx.x >= tiles[0]) return;
    const int e = tiles[1 + 3 * blockIdx.x], r0 = tiles[2 + 3 * blockIdx.x], nr = tiles[3 + 3 * blockIdx.x];
    for (int i = threadIdx.x; i < 16 * MT; i += blockDim.x) pair_s[i] = i < nr ? perm[r0 + i] : -1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int c0 = (blockIdx.y * MMA_WARPS + warp) * (8 * NT);
    const bf16* wrow[1][NT];
#pragma unroll
    for (int j = 0; j < NT; j++) wrow[0][j] = w_down + ((size_t)e * a.D + min(c0 + j * 8 + g, a.D - 1)) * a.F;
    float acc[1][MT][NT][4];
    tilemma::mma_tile<MT, NT, 1>(xs, pair_s, y, (size_t)a.F, 1, wrow, a.F, acc);
#pragma unroll
    for (int m = 0; m < MT; m++)
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int p = pair_s[m * 16 + g + 8 * half];
            if (p < 0) continue;
#pragma unroll
            for (int j = 0; j < NT; j++)
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    const int c = c0 + j * 8 + 2 * t + q;
                    if (c < a.D) o[(size_t)p * a.D + c] = acc[0][m][j][2 * half + q];
                }
        }
}

template <int MT, int ACT>
int launch_products_mma(const void* h, const void* w_gu, const void* w_down, void* y, float* o, const int* perm,
                        const int* tiles, int max_tiles, const MoeArgs& a, cudaStream_t stream) {
    constexpr int NT_GU = MT == 1 ? 1 : 2, NT_DOWN = MT == 1 ? 1 : 4;
    mynah_launch(moe_gate_up_mma_kernel<MT, NT_GU, ACT>, dim3(max_tiles, ceil_div(a.F, MMA_WARPS * 8 * NT_GU)), dim3(MMA_WARPS * 32), 0, stream,
                 (const bf16*)h, (const bf16*)w_gu, (bf16*)y, perm, tiles, a);
    if (mynah_check_launch("moe_gate_up") != 0) return -1;
    mynah_launch(moe_down_mma_kernel<MT, NT_DOWN>, dim3(max_tiles, ceil_div(a.D, MMA_WARPS * 8 * NT_DOWN)), dim3(MMA_WARPS * 32), 0, stream,
                 (const bf16*)y, (const bf16*)w_down, o, perm, tiles, a);
    return mynah_check_launch("moe_down");
}

// ---- prompts in bfloat16: the products as ONE grouped tcgen05 product each (gemm_tcgen05.cu) ----
// The pairs are sorted by expert with every expert's rows padded to whole tiles of 128 (rows that hold no pair are
// zeros), the token rows are gathered into that order, and the library's tensor-core kernel multiplies row tile m by the
// matrix of tile_group[m]: the gate/up product with the clamped gate in its epilogue, then the down product.
constexpr int GROUP_TILE = 128;

__global__ void __launch_bounds__(MOE_ROUTE_THREADS)
moe_route_padded_kernel(const int* __restrict__ tokens, const int* __restrict__ tok_seq, const int* __restrict__ table,
                        const int* __restrict__ choice, int T, int V, int top, int E, int m_pad, int* __restrict__ pair_expert, int* __restrict__ row_of_pair,
                        int* __restrict__ perm_pad, int* __restrict__ tile_group, int* __restrict__ status) {
    __shared__ int count[MOE_MAX_EXPERTS], start[MOE_MAX_EXPERTS];
    griddep_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    for (int r = threadIdx.x; r < m_pad; r += blockDim.x) perm_pad[r] = -1;
    __syncthreads();
    const int P = T * top;
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int t = p / top;
        int e = -1;
        if (tok_seq[t] >= 0) {
            if (choice != nullptr) {
                e = choice[p];                                    // a router picked it
            } else {
                const int tok = tokens[t];
                if (tok >= 0 && tok < V) e = table[(size_t)tok * top + p % top];
            }
            if (e < 0 || e >= E) {
                atomicOr(status, MYNAH_ST_TOKEN_RANGE);
                e = -1;
            }
        }
        pair_expert[p] = e;
        if (e >= 0) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        const int n_tiles = m_pad / GROUP_TILE;
        for (int e = 0; e < E; e++) {
            start[e] = at;
            for (int r = 0; r < count[e]; r += GROUP_TILE, at += GROUP_TILE)
                if (at / GROUP_TILE < n_tiles) tile_group[at / GROUP_TILE] = e;
        }
        for (int tile = at / GROUP_TILE; tile < n_tiles; tile++) tile_group[tile] = 0;      // tiles of zeros: any matrix
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = pair_expert[p];
        if (e < 0) continue;
        const int row = start[e] + atomicAdd(&count[e], 1);
        if (row < m_pad) {
            perm_pad[row] = p;
            row_of_pair[p] = row;
        }
    }
}

// a[r, :] = h[perm_pad[r] / top, :], zeros for the rows that hold no pair; 16 bytes a thread
__global__ void moe_gather_kernel(const bf16* __restrict__ h, const int* __restrict__ perm_pad, bf16* __restrict__ a, int top, int D) {
    griddep_wait();
    const int r = blockIdx.x, p = perm_pad[r];
    const uint4* src = p >= 0 ? reinterpret_cast<const uint4*>(h + (size_t)(p / top) * D) : nullptr;
    uint4* dst = reinterpret_cast<uint4*>(a + (size_t)r * D);
    for (int i = threadIdx.x; i < D / 8; i += blockDim.x) dst[i] = src != nullptr ? src[i] : make_uint4(0u, 0u, 0u, 0u);
}

template <typename TA, int BM, int ACT>
int launch_products(const void* h, const void* w_gu, const void* w_down, void* y, float* o, const int* perm,
                    const int* tiles, int max_tiles, const MoeArgs& a, cudaStream_t stream) {
    mynah_launch(moe_gate_up_kernel<TA, BM, ACT>, dim3(max_tiles, ceil_div(a.F, 64)), dim3(tilemm::THREADS), 0, stream,
                 (const TA*)h, (const TA*)w_gu, (TA*)y, perm, tiles, a);
    if (mynah_check_launch("moe_gate_up") != 0) return -1;
    mynah_launch(moe_down_kernel<TA, BM>, dim3(max_tiles, ceil_div(a.D, 64)), dim3(tilemm::THREADS), 0, stream,
                 (const TA*)y, (const TA*)w_down, o, perm, tiles, a);
    return mynah_check_launch("moe_down");
}

}  // namespace

// 1: the bfloat16 products run on the plain tiled kernels too (the tests compare the two).
static int g_moe_plain = 0;
MYNAH_API int mynah_moe_plain(int on) {
    const int before = g_moe_plain;
    g_moe_plain = on;
    return before;
}

// From how many (token, choice) pairs a bfloat16 step's products run as grouped tcgen05 products (0: never).
static int g_moe_grouped_min = 1024;
MYNAH_API int mynah_moe_grouped_min(int n) {
    const int before = g_moe_grouped_min;
    g_moe_grouped_min = n;
    return before;
}

extern "C" int mynah_gemm_tcgen05_grouped(const void* A, const void* W, void* C, int M, int N, int K, int ldc, int epilogue, int groups,
                               int group_rows, const int* tile_group, float gate_limit, float gate_alpha, int sm_count,
                               int* status, cudaStream_t stream);

// Rows of the sorted, padded layout of a step whose products run grouped; 0: the step runs tile by tile instead.
MYNAH_API int mynah_moe_grouped_rows(int T, int top, int E, int D, int F, int dtype) {
    const long long P = (long long)T * top;
    if (dtype != MYNAH_BF16 || g_moe_plain || g_moe_grouped_min <= 0 || P < g_moe_grouped_min || D % 8 || F % 8) return 0;
    return (int)((P + (long long)E * (GROUP_TILE - 1) + GROUP_TILE - 1) / GROUP_TILE * GROUP_TILE);
}

// Rows of a tile for a step of T tokens: small steps (decode) take 16-row tiles, prompts 64-row tiles.
MYNAH_API int mynah_moe_tile_rows(int T, int top) { return (long long)T * top <= 256 ? 16 : 64; }

// Most tiles a step of T tokens can have.
MYNAH_API int mynah_moe_max_tiles(int T, int top, int E) { return ceil_div(T * top, mynah_moe_tile_rows(T, top)) + E; }

// Both forms of the feed-forward. choice null: the table picks and every pair counts `weight`; else choice [T*top]
// (a router's picks) and pair_weight [T*top]. act: MOE_ACT_*; out_f32: the result leaves as fp32 rows.
static int moe_run(const void* h, int dtype, const int* tokens, const int* tok_seq, const int* table, const int* choice,
                   const float* pair_weight, const void* w_gu, const void* w_down, void* out, int out_f32, void* y, float* o,
                   int* ints, void* a_sorted, int T, int V, int top, int E, int D, int F, int act, float limit, float alpha,
                   float weight, int* status, cudaStream_t stream) {
    const int P = T * top, BM = mynah_moe_tile_rows(T, top), max_tiles = mynah_moe_max_tiles(T, top, E);
    int* pair_expert = ints;
    int* perm = ints + P;
    int* tiles = ints + 2 * P;
    const int threads = D >= 1024 ? 256 : 128;
    const int m_pad = mynah_moe_grouped_rows(T, top, E, D, F, dtype);
    if (m_pad > 0 && a_sorted != nullptr &&
        (((uintptr_t)h | (uintptr_t)w_gu | (uintptr_t)w_down | (uintptr_t)y | (uintptr_t)a_sorted | (uintptr_t)o) & 15) == 0) {
        int* perm_pad = ints + 2 * P + 1 + 3 * max_tiles;
        int* tile_group = perm_pad + m_pad;
        mynah_launch(moe_route_padded_kernel, dim3(1), dim3(MOE_ROUTE_THREADS), 0, stream, tokens, tok_seq, table, choice, T, V, top, E, m_pad,
                     pair_expert, perm, perm_pad, tile_group, status);
        if (mynah_check_launch("moe_route") != 0) return -1;
        mynah_launch(moe_gather_kernel, dim3(m_pad), dim3(128), 0, stream, (const bf16*)h, (const int*)perm_pad, (bf16*)a_sorted, top, D);
        if (mynah_check_launch("moe_gather") != 0) return -1;
        if (act == MOE_ACT_GELU) {
            if (mynah_gemm_tcgen05_grouped(a_sorted, w_gu, y, m_pad, F, D, F, 5, E, F, tile_group, 0.f, 0.f, 0, status, stream) != 0) return -1;
        } else {
            if (mynah_gemm_tcgen05_grouped(a_sorted, w_gu, y, m_pad, F, D, F, 4, E, 2 * F, tile_group, limit, alpha, 0, status, stream) != 0) return -1;
        }
        if (mynah_gemm_tcgen05_grouped(y, w_down, o, m_pad, D, F, D, 1, E, D, tile_group, 0.f, 0.f, 0, status, stream) != 0) return -1;
        if (out_f32)
            mynah_launch(moe_combine_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)o, (const int*)pair_expert,
                         (const int*)perm, pair_weight, (float*)out, top, D, weight);
        else
            mynah_launch(moe_combine_kernel<bf16>, dim3(T), dim3(threads), 0, stream, (const float*)o, (const int*)pair_expert,
                         (const int*)perm, pair_weight, (bf16*)out, top, D, weight);
        return mynah_check_launch("moe_combine");
    }
    mynah_launch(moe_route_kernel, dim3(1), dim3(MOE_ROUTE_THREADS), 0, stream, tokens, tok_seq, table, choice, T, V, top, E, BM,
                 pair_expert, perm, tiles, max_tiles, status);
    if (mynah_check_launch("moe_route") != 0) return -1;
    const MoeArgs a{top, D, F, limit, alpha};
    int rc;
    // bfloat16 rows that can move 16 bytes at a time take the tensor-core kernels
    const bool mma_ok = dtype == MYNAH_BF16 && D % 8 == 0 && F % 8 == 0 && !g_moe_plain &&
                        (((uintptr_t)h | (uintptr_t)w_gu | (uintptr_t)w_down | (uintptr_t)y) & 15) == 0;
#define MOE_GO(ACT_)                                                                                                   \
    if (mma_ok)                                                                                                        \
        rc = BM == 16 ? launch_products_mma<1, ACT_>(h, w_gu, w_down, y, o, perm, tiles, max_tiles, a, stream)         \
                      : launch_products_mma<4, ACT_>(h, w_gu, w_down, y, o, perm, tiles, max_tiles, a, stream);        \
    else if (dtype == MYNAH_F32)                                                                                       \
        rc = BM == 16 ? launch_products<float, 16, ACT_>(h, w_gu, w_down, y, o, perm, tiles, max_tiles, a, stream)     \
                      : launch_products<float, 64, ACT_>(h, w_gu, w_down, y, o, perm, tiles, max_tiles, a, stream);    \
    else                                                                                                               \
        rc = BM == 16 ? launch_products<bf16, 16, ACT_>(h, w_gu, w_down, y, o, perm, tiles, max_tiles, a, stream)      \
                      : launch_products<bf16, 64, ACT_>(h, w_gu, w_down, y, o, perm, tiles, max_tiles, a, stream)
    if (act == MOE_ACT_GELU) { MOE_GO(MOE_ACT_GELU); }
    else { MOE_GO(MOE_ACT_CLAMPED_GATE); }
#undef MOE_GO
    if (rc != 0) return rc;
    if (dtype == MYNAH_F32 || out_f32)
        mynah_launch(moe_combine_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)o, (const int*)pair_expert,
                     (const int*)nullptr, pair_weight, (float*)out, top, D, weight);
    else
        mynah_launch(moe_combine_kernel<bf16>, dim3(T), dim3(threads), 0, stream, (const float*)o, (const int*)pair_expert,
                     (const int*)nullptr, pair_weight, (bf16*)out, top, D, weight);
    return mynah_check_launch("moe_combine");
}

// The whole feed-forward with a table. h: [T][D]; table: int32 [V][top]; w_gu: [E][2][F][D]; w_down: [E][D][F]; out: [T][D] in the
// activation type. Scratch, with R = max(T*top, mynah_moe_grouped_rows(...)): y [R][F] (activation type), o fp32 [R][D],
// ints [2*T*top + 1 + 3*max_tiles + R + R/128], and, when the products run grouped, a [R][D] (activation type; else null).
MYNAH_API int mynah_moe_table_ffn(const void* h, int dtype, const int* tokens, const int* tok_seq, const int* table,
                                  const void* w_gu, const void* w_down, void* out, void* y, float* o, int* ints, void* a_sorted,
                                  int T, int V, int top, int E, int D, int F, float limit, float alpha, float weight,
                                  int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && V > 0 && top > 0 && E > 0 && D > 0 && F > 0, "moe_table_ffn: bad sizes");
    MYNAH_REQUIRE(E <= MOE_MAX_EXPERTS, "moe_table_ffn: %d experts exceed %d", E, MOE_MAX_EXPERTS);
    MYNAH_REQUIRE(dtype == MYNAH_F32 || dtype == MYNAH_BF16, "moe_table_ffn: unsupported dtype %d", dtype);
    return moe_run(h, dtype, tokens, tok_seq, table, nullptr, nullptr, w_gu, w_down, out, 0, y, o, ints, a_sorted, T, V, top, E,
                   D, F, MOE_ACT_CLAMPED_GATE, limit, alpha, weight, status, stream);
}

// The feed-forward with a learned router: logits W_r h + b_r in fp32, the `top` largest, softmax over the chosen; experts
// y = gelu(W_up h) (erf form), out = W_down y. w_router [E][D] in dtype, b_router [E] in b_dtype; w_up [E][F][D];
// w_down [E][D][F]; out fp32 [T][D]. Scratch as above plus choice int [T*top] and pair_weight fp32 [T*top].
MYNAH_API int mynah_moe_router_ffn(const void* h, int dtype, const int* tok_seq, const void* w_router, const void* b_router,
                                   int b_dtype, const void* w_up, const void* w_down, float* out, void* y, float* o, int* ints,
                                   void* a_sorted, int* choice, float* pair_weight, int T, int top, int E, int D, int F,
                                   int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && top > 0 && E > 0 && top <= E && D > 0 && F > 0, "moe_router_ffn: bad sizes");
    MYNAH_REQUIRE(E <= MOE_MAX_EXPERTS, "moe_router_ffn: %d experts exceed %d", E, MOE_MAX_EXPERTS);
    const VecRef bias{b_router, b_dtype};
    if (dtype == MYNAH_F32)
        mynah_launch(moe_router_kernel<float>, dim3(T), dim3(ROUTER_THREADS), 0, stream, (const float*)h, (const float*)w_router, bias,
                     tok_seq, choice, pair_weight, D, E, top);
    else if (dtype == MYNAH_BF16)
        mynah_launch(moe_router_kernel<bf16>, dim3(T), dim3(ROUTER_THREADS), 0, stream, (const bf16*)h, (const bf16*)w_router, bias,
                     tok_seq, choice, pair_weight, D, E, top);
    else
        return mynah_fail("moe_router_ffn: unsupported dtype %d", dtype);
    if (mynah_check_launch("moe_router") != 0) return -1;
    return moe_run(h, dtype, nullptr, tok_seq, nullptr, choice, pair_weight, w_up, w_down, out, 1, y, o, ints, a_sorted, T, 1, top,
                   E, D, F, MOE_ACT_GELU, 0.f, 0.f, 1.0f, status, stream);
}

// The feed-forward with the group-limited scored router and the clamped-gate experts: scores sigmoid(W_r h) in fp32, the
// choice by score + correction inside the `keep` best of `groups` equal groups of neighbouring experts, weights score *
// weight_scale (not renormalised). w_router [E][D] in dtype, correction [E] in c_dtype; w_gu [E][2][F][D]; w_down [E][D][F];
// out [T][D] in the activation type, or fp32 when out_f32. Scratch as for the learned router.
MYNAH_API int mynah_moe_group_router_ffn(const void* h, int dtype, const int* tok_seq, const void* w_router, const void* correction,
                                         int c_dtype, const void* w_gu, const void* w_down, void* out, int out_f32, void* y, float* o,
                                         int* ints, void* a_sorted, int* choice, float* pair_weight, int T, int top, int E, int D,
                                         int F, int groups, int keep, float weight_scale, float limit, float alpha, int* status,
                                         cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && top > 0 && E > 0 && top <= E && D > 0 && F > 0, "moe_group_router_ffn: bad sizes");
    MYNAH_REQUIRE(E <= MOE_MAX_EXPERTS, "moe_group_router_ffn: %d experts exceed %d", E, MOE_MAX_EXPERTS);
    MYNAH_REQUIRE(groups >= 1 && E % groups == 0 && keep >= 1 && keep <= groups, "moe_group_router_ffn: %d experts do not form %d groups of which %d are kept", E, groups, keep);
    MYNAH_REQUIRE(top <= keep * (E / groups), "moe_group_router_ffn: %d experts a token exceed those of %d kept groups", top, keep);
    const VecRef corr{correction, c_dtype};
    if (dtype == MYNAH_F32)
        mynah_launch(moe_group_router_kernel<float>, dim3(T), dim3(ROUTER_THREADS), 0, stream, (const float*)h, (const float*)w_router,
                     corr, tok_seq, choice, pair_weight, D, E, top, groups, keep, weight_scale);
    else if (dtype == MYNAH_BF16)
        mynah_launch(moe_group_router_kernel<bf16>, dim3(T), dim3(ROUTER_THREADS), 0, stream, (const bf16*)h, (const bf16*)w_router,
                     corr, tok_seq, choice, pair_weight, D, E, top, groups, keep, weight_scale);
    else
        return mynah_fail("moe_group_router_ffn: unsupported dtype %d", dtype);
    if (mynah_check_launch("moe_group_router") != 0) return -1;
    return moe_run(h, dtype, nullptr, tok_seq, nullptr, choice, pair_weight, w_gu, w_down, out, out_f32, y, o, ints, a_sorted, T, 1,
                   top, E, D, F, MOE_ACT_CLAMPED_GATE, limit, alpha, 1.0f, status, stream);
}
