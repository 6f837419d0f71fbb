// The sink attention with mixed heads (see sink_attn.cu for the equations) on tensor cores, bfloat16 activations and
// cache, head sizes 64 and 128. The weights of a key are mixed over all heads, so no head can be computed alone. Since
// the mixing is linear, the softmax is first finished per head and the rest is one pass over the keys:
//
//   sink_lse_tc     per query and head, the maximum and the sum of the denominator of the scaled scores: online over
//                   the visible keys, 64 queries of one head a CTA (mma.sync m16n8k16), a decode step's pages in
//                   shares; the mix kernel folds the shares and the sink into log2 of the denominator.
//   sink_mix_tc     a CTA takes 16 consecutive queries of a sequence, ALL score heads, up to 16 output heads, and a
//                   share of the key tiles (32 keys a tile). Per tile: for every kv head, its K tile and the queries
//                   of its heads stream through shared memory (several stages in flight); the warps form the scores and write
//                   w_g = exp2(s_g - lse_g) (fp32, zero where masked) to shared memory. Then every warp takes two
//                   output heads: it mixes the weights of all heads (fp32, m_h = sum_g talk[h, g] w_g) straight into
//                   the A fragments of the product with V, split in two bfloat16 terms (m = hi + lo, so that the
//                   weights keep 16 bits of mantissa), against the V tiles of all kv heads that lie in shared memory.
//   sink_finish     with more than one share of keys: adds the shares' partial sums (fp32) in their order and turns
//                   the sum back by the query's position. With one share the mix kernel does that itself.
//
// Sums over keys run in ascending tiles whatever else is in the step; a query's result depends on its tile of 16
// only through rounding-free zeros (masked weights are exactly zero).
#include "layout.cuh"
#include "mma_frag.cuh"

namespace {

constexpr int LQT = 64;               // queries per CTA of the lse kernel
constexpr int LKT = PAGE_TOKENS;      // its key tile: one page
constexpr int MROWS = 16;             // queries per CTA of the mix kernel
constexpr int MKEYS = 32;             // its key tile
constexpr int MWARPS = 8;
constexpr int MHO = 2 * MWARPS;       // output heads per CTA
constexpr int MSTAGES_MAX = 8;        // stages of (K tile, queries) in flight, at most
constexpr int PS_LD = MKEYS + 8;      // row stride of the weights in shared memory (floats)
static_assert(PAGE_TOKENS % MKEYS == 0, "a key tile lies inside a page");

using namespace mmafrag;
// waits until at most n of the newest groups are in flight (n below MSTAGES_MAX)
__device__ __forceinline__ void cp_async_wait_upto(int n) {
    switch (n) {
        case 0: cp_async_wait<0>(); break;
        case 1: cp_async_wait<1>(); break;
        case 2: cp_async_wait<2>(); break;
        case 3: cp_async_wait<3>(); break;
        case 4: cp_async_wait<4>(); break;
        case 5: cp_async_wait<5>(); break;
        default: cp_async_wait<6>(); break;
    }
}
// m = hi + lo in two bfloat16 terms: hi is m cut off behind bfloat16's bits (a bit pattern, no rounding), lo the exact
// remainder rounded to bfloat16, so hi + lo keeps 16 bits of m
__device__ __forceinline__ void split_bf16(float m0, float m1, uint32_t& hi, uint32_t& lo) {
    const uint32_t b0 = __float_as_uint(m0), b1 = __float_as_uint(m1);
    hi = __byte_perm(b0, b1, 0x7632);
    lo = pack_bf16(m0 - __uint_as_float(b0 & 0xffff0000u), m1 - __uint_as_float(b1 & 0xffff0000u));
}

struct SinkTcArgs {
    int B, H, G, T, window, splits, interleaved, n_pos_v, stages, cg;
    float scale_log2;                 // the score's scale times log2(e)
};

// ---------------------------------------------------------------------------------------------------------------
// Each head's maximum m and sum_j 2^(scale_log2 q.k_j - m) over one share (blockIdx.z) of the pages a query tile sees:
// stats[share, row, h] = (m, sum). The mix kernel folds the shares in their order and adds the sink.
template <int HD>
__global__ void __launch_bounds__(128)
sink_lse_tc_kernel(const bf16* __restrict__ q, float2* __restrict__ stats, const bf16* __restrict__ k_cache,
                   const int* __restrict__ cu_q, const int* __restrict__ kv_len, PageTable pt, SinkTcArgs a,
                   int* __restrict__ status) {
    constexpr int CH = HD / 8, KSTEPS = HD / 16, NT_S = LKT / 8;
    constexpr int TILE_BYTES = LKT * HD * 2;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* q_s = smem;                                  // [LQT][HD]
    unsigned char* k_s = smem + LQT * HD * 2;                   // 2 stages of a K tile
    griddep_wait();
    int b, tile;
    if (!find_query_tile(cu_q, a.B, LQT, blockIdx.x, b, tile)) return;
    const int h = blockIdx.y;
    const int q0 = cu_q[b], q_len = cu_q[b + 1] - q0;
    const int tile0 = tile * LQT;
    const int n_kv = kv_len[b];
    const int past = n_kv - q_len;
    const int nq = min(LQT, q_len - tile0);
    const int kvh = h / (a.H / a.G);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int p_first = past + tile0, p_last = p_first + nq - 1;
    const int k_lo = a.window > 0 ? max(0, p_first - a.window + 1) : 0;
    const int pg_lo = k_lo / LKT, pg_hi = p_last / LKT;
    const int pg_per = (pg_hi - pg_lo + 1 + a.splits - 1) / a.splits;
    const int pg_first = pg_lo + (int)blockIdx.z * pg_per, pg_last = min(pg_hi, pg_first + pg_per - 1);
    const size_t ldq = (size_t)a.H * HD;
    float2* st = stats + ((size_t)blockIdx.z * a.T + q0 + tile0) * a.H + h;
    if (pg_first > pg_last) {                                    // a share without pages
        for (int r = tid; r < nq; r += blockDim.x) st[(size_t)r * a.H] = make_float2(-INFINITY, 0.f);
        return;
    }

    const uint32_t q_base = smem_u32(q_s);
    for (int i = tid; i < LQT * CH; i += blockDim.x) {
        const int r = i / CH, c = i % CH;
        cp_async_16(q_base + swz<CH>(r, c), q + (size_t)(q0 + tile0 + (r < nq ? r : 0)) * ldq + (size_t)h * HD + c * 8, r < nq);
    }
    cp_async_commit();
    bool bad = false;
    auto load_tile = [&](int pg, int stage) {
        const int page = page_of(pt, b, pg * LKT);
        if (page < 0) bad = true;
        const size_t base = ((size_t)(page < 0 ? 0 : page) * a.G + kvh) * LKT * HD;
        const int rows = page < 0 ? 0 : min(LKT, n_kv - pg * LKT);
        const uint32_t kb = smem_u32(k_s + stage * TILE_BYTES);
        for (int i = tid; i < LKT * CH; i += blockDim.x) {
            const int r = i / CH, c = i % CH;
            cp_async_16(kb + swz<CH>(r, c), k_cache + base + (size_t)r * HD + c * 8, r < rows);
        }
        cp_async_commit();
    };
    load_tile(pg_first, 0);
    cp_async_wait<1>();
    __syncthreads();
    uint32_t qa[KSTEPS][4];
    const int mat = lane >> 3, rr = lane & 7;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ks++)
        ldmatrix_x4(qa[ks], q_base + swz<CH>(warp * 16 + (mat & 1) * 8 + rr, ks * 2 + (mat >> 1)));

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int pos_r[2] = {p_first + warp * 16 + g, p_first + warp * 16 + g + 8};
    for (int pg = pg_first; pg <= pg_last; pg++) {
        const int stage = (pg - pg_first) & 1;
        if (pg + 1 <= pg_last) {
            load_tile(pg + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t kb = smem_u32(k_s + stage * TILE_BYTES);
        float s[NT_S][4];
#pragma unroll
        for (int i = 0; i < NT_S; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
#pragma unroll
            for (int j = 0; j < NT_S / 2; j++) {
                uint32_t kf[4];
                ldmatrix_x4(kf, kb + swz<CH>(j * 16 + (mat >> 1) * 8 + rr, ks * 2 + (mat & 1)));
                mma_bf16(s[2 * j], qa[ks], kf[0], kf[1]);
                mma_bf16(s[2 * j + 1], qa[ks], kf[2], kf[3]);
            }
        }
        const int key0 = pg * LKT;
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int i = 0; i < NT_S; i++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int key = key0 + i * 8 + t * 2 + (e & 1), p = pos_r[e >> 1];
                bool vis = key <= p && key < n_kv;
                if (a.window > 0) vis = vis && key > p - a.window;
                const float v = vis ? s[i][e] * a.scale_log2 : -INFINITY;
                s[i][e] = v;
                m_new[e >> 1] = fmaxf(m_new[e >> 1], v);
            }
        }
#pragma unroll
        for (int j = 0; j < 2; j++) {
            m_new[j] = fmaxf(m_new[j], __shfl_xor_sync(0xffffffffu, m_new[j], 1));
            m_new[j] = fmaxf(m_new[j], __shfl_xor_sync(0xffffffffu, m_new[j], 2));
            const float alpha = m_new[j] == -INFINITY ? 1.f : exp2f(m_run[j] - m_new[j]);
            const float mm = m_new[j] == -INFINITY ? 0.f : m_new[j];
            float add = 0.f;
#pragma unroll
            for (int i = 0; i < NT_S; i++) add += exp2f(s[i][2 * j] - mm) + exp2f(s[i][2 * j + 1] - mm);
            l_run[j] = l_run[j] * alpha + add;
            m_run[j] = m_new[j];
        }
        __syncthreads();
    }
    if (bad && tid == 0) atomicOr(status, MYNAH_ST_PAGE_RANGE);
#pragma unroll
    for (int j = 0; j < 2; j++) {
        float l = l_run[j];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int r = warp * 16 + g + 8 * j;
        if (r >= nq || t != 0) continue;
        st[(size_t)r * a.H] = make_float2(m_run[j], l);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Shared memory of the mix kernel: V tiles of all kv heads, the weights of all heads, `stages` stages of (K tile of one
// kv head, queries of its heads), this CTA's rows of talk, the queries' lse2. A step's compute is short beside the
// latency of its loads, so as many stages are in flight as fit (at most as many as kv heads, two at least: a tile's
// V travels with the stage that is asked for at the tile's first step and must have landed by its last).
// A stage holds `cg` kv heads (two where that leaves room for three stages: half as many steps and barriers a tile, and
// two independent products a warp and step).
__host__ __device__ inline size_t mix_stage_bytes(int rep, int HD, int cg) { return (size_t)cg * (MKEYS + rep * MROWS) * HD * 2; }
__host__ __device__ inline size_t mix_smem_bytes(int H, int G, int HD, int VD, int stages, int cg) {
    return (size_t)G * MKEYS * VD * 2 + (size_t)H * MROWS * PS_LD * 4 + stages * mix_stage_bytes(H / G, HD, cg) + (size_t)MHO * H * 4 +
           (size_t)H * MROWS * 4;
}
inline int mix_heads_a_stage(int H, int G, int HD, int VD) {
    return G % 2 == 0 && mix_smem_bytes(H, G, HD, VD, 3, 2) <= 227 * 1024 ? 2 : 1;
}
inline int mix_stages(int H, int G, int HD, int VD, int cg) {
    int st = 2;
    while (st < MSTAGES_MAX && st < G / cg && mix_smem_bytes(H, G, HD, VD, st + 1, cg) <= 227 * 1024) st++;
    return st;
}

template <int HD, int VD>
__global__ void __launch_bounds__(MWARPS * 32, 1)
sink_mix_tc_kernel(const bf16* __restrict__ q, bf16* __restrict__ out, float* __restrict__ part,
                   const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, const float2* __restrict__ stats,
                   VecRef talk, VecRef sink, const float* __restrict__ cos_v, const float* __restrict__ sin_v,
                   const int* __restrict__ cu_q, const int* __restrict__ kv_len, PageTable pt, SinkTcArgs a,
                   int* __restrict__ status) {
    constexpr int CH = HD / 8, CHV = VD / 8, KSTEPS = HD / 16, NT_O = VD / 8;
    extern __shared__ __align__(128) unsigned char smem[];
    const int H = a.H, G = a.G, rep = H / G;
    const int CG = a.cg, GS = G / CG;                     // kv heads a step, steps a tile
    const size_t stage_bytes = mix_stage_bytes(rep, HD, CG);
    unsigned char* v_s = smem;                                                        // [G][MKEYS][VD]
    float* p_s = reinterpret_cast<float*>(v_s + (size_t)G * MKEYS * VD * 2);          // [H][MROWS][PS_LD]
    unsigned char* st_s = reinterpret_cast<unsigned char*>(p_s + (size_t)H * MROWS * PS_LD);   // stages x (K [MKEYS][HD], Q [rep][MROWS][HD])
    const int NST = a.stages;
    float* talk_s = reinterpret_cast<float*>(st_s + NST * stage_bytes);               // [MHO][H]
    float* lse_s = talk_s + MHO * H;                                                  // [H][MROWS]
    griddep_wait();
    int b, tile;
    if (!find_query_tile(cu_q, a.B, MROWS, blockIdx.x, b, tile)) return;
    const int split = blockIdx.y, hb = blockIdx.z * MHO;
    const int q0 = cu_q[b], q_len = cu_q[b + 1] - q0;
    const int tile0 = tile * MROWS;
    const int n_kv = kv_len[b];
    const int past = n_kv - q_len;
    const int nq = min(MROWS, q_len - tile0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3, mat = lane >> 3, rr = lane & 7;
    const int p_first = past + tile0, p_last = p_first + nq - 1;
    const int k_lo = a.window > 0 ? max(0, p_first - a.window + 1) : 0;
    const int kt_first = k_lo / MKEYS, kt_last = p_last / MKEYS;
    const int per = (kt_last - kt_first + 1 + a.splits - 1) / a.splits;
    const int kt0 = kt_first + split * per;
    const int n_my = max(0, min(kt_last + 1, kt0 + per) - kt0);
    const size_t ldq = (size_t)H * HD;

    for (int i = tid; i < MHO * H; i += MWARPS * 32) {           // [warp][score head][its two output heads]
        const int ho = i / H, hg = i % H;
        talk_s[((ho >> 1) * H + hg) * 2 + (ho & 1)] = hb + ho < H ? talk.at((hb + ho) * H + hg) : 0.f;
    }
    // log2 of each head's denominator: the shares' (maximum, sum) folded in their order, then the sink
    for (int i = tid; i < H * MROWS; i += MWARPS * 32) {
        const int r = i % MROWS, hh = i / MROWS;
        float lse = 0.f;
        if (r < nq) {
            const float2* st = stats + (size_t)(q0 + tile0 + r) * H + hh;
            const float sk2 = sink.at(hh) * 1.4426950408889634f;
            float m = sk2;
            for (int z = 0; z < a.splits; z++) m = fmaxf(m, st[(size_t)z * a.T * H].x);
            float tot = 0.f;
            for (int z = 0; z < a.splits; z++) {
                const float2 v = st[(size_t)z * a.T * H];
                if (v.y > 0.f) tot += v.y * exp2f(v.x - m);
            }
            lse = m + log2f(tot + exp2f(sk2 - m));
        }
        lse_s[i] = lse;
    }

    bool bad = false;
    // K tiles of CG kv heads and the queries of their heads, for step s = (tile, group of kv heads)
    int looked_kt = -1, looked_page = -1;                        // a tile's page is looked up once, not once a step
    auto load_stage = [&](int s) {
        const int kt = kt0 + s / GS, c_first = (s % GS) * CG;
        const uint32_t kb = smem_u32(st_s + (s % NST) * stage_bytes), qb = kb + CG * MKEYS * HD * 2;
        const int key0 = kt * MKEYS;
        if (kt != looked_kt) {
            looked_page = page_of(pt, b, key0);
            looked_kt = kt;
        }
        const int page = looked_page;
        if (page < 0) bad = true;
        const int rows = page < 0 ? 0 : min(MKEYS, n_kv - key0);
        for (int i = tid; i < CG * MKEYS * CH; i += MWARPS * 32) {
            const int r = i / CH, ch = i % CH, j = r / MKEYS, kr = r % MKEYS;
            const size_t base = (((size_t)(page < 0 ? 0 : page) * G + c_first + j) * PAGE_TOKENS + key0 % PAGE_TOKENS + kr) * HD;
            cp_async_16(kb + swz<CH>(r, ch), k_cache + base + ch * 8, kr < rows);
        }
        for (int i = tid; i < CG * rep * MROWS * CH; i += MWARPS * 32) {
            const int r = i / CH, ch = i % CH, row = r % MROWS, hh = c_first * rep + r / MROWS;
            cp_async_16(qb + swz<CH>(r, ch), q + (size_t)(q0 + tile0 + (row < nq ? row : 0)) * ldq + (size_t)hh * HD + ch * 8, row < nq);
        }
    };
    auto load_values = [&](int kt) {
        const int key0 = kt * MKEYS;
        const int page = page_of(pt, b, key0);
        const int rows = page < 0 ? 0 : min(MKEYS, n_kv - key0);
        const uint32_t vb = smem_u32(v_s);
        for (int i = tid; i < G * MKEYS * CHV; i += MWARPS * 32) {
            const int r = i / CHV, ch = i % CHV, c = r / MKEYS, kr = r % MKEYS;
            const size_t base = (((size_t)(page < 0 ? 0 : page) * G + c) * PAGE_TOKENS + key0 % PAGE_TOKENS + kr) * VD;
            cp_async_16(vb + swz<CHV>(r, ch), v_cache + base + ch * 8, kr < rows);
        }
    };

    float o[2][NT_O][4];
#pragma unroll
    for (int hh = 0; hh < 2; hh++)
#pragma unroll
        for (int i = 0; i < NT_O; i++) o[hh][i][0] = o[hh][i][1] = o[hh][i][2] = o[hh][i][3] = 0.f;
    const int pos_a = p_first + g, pos_b = p_first + g + 8;
    const int n_steps = n_my * GS;
    // one group of copies a step: step s asks for stage s + NST - 1 (and, at a tile's first step, for the tile's V)
    for (int i = 0; i < NST - 1; i++) {
        if (i < n_steps) load_stage(i);
        cp_async_commit();
    }

    for (int s = 0; s < n_steps; s++) {
        const int kt = kt0 + s / GS, cgi = s % GS;
        cp_async_wait_upto(NST - 2);                             // stage s has landed
        __syncthreads();                                         // and everyone has left step s - 1: its stage, the weights
        if (cgi == 0) load_values(kt);                             // and (behind a tile) the V tiles may be written again
        if (s + NST - 1 < n_steps) load_stage(s + NST - 1);
        cp_async_commit();
        // ---- weights of the heads of these kv heads: a warp takes a head and 8 keys at a time
        const uint32_t kb = smem_u32(st_s + (s % NST) * stage_bytes), qb = kb + CG * MKEYS * HD * 2;
        const int key0 = kt * MKEYS;
        for (int idx = warp; idx < CG * rep * (MKEYS / 8); idx += MWARPS) {
            const int r = idx / (MKEYS / 8), nt = idx % (MKEYS / 8), j = r / rep;
            float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};    // two chains over k, added at the end
#pragma unroll
            for (int k2 = 0; k2 < KSTEPS / 2; k2++) {
                uint32_t qa0[4], qa1[4], kf[4];
                ldmatrix_x4(qa0, qb + swz<CH>(r * MROWS + (mat & 1) * 8 + rr, k2 * 4 + (mat >> 1)));
                ldmatrix_x4(qa1, qb + swz<CH>(r * MROWS + (mat & 1) * 8 + rr, k2 * 4 + 2 + (mat >> 1)));
                ldmatrix_x4(kf, kb + swz<CH>(j * MKEYS + nt * 8 + rr, k2 * 4 + mat));
                mma_bf16(acc, qa0, kf[0], kf[1]);
                mma_bf16(acc1, qa1, kf[2], kf[3]);
            }
#pragma unroll
            for (int e = 0; e < 4; e++) acc[e] += acc1[e];
            const int head = cgi * CG * rep + r;
            float w[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int key = key0 + nt * 8 + t * 2 + (e & 1), p = e < 2 ? pos_a : pos_b, row = e < 2 ? g : g + 8;
                bool vis = row < nq && key <= p;
                if (a.window > 0) vis = vis && key > p - a.window;
                w[e] = vis ? exp2f(acc[e] * a.scale_log2 - lse_s[head * MROWS + row]) : 0.f;
            }
            float* pr = p_s + (size_t)head * MROWS * PS_LD + nt * 8 + t * 2;
            *reinterpret_cast<float2*>(pr + g * PS_LD) = make_float2(w[0], w[1]);
            *reinterpret_cast<float2*>(pr + (g + 8) * PS_LD) = make_float2(w[2], w[3]);
        }
        if (cgi + 1 < GS) continue;
        if (NST > GS) cp_async_wait<0>();                         // V came with a stage that nobody has waited for yet
        __syncthreads();                                         // every head's weights and the V tiles are in place
        // ---- this warp's two output heads: mix, split, multiply with V
        const int h0 = hb + 2 * warp;
        if (h0 < H) {
            const bool two = h0 + 1 < H;
            const float2* tk = reinterpret_cast<const float2*>(talk_s) + warp * H;
            const uint32_t vb = smem_u32(v_s);
            const int c0 = h0 / rep, c1 = two ? (h0 + 1) / rep : c0;
#pragma unroll
            for (int ks = 0; ks < MKEYS / 16; ks++) {
                float m0[8], m1[8];
#pragma unroll
                for (int e = 0; e < 8; e++) m0[e] = m1[e] = 0.f;
                const float* pr = p_s + ks * 16 + t * 2;
#pragma unroll 4
                for (int hg = 0; hg < H; hg++) {
                    const float* ph = pr + (size_t)hg * MROWS * PS_LD;
                    const float2 x0 = *reinterpret_cast<const float2*>(ph + g * PS_LD);
                    const float2 x1 = *reinterpret_cast<const float2*>(ph + (g + 8) * PS_LD);
                    const float2 x2 = *reinterpret_cast<const float2*>(ph + g * PS_LD + 8);
                    const float2 x3 = *reinterpret_cast<const float2*>(ph + (g + 8) * PS_LD + 8);
                    const float2 tt = tk[hg];
                    const float t0 = tt.x, t1 = tt.y;
                    m0[0] = fmaf(t0, x0.x, m0[0]); m0[1] = fmaf(t0, x0.y, m0[1]);
                    m0[2] = fmaf(t0, x1.x, m0[2]); m0[3] = fmaf(t0, x1.y, m0[3]);
                    m0[4] = fmaf(t0, x2.x, m0[4]); m0[5] = fmaf(t0, x2.y, m0[5]);
                    m0[6] = fmaf(t0, x3.x, m0[6]); m0[7] = fmaf(t0, x3.y, m0[7]);
                    m1[0] = fmaf(t1, x0.x, m1[0]); m1[1] = fmaf(t1, x0.y, m1[1]);
                    m1[2] = fmaf(t1, x1.x, m1[2]); m1[3] = fmaf(t1, x1.y, m1[3]);
                    m1[4] = fmaf(t1, x2.x, m1[4]); m1[5] = fmaf(t1, x2.y, m1[5]);
                    m1[6] = fmaf(t1, x3.x, m1[6]); m1[7] = fmaf(t1, x3.y, m1[7]);
                }
                uint32_t hi0[4], lo0[4], hi1[4], lo1[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    split_bf16(m0[2 * e], m0[2 * e + 1], hi0[e], lo0[e]);
                    split_bf16(m1[2 * e], m1[2 * e + 1], hi1[e], lo1[e]);
                }
#pragma unroll
                for (int i = 0; i < NT_O / 2; i++) {
                    uint32_t vf[4];
                    ldmatrix_x4_trans(vf, vb + swz<CHV>(c0 * MKEYS + ks * 16 + (mat & 1) * 8 + rr, i * 2 + (mat >> 1)));
                    mma_bf16(o[0][2 * i], hi0, vf[0], vf[1]);
                    mma_bf16(o[0][2 * i + 1], hi0, vf[2], vf[3]);
                    mma_bf16(o[0][2 * i], lo0, vf[0], vf[1]);
                    mma_bf16(o[0][2 * i + 1], lo0, vf[2], vf[3]);
                    if (c1 != c0) ldmatrix_x4_trans(vf, vb + swz<CHV>(c1 * MKEYS + ks * 16 + (mat & 1) * 8 + rr, i * 2 + (mat >> 1)));
                    if (two) {
                        mma_bf16(o[1][2 * i], hi1, vf[0], vf[1]);
                        mma_bf16(o[1][2 * i + 1], hi1, vf[2], vf[3]);
                        mma_bf16(o[1][2 * i], lo1, vf[0], vf[1]);
                        mma_bf16(o[1][2 * i + 1], lo1, vf[2], vf[3]);
                    }
                }
            }
        }
    }
    cp_async_wait<0>();
    if (bad && tid == 0) atomicOr(status, MYNAH_ST_PAGE_RANGE);

    // ---- store: turned back by the query's position (one share of keys), or the raw partial sums
    const int h0 = hb + 2 * warp;
    constexpr int HV = VD / 2;
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
        const int h = h0 + hh;
        if (h >= H) continue;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int r = g + 8 * j;
            if (r >= nq) continue;
            const size_t row = (size_t)(q0 + tile0 + r);
            if (a.splits > 1) {
                float* dst = part + ((size_t)split * a.T + row) * H * VD + (size_t)h * VD;
#pragma unroll
                for (int i = 0; i < NT_O; i++)
                    *reinterpret_cast<float2*>(dst + i * 8 + t * 2) = make_float2(o[hh][i][2 * j], o[hh][i][2 * j + 1]);
                continue;
            }
            const int p = p_first + r;
            if (p >= a.n_pos_v) {
                atomicOr(status, MYNAH_ST_POS_RANGE);
                continue;
            }
            const float* cv = cos_v + (size_t)p * HV;
            const float* sv = sin_v + (size_t)p * HV;
            bf16* dst = out + row * H * VD + (size_t)h * VD;
            if (a.interleaved) {
#pragma unroll
                for (int i = 0; i < NT_O; i++) {
                    const int e = i * 4 + t;
                    const float u = o[hh][i][2 * j], v = o[hh][i][2 * j + 1];
                    *reinterpret_cast<uint32_t*>(dst + i * 8 + t * 2) = pack_bf16(u * cv[e] + v * sv[e], v * cv[e] - u * sv[e]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < NT_O / 2; i++) {
#pragma unroll
                    for (int x = 0; x < 2; x++) {
                        const int e = i * 8 + t * 2 + x;
                        const float u = o[hh][i][2 * j + x], v = o[hh][i + NT_O / 2][2 * j + x];
                        dst[e] = __float2bfloat16_rn(u * cv[e] + v * sv[e]);
                        dst[e + HV] = __float2bfloat16_rn(v * cv[e] - u * sv[e]);
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// out[row] = R(-pos) sum_s part[s, row]: the shares in their order, then every pair turned back
__global__ void __launch_bounds__(64)
sink_finish_kernel(const float* __restrict__ part, bf16* __restrict__ out, const float* __restrict__ cos_v,
                   const float* __restrict__ sin_v, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                   int T, int H, int VD, int splits, int interleaved, int n_pos_v, int* __restrict__ status) {
    griddep_wait();
    const int row = blockIdx.x;
    if (tok_seq[row] < 0) return;
    const int p = tok_pos[row];
    if (p < 0 || p >= n_pos_v) {
        if (threadIdx.x == 0) atomicOr(status, MYNAH_ST_POS_RANGE);
        return;
    }
    const int hv = VD / 2;
    const size_t ld = (size_t)H * VD;
    for (int e = threadIdx.x; e < hv; e += blockDim.x) {
        const int h = blockIdx.y;
        const int i0 = h * VD + (interleaved ? 2 * e : e), i1 = h * VD + (interleaved ? 2 * e + 1 : e + hv);
        float u = 0.f, v = 0.f;
        for (int s = 0; s < splits; s++) {
            const float* src = part + ((size_t)s * T + row) * ld;
            u += src[i0];
            v += src[i1];
        }
        const float c = cos_v[(size_t)p * hv + e], sn = sin_v[(size_t)p * hv + e];
        out[(size_t)row * ld + i0] = __float2bfloat16_rn(u * c + v * sn);
        out[(size_t)row * ld + i1] = __float2bfloat16_rn(v * c - u * sn);
    }
}

template <int HD>
int launch_lse(const dim3& grid, cudaStream_t stream, const bf16* q, float2* stats, const bf16* k,
               const int* cu_q, const int* kv_len, const PageTable& pt, const SinkTcArgs& a, int* status) {
    const size_t smem = (size_t)LQT * HD * 2 + 2 * (size_t)LKT * HD * 2;
    if (cudaFuncSetAttribute(sink_lse_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return mynah_fail("sink_attn_tc: %zu bytes of shared memory are not to be had", smem);
    mynah_launch(sink_lse_tc_kernel<HD>, grid, dim3(128), smem, stream, q, stats, k, cu_q, kv_len, pt, a, status);
    return mynah_check_launch("sink_lse_tc");
}

template <int HD, int VD>
int launch_mix(const dim3& grid, cudaStream_t stream, const bf16* q, bf16* out, float* part, const bf16* k, const bf16* v,
               const float2* stats, const VecRef& talk, const VecRef& sink, const float* cos_v, const float* sin_v, const int* cu_q,
               const int* kv_len, const PageTable& pt, const SinkTcArgs& a, int* status) {
    const size_t smem = mix_smem_bytes(a.H, a.G, HD, VD, a.stages, a.cg);
    if (cudaFuncSetAttribute(sink_mix_tc_kernel<HD, VD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return mynah_fail("sink_attn_tc: %zu bytes of shared memory are not to be had", smem);
    mynah_launch(sink_mix_tc_kernel<HD, VD>, grid, dim3(MWARPS * 32), smem, stream, q, out, part, k, v, stats, talk, sink, cos_v, sin_v,
                 cu_q, kv_len, pt, a, status);
    return mynah_check_launch("sink_mix_tc");
}

}  // namespace

// Whether the tensor-core kernels take these sizes (bfloat16 only; the general kernel of sink_attn.cu takes the rest).
MYNAH_API int mynah_sink_attn_tc_supported(int H, int G, int dim, int vd) {
    if (!((dim == 64 || dim == 128) && (vd == 64 || vd == 128) && G > 0 && H > 0 && H % G == 0)) return 0;
    return mix_smem_bytes(H, G, dim, vd, 2, 1) <= 227 * 1024 ? 1 : 0;
}

// q [T, H*dim] (rotated), out [T, H*vd] bfloat16; lse2 fp32 [splits, T, H, 2] (8-byte aligned) and part fp32
// [splits, T, H*vd] are scratch (part may be null with one share of keys); talk [H, H], sink [H] in g_dtype. B sequences with rows cu_q[b]..cu_q[b+1] that
// end at position kv_len[b] - 1.
MYNAH_API int mynah_sink_attn_tc(const void* q, void* out, float* lse2, float* part, const void* k_cache, const void* v_cache,
                                 const void* talk, const void* sink, int g_dtype, const float* cos_v, const float* sin_v,
                                 int n_pos_v, const int* cu_q, const int* kv_len, const int* tok_seq, const int* tok_pos,
                                 const int* page_indptr, const int* page_ids, const int* page_base, int n_pages, int T, int B,
                                 int H, int G, int dim, int vd, int window, float scale, int interleaved, int splits,
                                 int* status, cudaStream_t stream) {
    if (T == 0 || B == 0) return 0;
    MYNAH_REQUIRE(mynah_sink_attn_tc_supported(H, G, dim, vd), "sink_attn_tc: H=%d G=%d dim=%d vd=%d is not taken by this kernel", H, G, dim, vd);
    MYNAH_REQUIRE(T > 0 && B > 0 && window >= 0 && splits >= 1 && splits <= 65535 && H <= 65535, "sink_attn_tc: bad sizes");
    MYNAH_REQUIRE(splits == 1 || part != nullptr, "sink_attn_tc: shares of keys need their scratch");
    const int cg = mix_heads_a_stage(H, G, dim, vd);
    const SinkTcArgs a{B, H, G, T, window, splits, interleaved, n_pos_v, mix_stages(H, G, dim, vd, cg), cg, scale * 1.4426950408889634f};
    const PageTable pt{page_indptr, page_ids, page_base, n_pages};
    const VecRef tk{talk, g_dtype}, sk{sink, g_dtype};
    const bf16 *qq = (const bf16*)q, *kk = (const bf16*)k_cache, *vv = (const bf16*)v_cache;
    MYNAH_REQUIRE((reinterpret_cast<uintptr_t>(lse2) & 7) == 0, "sink_attn_tc: scratch is not 8-byte aligned");
    float2* stats = reinterpret_cast<float2*>(lse2);
    const dim3 lgrid(ceil_div(T, LQT) + B, H, splits);
    int rc = dim == 128 ? launch_lse<128>(lgrid, stream, qq, stats, kk, cu_q, kv_len, pt, a, status)
                        : launch_lse<64>(lgrid, stream, qq, stats, kk, cu_q, kv_len, pt, a, status);
    if (rc) return rc;
    const dim3 mgrid(ceil_div(T, MROWS) + B, splits, ceil_div(H, MHO));
#define SINK_MIX(HD_, VD_)                                                                                              \
    rc = launch_mix<HD_, VD_>(mgrid, stream, qq, (bf16*)out, part, kk, vv, stats, tk, sk, cos_v, sin_v, cu_q, kv_len, pt, a, status)
    if (dim == 128 && vd == 128) SINK_MIX(128, 128);
    else if (dim == 128) SINK_MIX(128, 64);
    else if (vd == 128) SINK_MIX(64, 128);
    else SINK_MIX(64, 64);
#undef SINK_MIX
    if (rc || splits == 1) return rc;
    mynah_launch(sink_finish_kernel, dim3(T, H), dim3(64), 0, stream, (const float*)part, (bf16*)out, cos_v, sin_v, tok_seq, tok_pos,
                 T, H, vd, splits, interleaved, n_pos_v, status);
    return mynah_check_launch("sink_finish");
}
