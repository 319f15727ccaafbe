// VSA2 with 64 / RM / 1 representative tiers: every (query block, kv block) pair is attended at one of three resolutions,
// one online softmax over all of them.
//   tier A: the pair is in the CSR selection (and in bits_a): the block's valid tokens, bias 0;
//   tier B: bits_ab & ~bits_a: the block's RM group means (groups of 64 / RM tokens), each with bias log2(tokens in the group);
//   tier C: ~bits_ab: the block mean, bias log2(tokens in the block).
// Reference: experiments/vsa2_representative/vsa2_rep/reference.py:53-96 (the math) and csrc/rep/rep_api.cpp:90-505 of
// shaoshitong/self_trainable_or_free_attn (rep_attn_fwd, rep_attn_bwd_q, tier_a_bwd_kv, rep_unpool). The representative
// tables are the pooled means the router already needs (group means of K and V, block means of K and V).
//
// Forward and the dQ pass: one CTA per query block walks "column tiles" of 64 columns: tier-A blocks from the CSR list,
// then tier-B tiles (64 / RM blocks x RM representatives, gathered through a block list built from the bitmaps), then
// tier-C tiles (64 block means). The gradients of the representatives come from a second pass with one CTA per tile of 64
// consecutive table rows walking the query blocks that use any of them: every table row has one owner, no atomics.
#include <string>

#include "es_api_internal.h"
#include "es_vsa_mma.cuh"

namespace es {
namespace vsa {

constexpr int PH_A = 1, PH_B = 2, PH_C = 4;

struct TierArgs {
    const void *q, *k, *v, *dout;
    const void *k_mid, *v_mid, *k_tail, *v_tail;      // [BH, mid_stride, D], [BH, tail_stride, D]
    void* o;                                          // forward: O; dQ pass: dQ (element type)
    float* lse;                                       // forward: out; backward: in
    const float* delta;
    const float* add;                                 // dQ pass: optional per-block gradient [BH, add_nb, D]
    float *dk_mid, *dv_mid, *dk_tail, *dv_tail;        // representative pass: fp32 tables like k_mid / k_tail
    const int *row_ptr, *col_idx;                     // tier A, q -> kv
    const uint32_t *bits_a, *bits_ab;                 // [BH, NB, W]
    const int* blk_cnt;
    int L, NB, W, RM, mid_stride, tail_stride, add_nb, phases;
    float scale, scale_log2;
};

// Lists of the tier-B and tier-C blocks of one query block, ascending, built by warp 0 from the two bitmap rows.
__device__ __forceinline__ void build_lists(const TierArgs& a, int bh, int qb, int* listB, int* listC, int* counts,
                                            int lane) {
    const uint32_t* ra = a.bits_a + ((size_t)bh * a.NB + qb) * a.W;
    const uint32_t* rab = a.bits_ab + ((size_t)bh * a.NB + qb) * a.W;
    int nB = 0, nC = 0;
    for (int w0 = 0; w0 < a.W; w0 += 32) {
        const int w = w0 + lane;
        uint32_t wa = 0, wab = 0xFFFFFFFFu;
        if (w < a.W) { wa = ra[w]; wab = rab[w]; }
        const int left = a.NB - w * 32;                                   // blocks covered by this word
        const uint32_t live = left >= 32 ? 0xFFFFFFFFu : (left > 0 ? (1u << left) - 1u : 0u);
        uint32_t mb = (a.phases & PH_B) ? (wab & ~wa & live) : 0u;
        uint32_t mc = (a.phases & PH_C) ? (~wab & live) : 0u;
        int pb = __popc(mb), pc = __popc(mc), sb = pb, sc = pc;
        for (int o = 1; o < 32; o <<= 1) {
            const int xb = __shfl_up_sync(0xffffffffu, sb, o), xc = __shfl_up_sync(0xffffffffu, sc, o);
            if (lane >= o) { sb += xb; sc += xc; }
        }
        int ob = nB + sb - pb, oc = nC + sc - pc;
        while (mb) { const int b = __ffs(mb) - 1; mb &= mb - 1; listB[ob++] = w * 32 + b; }
        while (mc) { const int b = __ffs(mc) - 1; mc &= mc - 1; listC[oc++] = w * 32 + b; }
        nB += __shfl_sync(0xffffffffu, sb, 31);
        nC += __shfl_sync(0xffffffffu, sc, 31);
    }
    if (lane == 0) { counts[0] = nB; counts[1] = nC; }
}

// Column tile t of a query block -> K / V tiles of a stage and the 64 column biases (log2 count, -inf = masked).
template <typename T, int D>
__device__ __forceinline__ void load_col_tile(const TierArgs& a, int bh, int t, int nA, int nBt, int beg, const int* listB,
                                              int nB, const int* listC, int nC, uint32_t sK, uint32_t sV, float* bias,
                                              int tid) {
    constexpr int CH = D / 8;
    if (t < nA) {
        const int j = a.col_idx[beg + t];
        const size_t off = ((size_t)bh * a.L + (size_t)j * TB) * D;
        load_tile<T, D>(sK, static_cast<const T*>(a.k) + off, D, tid);
        load_tile<T, D>(sV, static_cast<const T*>(a.v) + off, D, tid);
        if (tid < TB) bias[tid] = tid < a.blk_cnt[j] ? 0.f : -INFINITY;
        return;
    }
    const bool mid = t < nA + nBt;
    const int tt = mid ? t - nA : t - nA - nBt;
    const int per = mid ? TB / a.RM : TB;                 // list entries per tile
    const int R = TB / a.RM;                              // tokens per group
#pragma unroll
    for (int i = 0; i < TB * CH / 128; ++i) {
        const int idx = i * 128 + tid, row = idx / CH, ch = idx % CH;
        const int e = tt * per + (mid ? row / a.RM : row);
        size_t src_row;
        if (mid) src_row = (size_t)bh * a.mid_stride + (e < nB ? (size_t)listB[e] * a.RM + row % a.RM : 0);
        else src_row = (size_t)bh * a.tail_stride + (e < nC ? listC[e] : 0);
        const T* kt = static_cast<const T*>(mid ? a.k_mid : a.k_tail) + src_row * D + ch * 8;
        const T* vt = static_cast<const T*>(mid ? a.v_mid : a.v_tail) + src_row * D + ch * 8;
        cp16(sK + tile_off<D>(row, ch), kt);
        cp16(sV + tile_off<D>(row, ch), vt);
    }
    if (tid < TB) {
        const int e = tt * per + (mid ? tid / a.RM : tid);
        float b = -INFINITY;
        if (mid && e < nB) {
            const int c = min(max(a.blk_cnt[listB[e]] - (tid % a.RM) * R, 0), R);
            if (c > 0) b = log2f((float)c);
        } else if (!mid && e < nC) {
            b = log2f((float)a.blk_cnt[listC[e]]);
        }
        bias[tid] = b;
    }
}

// BWD = false: forward (O, lse). BWD = true: dQ of all three tiers (P = exp(scale S + bias - lse), dQ += scale dS K_col).
template <typename T, int D, bool BWD>
__global__ void __launch_bounds__(128) tier_q_kernel(const TierArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t TILE = TB * D * 2;
    constexpr int NT = BWD ? 6 : 5;                                  // Q (+ dO) and two stages of K, V
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int qb = blockIdx.x, bh = blockIdx.y;
    const uint32_t sQ = smem_addr(smem), sDO = sQ + TILE, sKV = sQ + (BWD ? 2 : 1) * TILE;
    float* sBias = reinterpret_cast<float*>(smem + NT * TILE);       // [2][64]
    int* counts = reinterpret_cast<int*>(sBias + 128);               // [2] (+2 pad)
    int* listB = counts + 4;
    int* listC = listB + a.NB;
    const size_t seq = (size_t)bh * a.L;
    const int beg = a.row_ptr[(size_t)bh * (a.NB + 1) + qb], end = a.row_ptr[(size_t)bh * (a.NB + 1) + qb + 1];
    const int nA = (a.phases & PH_A) ? end - beg : 0;
    const int cnt_q = a.blk_cnt[qb];

    load_tile<T, D>(sQ, static_cast<const T*>(a.q) + (seq + (size_t)qb * TB) * D, D, tid);
    if (BWD) load_tile<T, D>(sDO, static_cast<const T*>(a.dout) + (seq + (size_t)qb * TB) * D, D, tid);
    if (warp == 0) build_lists(a, bh, qb, listB, listC, counts, lane);
    __syncthreads();
    const int nB = counts[0], nC = counts[1];
    const int nBt = (nB * a.RM + TB - 1) / TB, nCt = (nC + TB - 1) / TB;
    const int n = nA + nBt + nCt;
    if (n > 0) load_col_tile<T, D>(a, bh, 0, nA, nBt, beg, listB, nB, listC, nC, sKV, sKV + TILE, sBias, tid);
    cp_commit();

    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
    float acc[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float ls0 = 0.f, ls1 = 0.f, d0 = 0.f, d1 = 0.f;
    bool ok0 = true, ok1 = true;
    if (BWD) {
        ls0 = a.lse[seq + (size_t)qb * TB + r0] * LOG2E; ls1 = a.lse[seq + (size_t)qb * TB + r1] * LOG2E;
        d0 = a.delta[seq + (size_t)qb * TB + r0]; d1 = a.delta[seq + (size_t)qb * TB + r1];
        ok0 = r0 < cnt_q && ls0 != -INFINITY; ok1 = r1 < cnt_q && ls1 != -INFINITY;
    }
    uint32_t qa[D / 16][4];
    for (int e = 0; e < n; ++e) {
        const int stage = e & 1;
        const uint32_t sK = sKV + (uint32_t)stage * 2 * TILE, sV = sK + TILE;
        const float* bias = sBias + stage * 64;
        if (e + 1 < n) {
            const uint32_t nk = sKV + (uint32_t)(stage ^ 1) * 2 * TILE;
            load_col_tile<T, D>(a, bh, e + 1, nA, nBt, beg, listB, nB, listC, nC, nk, nk + TILE, sBias + (stage ^ 1) * 64, tid);
        }
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        if (e == 0) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) load_a<D>(sQ, warp * 16, ks, lane, qa[ks]);
        }
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                load_b_nk<D>(sK, np, ks, lane, b);
                Elt<T>::mma(s[2 * np], qa[ks], b[0], b[1]);
                Elt<T>::mma(s[2 * np + 1], qa[ks], b[2], b[3]);
            }
        uint32_t p[8][2];
        if (!BWD) {
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int c = i * 8 + 2 * (lane & 3);
                const float b0 = bias[c], b1 = bias[c + 1];
                s[i][0] = s[i][0] * a.scale_log2 + b0; s[i][1] = s[i][1] * a.scale_log2 + b1;
                s[i][2] = s[i][2] * a.scale_log2 + b0; s[i][3] = s[i][3] * a.scale_log2 + b1;
                mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
                mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
            }
            const float mn0 = fmaxf(m0, quad_max(mx0)), mn1 = fmaxf(m1, quad_max(mx1));
            const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
            const float al0 = ex2(m0 - ms0), al1 = ex2(m1 - ms1);
            m0 = mn0; m1 = mn1;
            float t0 = 0.f, t1 = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float p0 = ex2(s[i][0] - ms0), p1 = ex2(s[i][1] - ms0), p2 = ex2(s[i][2] - ms1), p3 = ex2(s[i][3] - ms1);
                t0 += p0 + p1; t1 += p2 + p3;
                p[i][0] = Elt<T>::pack(p0, p1);
                p[i][1] = Elt<T>::pack(p2, p3);
            }
            l0 = l0 * al0 + t0; l1 = l1 * al1 + t1;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) { acc[i][0] *= al0; acc[i][1] *= al0; acc[i][2] *= al1; acc[i][3] *= al1; }
#pragma unroll
            for (int kt = 0; kt < 4; ++kt) {
                const uint32_t pa[4] = {p[2 * kt][0], p[2 * kt][1], p[2 * kt + 1][0], p[2 * kt + 1][1]};
#pragma unroll
                for (int dp = 0; dp < D / 16; ++dp) {
                    uint32_t b[4];
                    load_b_kn<D>(sV, kt, dp, lane, b);
                    Elt<T>::mma(acc[2 * dp], pa, b[0], b[1]);
                    Elt<T>::mma(acc[2 * dp + 1], pa, b[2], b[3]);
                }
            }
        } else {
            float dp[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t da[4];
                load_a<D>(sDO, warp * 16, ks, lane, da);
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t b[4];
                    load_b_nk<D>(sV, np, ks, lane, b);
                    Elt<T>::mma(dp[2 * np], da, b[0], b[1]);
                    Elt<T>::mma(dp[2 * np + 1], da, b[2], b[3]);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int c = i * 8 + 2 * (lane & 3);
                const float b0 = bias[c], b1 = bias[c + 1];
                const float p0 = (ok0 && b0 != -INFINITY) ? ex2(s[i][0] * a.scale_log2 + b0 - ls0) : 0.f;
                const float p1 = (ok0 && b1 != -INFINITY) ? ex2(s[i][1] * a.scale_log2 + b1 - ls0) : 0.f;
                const float p2 = (ok1 && b0 != -INFINITY) ? ex2(s[i][2] * a.scale_log2 + b0 - ls1) : 0.f;
                const float p3 = (ok1 && b1 != -INFINITY) ? ex2(s[i][3] * a.scale_log2 + b1 - ls1) : 0.f;
                p[i][0] = Elt<T>::pack(p0 * (dp[i][0] - d0), p1 * (dp[i][1] - d0));
                p[i][1] = Elt<T>::pack(p2 * (dp[i][2] - d1), p3 * (dp[i][3] - d1));
            }
#pragma unroll
            for (int kt = 0; kt < 4; ++kt) {
                const uint32_t da[4] = {p[2 * kt][0], p[2 * kt][1], p[2 * kt + 1][0], p[2 * kt + 1][1]};
#pragma unroll
                for (int dpi = 0; dpi < D / 16; ++dpi) {
                    uint32_t b[4];
                    load_b_kn<D>(sK, kt, dpi, lane, b);
                    Elt<T>::mma(acc[2 * dpi], da, b[0], b[1]);
                    Elt<T>::mma(acc[2 * dpi + 1], da, b[2], b[3]);
                }
            }
        }
        __syncthreads();
    }
    cp_wait<0>();

    T* out = static_cast<T*>(a.o) + (seq + (size_t)qb * TB) * D;
    if (!BWD) {
        l0 = quad_sum(l0); l1 = quad_sum(l1);
        const bool v0 = r0 < cnt_q && l0 > 0.f, v1 = r1 < cnt_q && l1 > 0.f;
        const float i0 = v0 ? 1.f / l0 : 0.f, i1 = v1 ? 1.f / l1 : 0.f;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            const int c = i * 8 + 2 * (lane & 3);
            *reinterpret_cast<uint32_t*>(out + (size_t)r0 * D + c) = Elt<T>::pack(acc[i][0] * i0, acc[i][1] * i0);
            *reinterpret_cast<uint32_t*>(out + (size_t)r1 * D + c) = Elt<T>::pack(acc[i][2] * i1, acc[i][3] * i1);
        }
        if ((lane & 3) == 0) {
            a.lse[seq + (size_t)qb * TB + r0] = v0 ? (m0 + log2f(l0)) * LN2 : -INFINITY;
            a.lse[seq + (size_t)qb * TB + r1] = v1 ? (m1 + log2f(l1)) * LN2 : -INFINITY;
        }
    } else {
        const float inv = 1.f / (float)cnt_q;
        const float* ad = a.add ? a.add + ((size_t)bh * a.add_nb + qb) * D : nullptr;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            const int c = i * 8 + 2 * (lane & 3);
            const float a0 = ad ? ad[c] * inv : 0.f, a1 = ad ? ad[c + 1] * inv : 0.f;
            const uint32_t w0 = r0 < cnt_q ? Elt<T>::pack(acc[i][0] * a.scale + a0, acc[i][1] * a.scale + a1) : 0u;
            const uint32_t w1 = r1 < cnt_q ? Elt<T>::pack(acc[i][2] * a.scale + a0, acc[i][3] * a.scale + a1) : 0u;
            *reinterpret_cast<uint32_t*>(out + (size_t)r0 * D + c) = w0;
            *reinterpret_cast<uint32_t*>(out + (size_t)r1 * D + c) = w1;
        }
    }
}

// Gradients of the representatives. Grid x = tiles of 64 consecutive table rows: first the group-mean table (tile t covers
// the blocks t * 64 / RM ..), then the block-mean table (tile covers 64 blocks). The CTA walks the query blocks that use at
// least one of its rows (tier B resp. tier C for that pair): P^T = exp(scale S^T + bias_row - lse_q) on the used pairs,
// dV_row += P^T dO, dK_row += scale (P^T (V_row dO^T - delta_q)) Q, and stores its rows of the fp32 tables.
template <typename T, int D>
__global__ void __launch_bounds__(128) tier_rep_kernel(const TierArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t TILE = TB * D * 2;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int bh = blockIdx.y;
    const int nMidTiles = (a.phases & PH_B) ? (a.NB * a.RM + TB - 1) / TB : 0;
    const bool mid = (int)blockIdx.x < nMidTiles;
    const int tt = mid ? blockIdx.x : blockIdx.x - nMidTiles;
    const int per = mid ? TB / a.RM : TB;                 // blocks covered by this tile
    const int j0 = tt * per;
    const int R = TB / a.RM;
    const uint32_t sK = smem_addr(smem), sV = sK + TILE, sQD = sV + TILE;
    float* sLse = reinterpret_cast<float*>(smem + 6 * TILE);               // [2][lse 64, delta 64]
    int* s_n = reinterpret_cast<int*>(sLse + 256);
    int* listQ = s_n + 4;                                                  // active query blocks
    unsigned long long* maskQ = reinterpret_cast<unsigned long long*>(listQ + ((a.NB + 1) & ~1));   // their block masks
    const size_t seq = (size_t)bh * a.L;
    const T* ktab = static_cast<const T*>(mid ? a.k_mid : a.k_tail) + ((size_t)bh * (mid ? a.mid_stride : a.tail_stride) + (size_t)tt * TB) * D;
    const T* vtab = static_cast<const T*>(mid ? a.v_mid : a.v_tail) + ((size_t)bh * (mid ? a.mid_stride : a.tail_stride) + (size_t)tt * TB) * D;
    load_tile<T, D>(sK, ktab, D, tid);
    load_tile<T, D>(sV, vtab, D, tid);
    // the query blocks that use a row of this tile, ascending, with the mask of the tile's blocks they use
    if (warp == 0) {
        int nq = 0;
        for (int i0 = 0; i0 < a.NB; i0 += 32) {
            const int i = i0 + lane;
            unsigned long long m = 0ull;
            if (i < a.NB) {
                const uint32_t* ra = a.bits_a + ((size_t)bh * a.NB + i) * a.W;
                const uint32_t* rab = a.bits_ab + ((size_t)bh * a.NB + i) * a.W;
                for (int h2 = 0; h2 < 2; ++h2) {
                    const int jb = j0 + 32 * h2;              // 32 blocks of the tile
                    if (jb >= a.NB || 32 * h2 >= per) break;
                    const int w = jb >> 5, sh = jb & 31;      // per <= 32 tiles start inside a word; 64-block tiles are aligned
                    uint32_t wa = ra[w] >> sh, wab = rab[w] >> sh;
                    uint32_t bits = mid ? (wab & ~wa) : ~wab;
                    const int live = min(min(per - 32 * h2, 32), a.NB - jb);
                    bits &= live >= 32 ? 0xFFFFFFFFu : ((1u << live) - 1u);
                    m |= (unsigned long long)bits << (32 * h2);
                }
            }
            const unsigned act = __ballot_sync(0xffffffffu, m != 0ull);
            if (m != 0ull) {
                const int pos = nq + __popc(act & ((1u << lane) - 1));
                listQ[pos] = i; maskQ[pos] = m;
            }
            nq += __popc(act);
        }
        if (lane == 0) s_n[0] = nq;
    }
    __syncthreads();
    const int n = s_n[0];
    const T* qbase = static_cast<const T*>(a.q) + seq * D;
    const T* dobase = static_cast<const T*>(a.dout) + seq * D;
    auto load_pair = [&](int stage, int i) {
        const uint32_t t = sQD + (uint32_t)stage * 2 * TILE;
        load_tile<T, D>(t, qbase + (size_t)i * TB * D, D, tid);
        load_tile<T, D>(t + TILE, dobase + (size_t)i * TB * D, D, tid);
        if (tid < 32) {
            const float* src = (tid < 16 ? a.lse : a.delta) + seq + (size_t)i * TB + (tid & 15) * 4;
            cp16(smem_addr(sLse + stage * 128 + (tid < 16 ? 0 : 64) + (tid & 15) * 4), src);
        }
    };
    if (n > 0) load_pair(0, listQ[0]);
    cp_commit();

    // this thread's two table rows: their block (relative to the tile) and bias
    const int kr0 = warp * 16 + (lane >> 2), kr1 = kr0 + 8;
    int rb0, rb1;
    float bias0 = -INFINITY, bias1 = -INFINITY;
    {
        const int rows[2] = {kr0, kr1};
        float* bs[2] = {&bias0, &bias1};
        int* rb[2] = {&rb0, &rb1};
        for (int u = 0; u < 2; ++u) {
            const int r = rows[u];
            const int jb = mid ? r / a.RM : r;
            *rb[u] = jb;
            const int j = j0 + jb;
            if (j < a.NB) {
                const int c = mid ? min(max(a.blk_cnt[j] - (r % a.RM) * R, 0), R) : a.blk_cnt[j];
                if (c > 0) *bs[u] = log2f((float)c);
            }
        }
    }
    float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
        dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f;
    }
    for (int e = 0; e < n; ++e) {
        const int stage = e & 1;
        const uint32_t sQ = sQD + (uint32_t)stage * 2 * TILE, sDO = sQ + TILE;
        const int qb = listQ[e];
        const unsigned long long um = maskQ[e];
        if (e + 1 < n) load_pair(stage ^ 1, listQ[e + 1]);
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        const int cnt_q = a.blk_cnt[qb];
        const float* lse = sLse + stage * 128;
        const float* dl = lse + 64;
        const bool use0 = ((um >> rb0) & 1ull) && bias0 != -INFINITY, use1 = ((um >> rb1) & 1ull) && bias1 != -INFINITY;
        float s[8][4], dp[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
            dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
        }
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t ka[4], va[4];
            load_a<D>(sK, warp * 16, ks, lane, ka);
            load_a<D>(sV, warp * 16, ks, lane, va);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                load_b_nk<D>(sQ, np, ks, lane, b);
                Elt<T>::mma(s[2 * np], ka, b[0], b[1]);
                Elt<T>::mma(s[2 * np + 1], ka, b[2], b[3]);
                load_b_nk<D>(sDO, np, ks, lane, b);
                Elt<T>::mma(dp[2 * np], va, b[0], b[1]);
                Elt<T>::mma(dp[2 * np + 1], va, b[2], b[3]);
            }
        }
        uint32_t p[8][2], ds[8][2];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = i * 8 + 2 * (lane & 3);
            const float ls0 = lse[c] * LOG2E, ls1 = lse[c + 1] * LOG2E, e0 = dl[c], e1 = dl[c + 1];
            const bool q0 = c < cnt_q && ls0 != -INFINITY, q1 = c + 1 < cnt_q && ls1 != -INFINITY;
            const float p0 = (q0 && use0) ? ex2(s[i][0] * a.scale_log2 + bias0 - ls0) : 0.f;
            const float p1 = (q1 && use0) ? ex2(s[i][1] * a.scale_log2 + bias0 - ls1) : 0.f;
            const float p2 = (q0 && use1) ? ex2(s[i][2] * a.scale_log2 + bias1 - ls0) : 0.f;
            const float p3 = (q1 && use1) ? ex2(s[i][3] * a.scale_log2 + bias1 - ls1) : 0.f;
            p[i][0] = Elt<T>::pack(p0, p1);
            p[i][1] = Elt<T>::pack(p2, p3);
            ds[i][0] = Elt<T>::pack(p0 * (dp[i][0] - e0), p1 * (dp[i][1] - e1));
            ds[i][1] = Elt<T>::pack(p2 * (dp[i][2] - e0), p3 * (dp[i][3] - e1));
        }
#pragma unroll
        for (int kt = 0; kt < 4; ++kt) {
            const uint32_t pa[4] = {p[2 * kt][0], p[2 * kt][1], p[2 * kt + 1][0], p[2 * kt + 1][1]};
            const uint32_t da[4] = {ds[2 * kt][0], ds[2 * kt][1], ds[2 * kt + 1][0], ds[2 * kt + 1][1]};
#pragma unroll
            for (int dpi = 0; dpi < D / 16; ++dpi) {
                uint32_t b[4];
                load_b_kn<D>(sDO, kt, dpi, lane, b);
                Elt<T>::mma(dv[2 * dpi], pa, b[0], b[1]);
                Elt<T>::mma(dv[2 * dpi + 1], pa, b[2], b[3]);
                load_b_kn<D>(sQ, kt, dpi, lane, b);
                Elt<T>::mma(dk[2 * dpi], da, b[0], b[1]);
                Elt<T>::mma(dk[2 * dpi + 1], da, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    cp_wait<0>();
    // rows of the fp32 tables (rows past the table's real size stay untouched: the caller zero-fills the tables)
    const int stride = mid ? a.mid_stride : a.tail_stride;
    const int limit = mid ? a.NB * a.RM : a.NB;
    float* dkt = (mid ? a.dk_mid : a.dk_tail) + ((size_t)bh * stride + (size_t)tt * TB) * D;
    float* dvt = (mid ? a.dv_mid : a.dv_tail) + ((size_t)bh * stride + (size_t)tt * TB) * D;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        const int c = i * 8 + 2 * (lane & 3);
        if (tt * TB + kr0 < limit) {
            *reinterpret_cast<float2*>(dkt + (size_t)kr0 * D + c) = make_float2(dk[i][0] * a.scale, dk[i][1] * a.scale);
            *reinterpret_cast<float2*>(dvt + (size_t)kr0 * D + c) = make_float2(dv[i][0], dv[i][1]);
        }
        if (tt * TB + kr1 < limit) {
            *reinterpret_cast<float2*>(dkt + (size_t)kr1 * D + c) = make_float2(dk[i][2] * a.scale, dk[i][3] * a.scale);
            *reinterpret_cast<float2*>(dvt + (size_t)kr1 * D + c) = make_float2(dv[i][2], dv[i][3]);
        }
    }
}

// Token gradients from the three sources: out = valid ? tok[t] + mid[block * RM + group] / tokens in the group
// + (tail[block] + add[block]) / tokens in the block : 0. tok, mid, tail, add are fp32 and optional.
struct UnpoolArgs {
    const float *tok, *mid, *tail, *add;
    void* out;
    const int* blk_cnt;
    int L, RM, mid_stride, tail_stride, add_nb;
};
template <typename T, int D>
__global__ void __launch_bounds__(D / 2) tier_unpool_kernel(const UnpoolArgs a) {
    const int blk = blockIdx.x, bh = blockIdx.y, c = 2 * threadIdx.x;
    const int cnt = a.blk_cnt[blk], R = TB / a.RM;
    float tx = 0.f, ty = 0.f;
    if (a.tail) { const float* p = a.tail + ((size_t)bh * a.tail_stride + blk) * D + c; tx = p[0]; ty = p[1]; }
    if (a.add) { const float* p = a.add + ((size_t)bh * a.add_nb + blk) * D + c; tx += p[0]; ty += p[1]; }
    tx /= (float)cnt; ty /= (float)cnt;
    for (int r = 0; r < TB; ++r) {
        const size_t row = (size_t)bh * a.L + (size_t)blk * TB + r;
        uint32_t out = 0u;
        if (r < cnt) {
            float x = tx, y = ty;
            if (a.mid) {
                const int g = r / R, cg = min(cnt - g * R, R);
                const float* p = a.mid + ((size_t)bh * a.mid_stride + (size_t)blk * a.RM + g) * D + c;
                x += p[0] / (float)cg; y += p[1] / (float)cg;
            }
            if (a.tok) { x += a.tok[row * D + c]; y += a.tok[row * D + c + 1]; }
            out = Elt<T>::pack(x, y);
        }
        *reinterpret_cast<uint32_t*>(static_cast<T*>(a.out) + row * D + c) = out;
    }
}

static int check_tier(const char* name, int BH, int L, int D, int dtype, int RM, int phases, int mid_stride, int tail_stride) {
    if (BH <= 0 || L <= 0 || L % TB != 0) return set_error(-1, (std::string(name) + ": BH > 0 and L a positive multiple of 64").c_str());
    if (D != 64 && D != 128) return set_error(-1, (std::string(name) + ": head dim must be 64 or 128").c_str());
    if (dtype != 0 && dtype != 1) return set_error(-1, (std::string(name) + ": dtype must be 0 (bf16) or 1 (fp16)").c_str());
    if (RM != 2 && RM != 4 && RM != 8 && RM != 16) return set_error(-1, (std::string(name) + ": mid_reps must be 2, 4, 8 or 16").c_str());
    if (phases < 0 || phases > 7) return set_error(-1, (std::string(name) + ": phases is a mask of 1 (A), 2 (B), 4 (C)").c_str());
    const int NB = L / TB;
    if (mid_stride < (NB * RM + TB - 1) / TB * TB || tail_stride < (NB + TB - 1) / TB * TB)
        return set_error(-1, (std::string(name) + ": the tables must be padded to multiples of 64 rows").c_str());
    if (NB > 4096) return set_error(-1, (std::string(name) + ": at most 4096 blocks").c_str());
    return 0;
}

template <typename K> static int set_smem_t(K kern, size_t bytes) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    return e == cudaSuccess ? 0 : set_error(-2, cudaGetErrorString(e));
}

#define TIER_DISPATCH(KERNEL, SMEM, GRID, ARGS, ...)                                                                     \
    do {                                                                                                                \
        int rc__ = 0;                                                                                                   \
        if (dtype == 0 && D == 128) { if ((rc__ = set_smem_t(KERNEL<__nv_bfloat16, 128 __VA_ARGS__>, SMEM))) return rc__; KERNEL<__nv_bfloat16, 128 __VA_ARGS__><<<GRID, 128, SMEM, st>>>(ARGS); } \
        else if (dtype == 0) { if ((rc__ = set_smem_t(KERNEL<__nv_bfloat16, 64 __VA_ARGS__>, SMEM))) return rc__; KERNEL<__nv_bfloat16, 64 __VA_ARGS__><<<GRID, 128, SMEM, st>>>(ARGS); } \
        else if (D == 128) { if ((rc__ = set_smem_t(KERNEL<__half, 128 __VA_ARGS__>, SMEM))) return rc__; KERNEL<__half, 128 __VA_ARGS__><<<GRID, 128, SMEM, st>>>(ARGS); } \
        else { if ((rc__ = set_smem_t(KERNEL<__half, 64 __VA_ARGS__>, SMEM))) return rc__; KERNEL<__half, 64 __VA_ARGS__><<<GRID, 128, SMEM, st>>>(ARGS); } \
    } while (0)

}  // namespace vsa
}  // namespace es

using namespace es;
using namespace es::vsa;

static void fill_tier(TierArgs& a, int L, int D, int RM, int phases, int mid_stride, int tail_stride) {
    a.L = L; a.NB = L / TB; a.W = (a.NB + 31) / 32; a.RM = RM; a.phases = phases;
    a.mid_stride = mid_stride; a.tail_stride = tail_stride;
    a.scale = 1.f / sqrtf((float)D);
    a.scale_log2 = LOG2E * a.scale;
}

extern "C" int es_vsa_tier_attn_fwd(const void* q, const void* k, const void* v, const void* k_mid, const void* v_mid,
                                    const void* k_tail, const void* v_tail, void* o, float* lse, const int32_t* q2k_ptr,
                                    const int32_t* q2k_idx, const int32_t* bits_a, const int32_t* bits_ab,
                                    const int32_t* blk_cnt, int32_t BH, int32_t L, int32_t D, int32_t mid_reps,
                                    int32_t mid_stride, int32_t tail_stride, int32_t phases, int32_t dtype, void* stream) {
    if (!q || !k || !v || !k_mid || !v_mid || !k_tail || !v_tail || !o || !lse || !q2k_ptr || !q2k_idx || !bits_a || !bits_ab || !blk_cnt)
        return set_error(-1, "es_vsa_tier_attn_fwd: null pointer");
    if (int rc = check_tier("es_vsa_tier_attn_fwd", BH, L, D, dtype, mid_reps, phases, mid_stride, tail_stride)) return rc;
    TierArgs a{};
    a.q = q; a.k = k; a.v = v; a.k_mid = k_mid; a.v_mid = v_mid; a.k_tail = k_tail; a.v_tail = v_tail; a.o = o; a.lse = lse;
    a.row_ptr = q2k_ptr; a.col_idx = q2k_idx; a.bits_a = (const uint32_t*)bits_a; a.bits_ab = (const uint32_t*)bits_ab;
    a.blk_cnt = blk_cnt;
    fill_tier(a, L, D, mid_reps, phases, mid_stride, tail_stride);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)5 * TB * D * 2 + 128 * 4 + 16 + 2 * (size_t)a.NB * 4;
    const dim3 grid(a.NB, BH);
#define COMMA_FALSE , false
    TIER_DISPATCH(tier_q_kernel, smem, grid, a, COMMA_FALSE);
#undef COMMA_FALSE
    ES_CHECK_LAUNCH("tier_q_kernel");
    return 0;
}

extern "C" int es_vsa_tier_attn_bwd_q(const void* q, const void* k, const void* v, const void* k_mid, const void* v_mid,
                                      const void* k_tail, const void* v_tail, const void* dout, const float* lse,
                                      const float* delta, void* dq, const float* add_dq, int32_t add_nb,
                                      const int32_t* q2k_ptr, const int32_t* q2k_idx, const int32_t* bits_a,
                                      const int32_t* bits_ab, const int32_t* blk_cnt, int32_t BH, int32_t L, int32_t D,
                                      int32_t mid_reps, int32_t mid_stride, int32_t tail_stride, int32_t phases,
                                      int32_t dtype, void* stream) {
    if (!q || !k || !v || !k_mid || !v_mid || !k_tail || !v_tail || !dout || !lse || !delta || !dq || !q2k_ptr || !q2k_idx || !bits_a || !bits_ab || !blk_cnt)
        return set_error(-1, "es_vsa_tier_attn_bwd_q: null pointer");
    if (int rc = check_tier("es_vsa_tier_attn_bwd_q", BH, L, D, dtype, mid_reps, phases, mid_stride, tail_stride)) return rc;
    if (add_dq && add_nb < L / TB) return set_error(-1, "es_vsa_tier_attn_bwd_q: add_nb smaller than the block count");
    TierArgs a{};
    a.q = q; a.k = k; a.v = v; a.dout = dout; a.k_mid = k_mid; a.v_mid = v_mid; a.k_tail = k_tail; a.v_tail = v_tail;
    a.o = dq; a.lse = const_cast<float*>(lse); a.delta = delta; a.add = add_dq; a.add_nb = add_nb;
    a.row_ptr = q2k_ptr; a.col_idx = q2k_idx; a.bits_a = (const uint32_t*)bits_a; a.bits_ab = (const uint32_t*)bits_ab;
    a.blk_cnt = blk_cnt;
    fill_tier(a, L, D, mid_reps, phases, mid_stride, tail_stride);
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)6 * TB * D * 2 + 128 * 4 + 16 + 2 * (size_t)a.NB * 4;
    const dim3 grid(a.NB, BH);
#define COMMA_TRUE , true
    TIER_DISPATCH(tier_q_kernel, smem, grid, a, COMMA_TRUE);
#undef COMMA_TRUE
    ES_CHECK_LAUNCH("tier_q_kernel");
    return 0;
}

extern "C" int es_vsa_tier_rep_bwd(const void* q, const void* k_mid, const void* v_mid, const void* k_tail,
                                   const void* v_tail, const void* dout, const float* lse, const float* delta,
                                   float* dk_mid, float* dv_mid, float* dk_tail, float* dv_tail, const int32_t* bits_a,
                                   const int32_t* bits_ab, const int32_t* blk_cnt, int32_t BH, int32_t L, int32_t D,
                                   int32_t mid_reps, int32_t mid_stride, int32_t tail_stride, int32_t phases, int32_t dtype,
                                   void* stream) {
    if (!q || !k_mid || !v_mid || !k_tail || !v_tail || !dout || !lse || !delta || !dk_mid || !dv_mid || !dk_tail || !dv_tail || !bits_a || !bits_ab || !blk_cnt)
        return set_error(-1, "es_vsa_tier_rep_bwd: null pointer");
    if (int rc = check_tier("es_vsa_tier_rep_bwd", BH, L, D, dtype, mid_reps, phases, mid_stride, tail_stride)) return rc;
    TierArgs a{};
    a.q = q; a.dout = dout; a.k_mid = k_mid; a.v_mid = v_mid; a.k_tail = k_tail; a.v_tail = v_tail;
    a.lse = const_cast<float*>(lse); a.delta = delta; a.dk_mid = dk_mid; a.dv_mid = dv_mid; a.dk_tail = dk_tail; a.dv_tail = dv_tail;
    a.bits_a = (const uint32_t*)bits_a; a.bits_ab = (const uint32_t*)bits_ab; a.blk_cnt = blk_cnt;
    fill_tier(a, L, D, mid_reps, phases, mid_stride, tail_stride);
    const int tiles = ((phases & PH_B) ? (a.NB * mid_reps + TB - 1) / TB : 0) + ((phases & PH_C) ? (a.NB + TB - 1) / TB : 0);
    if (tiles == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)6 * TB * D * 2 + 256 * 4 + 16 + (size_t)((a.NB + 1) & ~1) * 4 + (size_t)a.NB * 8;
    const dim3 grid(tiles, BH);
    TIER_DISPATCH(tier_rep_kernel, smem, grid, a);
    ES_CHECK_LAUNCH("tier_rep_kernel");
    return 0;
}

extern "C" int es_vsa_tier_unpool(const float* tok, const float* mid, const float* tail, const float* add, int32_t add_nb,
                                  void* out, const int32_t* blk_cnt, int32_t BH, int32_t L, int32_t D, int32_t mid_reps,
                                  int32_t mid_stride, int32_t tail_stride, int32_t dtype, void* stream) {
    if (!out || !blk_cnt) return set_error(-1, "es_vsa_tier_unpool: null pointer");
    if (int rc = check_tier("es_vsa_tier_unpool", BH, L, D, dtype, mid_reps, 7, mid ? mid_stride : 1 << 30, tail ? tail_stride : 1 << 30)) return rc;
    if (add && add_nb < L / TB) return set_error(-1, "es_vsa_tier_unpool: add_nb smaller than the block count");
    UnpoolArgs a{tok, mid, tail, add, out, blk_cnt, L, mid_reps, mid_stride, tail_stride, add_nb};
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid(L / TB, BH);
    if (dtype == 0 && D == 128) tier_unpool_kernel<__nv_bfloat16, 128><<<grid, 64, 0, st>>>(a);
    else if (dtype == 0) tier_unpool_kernel<__nv_bfloat16, 64><<<grid, 32, 0, st>>>(a);
    else if (D == 128) tier_unpool_kernel<__half, 128><<<grid, 64, 0, st>>>(a);
    else tier_unpool_kernel<__half, 64><<<grid, 32, 0, st>>>(a);
    ES_CHECK_LAUNCH("tier_unpool_kernel");
    return 0;
}
