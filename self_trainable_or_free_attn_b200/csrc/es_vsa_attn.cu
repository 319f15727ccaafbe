// VSA2 block-sparse attention over CSR block lists: forward (online softmax), backward for dK / dV (one CTA per kv block
// walking the kv -> q lists) and for dQ (one CTA per query block walking the q -> kv lists). No atomics: every output
// row has one owner, so results are reproducible bit for bit.
//
// Conventions (reference: csrc/vsa/vsa2_kernels.h:1-12 of shaoshitong/self_trainable_or_free_attn):
//   token tensors [BH, L, D], L = NB * 64, blk_cnt [NB] valid tokens per block (valid tokens first);
//   CSR: row_ptr [BH * (NB + 1)] absolute offsets into col_idx; lse [BH, L] natural log, -inf for rows without a key
//   and for padded rows; padded rows output 0 and receive zero gradient.
// The same kernels serve the coarse branch (block means as a sequence of NBc_pad rows, 64-row tiles with their own counts).
//
// One CTA = 4 warps x 16 rows of a 64-row block; K / V (or Q / dO) tiles of the walked list are double-buffered in
// shared memory with cp.async; products on the tensor cores (mma.sync m16n8k16, fp32 accumulation).
#include <string>

#include "es_api_internal.h"
#include "es_vsa_mma.cuh"

namespace es {
namespace vsa {

struct FwdArgs {
    const void *q, *k, *v;
    void* o;
    float* lse;
    const int *row_ptr, *col_idx, *blk_cnt;
    int L, NB;
    float scale_log2;
    // Split-KV task mode (es_vsa_split_plan), all null in the plain (block, bh) grid: tasks[t] = {row = bh * NB + block,
    // first edge, one past the last edge, slot}; slot < 0 writes o / lse, slot >= 0 writes the fp32 normalised partial
    // part_o[slot] [64, D] and its log2-domain lse part_lse[slot] [64].
    const int* tasks;
    const int* task_info;
    float* part_o;
    float* part_lse;
};

// The work item of a CTA: (block, bh) of the grid, or a task of the split plan. False: nothing to do.
__device__ __forceinline__ bool work_item(const int* tasks, const int* info, const int* row_ptr, int NB, int& blk, int& bh,
                                          int& beg, int& end, int& slot) {
    if (tasks) {
        if ((int)blockIdx.x >= info[0]) return false;
        const int4 t = reinterpret_cast<const int4*>(tasks)[blockIdx.x];
        bh = t.x / NB; blk = t.x - bh * NB; beg = t.y; end = t.z; slot = t.w;
    } else {
        blk = blockIdx.x; bh = blockIdx.y; slot = -1;
        beg = row_ptr[(size_t)bh * (NB + 1) + blk];
        end = row_ptr[(size_t)bh * (NB + 1) + blk + 1];
    }
    return true;
}

template <typename T, int D>
__global__ void __launch_bounds__(128) attn_fwd_kernel(const FwdArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t TILE = TB * D * 2;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int qb, bh, beg, end, slot;
    if (!work_item(a.tasks, a.task_info, a.row_ptr, a.NB, qb, bh, beg, end, slot)) return;
    const uint32_t sQ = smem_addr(smem), sKV = sQ + TILE;           // [stage][K, V]
    const T* q = static_cast<const T*>(a.q) + ((size_t)bh * a.L + (size_t)qb * TB) * D;
    const T* kbase = static_cast<const T*>(a.k) + (size_t)bh * a.L * D;
    const T* vbase = static_cast<const T*>(a.v) + (size_t)bh * a.L * D;
    const int n = end - beg;
    const int cnt_q = a.blk_cnt[qb];

    load_tile<T, D>(sQ, q, D, tid);
    if (n > 0) {
        const int j = a.col_idx[beg];
        load_tile<T, D>(sKV, kbase + (size_t)j * TB * D, D, tid);
        load_tile<T, D>(sKV + TILE, vbase + (size_t)j * TB * D, D, tid);
    }
    cp_commit();

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    uint32_t qa[D / 16][4];

    for (int e = 0; e < n; ++e) {
        const uint32_t sK = sKV + (uint32_t)(e & 1) * 2 * TILE, sV = sK + TILE;
        const int kvb = a.col_idx[beg + e];
        if (e + 1 < n) {
            const int j = a.col_idx[beg + e + 1];
            const uint32_t nk = sKV + (uint32_t)((e + 1) & 1) * 2 * TILE;
            load_tile<T, D>(nk, kbase + (size_t)j * TB * D, D, tid);
            load_tile<T, D>(nk + TILE, vbase + (size_t)j * TB * D, D, tid);
        }
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        if (e == 0) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) load_a<D>(sQ, warp * 16, ks, lane, qa[ks]);
        }
        // S = Q K^T (16 rows x 64 keys per warp)
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
        // online softmax in the log2 domain; keys past the block's count are masked
        const int cnt_k = a.blk_cnt[kvb];
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = i * 8 + 2 * (lane & 3);
            s[i][0] = c < cnt_k ? s[i][0] * a.scale_log2 : -INFINITY;
            s[i][1] = c + 1 < cnt_k ? s[i][1] * a.scale_log2 : -INFINITY;
            s[i][2] = c < cnt_k ? s[i][2] * a.scale_log2 : -INFINITY;
            s[i][3] = c + 1 < cnt_k ? s[i][3] * a.scale_log2 : -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
            mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
        }
        const float mn0 = fmaxf(m0, quad_max(mx0)), mn1 = fmaxf(m1, quad_max(mx1));
        const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
        const float al0 = ex2(m0 - ms0), al1 = ex2(m1 - ms1);
        m0 = mn0; m1 = mn1;
        float r0 = 0.f, r1 = 0.f;
        uint32_t p[8][2];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float p0 = ex2(s[i][0] - ms0), p1 = ex2(s[i][1] - ms0), p2 = ex2(s[i][2] - ms1), p3 = ex2(s[i][3] - ms1);
            r0 += p0 + p1; r1 += p2 + p3;
            p[i][0] = Elt<T>::pack(p0, p1);
            p[i][1] = Elt<T>::pack(p2, p3);
        }
        l0 = l0 * al0 + r0; l1 = l1 * al1 + r1;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1; }
        // O += P V
#pragma unroll
        for (int kt = 0; kt < 4; ++kt) {
            const uint32_t pa[4] = {p[2 * kt][0], p[2 * kt][1], p[2 * kt + 1][0], p[2 * kt + 1][1]};
#pragma unroll
            for (int dp = 0; dp < D / 16; ++dp) {
                uint32_t b[4];
                load_b_kn<D>(sV, kt, dp, lane, b);
                Elt<T>::mma(o[2 * dp], pa, b[0], b[1]);
                Elt<T>::mma(o[2 * dp + 1], pa, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    cp_wait<0>();

    l0 = quad_sum(l0); l1 = quad_sum(l1);
    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
    if (slot >= 0) {
        // a chunk of a split row: the normalised partial and its log2 lse; the merge masks the padded rows
        const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
        float* po = a.part_o + (size_t)slot * TB * D;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            const int c = i * 8 + 2 * (lane & 3);
            *reinterpret_cast<float2*>(po + (size_t)r0 * D + c) = make_float2(o[i][0] * i0, o[i][1] * i0);
            *reinterpret_cast<float2*>(po + (size_t)r1 * D + c) = make_float2(o[i][2] * i1, o[i][3] * i1);
        }
        if ((lane & 3) == 0) {
            a.part_lse[(size_t)slot * TB + r0] = l0 > 0.f ? m0 + log2f(l0) : -INFINITY;
            a.part_lse[(size_t)slot * TB + r1] = l1 > 0.f ? m1 + log2f(l1) : -INFINITY;
        }
        return;
    }
    const bool ok0 = r0 < cnt_q && l0 > 0.f, ok1 = r1 < cnt_q && l1 > 0.f;
    const float i0 = ok0 ? 1.f / l0 : 0.f, i1 = ok1 ? 1.f / l1 : 0.f;
    T* out = static_cast<T*>(a.o) + ((size_t)bh * a.L + (size_t)qb * TB) * D;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        const int c = i * 8 + 2 * (lane & 3);
        *reinterpret_cast<uint32_t*>(out + (size_t)r0 * D + c) = Elt<T>::pack(o[i][0] * i0, o[i][1] * i0);
        *reinterpret_cast<uint32_t*>(out + (size_t)r1 * D + c) = Elt<T>::pack(o[i][2] * i1, o[i][3] * i1);
    }
    if ((lane & 3) == 0) {
        float* lse = a.lse + (size_t)bh * a.L + (size_t)qb * TB;
        lse[r0] = ok0 ? (m0 + log2f(l0)) * LN2 : -INFINITY;
        lse[r1] = ok1 ? (m1 + log2f(l1)) * LN2 : -INFINITY;
    }
}

// ---------------------------------------------------------------------------------------------- backward, dK / dV
struct BwdArgs {
    const void *q, *k, *v, *dout;
    const float *lse, *delta;
    void *d0, *d1;                 // kv owner: dK, dV; q owner: dQ, unused (element type)
    float *f0, *f1;                // fp32 outputs instead, when not null
    const float *add0, *add1;      // optional per-block gradients [BH, add_nb, D], added as add / count to every valid token
    int add_nb;
    const int *row_ptr, *col_idx, *blk_cnt;
    int L, NB;
    float scale, scale_log2;
    // Split-KV task mode over the walked lists (see FwdArgs): slot >= 0 writes fp32 partial gradients to part0 / part1
    // [slot] [64, D] without the per-block add (the merge adds it once and zeroes the padded rows).
    const int* tasks;
    const int* task_info;
    float *part0, *part1;
};

template <typename T, int D>
__device__ __forceinline__ void store_rows(const BwdArgs& a, float (&acc)[D / 8][4], void* dst_e, float* dst_f,
                                           const float* add, int bh, int blk, int cnt, int warp, int lane, float mul) {
    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
    const float inv = 1.f / (float)cnt;
    const float* ad = add ? add + ((size_t)bh * a.add_nb + blk) * D : nullptr;
    const size_t base = ((size_t)bh * a.L + (size_t)blk * TB) * D;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        const int c = i * 8 + 2 * (lane & 3);
        const float a0 = ad ? ad[c] * inv : 0.f, a1 = ad ? ad[c + 1] * inv : 0.f;
        float v0 = r0 < cnt ? acc[i][0] * mul + a0 : 0.f, v1 = r0 < cnt ? acc[i][1] * mul + a1 : 0.f;
        float v2 = r1 < cnt ? acc[i][2] * mul + a0 : 0.f, v3 = r1 < cnt ? acc[i][3] * mul + a1 : 0.f;
        if (dst_f) {
            *reinterpret_cast<float2*>(dst_f + base + (size_t)r0 * D + c) = make_float2(v0, v1);
            *reinterpret_cast<float2*>(dst_f + base + (size_t)r1 * D + c) = make_float2(v2, v3);
        } else {
            T* d = static_cast<T*>(dst_e) + base;
            *reinterpret_cast<uint32_t*>(d + (size_t)r0 * D + c) = Elt<T>::pack(v0, v1);
            *reinterpret_cast<uint32_t*>(d + (size_t)r1 * D + c) = Elt<T>::pack(v2, v3);
        }
    }
}

template <int D>
__device__ __forceinline__ void store_part(float (&acc)[D / 8][4], float* dst, int warp, int lane, float mul) {
    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        const int c = i * 8 + 2 * (lane & 3);
        *reinterpret_cast<float2*>(dst + (size_t)r0 * D + c) = make_float2(acc[i][0] * mul, acc[i][1] * mul);
        *reinterpret_cast<float2*>(dst + (size_t)r1 * D + c) = make_float2(acc[i][2] * mul, acc[i][3] * mul);
    }
}

// One CTA per kv block j: walks the query blocks i that selected it. Per pair, with S^T = K Q^T (kv rows x q columns):
//   P^T = exp(scale S^T - lse_q), dV += P^T dO, dP^T = V dO^T, dS^T = P^T (dP^T - delta_q), dK += scale dS^T Q.
template <typename T, int D>
__global__ void __launch_bounds__(128) attn_bwd_kv_kernel(const BwdArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t TILE = TB * D * 2;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int kb, bh, beg, end, slot;
    if (!work_item(a.tasks, a.task_info, a.row_ptr, a.NB, kb, bh, beg, end, slot)) return;
    const uint32_t sK = smem_addr(smem), sV = sK + TILE, sQD = sV + TILE;      // [stage][Q, dO]
    float* sLse = reinterpret_cast<float*>(smem + 6 * TILE);                   // [stage][lse 64, delta 64]
    const size_t seq = (size_t)bh * a.L;
    const T* qbase = static_cast<const T*>(a.q) + seq * D;
    const T* dobase = static_cast<const T*>(a.dout) + seq * D;
    const int n = end - beg;
    const int cnt_k = a.blk_cnt[kb];

    auto load_pair = [&](int stage, int i) {
        const uint32_t t = sQD + (uint32_t)stage * 2 * TILE;
        load_tile<T, D>(t, qbase + (size_t)i * TB * D, D, tid);
        load_tile<T, D>(t + TILE, dobase + (size_t)i * TB * D, D, tid);
        if (tid < 32) {
            const float* src = (tid < 16 ? a.lse : a.delta) + seq + (size_t)i * TB + (tid & 15) * 4;
            cp16(smem_addr(sLse + stage * 128 + (tid < 16 ? 0 : 64) + (tid & 15) * 4), src);
        }
    };
    load_tile<T, D>(sK, static_cast<const T*>(a.k) + (seq + (size_t)kb * TB) * D, D, tid);
    load_tile<T, D>(sV, static_cast<const T*>(a.v) + (seq + (size_t)kb * TB) * D, D, tid);
    if (n > 0) load_pair(0, a.col_idx[beg]);
    cp_commit();

    float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
        dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f;
    }
    const int kr0 = warp * 16 + (lane >> 2), kr1 = kr0 + 8;        // this thread's kv rows
    for (int e = 0; e < n; ++e) {
        const int stage = e & 1;
        const uint32_t sQ = sQD + (uint32_t)stage * 2 * TILE, sDO = sQ + TILE;
        const int qb = a.col_idx[beg + e];
        if (e + 1 < n) load_pair(stage ^ 1, a.col_idx[beg + e + 1]);
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        const int cnt_q = a.blk_cnt[qb];
        const float* lse = sLse + stage * 128;
        const float* dl = lse + 64;
        // S^T = K Q^T and dP^T = V dO^T
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
            const float ls0 = lse[c] * LOG2E, ls1 = lse[c + 1] * LOG2E, d0 = dl[c], d1 = dl[c + 1];
            const bool q0 = c < cnt_q && ls0 != -INFINITY, q1 = c + 1 < cnt_q && ls1 != -INFINITY;
            const float p0 = (q0 && kr0 < cnt_k) ? ex2(s[i][0] * a.scale_log2 - ls0) : 0.f;
            const float p1 = (q1 && kr0 < cnt_k) ? ex2(s[i][1] * a.scale_log2 - ls1) : 0.f;
            const float p2 = (q0 && kr1 < cnt_k) ? ex2(s[i][2] * a.scale_log2 - ls0) : 0.f;
            const float p3 = (q1 && kr1 < cnt_k) ? ex2(s[i][3] * a.scale_log2 - ls1) : 0.f;
            p[i][0] = Elt<T>::pack(p0, p1);
            p[i][1] = Elt<T>::pack(p2, p3);
            ds[i][0] = Elt<T>::pack(p0 * (dp[i][0] - d0), p1 * (dp[i][1] - d1));
            ds[i][1] = Elt<T>::pack(p2 * (dp[i][2] - d0), p3 * (dp[i][3] - d1));
        }
        // dV += P^T dO and dK += dS^T Q (k dimension = the 64 query rows)
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
    if (slot >= 0) {
        store_part<D>(dk, a.part0 + (size_t)slot * TB * D, warp, lane, a.scale);
        store_part<D>(dv, a.part1 + (size_t)slot * TB * D, warp, lane, 1.f);
        return;
    }
    store_rows<T, D>(a, dk, a.d0, a.f0, a.add0, bh, kb, cnt_k, warp, lane, a.scale);
    store_rows<T, D>(a, dv, a.d1, a.f1, a.add1, bh, kb, cnt_k, warp, lane, 1.f);
}

// One CTA per query block i: walks its kv blocks. Per pair: P = exp(scale S - lse), dP = dO V^T, dS = P (dP - delta),
// dQ += scale dS K.
template <typename T, int D>
__global__ void __launch_bounds__(128) attn_bwd_q_kernel(const BwdArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t TILE = TB * D * 2;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int qb, bh, beg, end, slot;
    if (!work_item(a.tasks, a.task_info, a.row_ptr, a.NB, qb, bh, beg, end, slot)) return;
    const uint32_t sQ = smem_addr(smem), sDO = sQ + TILE, sKV = sDO + TILE;
    const size_t seq = (size_t)bh * a.L;
    const T* kbase = static_cast<const T*>(a.k) + seq * D;
    const T* vbase = static_cast<const T*>(a.v) + seq * D;
    const int n = end - beg;
    const int cnt_q = a.blk_cnt[qb];

    auto load_pair = [&](int stage, int j) {
        const uint32_t t = sKV + (uint32_t)stage * 2 * TILE;
        load_tile<T, D>(t, kbase + (size_t)j * TB * D, D, tid);
        load_tile<T, D>(t + TILE, vbase + (size_t)j * TB * D, D, tid);
    };
    load_tile<T, D>(sQ, static_cast<const T*>(a.q) + (seq + (size_t)qb * TB) * D, D, tid);
    load_tile<T, D>(sDO, static_cast<const T*>(a.dout) + (seq + (size_t)qb * TB) * D, D, tid);
    if (n > 0) load_pair(0, a.col_idx[beg]);
    cp_commit();

    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
    const float* lsep = a.lse + seq + (size_t)qb * TB;
    const float* dlp = a.delta + seq + (size_t)qb * TB;
    const float ls0 = lsep[r0] * LOG2E, ls1 = lsep[r1] * LOG2E, d0 = dlp[r0], d1 = dlp[r1];
    const bool ok0 = r0 < cnt_q && ls0 != -INFINITY, ok1 = r1 < cnt_q && ls1 != -INFINITY;
    float dq[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;
    for (int e = 0; e < n; ++e) {
        const int stage = e & 1;
        const uint32_t sK = sKV + (uint32_t)stage * 2 * TILE, sV = sK + TILE;
        const int kb = a.col_idx[beg + e];
        if (e + 1 < n) load_pair(stage ^ 1, a.col_idx[beg + e + 1]);
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        const int cnt_k = a.blk_cnt[kb];
        float s[8][4], dp[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
            dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
        }
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t qa[4], da[4];
            load_a<D>(sQ, warp * 16, ks, lane, qa);
            load_a<D>(sDO, warp * 16, ks, lane, da);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                load_b_nk<D>(sK, np, ks, lane, b);
                Elt<T>::mma(s[2 * np], qa, b[0], b[1]);
                Elt<T>::mma(s[2 * np + 1], qa, b[2], b[3]);
                load_b_nk<D>(sV, np, ks, lane, b);
                Elt<T>::mma(dp[2 * np], da, b[0], b[1]);
                Elt<T>::mma(dp[2 * np + 1], da, b[2], b[3]);
            }
        }
        uint32_t ds[8][2];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = i * 8 + 2 * (lane & 3);
            const bool c0 = c < cnt_k, c1 = c + 1 < cnt_k;
            const float p0 = (ok0 && c0) ? ex2(s[i][0] * a.scale_log2 - ls0) : 0.f;
            const float p1 = (ok0 && c1) ? ex2(s[i][1] * a.scale_log2 - ls0) : 0.f;
            const float p2 = (ok1 && c0) ? ex2(s[i][2] * a.scale_log2 - ls1) : 0.f;
            const float p3 = (ok1 && c1) ? ex2(s[i][3] * a.scale_log2 - ls1) : 0.f;
            ds[i][0] = Elt<T>::pack(p0 * (dp[i][0] - d0), p1 * (dp[i][1] - d0));
            ds[i][1] = Elt<T>::pack(p2 * (dp[i][2] - d1), p3 * (dp[i][3] - d1));
        }
#pragma unroll
        for (int kt = 0; kt < 4; ++kt) {
            const uint32_t da[4] = {ds[2 * kt][0], ds[2 * kt][1], ds[2 * kt + 1][0], ds[2 * kt + 1][1]};
#pragma unroll
            for (int dpi = 0; dpi < D / 16; ++dpi) {
                uint32_t b[4];
                load_b_kn<D>(sK, kt, dpi, lane, b);
                Elt<T>::mma(dq[2 * dpi], da, b[0], b[1]);
                Elt<T>::mma(dq[2 * dpi + 1], da, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    cp_wait<0>();
    if (slot >= 0) {
        store_part<D>(dq, a.part0 + (size_t)slot * TB * D, warp, lane, a.scale);
        return;
    }
    store_rows<T, D>(a, dq, a.d0, a.f0, a.add0, bh, qb, cnt_q, warp, lane, a.scale);
}

// ---------------------------------------------------------------------------------------------- host side
static int check_common(const char* name, int BH, int L, int D, int dtype) {
    if (BH <= 0 || L <= 0 || L % TB != 0) return set_error(-1, (std::string(name) + ": BH > 0 and L a positive multiple of 64").c_str());
    if (D != 64 && D != 128) return set_error(-1, (std::string(name) + ": head dim must be 64 or 128").c_str());
    if (dtype != 0 && dtype != 1) return set_error(-1, (std::string(name) + ": dtype must be 0 (bf16) or 1 (fp16)").c_str());
    return 0;
}

template <typename K> static int set_smem(K kern, size_t bytes) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    return e == cudaSuccess ? 0 : set_error(-2, cudaGetErrorString(e));
}

#define VSA_DISPATCH(KERNEL, SMEM, GRID, ARGS)                                                        \
    do {                                                                                              \
        int rc__ = 0;                                                                                 \
        if (dtype == 0 && D == 128) { if ((rc__ = set_smem(KERNEL<__nv_bfloat16, 128>, SMEM))) return rc__; KERNEL<__nv_bfloat16, 128><<<GRID, 128, SMEM, st>>>(ARGS); } \
        else if (dtype == 0) { if ((rc__ = set_smem(KERNEL<__nv_bfloat16, 64>, SMEM))) return rc__; KERNEL<__nv_bfloat16, 64><<<GRID, 128, SMEM, st>>>(ARGS); } \
        else if (D == 128) { if ((rc__ = set_smem(KERNEL<__half, 128>, SMEM))) return rc__; KERNEL<__half, 128><<<GRID, 128, SMEM, st>>>(ARGS); } \
        else { if ((rc__ = set_smem(KERNEL<__half, 64>, SMEM))) return rc__; KERNEL<__half, 64><<<GRID, 128, SMEM, st>>>(ARGS); } \
    } while (0)

}  // namespace vsa
}  // namespace es

using namespace es;
using namespace es::vsa;

extern "C" int es_vsa_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int32_t* row_ptr,
                               const int32_t* col_idx, const int32_t* blk_cnt, int32_t BH, int32_t L, int32_t D,
                               int32_t dtype, void* stream) {
    if (!q || !k || !v || !o || !lse || !row_ptr || !col_idx || !blk_cnt) return set_error(-1, "es_vsa_attn_fwd: null pointer");
    if (int rc = check_common("es_vsa_attn_fwd", BH, L, D, dtype)) return rc;
    FwdArgs a{q, k, v, o, lse, row_ptr, col_idx, blk_cnt, L, L / TB, LOG2E / sqrtf((float)D)};
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)5 * TB * D * 2;
    const dim3 grid(L / TB, BH);
    VSA_DISPATCH(attn_fwd_kernel, smem, grid, a);
    ES_CHECK_LAUNCH("attn_fwd_kernel");
    return 0;
}

static int fill_bwd(BwdArgs& a, const void* q, const void* k, const void* v, const void* dout, const float* lse,
                    const float* delta, const int32_t* row_ptr, const int32_t* col_idx, const int32_t* blk_cnt, int L,
                    int D) {
    a.q = q; a.k = k; a.v = v; a.dout = dout; a.lse = lse; a.delta = delta;
    a.row_ptr = row_ptr; a.col_idx = col_idx; a.blk_cnt = blk_cnt; a.L = L; a.NB = L / TB;
    a.scale = 1.f / sqrtf((float)D);
    a.scale_log2 = LOG2E * a.scale;
    return 0;
}

extern "C" int es_vsa_attn_bwd_kv(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                                  const float* delta, void* dk, void* dv, float* dk_f32, float* dv_f32,
                                  const float* add_dk, const float* add_dv, int32_t add_nb, const int32_t* k2q_ptr,
                                  const int32_t* k2q_idx, const int32_t* blk_cnt, int32_t BH, int32_t L, int32_t D,
                                  int32_t dtype, void* stream) {
    if (!q || !k || !v || !dout || !lse || !delta || !k2q_ptr || !k2q_idx || !blk_cnt)
        return set_error(-1, "es_vsa_attn_bwd_kv: null pointer");
    if ((!dk && !dk_f32) || (!dv && !dv_f32)) return set_error(-1, "es_vsa_attn_bwd_kv: no output for dK or dV");
    if ((add_dk || add_dv) && add_nb < L / TB) return set_error(-1, "es_vsa_attn_bwd_kv: add_nb smaller than the block count");
    if (int rc = check_common("es_vsa_attn_bwd_kv", BH, L, D, dtype)) return rc;
    BwdArgs a{};
    fill_bwd(a, q, k, v, dout, lse, delta, k2q_ptr, k2q_idx, blk_cnt, L, D);
    a.d0 = dk; a.d1 = dv; a.f0 = dk_f32; a.f1 = dv_f32; a.add0 = add_dk; a.add1 = add_dv; a.add_nb = add_nb;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)6 * TB * D * 2 + 2 * 128 * sizeof(float);
    const dim3 grid(L / TB, BH);
    VSA_DISPATCH(attn_bwd_kv_kernel, smem, grid, a);
    ES_CHECK_LAUNCH("attn_bwd_kv_kernel");
    return 0;
}

extern "C" int es_vsa_attn_bwd_q(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                                 const float* delta, void* dq, float* dq_f32, const float* add_dq, int32_t add_nb,
                                 const int32_t* q2k_ptr, const int32_t* q2k_idx, const int32_t* blk_cnt, int32_t BH,
                                 int32_t L, int32_t D, int32_t dtype, void* stream) {
    if (!q || !k || !v || !dout || !lse || !delta || !q2k_ptr || !q2k_idx || !blk_cnt)
        return set_error(-1, "es_vsa_attn_bwd_q: null pointer");
    if (!dq && !dq_f32) return set_error(-1, "es_vsa_attn_bwd_q: no output for dQ");
    if (add_dq && add_nb < L / TB) return set_error(-1, "es_vsa_attn_bwd_q: add_nb smaller than the block count");
    if (int rc = check_common("es_vsa_attn_bwd_q", BH, L, D, dtype)) return rc;
    BwdArgs a{};
    fill_bwd(a, q, k, v, dout, lse, delta, q2k_ptr, q2k_idx, blk_cnt, L, D);
    a.d0 = dq; a.f0 = dq_f32; a.add0 = add_dq; a.add_nb = add_nb;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)6 * TB * D * 2;
    const dim3 grid(L / TB, BH);
    VSA_DISPATCH(attn_bwd_q_kernel, smem, grid, a);
    ES_CHECK_LAUNCH("attn_bwd_q_kernel");
    return 0;
}

// ---------------------------------------------------------------------------------------------- split-KV task launches
static int check_tasks(const char* name, const int32_t* tasks, const int32_t* info, int n_tasks_cap) {
    if (!tasks || !info) return set_error(-1, (std::string(name) + ": null task list").c_str());
    if (n_tasks_cap <= 0) return set_error(-1, (std::string(name) + ": the task grid is empty").c_str());
    if ((uintptr_t)tasks & 15) return set_error(-1, (std::string(name) + ": tasks must be 16-byte aligned").c_str());
    return 0;
}

extern "C" int es_vsa_attn_fwd_tasks(const void* q, const void* k, const void* v, void* o, float* lse,
                                     const int32_t* q2k_idx, const int32_t* blk_cnt, const int32_t* tasks,
                                     const int32_t* task_info, int32_t n_tasks_cap, float* part_o, float* part_lse,
                                     int32_t BH, int32_t L, int32_t D, int32_t dtype, void* stream) {
    if (!q || !k || !v || !o || !lse || !q2k_idx || !blk_cnt) return set_error(-1, "es_vsa_attn_fwd_tasks: null pointer");
    if (int rc = check_common("es_vsa_attn_fwd_tasks", BH, L, D, dtype)) return rc;
    if (int rc = check_tasks("es_vsa_attn_fwd_tasks", tasks, task_info, n_tasks_cap)) return rc;
    FwdArgs a{q, k, v, o, lse, nullptr, q2k_idx, blk_cnt, L, L / TB, LOG2E / sqrtf((float)D), tasks, task_info, part_o, part_lse};
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)5 * TB * D * 2;
    const dim3 grid(n_tasks_cap, 1);
    VSA_DISPATCH(attn_fwd_kernel, smem, grid, a);
    ES_CHECK_LAUNCH("attn_fwd_kernel");
    return 0;
}

extern "C" int es_vsa_attn_bwd_kv_tasks(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                                        const float* delta, void* dk, void* dv, float* dk_f32, float* dv_f32,
                                        const float* add_dk, const float* add_dv, int32_t add_nb, const int32_t* k2q_idx,
                                        const int32_t* blk_cnt, const int32_t* tasks, const int32_t* task_info,
                                        int32_t n_tasks_cap, float* part_dk, float* part_dv, int32_t BH, int32_t L,
                                        int32_t D, int32_t dtype, void* stream) {
    if (!q || !k || !v || !dout || !lse || !delta || !k2q_idx || !blk_cnt)
        return set_error(-1, "es_vsa_attn_bwd_kv_tasks: null pointer");
    if ((!dk && !dk_f32) || (!dv && !dv_f32)) return set_error(-1, "es_vsa_attn_bwd_kv_tasks: no output for dK or dV");
    if ((add_dk || add_dv) && add_nb < L / TB) return set_error(-1, "es_vsa_attn_bwd_kv_tasks: add_nb smaller than the block count");
    if (int rc = check_common("es_vsa_attn_bwd_kv_tasks", BH, L, D, dtype)) return rc;
    if (int rc = check_tasks("es_vsa_attn_bwd_kv_tasks", tasks, task_info, n_tasks_cap)) return rc;
    BwdArgs a{};
    fill_bwd(a, q, k, v, dout, lse, delta, nullptr, k2q_idx, blk_cnt, L, D);
    a.d0 = dk; a.d1 = dv; a.f0 = dk_f32; a.f1 = dv_f32; a.add0 = add_dk; a.add1 = add_dv; a.add_nb = add_nb;
    a.tasks = tasks; a.task_info = task_info; a.part0 = part_dk; a.part1 = part_dv;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)6 * TB * D * 2 + 2 * 128 * sizeof(float);
    const dim3 grid(n_tasks_cap, 1);
    VSA_DISPATCH(attn_bwd_kv_kernel, smem, grid, a);
    ES_CHECK_LAUNCH("attn_bwd_kv_kernel");
    return 0;
}

extern "C" int es_vsa_attn_bwd_q_tasks(const void* q, const void* k, const void* v, const void* dout, const float* lse,
                                       const float* delta, void* dq, float* dq_f32, const float* add_dq, int32_t add_nb,
                                       const int32_t* q2k_idx, const int32_t* blk_cnt, const int32_t* tasks,
                                       const int32_t* task_info, int32_t n_tasks_cap, float* part_dq, int32_t BH,
                                       int32_t L, int32_t D, int32_t dtype, void* stream) {
    if (!q || !k || !v || !dout || !lse || !delta || !q2k_idx || !blk_cnt)
        return set_error(-1, "es_vsa_attn_bwd_q_tasks: null pointer");
    if (!dq && !dq_f32) return set_error(-1, "es_vsa_attn_bwd_q_tasks: no output for dQ");
    if (add_dq && add_nb < L / TB) return set_error(-1, "es_vsa_attn_bwd_q_tasks: add_nb smaller than the block count");
    if (int rc = check_common("es_vsa_attn_bwd_q_tasks", BH, L, D, dtype)) return rc;
    if (int rc = check_tasks("es_vsa_attn_bwd_q_tasks", tasks, task_info, n_tasks_cap)) return rc;
    BwdArgs a{};
    fill_bwd(a, q, k, v, dout, lse, delta, nullptr, q2k_idx, blk_cnt, L, D);
    a.d0 = dq; a.f0 = dq_f32; a.add0 = add_dq; a.add_nb = add_nb;
    a.tasks = tasks; a.task_info = task_info; a.part0 = part_dq;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)6 * TB * D * 2;
    const dim3 grid(n_tasks_cap, 1);
    VSA_DISPATCH(attn_bwd_q_kernel, smem, grid, a);
    ES_CHECK_LAUNCH("attn_bwd_q_kernel");
    return 0;
}
