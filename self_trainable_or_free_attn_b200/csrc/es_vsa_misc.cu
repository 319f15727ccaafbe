// VSA2 stages around the attention kernels: pooling, the PSP router (pooled-row LSE, block scores), the exact global
// top-k with its CSR lists in both directions, gate fusion forward / backward and the final gradient assembly.
// Reference: csrc/vsa/vsa2_kernels.h:179-302 of shaoshitong/self_trainable_or_free_attn (parameter structs of the same
// stages) and tests/vsa_reference.py:28-87 (what they compute). Vectorised loads, warp shuffles and, for the two router
// passes, mma.sync tiles; integer stages (top-k, CSR) are exact and deterministic.
#include <string>

#include "es_api_internal.h"
#include "es_vsa_mma.cuh"

namespace es {
namespace vsa {

// ---------------------------------------------------------------------------------------------- pooling
// One CTA per (block, bh): means of the R-token router groups of q and k (optionally v) over their valid tokens, and the
// block means of q, k, v, fp32 sums rounded once to the element type. Empty groups and the padding rows of the pooled
// tensors are zero.
struct PoolArgs {
    const void *q, *k, *v;
    void *qr, *kr, *vr, *qc, *kc, *vc;
    const int* blk_cnt;
    int L, NB, R, G, Lr_pad, NBc_pad;
};

template <typename T, int D>
__global__ void __launch_bounds__(D / 2) pool_kernel(const PoolArgs a) {
    const int blk = blockIdx.x, bh = blockIdx.y, c = 2 * threadIdx.x;
    const int tiles_c = a.NBc_pad, rows_r = a.Lr_pad;
    const void* src[3] = {a.q, a.k, a.v};
    void* dst_r[3] = {a.qr, a.kr, a.vr};
    void* dst_c[3] = {a.qc, a.kc, a.vc};
    if (blk >= a.NB) {                       // padding rows of the pooled tensors
#pragma unroll
        for (int t = 0; t < 3; ++t) {
            if (blk < tiles_c && dst_c[t])
                *reinterpret_cast<uint32_t*>(static_cast<T*>(dst_c[t]) + ((size_t)bh * tiles_c + blk) * D + c) = 0u;
            if (dst_r[t])
                for (int r = blk * a.G; r < (blk + 1) * a.G; ++r)
                    if (r < rows_r)
                        *reinterpret_cast<uint32_t*>(static_cast<T*>(dst_r[t]) + ((size_t)bh * rows_r + r) * D + c) = 0u;
        }
        return;
    }
    const int cnt = a.blk_cnt[blk];
#pragma unroll
    for (int t = 0; t < 3; ++t) {
        if (!src[t]) continue;
        const T* x = static_cast<const T*>(src[t]) + ((size_t)bh * a.L + (size_t)blk * TB) * D + c;
        float bx = 0.f, by = 0.f;
        for (int g = 0; g < a.G; ++g) {
            float sx = 0.f, sy = 0.f;
            const int lo = g * a.R, hi = min(lo + a.R, cnt);
            for (int r = lo; r < hi; ++r) {
                const float2 w = Elt<T>::unpack(*reinterpret_cast<const uint32_t*>(x + (size_t)r * D));
                sx += w.x; sy += w.y;
            }
            bx += sx; by += sy;
            if (dst_r[t]) {
                const float inv = hi > lo ? 1.f / (float)(hi - lo) : 0.f;
                *reinterpret_cast<uint32_t*>(static_cast<T*>(dst_r[t]) + ((size_t)bh * rows_r + blk * a.G + g) * D + c) =
                    Elt<T>::pack(sx * inv, sy * inv);
            }
        }
        if (dst_c[t]) {
            const float inv = 1.f / (float)cnt;
            *reinterpret_cast<uint32_t*>(static_cast<T*>(dst_c[t]) + ((size_t)bh * tiles_c + blk) * D + c) =
                Elt<T>::pack(bx * inv, by * inv);
        }
    }
}

// ---------------------------------------------------------------------------------------------- router
// Pooled rows: row r = blk * G + g is valid when group g of block blk holds a token (g * R < blk_cnt[blk]).
struct RouterArgs {
    const void *qr, *kr;
    float* lse2;          // [BH, Lr_pad] log2-domain LSE over the valid pooled keys
    float* scores;        // [bh_count, NB, NB]
    const int* blk_cnt;
    int NB, R, G, Lr, Lr_pad, bh0, row_norm;
    float scale_log2;
};

// MODE 0: lse2 of 64 pooled query rows over all pooled keys. MODE 1: block scores of the 64 / G query blocks of the tile:
// score[i][j] = sum over the groups a of i and b of j of 2^(s - lse2), times the row normalisation; the G x G sums are
// taken from a shared-memory copy of the probabilities in a fixed order (reproducible).
template <typename T, int D, int MODE>
__global__ void __launch_bounds__(128) router_kernel(const RouterArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr uint32_t TILE = TB * D * 2;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int qt = blockIdx.x, bh = a.bh0 + blockIdx.y;
    const uint32_t sQ = smem_addr(smem), sK = sQ + TILE;                 // K: two stages
    float* sP = reinterpret_cast<float*>(smem + 3 * TILE);               // MODE 1: [64][65] probabilities
    const T* q = static_cast<const T*>(a.qr) + ((size_t)bh * a.Lr_pad + (size_t)qt * TB) * D;
    const T* kbase = static_cast<const T*>(a.kr) + (size_t)bh * a.Lr_pad * D;
    const int nkt = a.Lr_pad / TB;
    load_tile<T, D>(sQ, q, D, tid);
    load_tile<T, D>(sK, kbase, D, tid);
    cp_commit();
    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f, ls0 = 0.f, ls1 = 0.f;
    if (MODE == 1) {
        const float* lse = a.lse2 + (size_t)bh * a.Lr_pad + (size_t)qt * TB;
        ls0 = lse[r0]; ls1 = lse[r1];
    }
    uint32_t qa[D / 16][4];
    for (int kt = 0; kt < nkt; ++kt) {
        const uint32_t sKt = sK + (uint32_t)(kt & 1) * TILE;
        if (kt + 1 < nkt) load_tile<T, D>(sK + (uint32_t)((kt + 1) & 1) * TILE, kbase + (size_t)(kt + 1) * TB * D, D, tid);
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        if (kt == 0) {
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
                load_b_nk<D>(sKt, np, ks, lane, b);
                Elt<T>::mma(s[2 * np], qa[ks], b[0], b[1]);
                Elt<T>::mma(s[2 * np + 1], qa[ks], b[2], b[3]);
            }
        // validity of the pooled keys of this tile
        bool kv[8][2];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int r = kt * TB + i * 8 + 2 * (lane & 3) + u;
                kv[i][u] = r < a.Lr && (r % a.G) * a.R < a.blk_cnt[r / a.G];
            }
        if (MODE == 0) {
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                s[i][0] = kv[i][0] ? s[i][0] * a.scale_log2 : -INFINITY;
                s[i][1] = kv[i][1] ? s[i][1] * a.scale_log2 : -INFINITY;
                s[i][2] = kv[i][0] ? s[i][2] * a.scale_log2 : -INFINITY;
                s[i][3] = kv[i][1] ? s[i][3] * a.scale_log2 : -INFINITY;
                mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
                mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
            }
            const float mn0 = fmaxf(m0, quad_max(mx0)), mn1 = fmaxf(m1, quad_max(mx1));
            const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
            float t0 = 0.f, t1 = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                t0 += exp2f(s[i][0] - ms0) + exp2f(s[i][1] - ms0);
                t1 += exp2f(s[i][2] - ms1) + exp2f(s[i][3] - ms1);
            }
            l0 = l0 * exp2f(m0 - ms0) + t0; l1 = l1 * exp2f(m1 - ms1) + t1;
            m0 = mn0; m1 = mn1;
        } else {
            // probabilities of this key tile -> shared memory, then fixed-order G x G sums
            const int qrow0 = qt * TB + r0, qrow1 = qt * TB + r1;
            const bool qv0 = qrow0 < a.Lr && (qrow0 % a.G) * a.R < a.blk_cnt[qrow0 / a.G];
            const bool qv1 = qrow1 < a.Lr && (qrow1 % a.G) * a.R < a.blk_cnt[qrow1 / a.G];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int c = i * 8 + 2 * (lane & 3);
                sP[r0 * 65 + c] = (qv0 && kv[i][0]) ? exp2f(s[i][0] * a.scale_log2 - ls0) : 0.f;
                sP[r0 * 65 + c + 1] = (qv0 && kv[i][1]) ? exp2f(s[i][1] * a.scale_log2 - ls0) : 0.f;
                sP[r1 * 65 + c] = (qv1 && kv[i][0]) ? exp2f(s[i][2] * a.scale_log2 - ls1) : 0.f;
                sP[r1 * 65 + c + 1] = (qv1 && kv[i][1]) ? exp2f(s[i][3] * a.scale_log2 - ls1) : 0.f;
            }
            __syncthreads();
            const int per = TB / a.G;                        // blocks per tile side
            for (int e = tid; e < per * per; e += 128) {
                const int bi = e / per, bj = e % per;
                const int qblk = qt * per + bi, kblk = kt * per + bj;
                if (qblk < a.NB && kblk < a.NB) {
                    float acc = 0.f;
                    for (int x = 0; x < a.G; ++x)
                        for (int y = 0; y < a.G; ++y) acc += sP[(bi * a.G + x) * 65 + bj * a.G + y];
                    float norm;
                    if (a.row_norm == 1) norm = 1.f / (float)(a.G * a.G);
                    else norm = 1.f / (float)((a.blk_cnt[qblk] + a.R - 1) / a.R);
                    a.scores[((size_t)blockIdx.y * a.NB + qblk) * a.NB + kblk] = acc * norm;
                }
            }
        }
        __syncthreads();
    }
    cp_wait<0>();
    if (MODE == 0) {
        l0 = quad_sum(l0); l1 = quad_sum(l1);
        if ((lane & 3) == 0) {
            float* lse = a.lse2 + (size_t)bh * a.Lr_pad + (size_t)qt * TB;
            lse[r0] = l0 > 0.f ? m0 + log2f(l0) : -INFINITY;
            lse[r1] = l1 > 0.f ? m1 + log2f(l1) : -INFINITY;
        }
    }
}

// ---------------------------------------------------------------------------------------------- exact global top-k
// Per (b, h): the `budget` largest of the NB x NB scores in the order (score descending, flat index ascending). Scores are
// non-negative, so their bit patterns order like the values. Stages: (1) 4-pass radix select of the threshold key and the
// number of entries equal to it that are taken; (2) per row, counts of larger and equal entries; (3) scans: equal-rank base
// of every row, row pointers; (4) per row, the ascending list and the selection bitmap; (5) per column, count, scan, list.
struct TopkArgs {
    const float* scores;    // [bh_count, NB, NB]
    int NB, W, bh0;
    long long budget;       // clamped to NB * NB
    int *q2k_ptr, *q2k_idx, *k2q_ptr, *k2q_idx;
    int* state;             // [bh_count, 4]: threshold key, equal entries to take
    int *gtcnt, *eqcnt, *eqbase, *colcnt;     // [bh_count, NB] each
    uint32_t* selbits;      // [bh_count, NB, W]
};

__device__ __forceinline__ uint32_t score_key(float x) {
    x += 0.0f;                                     // -0 -> +0
    const uint32_t u = __float_as_uint(x);
    return (u & 0x80000000u) ? 0u : u;             // negative values (never produced by the router) order as zero
}

__global__ void __launch_bounds__(1024) topk_select_kernel(const TopkArgs a) {
    __shared__ uint32_t hist[256];
    __shared__ uint32_t s_prefix, s_need;
    const int b = blockIdx.x, tid = threadIdx.x;
    const float* sc = a.scores + (size_t)b * a.NB * a.NB;
    const long long N = (long long)a.NB * a.NB;
    if (tid == 0) { s_prefix = 0; s_need = (uint32_t)a.budget; }
    __syncthreads();
    if (a.budget <= 0) {
        if (tid == 0) { a.state[b * 4] = (int)0xFFFFFFFFu; a.state[b * 4 + 1] = 0; }
        return;
    }
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix, mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
        for (long long i = tid; i < N; i += 1024) {
            const uint32_t key = score_key(sc[i]);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            uint32_t need = s_need, d = 255;
            for (;; --d) {
                if (hist[d] >= need) break;
                need -= hist[d];
                if (d == 0) break;
            }
            s_prefix = prefix | (d << shift);
            s_need = need;
        }
        __syncthreads();
    }
    if (tid == 0) { a.state[b * 4] = (int)s_prefix; a.state[b * 4 + 1] = (int)s_need; }
}

// one warp per row
__global__ void __launch_bounds__(128) topk_count_kernel(const TopkArgs a) {
    const int b = blockIdx.y, row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= a.NB) return;
    const uint32_t thr = (uint32_t)a.state[b * 4];
    const float* sc = a.scores + ((size_t)b * a.NB + row) * a.NB;
    int gt = 0, eq = 0;
    for (int j = lane; j < a.NB; j += 32) {
        const uint32_t key = score_key(sc[j]);
        gt += key > thr; eq += key == thr;
    }
    for (int o = 16; o > 0; o >>= 1) {
        gt += __shfl_xor_sync(0xffffffffu, gt, o);
        eq += __shfl_xor_sync(0xffffffffu, eq, o);
    }
    if (lane == 0) { a.gtcnt[b * a.NB + row] = gt; a.eqcnt[b * a.NB + row] = eq; }
}

// one CTA per (b, h): exclusive scans over the rows (kind 0: rows -> eqbase and q2k_ptr; kind 1: columns -> k2q_ptr)
__global__ void __launch_bounds__(1024) topk_scan_kernel(const TopkArgs a, int kind) {
    __shared__ int part[1024];
    const int b = blockIdx.x, tid = threadIdx.x, bh = a.bh0 + b;
    const int per = (a.NB + 1023) / 1024, lo = tid * per, hi = min(lo + per, a.NB);
    const int need = a.state[b * 4 + 1];
    const long long base = (long long)bh * a.budget;
    auto scan = [&](int v) -> int {          // exclusive prefix of v over the threads
        part[tid] = v;
        __syncthreads();
        for (int o = 1; o < 1024; o <<= 1) {
            const int x = tid >= o ? part[tid - o] : 0;
            __syncthreads();
            part[tid] += x;
            __syncthreads();
        }
        const int r = part[tid] - v;
        __syncthreads();
        return r;
    };
    if (kind == 0) {
        int se = 0;
        for (int r = lo; r < hi; ++r) se += a.eqcnt[b * a.NB + r];
        int eb = scan(se);
        int sc = 0;
        for (int r = lo; r < hi; ++r) {
            a.eqbase[b * a.NB + r] = eb;
            const int e = a.eqcnt[b * a.NB + r];
            sc += a.gtcnt[b * a.NB + r] + max(0, min(e, need - eb));
            eb += e;
        }
        int pos = scan(sc);
        eb = a.eqbase[b * a.NB + (lo < a.NB ? lo : 0)];
        for (int r = lo; r < hi; ++r) {
            a.q2k_ptr[(size_t)bh * (a.NB + 1) + r] = (int)(base + pos);
            const int e = a.eqcnt[b * a.NB + r];
            pos += a.gtcnt[b * a.NB + r] + max(0, min(e, need - eb));
            eb += e;
        }
        if (tid == 1023) a.q2k_ptr[(size_t)bh * (a.NB + 1) + a.NB] = (int)(base + pos);   // the last thread ends at the total
    } else {
        int sc = 0;
        for (int r = lo; r < hi; ++r) sc += a.colcnt[b * a.NB + r];
        int pos = scan(sc);
        for (int r = lo; r < hi; ++r) {
            a.k2q_ptr[(size_t)bh * (a.NB + 1) + r] = (int)(base + pos);
            pos += a.colcnt[b * a.NB + r];
        }
        if (tid == 1023) a.k2q_ptr[(size_t)bh * (a.NB + 1) + a.NB] = (int)(base + pos);
    }
}

// one warp per row: the ascending kv list and the selection bits
__global__ void __launch_bounds__(128) topk_emit_rows_kernel(const TopkArgs a) {
    const int b = blockIdx.y, row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31, bh = a.bh0 + b;
    if (row >= a.NB) return;
    const uint32_t thr = (uint32_t)a.state[b * 4];
    const int need = a.state[b * 4 + 1];
    const float* sc = a.scores + ((size_t)b * a.NB + row) * a.NB;
    int eqrank = a.eqbase[b * a.NB + row];
    int pos = a.q2k_ptr[(size_t)bh * (a.NB + 1) + row];
    for (int j0 = 0; j0 < a.NB; j0 += 32) {
        const int j = j0 + lane;
        const uint32_t key = j < a.NB ? score_key(sc[j]) : 0u;
        const bool gt = j < a.NB && key > thr, eq = j < a.NB && key == thr;
        const unsigned em = __ballot_sync(0xffffffffu, eq);
        const bool take = gt || (eq && eqrank + __popc(em & ((1u << lane) - 1)) < need);
        const unsigned tm = __ballot_sync(0xffffffffu, take);
        if (take) a.q2k_idx[pos + __popc(tm & ((1u << lane) - 1))] = j;
        if (lane == 0) a.selbits[((size_t)b * a.NB + row) * a.W + (j0 >> 5)] = tm;
        pos += __popc(tm);
        eqrank += __popc(em);
    }
}

// one thread per column: count (pass 0) or emit the ascending query list (pass 1)
__global__ void __launch_bounds__(128) topk_cols_kernel(const TopkArgs a, int pass) {
    const int b = blockIdx.y, col = blockIdx.x * 128 + threadIdx.x, bh = a.bh0 + b;
    if (col >= a.NB) return;
    const uint32_t* bits = a.selbits + (size_t)b * a.NB * a.W + (col >> 5);
    const uint32_t m = 1u << (col & 31);
    if (pass == 0) {
        int n = 0;
        for (int r = 0; r < a.NB; ++r) n += (bits[(size_t)r * a.W] & m) != 0;
        a.colcnt[b * a.NB + col] = n;
    } else {
        int pos = a.k2q_ptr[(size_t)bh * (a.NB + 1) + col];
        for (int r = 0; r < a.NB; ++r)
            if (bits[(size_t)r * a.W] & m) a.k2q_idx[pos++] = r;
    }
}

// ---------------------------------------------------------------------------------------------- original-VSA router
// Whole-block scores in the original's rounding (reference: BlockScoreParams, csrc/vsa/vsa2_kernels.h:243-253):
// S = rnd(rnd(qc . kc) * scale), rnd = round to the element type, scale = the fp32 reciprocal of sqrt(D): what Torch's
// `(q_c @ k_c^T) / sqrt(D)` computes in bf16 / fp16 (fp32-accumulated product rounded once, then multiplied by the fp32
// reciprocal of the scalar and rounded again). One thread per score; the means are small and stay in cache.
struct BlockScoreArgs {
    const void *qc, *kc;
    void* scores;            // [bh_count, NB, NB] element type
    int NB, NBc_pad, bh0;
    float inv_scale;
};
template <typename T, int D>
__global__ void __launch_bounds__(128) block_scores_kernel(const BlockScoreArgs a) {
    const int j = blockIdx.x * 128 + threadIdx.x, i = blockIdx.y, b = blockIdx.z, bh = a.bh0 + b;
    if (j >= a.NB) return;
    const T* q = static_cast<const T*>(a.qc) + ((size_t)bh * a.NBc_pad + i) * D;
    const T* k = static_cast<const T*>(a.kc) + ((size_t)bh * a.NBc_pad + j) * D;
    float acc = 0.f;
#pragma unroll 8
    for (int d = 0; d < D; d += 2) {
        const float2 x = Elt<T>::unpack(*reinterpret_cast<const uint32_t*>(q + d));
        const float2 y = Elt<T>::unpack(*reinterpret_cast<const uint32_t*>(k + d));
        acc = fmaf(x.x, y.x, acc);
        acc = fmaf(x.y, y.y, acc);
    }
    const float once = Elt<T>::to_float(Elt<T>::from_float(acc));
    static_cast<T*>(a.scores)[((size_t)b * a.NB + i) * a.NB + j] = Elt<T>::from_float(once * a.inv_scale);
}

// Per query row: exactly K = min(topk, NB) kv blocks, larger score first, ties to the smaller kv index, -0 == +0
// (reference: RowTopkParams, csrc/vsa/vsa2_kernels.h:255-270). One CTA per row: two-pass radix select of the K-th largest
// 16-bit key, then the ascending list and the selection bits. Row r of (b, h) owns idx[((b, h) * NB + r) * K ..).
struct RowTopkArgs {
    const uint16_t* scores;  // [bh_count, NB, NB]
    int NB, W, bh0, K, fp16;
    int *q2k_ptr, *q2k_idx;
    uint32_t* selbits;       // [bh_count, NB, W]
};
__device__ __forceinline__ uint32_t key16(uint16_t u, int fp16) {
    // bf16 and fp16 order like their bit patterns once the sign is handled; -0 becomes +0
    if ((u & 0x7FFFu) == 0) u = 0;
    (void)fp16;
    return (u & 0x8000u) ? (uint32_t)(uint16_t)~u : (uint32_t)(u | 0x8000u);
}
__global__ void __launch_bounds__(128) row_topk_kernel(const RowTopkArgs a) {
    __shared__ uint32_t hist[256];
    __shared__ uint32_t s_prefix, s_need;
    __shared__ int warp_gt[4], warp_eq[4];
    const int row = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, bh = a.bh0 + b;
    const uint16_t* sc = a.scores + ((size_t)b * a.NB + row) * a.NB;
    const long long base = ((long long)bh * a.NB + row) * a.K;
    if (tid == 0) {
        a.q2k_ptr[(size_t)bh * (a.NB + 1) + row] = (int)base;
        if (row == a.NB - 1) a.q2k_ptr[(size_t)bh * (a.NB + 1) + a.NB] = (int)(base + a.K);
        s_prefix = 0; s_need = (uint32_t)a.K;
    }
    __syncthreads();
    uint32_t thr = 0xFFFFFFFFu;
    int need = 0;
    if (a.K > 0) {
        for (int pass = 0; pass < 2; ++pass) {
            const int shift = 8 - 8 * pass;
            for (int x = tid; x < 256; x += 128) hist[x] = 0;
            __syncthreads();
            const uint32_t prefix = s_prefix, mask = pass == 0 ? 0u : 0xFF00u;
            for (int j = tid; j < a.NB; j += 128) {
                const uint32_t key = key16(sc[j], a.fp16);
                if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                uint32_t nd = s_need, d = 255;
                for (;; --d) {
                    if (hist[d] >= nd) break;
                    nd -= hist[d];
                    if (d == 0) break;
                }
                s_prefix = prefix | (d << shift);
                s_need = nd;
            }
            __syncthreads();
        }
        thr = s_prefix; need = (int)s_need;
    }
    // ascending emission, 128 columns at a time
    int pos = 0, eqrank = 0;
    for (int j0 = 0; j0 < a.NB; j0 += 128) {
        const int j = j0 + tid;
        const uint32_t key = j < a.NB ? key16(sc[j], a.fp16) : 0u;
        const bool gt = j < a.NB && a.K > 0 && key > thr, eq = j < a.NB && a.K > 0 && key == thr;
        const unsigned gm = __ballot_sync(0xffffffffu, gt), em = __ballot_sync(0xffffffffu, eq);
        if (lane == 0) { warp_gt[warp] = __popc(gm); warp_eq[warp] = __popc(em); }
        __syncthreads();
        int eq_before = eqrank, take_before = 0;
        for (int w = 0; w < warp; ++w) eq_before += warp_eq[w];
        const int my_eq = eq_before + __popc(em & ((1u << lane) - 1));
        const bool take = gt || (eq && my_eq < need);
        const unsigned tm = __ballot_sync(0xffffffffu, take);
        // positions: takes of the earlier warps of this chunk = their gt + their eq clipped to the remaining need
        int run_eq = eqrank;
        for (int w = 0; w < warp; ++w) {
            take_before += warp_gt[w] + max(0, min(warp_eq[w], need - run_eq));
            run_eq += warp_eq[w];
        }
        if (take) a.q2k_idx[base + pos + take_before + __popc(tm & ((1u << lane) - 1))] = j;
        if (lane == 0 && j0 + 32 * warp < a.W * 32) a.selbits[((size_t)b * a.NB + row) * a.W + (j0 >> 5) + warp] = tm;
        int chunk_take = 0, chunk_eq = 0, r2 = eqrank;
        for (int w = 0; w < 4; ++w) {
            chunk_take += warp_gt[w] + max(0, min(warp_eq[w], need - r2));
            r2 += warp_eq[w];
            chunk_eq += warp_eq[w];
        }
        pos += chunk_take; eqrank += chunk_eq;
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------- gate fusion
// gate_mode: 0 none (weight 1), 1 one value per token [BH, L], 2 one per element [BH, L, D]; gate_act: 0 tanh, 1 identity.
struct FuseArgs {
    const void *of, *oc, *gate, *dout;
    void *o, *dout_f, *dout_c, *dgate;
    float *delta_f, *delta_c;
    const int* blk_cnt;
    int L, NB, NBc_pad, gate_mode, gate_act;
};

template <typename T, int D>
__global__ void __launch_bounds__(D / 2) fuse_fwd_kernel(const FuseArgs a) {
    const int blk = blockIdx.x, bh = blockIdx.y, c = 2 * threadIdx.x;
    const int cnt = a.blk_cnt[blk];
    const float2 oc = Elt<T>::unpack(*reinterpret_cast<const uint32_t*>(static_cast<const T*>(a.oc) + ((size_t)bh * a.NBc_pad + blk) * D + c));
    for (int r = 0; r < TB; ++r) {
        const size_t row = (size_t)bh * a.L + (size_t)blk * TB + r;
        uint32_t out = 0u;
        if (r < cnt) {
            const float2 f = Elt<T>::unpack(*reinterpret_cast<const uint32_t*>(static_cast<const T*>(a.of) + row * D + c));
            float gx = 1.f, gy = 1.f;
            if (a.gate_mode == 1) gx = gy = Elt<T>::to_float(static_cast<const T*>(a.gate)[row]);
            else if (a.gate_mode == 2) {
                const float2 g = Elt<T>::unpack(*reinterpret_cast<const uint32_t*>(static_cast<const T*>(a.gate) + row * D + c));
                gx = g.x; gy = g.y;
            }
            if (a.gate_mode != 0 && a.gate_act == 0) { gx = tanhf(gx); gy = tanhf(gy); }
            out = Elt<T>::pack(f.x + gx * oc.x, f.y + gy * oc.y);
        }
        *reinterpret_cast<uint32_t*>(static_cast<T*>(a.o) + row * D + c) = out;
    }
}

// One CTA per (block, bh), D / 2 threads: delta_f = rowsum(dO O_f); dO_c = sum over the block's valid rows of w dO;
// delta_c = rowsum(dO_c O_c); dgate = act'(g) * (dO . O_c) per token or per element; dout_f = dO on valid rows, else 0.
template <typename T, int D>
__global__ void __launch_bounds__(D / 2) fuse_bwd_kernel(const FuseArgs a) {
    __shared__ float red[2][D / 64];
    const int blk = blockIdx.x, bh = blockIdx.y, tid = threadIdx.x, c = 2 * tid, warp = tid >> 5, lane = tid & 31;
    const int cnt = a.blk_cnt[blk];
    const float2 oc = Elt<T>::unpack(*reinterpret_cast<const uint32_t*>(static_cast<const T*>(a.oc) + ((size_t)bh * a.NBc_pad + blk) * D + c));
    float cx = 0.f, cy = 0.f;
    auto block_sum = [&](float v, int slot) -> float {
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) red[slot][warp] = v;
        __syncthreads();
        float t = 0.f;
        for (int w = 0; w < D / 64; ++w) t += red[slot][w];
        __syncthreads();
        return t;
    };
    for (int r = 0; r < TB; ++r) {
        const size_t row = (size_t)bh * a.L + (size_t)blk * TB + r;
        const bool ok = r < cnt;
        float2 d = make_float2(0.f, 0.f), f = make_float2(0.f, 0.f);
        if (ok) {
            d = Elt<T>::unpack(*reinterpret_cast<const uint32_t*>(static_cast<const T*>(a.dout) + row * D + c));
            f = Elt<T>::unpack(*reinterpret_cast<const uint32_t*>(static_cast<const T*>(a.of) + row * D + c));
        }
        if (a.dout_f) *reinterpret_cast<uint32_t*>(static_cast<T*>(a.dout_f) + row * D + c) = ok ? Elt<T>::pack(d.x, d.y) : 0u;
        float gx = 1.f, gy = 1.f, rx = 1.f, ry = 1.f;       // weight and its derivative factor
        if (a.gate_mode == 1) gx = gy = Elt<T>::to_float(static_cast<const T*>(a.gate)[row]);
        else if (a.gate_mode == 2) {
            const float2 g = Elt<T>::unpack(*reinterpret_cast<const uint32_t*>(static_cast<const T*>(a.gate) + row * D + c));
            gx = g.x; gy = g.y;
        }
        if (a.gate_mode != 0 && a.gate_act == 0) {
            gx = tanhf(gx); gy = tanhf(gy);
            rx = 1.f - gx * gx; ry = 1.f - gy * gy;
        }
        const float df = block_sum(d.x * f.x + d.y * f.y, 0);
        if (tid == 0) a.delta_f[row] = ok ? df : 0.f;
        if (a.gate_mode == 1) {
            const float dg = block_sum(d.x * oc.x + d.y * oc.y, 1);
            if (tid == 0) static_cast<T*>(a.dgate)[row] = Elt<T>::from_float(ok ? dg * rx : 0.f);
        } else if (a.gate_mode == 2) {
            *reinterpret_cast<uint32_t*>(static_cast<T*>(a.dgate) + row * D + c) =
                ok ? Elt<T>::pack(d.x * oc.x * rx, d.y * oc.y * ry) : 0u;
        }
        cx += gx * d.x; cy += gy * d.y;
    }
    // the coarse branch sees dO_c rounded to the element type, like every tensor that crosses a kernel boundary
    const uint32_t packed = Elt<T>::pack(cx, cy);
    *reinterpret_cast<uint32_t*>(static_cast<T*>(a.dout_c) + ((size_t)bh * a.NBc_pad + blk) * D + c) = packed;
    const float2 dc = Elt<T>::unpack(packed);
    const float t = block_sum(dc.x * oc.x + dc.y * oc.y, 0);
    if (tid == 0) a.delta_c[(size_t)bh * a.NBc_pad + blk] = t;
}

// out = valid ? acc + add[block] / count : 0, cast to the element type (acc and add optional).
struct FinalArgs {
    const float *acc, *add;
    void* out;
    const int* blk_cnt;
    int L, add_nb;
};
template <typename T, int D>
__global__ void __launch_bounds__(D / 2) finalize_kernel(const FinalArgs a) {
    const int blk = blockIdx.x, bh = blockIdx.y, c = 2 * threadIdx.x;
    const int cnt = a.blk_cnt[blk];
    float ax = 0.f, ay = 0.f;
    if (a.add) {
        const float* p = a.add + ((size_t)bh * a.add_nb + blk) * D + c;
        ax = p[0] / (float)cnt; ay = p[1] / (float)cnt;
    }
    for (int r = 0; r < TB; ++r) {
        const size_t row = (size_t)bh * a.L + (size_t)blk * TB + r;
        uint32_t out = 0u;
        if (r < cnt) {
            float x = ax, y = ay;
            if (a.acc) { x += a.acc[row * D + c]; y += a.acc[row * D + c + 1]; }
            out = Elt<T>::pack(x, y);
        }
        *reinterpret_cast<uint32_t*>(static_cast<T*>(a.out) + row * D + c) = out;
    }
}

static int check_shape(const char* name, int BH, int L, int D, int dtype) {
    if (BH <= 0 || L <= 0 || L % TB != 0) return set_error(-1, (std::string(name) + ": BH > 0 and L a positive multiple of 64").c_str());
    if (D != 64 && D != 128) return set_error(-1, (std::string(name) + ": head dim must be 64 or 128").c_str());
    if (dtype != 0 && dtype != 1) return set_error(-1, (std::string(name) + ": dtype must be 0 (bf16) or 1 (fp16)").c_str());
    return 0;
}

#define VSA_LAUNCH(KERNEL, GRID, THREADS, SMEM, ARGS)                                              \
    do {                                                                                           \
        if (dtype == 0 && D == 128) KERNEL<__nv_bfloat16, 128><<<GRID, THREADS, SMEM, st>>>(ARGS);  \
        else if (dtype == 0) KERNEL<__nv_bfloat16, 64><<<GRID, THREADS, SMEM, st>>>(ARGS);          \
        else if (D == 128) KERNEL<__half, 128><<<GRID, THREADS, SMEM, st>>>(ARGS);                  \
        else KERNEL<__half, 64><<<GRID, THREADS, SMEM, st>>>(ARGS);                                 \
    } while (0)

}  // namespace vsa
}  // namespace es

using namespace es;
using namespace es::vsa;

extern "C" int es_vsa_pool(const void* q, const void* k, const void* v, void* qr, void* kr, void* vr, void* qc, void* kc,
                           void* vc, const int32_t* blk_cnt, int32_t BH, int32_t L, int32_t D, int32_t R, int32_t Lr_pad,
                           int32_t NBc_pad, int32_t dtype, void* stream) {
    if ((!q && !k && !v) || !blk_cnt) return set_error(-1, "es_vsa_pool: null pointer");
    if ((!q && (qr || qc)) || (!k && (kr || kc))) return set_error(-1, "es_vsa_pool: an output without its input");
    if (int rc = check_shape("es_vsa_pool", BH, L, D, dtype)) return rc;
    if (R < 1 || R > 64 || 64 % R != 0) return set_error(-1, "es_vsa_pool: R must divide 64");
    const int NB = L / TB, G = 64 / R;
    if (Lr_pad < NB * G || NBc_pad < NB) return set_error(-1, "es_vsa_pool: padded sizes smaller than the real ones");
    if ((vr || vc) && !v) return set_error(-1, "es_vsa_pool: v outputs without v");
    PoolArgs a{q, k, v, qr, kr, vr, qc, kc, vc, blk_cnt, L, NB, R, G, Lr_pad, NBc_pad};
    cudaStream_t st = (cudaStream_t)stream;
    const int rows = max(max(NB, NBc_pad), (Lr_pad + G - 1) / G);
    const dim3 grid(rows, BH);
    VSA_LAUNCH(pool_kernel, grid, D / 2, 0, a);
    ES_CHECK_LAUNCH("pool_kernel");
    return 0;
}

template <int MODE>
static int launch_router(const RouterArgs& a, int D, int dtype, int bh_count, cudaStream_t st) {
    const size_t smem = (size_t)3 * TB * D * 2 + (MODE == 1 ? 64 * 65 * sizeof(float) : 0);
    const dim3 grid(a.Lr_pad / TB, bh_count);
#define ROUTER_CASE(TT, DD)                                                                                             \
    {                                                                                                                   \
        cudaError_t e = cudaFuncSetAttribute(router_kernel<TT, DD, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e != cudaSuccess) return set_error(-2, cudaGetErrorString(e));                                              \
        router_kernel<TT, DD, MODE><<<grid, 128, smem, st>>>(a);                                                        \
    }
    if (dtype == 0 && D == 128) ROUTER_CASE(__nv_bfloat16, 128)
    else if (dtype == 0) ROUTER_CASE(__nv_bfloat16, 64)
    else if (D == 128) ROUTER_CASE(__half, 128)
    else ROUTER_CASE(__half, 64)
#undef ROUTER_CASE
    ES_CHECK_LAUNCH("router_kernel");
    return 0;
}

extern "C" int es_vsa_router_lse(const void* qr, const void* kr, float* lse2, const int32_t* blk_cnt, int32_t BH,
                                 int32_t NB, int32_t D, int32_t R, int32_t Lr_pad, int32_t dtype, void* stream) {
    if (!qr || !kr || !lse2 || !blk_cnt) return set_error(-1, "es_vsa_router_lse: null pointer");
    if (int rc = check_shape("es_vsa_router_lse", BH, NB * TB, D, dtype)) return rc;
    if (R < 1 || R > 64 || 64 % R != 0 || Lr_pad % TB != 0 || Lr_pad < NB * (64 / R))
        return set_error(-1, "es_vsa_router_lse: R must divide 64 and Lr_pad be a multiple of 64 covering NB * 64 / R");
    RouterArgs a{qr, kr, lse2, nullptr, blk_cnt, NB, R, 64 / R, NB * (64 / R), Lr_pad, 0, 1, LOG2E / sqrtf((float)D)};
    return launch_router<0>(a, D, dtype, BH, (cudaStream_t)stream);
}

extern "C" int es_vsa_router_scores(const void* qr, const void* kr, const float* lse2, float* scores,
                                    const int32_t* blk_cnt, int32_t BH, int32_t NB, int32_t D, int32_t R, int32_t Lr_pad,
                                    int32_t bh0, int32_t bh_count, int32_t row_norm, int32_t dtype, void* stream) {
    if (!qr || !kr || !lse2 || !scores || !blk_cnt) return set_error(-1, "es_vsa_router_scores: null pointer");
    if (int rc = check_shape("es_vsa_router_scores", BH, NB * TB, D, dtype)) return rc;
    if (R < 1 || R > 64 || 64 % R != 0 || Lr_pad % TB != 0 || Lr_pad < NB * (64 / R))
        return set_error(-1, "es_vsa_router_scores: R must divide 64 and Lr_pad be a multiple of 64 covering NB * 64 / R");
    if (bh0 < 0 || bh_count < 1 || bh0 + bh_count > BH) return set_error(-1, "es_vsa_router_scores: bad (b, h) range");
    if (row_norm != 0 && row_norm != 1) return set_error(-1, "es_vsa_router_scores: row_norm must be 0 or 1");
    RouterArgs a{qr, kr, const_cast<float*>(lse2), scores, blk_cnt, NB, R, 64 / R, NB * (64 / R), Lr_pad, bh0, row_norm,
                 LOG2E / sqrtf((float)D)};
    return launch_router<1>(a, D, dtype, bh_count, (cudaStream_t)stream);
}

extern "C" long long es_vsa_topk_workspace_bytes(int32_t bh_count, int32_t NB) {
    if (bh_count <= 0 || NB <= 0) return 0;
    const long long W = (NB + 31) / 32;
    return (long long)bh_count * (4 + 4LL * NB + W * NB) * 4;
}

// Byte offset of the selection bitmap [bh_count, NB, ceil(NB / 32)] that es_vsa_global_topk leaves in its workspace.
extern "C" long long es_vsa_topk_bits_offset(int32_t bh_count, int32_t NB) {
    if (bh_count <= 0 || NB <= 0) return 0;
    return (long long)bh_count * (4 + 4LL * NB) * 4;
}

extern "C" int es_vsa_global_topk(const float* scores, int32_t NB, int32_t bh0, int32_t bh_count, long long budget,
                                  int32_t* q2k_ptr, int32_t* q2k_idx, int32_t* k2q_ptr, int32_t* k2q_idx, void* workspace,
                                  void* stream) {
    if (!scores || !q2k_ptr || !q2k_idx || !k2q_ptr || !k2q_idx || !workspace)
        return set_error(-1, "es_vsa_global_topk: null pointer");
    if (NB <= 0 || bh_count <= 0 || bh0 < 0) return set_error(-1, "es_vsa_global_topk: bad sizes");
    if (budget < 0 || budget > (long long)NB * NB) return set_error(-1, "es_vsa_global_topk: budget outside [0, NB * NB]");
    if ((long long)(bh0 + bh_count) * budget > 0x7FFFFFFFLL) return set_error(-1, "es_vsa_global_topk: offsets exceed int32");
    TopkArgs a{};
    a.scores = scores; a.NB = NB; a.W = (NB + 31) / 32; a.bh0 = bh0; a.budget = budget;
    a.q2k_ptr = q2k_ptr; a.q2k_idx = q2k_idx; a.k2q_ptr = k2q_ptr; a.k2q_idx = k2q_idx;
    int* w = static_cast<int*>(workspace);
    a.state = w; w += (size_t)bh_count * 4;
    a.gtcnt = w; w += (size_t)bh_count * NB;
    a.eqcnt = w; w += (size_t)bh_count * NB;
    a.eqbase = w; w += (size_t)bh_count * NB;
    a.colcnt = w; w += (size_t)bh_count * NB;
    a.selbits = reinterpret_cast<uint32_t*>(w);
    cudaStream_t st = (cudaStream_t)stream;
    topk_select_kernel<<<bh_count, 1024, 0, st>>>(a);
    ES_CHECK_LAUNCH("topk_select_kernel");
    const dim3 rows((NB + 3) / 4, bh_count), cols((NB + 127) / 128, bh_count);
    topk_count_kernel<<<rows, 128, 0, st>>>(a);
    ES_CHECK_LAUNCH("topk_count_kernel");
    topk_scan_kernel<<<bh_count, 1024, 0, st>>>(a, 0);
    ES_CHECK_LAUNCH("topk_scan_kernel");
    topk_emit_rows_kernel<<<rows, 128, 0, st>>>(a);
    ES_CHECK_LAUNCH("topk_emit_rows_kernel");
    topk_cols_kernel<<<cols, 128, 0, st>>>(a, 0);
    ES_CHECK_LAUNCH("topk_cols_kernel");
    topk_scan_kernel<<<bh_count, 1024, 0, st>>>(a, 1);
    ES_CHECK_LAUNCH("topk_scan_kernel");
    topk_cols_kernel<<<cols, 128, 0, st>>>(a, 1);
    ES_CHECK_LAUNCH("topk_cols_kernel");
    return 0;
}

extern "C" int es_vsa_fuse_fwd(const void* of, const void* oc, const void* gate, void* o, const int32_t* blk_cnt,
                               int32_t BH, int32_t L, int32_t D, int32_t NBc_pad, int32_t gate_mode, int32_t gate_act,
                               int32_t dtype, void* stream) {
    if (!of || !oc || !o || !blk_cnt) return set_error(-1, "es_vsa_fuse_fwd: null pointer");
    if (int rc = check_shape("es_vsa_fuse_fwd", BH, L, D, dtype)) return rc;
    if (gate_mode < 0 || gate_mode > 2 || (gate_mode != 0 && !gate)) return set_error(-1, "es_vsa_fuse_fwd: bad gate mode");
    if (gate_act < 0 || gate_act > 1 || NBc_pad < L / TB) return set_error(-1, "es_vsa_fuse_fwd: bad gate_act or NBc_pad");
    FuseArgs a{};
    a.of = of; a.oc = oc; a.gate = gate; a.o = o; a.blk_cnt = blk_cnt; a.L = L; a.NB = L / TB; a.NBc_pad = NBc_pad;
    a.gate_mode = gate_mode; a.gate_act = gate_act;
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid(L / TB, BH);
    VSA_LAUNCH(fuse_fwd_kernel, grid, D / 2, 0, a);
    ES_CHECK_LAUNCH("fuse_fwd_kernel");
    return 0;
}

extern "C" int es_vsa_fuse_bwd(const void* dout, const void* of, const void* oc, const void* gate, void* dout_f,
                               float* delta_f, void* dout_c, float* delta_c, void* dgate, const int32_t* blk_cnt,
                               int32_t BH, int32_t L, int32_t D, int32_t NBc_pad, int32_t gate_mode, int32_t gate_act,
                               int32_t dtype, void* stream) {
    if (!dout || !of || !oc || !delta_f || !dout_c || !delta_c || !blk_cnt) return set_error(-1, "es_vsa_fuse_bwd: null pointer");
    if (int rc = check_shape("es_vsa_fuse_bwd", BH, L, D, dtype)) return rc;
    if (gate_mode < 0 || gate_mode > 2 || (gate_mode != 0 && (!gate || !dgate))) return set_error(-1, "es_vsa_fuse_bwd: bad gate mode");
    if (gate_act < 0 || gate_act > 1 || NBc_pad < L / TB) return set_error(-1, "es_vsa_fuse_bwd: bad gate_act or NBc_pad");
    FuseArgs a{};
    a.dout = dout; a.of = of; a.oc = oc; a.gate = gate; a.dout_f = dout_f; a.delta_f = delta_f; a.dout_c = dout_c;
    a.delta_c = delta_c; a.dgate = dgate; a.blk_cnt = blk_cnt; a.L = L; a.NB = L / TB; a.NBc_pad = NBc_pad;
    a.gate_mode = gate_mode; a.gate_act = gate_act;
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid(L / TB, BH);
    VSA_LAUNCH(fuse_bwd_kernel, grid, D / 2, 0, a);
    ES_CHECK_LAUNCH("fuse_bwd_kernel");
    return 0;
}

extern "C" int es_vsa_finalize(const float* acc, const float* add, void* out, const int32_t* blk_cnt, int32_t BH,
                               int32_t L, int32_t D, int32_t add_nb, int32_t dtype, void* stream) {
    if (!out || !blk_cnt) return set_error(-1, "es_vsa_finalize: null pointer");
    if (int rc = check_shape("es_vsa_finalize", BH, L, D, dtype)) return rc;
    if (add && add_nb < L / TB) return set_error(-1, "es_vsa_finalize: add_nb smaller than the block count");
    FinalArgs a{acc, add, out, blk_cnt, L, add_nb};
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid(L / TB, BH);
    VSA_LAUNCH(finalize_kernel, grid, D / 2, 0, a);
    ES_CHECK_LAUNCH("finalize_kernel");
    return 0;
}

extern "C" int es_vsa_block_scores(const void* qc, const void* kc, void* scores, int32_t BH, int32_t NB, int32_t D,
                                   int32_t NBc_pad, int32_t bh0, int32_t bh_count, int32_t dtype, void* stream) {
    if (!qc || !kc || !scores) return set_error(-1, "es_vsa_block_scores: null pointer");
    if (int rc = check_shape("es_vsa_block_scores", BH, NB * TB, D, dtype)) return rc;
    if (NBc_pad < NB || bh0 < 0 || bh_count < 1 || bh0 + bh_count > BH) return set_error(-1, "es_vsa_block_scores: bad sizes");
    BlockScoreArgs a{qc, kc, scores, NB, NBc_pad, bh0, 1.0f / sqrtf((float)D)};
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid((NB + 127) / 128, NB, bh_count);
    VSA_LAUNCH(block_scores_kernel, grid, 128, 0, a);
    ES_CHECK_LAUNCH("block_scores_kernel");
    return 0;
}

extern "C" int es_vsa_row_topk(const void* scores, int32_t NB, int32_t bh0, int32_t bh_count, int32_t topk,
                               int32_t* q2k_ptr, int32_t* q2k_idx, int32_t* k2q_ptr, int32_t* k2q_idx, void* workspace,
                               int32_t dtype, void* stream) {
    if (!scores || !q2k_ptr || !q2k_idx || !k2q_ptr || !k2q_idx || !workspace) return set_error(-1, "es_vsa_row_topk: null pointer");
    if (NB <= 0 || bh_count <= 0 || bh0 < 0 || topk < 0) return set_error(-1, "es_vsa_row_topk: bad sizes");
    if (dtype != 0 && dtype != 1) return set_error(-1, "es_vsa_row_topk: dtype must be 0 (bf16) or 1 (fp16)");
    const int K = topk < NB ? topk : NB;
    if ((long long)(bh0 + bh_count) * NB * K > 0x7FFFFFFFLL) return set_error(-1, "es_vsa_row_topk: offsets exceed int32");
    // the workspace has the layout of es_vsa_global_topk's: the column stages are shared with it
    TopkArgs t{};
    t.NB = NB; t.W = (NB + 31) / 32; t.bh0 = bh0; t.budget = (long long)NB * K;
    t.q2k_ptr = q2k_ptr; t.q2k_idx = q2k_idx; t.k2q_ptr = k2q_ptr; t.k2q_idx = k2q_idx;
    int* w = static_cast<int*>(workspace);
    t.state = w; w += (size_t)bh_count * 4;
    t.gtcnt = w; w += (size_t)bh_count * NB;
    t.eqcnt = w; w += (size_t)bh_count * NB;
    t.eqbase = w; w += (size_t)bh_count * NB;
    t.colcnt = w; w += (size_t)bh_count * NB;
    t.selbits = reinterpret_cast<uint32_t*>(w);
    RowTopkArgs a{static_cast<const uint16_t*>(scores), NB, t.W, bh0, K, dtype, q2k_ptr, q2k_idx, t.selbits};
    cudaStream_t st = (cudaStream_t)stream;
    row_topk_kernel<<<dim3(NB, bh_count), 128, 0, st>>>(a);
    ES_CHECK_LAUNCH("row_topk_kernel");
    const dim3 cols((NB + 127) / 128, bh_count);
    topk_cols_kernel<<<cols, 128, 0, st>>>(t, 0);
    ES_CHECK_LAUNCH("topk_cols_kernel");
    topk_scan_kernel<<<bh_count, 1024, 0, st>>>(t, 1);
    ES_CHECK_LAUNCH("topk_scan_kernel");
    topk_cols_kernel<<<cols, 128, 0, st>>>(t, 1);
    ES_CHECK_LAUNCH("topk_cols_kernel");
    return 0;
}
