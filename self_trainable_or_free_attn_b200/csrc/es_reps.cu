// Four representatives per 64-token kv block, clustered in the query metric
// (reference: echosparse/kernels/representatives.py:1-166).
//
//   G_h = Q_h^T Q_h / (D L) + 1e-3 mean(diag) I;  M_h = chol(G_h) (lower, pivots clamped), stored bf16
//   64 probes per head: scaled means of evenly spaced 64-row query blocks, bf16
//   per kv block: X = K M, token weights from the probes' softmaxes, weighted Lloyd from four 16-token groups,
//   output = plain means of K and V over each final cluster (bf16) and log2 of the cluster sizes (-inf when empty).
//
// The Gram matrix is accumulated as per-split partial sums that the Cholesky kernel adds in a fixed order, so the
// metric is reproducible bit for bit (the reference adds with atomics).
#include "es_api_internal.h"

#include <cuda_bf16.h>
#include <math.h>

namespace es {

constexpr int HD = 128;
constexpr int NP = 64;            // probes per head

__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// ------------------------------------------------------------------------------------------------ Gram partials
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// 16-byte asynchronous copy global -> shared; `bytes` = 0 fills the destination with zeros
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// parts[h][split] = sum over the split's rows of q_r q_r^T (bf16 products, float32 sums). The rows stream through two
// 64-row shared-memory tiles (cp.async); both MMA operands are transposed views of the same tile (ldmatrix.trans): warp
// (wm, wn) owns the 32 x 64 patch at (32 wm, 64 wn) of the 128 x 128 result.
constexpr int GS = 136;           // bf16 row stride of a row tile: 272 B, conflict-free for ldmatrix
__global__ void __launch_bounds__(256)
gram_kernel(const __nv_bfloat16* __restrict__ q, float* __restrict__ parts, int L, int H, int rows_per_split,
            int nsplit) {
    __shared__ __align__(16) __nv_bfloat16 tile[2][64 * GS];
    const int h = blockIdx.x, sp = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp >> 1, wn = warp & 1, g = lane >> 2, tg = lane & 3;
    float acc[2][8][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int x = 0; x < 4; ++x) acc[i][j][x] = 0.f;
    const int r_begin = sp * rows_per_split, r_end = min(L, r_begin + rows_per_split);
    const int nchunk = (r_end - r_begin + 63) / 64;
    auto load = [&](int c, int buf) {
        // 64 rows x 256 B: thread -> row tid / 4 (+ 0), four 16-byte pieces
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int rr = tid >> 2, c16 = (tid & 3) * 4 + x;
            const int row = r_begin + c * 64 + rr;
            const bool okr = row < r_end;
            cp_async16_zfill((uint32_t)__cvta_generic_to_shared(&tile[buf][rr * GS + c16 * 8]),
                             q + ((size_t)(okr ? row : 0) * H + h) * HD + c16 * 8, okr ? 16 : 0);
        }
        cp_async_commit();
    };
    if (nchunk > 0) load(0, 0);
    const int lj = lane & 7, lm = lane >> 3;
    for (int c = 0; c < nchunk; ++c) {
        if (c + 1 < nchunk) { load(c + 1, (c + 1) & 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncthreads();
        const uint32_t tb = (uint32_t)__cvta_generic_to_shared(&tile[c & 1][0]);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const int k0 = ks * 16;
            uint32_t a[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                // A[m][k] = tile[k][m]: matrices (m lo, k lo), (m hi, k lo), (m lo, k hi), (m hi, k hi)
                const int row = k0 + lj + (lm >> 1) * 8, col = 32 * wm + 16 * i + (lm & 1) * 8;
                ldmatrix_x4_trans(tb + (uint32_t)(row * GS + col) * 2, a[i][0], a[i][1], a[i][2], a[i][3]);
            }
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {
                // B[k][n] = tile[k][n]: matrices (k lo, n0), (k hi, n0), (k lo, n0 + 8), (k hi, n0 + 8)
                const int row = k0 + lj + (lm & 1) * 8, col = 64 * wn + 16 * jp + (lm >> 1) * 8;
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(tb + (uint32_t)(row * GS + col) * 2, b0, b1, b2, b3);
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    mma16816(acc[i][2 * jp], a[i][0], a[i][1], a[i][2], a[i][3], b0, b1);
                    mma16816(acc[i][2 * jp + 1], a[i][0], a[i][1], a[i][2], a[i][3], b2, b3);
                }
            }
        }
        __syncthreads();
    }
    float* out = parts + ((size_t)h * nsplit + sp) * HD * HD;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int m = 32 * wm + 16 * i + g, nn = 64 * wn + 8 * j + 2 * tg;
            *reinterpret_cast<float2*>(out + m * HD + nn) = make_float2(acc[i][j][0], acc[i][j][1]);
            *reinterpret_cast<float2*>(out + (m + 8) * HD + nn) = make_float2(acc[i][j][2], acc[i][j][3]);
        }
}

// ------------------------------------------------------------------------------------------------ metric
// Sum of the Gram partials of a head, scaled: parts[h][0] <- norm * sum_p parts[h][p], in the fixed order the sums have
// always been taken in (four running sums over p % 4, then (s0 + s1) + (s2 + s3)). Sixteen CTAs per head, so that the
// reduction of the 2 MB of partials is not one CTA's chain of loads (with a handful of heads per GPU it was).
__global__ void __launch_bounds__(256)
gram_reduce_kernel(float* __restrict__ parts, int nsplit, float norm) {
    const int h = blockIdx.x, e0 = (blockIdx.y * 256 + threadIdx.x) * 4;
    float* src = parts + (size_t)h * nsplit * HD * HD + e0;
    float4 s4[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) s4[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    int p = 0;
    for (; p + 4 <= nsplit; p += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float4 x = *reinterpret_cast<const float4*>(src + (size_t)(p + u) * HD * HD);
            s4[u].x += x.x; s4[u].y += x.y; s4[u].z += x.z; s4[u].w += x.w;
        }
    }
    for (int u = 0; p < nsplit; ++p, ++u) {
        const float4 x = *reinterpret_cast<const float4*>(src + (size_t)p * HD * HD);
        s4[u].x += x.x; s4[u].y += x.y; s4[u].z += x.z; s4[u].w += x.w;
    }
    float4 r;
    r.x = ((s4[0].x + s4[1].x) + (s4[2].x + s4[3].x)) * norm;
    r.y = ((s4[0].y + s4[1].y) + (s4[2].y + s4[3].y)) * norm;
    r.z = ((s4[0].z + s4[1].z) + (s4[2].z + s4[3].z)) * norm;
    r.w = ((s4[0].w + s4[1].w) + (s4[2].w + s4[3].w)) * norm;
    *reinterpret_cast<float4*>(src) = r;              // the slot of split 0: only this thread reads or writes these elements
}

// G (from gram_reduce_kernel) regularised, then its Cholesky factor with clamped pivots (representatives.py:49-63,
// 163-165), blocked: per panel of 16 columns one warp factors the 16 x 16 diagonal block in registers (a lane per row,
// the pivot row's values by shuffle), every row below solves its 16 entries against that block, and the trailing matrix
// takes the rank-16 update: three barriers per panel, 24 in all, against two per column in the unblocked form. One CTA
// per head; the matrix lives in shared memory.
constexpr int CH_PANEL = 16;
__global__ void __launch_bounds__(256)
metric_kernel(const float* __restrict__ parts, __nv_bfloat16* __restrict__ metric, float* __restrict__ gram_out,
              int nsplit) {
    extern __shared__ float sm[];
    float* A = sm;                 // [128][129]
    float* Lm = A + HD * 129;      // [128][129]
    float* sq = Lm + HD * 129;     // [128] square roots of the clamped pivots
    __shared__ float red[8];
    __shared__ float s_eps, s_diag;
    const int h = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const float* src = parts + (size_t)h * nsplit * HD * HD;
    for (int e = tid * 4; e < HD * HD; e += 1024) {
        const float4 x = *reinterpret_cast<const float4*>(src + e);
        float* dst = A + (e >> 7) * 129 + (e & 127);
        dst[0] = x.x; dst[1] = x.y; dst[2] = x.z; dst[3] = x.w;
        float* dl = Lm + (e >> 7) * 129 + (e & 127);
        dl[0] = 0.f; dl[1] = 0.f; dl[2] = 0.f; dl[3] = 0.f;
    }
    __syncthreads();
    float dg = tid < HD ? A[tid * 129 + tid] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dg += __shfl_xor_sync(0xffffffffu, dg, o);
    if (lane == 0) red[warp] = dg;
    __syncthreads();
    if (tid == 0) s_diag = (((red[0] + red[1]) + (red[2] + red[3])) + ((red[4] + red[5]) + (red[6] + red[7]))) / HD;
    __syncthreads();
    if (tid < HD) A[tid * 129 + tid] += 1e-3f * s_diag;
    __syncthreads();
    if (gram_out)
        for (int e = tid; e < HD * HD; e += 256) gram_out[(size_t)h * HD * HD + e] = A[(e >> 7) * 129 + (e & 127)];
    dg = tid < HD ? A[tid * 129 + tid] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dg += __shfl_xor_sync(0xffffffffu, dg, o);
    __syncthreads();
    if (lane == 0) red[warp] = dg;
    __syncthreads();
    if (tid == 0)
        s_eps = (((red[0] + red[1]) + (red[2] + red[3])) + ((red[4] + red[5]) + (red[6] + red[7]))) / HD * 1e-12f;
    __syncthreads();
    const float eps = s_eps;
    for (int j0 = 0; j0 < HD; j0 += CH_PANEL) {
        // (1) the diagonal block: lane i (and its duplicate i + 16) holds row j0 + i of the block
        if (warp == 0) {
            const int i = lane & 15, r = j0 + i;
            float a[CH_PANEL];
#pragma unroll
            for (int c = 0; c < CH_PANEL; ++c) a[c] = A[r * 129 + j0 + c];
#pragma unroll
            for (int j = 0; j < CH_PANEL; ++j) {
                const float root = sqrtf(fmaxf(__shfl_sync(0xffffffffu, a[j], j), eps));
                const float l = i >= j ? a[j] / root : 0.f;
                a[j] = l;
                if (lane == j) sq[j0 + j] = root;
#pragma unroll
                for (int c = j + 1; c < CH_PANEL; ++c) {
                    const float lc = __shfl_sync(0xffffffffu, l, c);
                    if (i >= c) a[c] -= l * lc;
                }
            }
            if (lane < 16) {
#pragma unroll
                for (int c = 0; c < CH_PANEL; ++c) Lm[r * 129 + j0 + c] = c <= i ? a[c] : 0.f;
            }
        }
        __syncthreads();
        // (2) the rows below: L[r][j0 + j] = (A[r][j0 + j] - sum_{k < j} L[r][j0 + k] L[j0 + j][j0 + k]) / root_j
        if (tid < HD && tid >= j0 + CH_PANEL) {
            float x[CH_PANEL];
#pragma unroll
            for (int c = 0; c < CH_PANEL; ++c) x[c] = A[tid * 129 + j0 + c];
#pragma unroll
            for (int j = 0; j < CH_PANEL; ++j) {
                float sacc = x[j];
#pragma unroll
                for (int k2 = 0; k2 < j; ++k2) sacc -= x[k2] * Lm[(j0 + j) * 129 + j0 + k2];
                x[j] = sacc / sq[j0 + j];
            }
#pragma unroll
            for (int c = 0; c < CH_PANEL; ++c) Lm[tid * 129 + j0 + c] = x[c];
        }
        __syncthreads();
        // (3) A -= L_panel L_panel^T on the lower triangle of the trailing block: two threads per row, columns alternating
        {
            const int r = tid >> 1;
            if (r >= j0 + CH_PANEL) {
                float lr[CH_PANEL];
#pragma unroll
                for (int k2 = 0; k2 < CH_PANEL; ++k2) lr[k2] = Lm[r * 129 + j0 + k2];
                float* row = A + r * 129;
                for (int c = j0 + CH_PANEL + (tid & 1); c <= r; c += 2) {
                    const float* lc = Lm + c * 129 + j0;
                    float sacc = row[c];
#pragma unroll
                    for (int k2 = 0; k2 < CH_PANEL; ++k2) sacc -= lr[k2] * lc[k2];
                    row[c] = sacc;
                }
            }
        }
        __syncthreads();
    }
    for (int e = tid; e < HD * HD; e += 256)
        metric[(size_t)h * HD * HD + e] = __float2bfloat16_rn(Lm[(e >> 7) * 129 + (e & 127)]);
}

// ------------------------------------------------------------------------------------------------ probes
// Probe i of a head = scale * mean of the query rows of 64-row block floor(i (nb - 1) / 63 + 0.5) (representatives.py:36-46).
__global__ void __launch_bounds__(HD)
probe_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ probes, int L, int H, int nb, float scale) {
    const int i = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
    const int blk = (int)((float)(i * (nb - 1)) / (float)(NP - 1) + 0.5f);
    float s = 0.f;
    int n = 0;
    for (int r = 0; r < 64; ++r) {
        const int row = blk * 64 + r;
        if (row < L) { s += __bfloat162float(q[((size_t)row * H + h) * HD + d]); ++n; }
    }
    probes[((size_t)h * NP + i) * HD + d] = __float2bfloat16_rn(s * scale / fmaxf((float)n, 1.0f));
}

// ------------------------------------------------------------------------------------------------ k-means
// One CTA (8 warps) per (kv block, head). The two contractions (X = K M, probe scores = P K^T) run on the tensor cores
// (mma.sync m16n8k16, bf16 products with float32 sums, the arithmetic of the reference's tl.dot on bf16 inputs); the
// Lloyd iterations work on X in shared memory in float32 with all 256 threads busy in every phase.
constexpr int KS = 136;           // bf16 row stride of the K tile: 272 B, so the 8 rows of an ldmatrix hit distinct banks
constexpr int XS = 132;           // float row stride of X and of the centroids
constexpr int PS = 65;            // float row stride of the probe scores
constexpr int MS = 136;           // bf16 row stride of the metric in shared memory
constexpr int KM_BLOCKS = 4;      // kv blocks per CTA: the metric is loaded into shared memory once for all of them
constexpr int KM_SMEM = 128 * MS * 2 + 64 * KS * 2 + 64 * XS * 4 + 64 * PS * 4 + 4 * XS * 4 + 4 * 64 * 4 + 64 * 4 + 64 * 4 +
                        4 * 64 * 4 * 4 + 2 * 4 * 128 * 4;      // + partial dots [4][64][4] and partial centroid sums [2][4][128]

__global__ void __launch_bounds__(256, 2)
kmeans_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
              const __nv_bfloat16* __restrict__ metric, const __nv_bfloat16* __restrict__ probes,
              __nv_bfloat16* __restrict__ k4, __nv_bfloat16* __restrict__ v4, float* __restrict__ c4,
              __nv_bfloat16* __restrict__ km, __nv_bfloat16* __restrict__ vm, int L, int H, int nb4, int iters,
              int blocks_per_cta) {
    extern __shared__ __align__(16) uint8_t raw[];
    __nv_bfloat16* sM = reinterpret_cast<__nv_bfloat16*>(raw);                     // [128][MS] the head's metric
    __nv_bfloat16* sK = sM + 128 * MS;                                             // [64][KS]
    float* sX = reinterpret_cast<float*>(raw + 128 * MS * 2 + 64 * KS * 2);         // [64][XS]
    float* sP = sX + 64 * XS;                                                       // [64 probes][PS]
    float* cen = sP + 64 * PS;                                                      // [4][XS]
    float* wpart = cen + 4 * XS;                                                    // [4][64]
    float* w = wpart + 4 * 64;                                                      // [64]
    int* lab = reinterpret_cast<int*>(w + 64);                                      // [64]
    float* dpart = reinterpret_cast<float*>(lab + 64);                              // [4 d quarters][64 tokens][4 clusters]
    // dpart is followed by 4 KB more, so that the two together hold [4][4][128] partial sums
    __shared__ float cw[4], nnp[8];
    float4* ohw = reinterpret_cast<float4*>(wpart);    // [64 tokens]: the token's weight in the slot of its cluster (wpart is dead by then)
    __shared__ float s_cnt[4];
    const int h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tg = lane & 3;
    const int nb = (L + 63) / 64;
    // the metric of this head: 128 x 128 bf16, once per CTA
    for (int e = tid; e < 128 * 16; e += 256) {
        const int r = e >> 4, c16 = e & 15;
        cp_async16_zfill((uint32_t)__cvta_generic_to_shared(sM + r * MS + c16 * 8),
                         metric + ((size_t)h * HD + r) * HD + c16 * 8, 16);
    }
    cp_async_commit();
    const int mt = warp & 3, nh = warp >> 2;
    // this thread's A fragments of the probe scores (probes 16 mt .. +15), the same for every block of the head
    uint32_t pa[8][4];
    {
        const __nv_bfloat16* p0 = probes + ((size_t)h * NP + 16 * mt + g) * HD + 2 * tg;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            pa[ks][0] = __ldg(reinterpret_cast<const uint32_t*>(p0 + ks * 16));
            pa[ks][1] = __ldg(reinterpret_cast<const uint32_t*>(p0 + 8 * HD + ks * 16));
            pa[ks][2] = __ldg(reinterpret_cast<const uint32_t*>(p0 + ks * 16 + 8));
            pa[ks][3] = __ldg(reinterpret_cast<const uint32_t*>(p0 + 8 * HD + ks * 16 + 8));
        }
    }
  for (int j = blockIdx.x * blocks_per_cta; j < min(nb, (int)(blockIdx.x + 1) * blocks_per_cta); ++j) {
    const int nvalid = min(L - j * 64, 64);
    __syncthreads();                       // the previous block's readers of the shared tiles are done
    // K tile (rows past L are zero)
    for (int e = tid; e < 64 * 16; e += 256) {
        const int r = e >> 4, c16 = e & 15;
        const bool okr = r < nvalid;
        cp_async16_zfill((uint32_t)__cvta_generic_to_shared(sK + r * KS + c16 * 8),
                         k + ((size_t)(j * 64 + (okr ? r : 0)) * H + h) * HD + c16 * 8, okr ? 16 : 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    // A fragments of this warp's 16 tokens (rows 16 mt ..), all 8 k-steps: shared by both contractions below? No: the
    // probe scores use K as the B operand. Only X uses these.
    {
        // X = K M: rows 16 mt .. +15, columns 64 nh .. +63
        float acc[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int x = 0; x < 4; ++x) acc[nt][x] = 0.f;
        const uint32_t a_addr = (uint32_t)__cvta_generic_to_shared(sK + (16 * mt + (lane & 15)) * KS + (lane >> 4) * 8);
        const uint32_t m_addr = (uint32_t)__cvta_generic_to_shared(sM);
        const int lj = lane & 7, lm = lane >> 3;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t a0, a1, a2, a3;
            ldmatrix_x4(a_addr + ks * 32, a0, a1, a2, a3);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                // B[k][n] = M[k][n], row-major in shared memory: transposed 8 x 8 loads, matrices (k lo, n0), (k hi, n0),
                // (k lo, n0 + 8), (k hi, n0 + 8)
                const int row = ks * 16 + lj + (lm & 1) * 8, col = 64 * nh + 16 * np + (lm >> 1) * 8;
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(m_addr + (uint32_t)(row * MS + col) * 2, b0, b1, b2, b3);
                mma16816(acc[2 * np], a0, a1, a2, a3, b0, b1);
                mma16816(acc[2 * np + 1], a0, a1, a2, a3, b2, b3);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int col = 64 * nh + 8 * nt + 2 * tg;
            *reinterpret_cast<float2*>(sX + (16 * mt + g) * XS + col) = make_float2(acc[nt][0], acc[nt][1]);
            *reinterpret_cast<float2*>(sX + (16 * mt + g + 8) * XS + col) = make_float2(acc[nt][2], acc[nt][3]);
        }
    }
    {
        // probe scores: probes 16 mt .. +15 (A, in registers), tokens 32 nh .. +31 (B = K rows, from shared memory)
        float acc[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int x = 0; x < 4; ++x) acc[nt][x] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            const uint32_t a0 = pa[ks][0], a1 = pa[ks][1], a2 = pa[ks][2], a3 = pa[ks][3];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const __nv_bfloat16* kr = sK + (32 * nh + 8 * nt + g) * KS + ks * 16 + 2 * tg;
                mma16816(acc[nt], a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(kr),
                         *reinterpret_cast<const uint32_t*>(kr + 8));
            }
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int col = 32 * nh + 8 * nt + 2 * tg;
            sP[(16 * mt + g) * PS + col] = acc[nt][0];
            sP[(16 * mt + g) * PS + col + 1] = acc[nt][1];
            sP[(16 * mt + g + 8) * PS + col] = acc[nt][2];
            sP[(16 * mt + g + 8) * PS + col + 1] = acc[nt][3];
        }
    }
    __syncthreads();
    // each probe's softmax over the block's valid tokens (natural exponent): four threads per probe, 16 tokens each
    {
        float* row = sP + (tid >> 2) * PS + (tid & 3) * 16;
        const int t0 = (tid & 3) * 16;
        float mx = -INFINITY;
#pragma unroll
        for (int t = 0; t < 16; ++t) mx = (t0 + t < nvalid) ? fmaxf(mx, row[t]) : mx;
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        float e[16], sum = 0.f;
#pragma unroll
        for (int t = 0; t < 16; ++t) {
            e[t] = (t0 + t < nvalid) ? expf(row[t] - mx) : 0.f;
            sum += e[t];
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const float inv = 1.0f / sum;
#pragma unroll
        for (int t = 0; t < 16; ++t) row[t] = e[t] * inv;
    }
    __syncthreads();
    // token weights: sum over the probes (four partial sums of 16 probes, added in a fixed order)
    {
        const int t = tid & 63, qp = tid >> 6;
        float sacc = 0.f;
#pragma unroll
        for (int p = 0; p < 16; ++p) sacc += sP[(16 * qp + p) * PS + t];
        wpart[qp * 64 + t] = sacc;
    }
    __syncthreads();
    if (tid < 64) {
        const float sacc = (wpart[tid] + wpart[64 + tid]) + (wpart[128 + tid] + wpart[192 + tid]);
        const float wt = tid < nvalid ? sacc * ((float)nvalid / (float)NP) : 0.f;
        w[tid] = wt;
        lab[tid] = tid >> 4;
        asm volatile("bar.sync 1, 64;" ::: "memory");          // warps 0 and 1 have read the partial sums that ohw overlays
        ohw[tid] = make_float4(tid < 16 ? wt : 0.f, (tid >> 4) == 1 ? wt : 0.f, (tid >> 4) == 2 ? wt : 0.f, tid >= 48 ? wt : 0.f);
    }
    // The probe scores are dead now: their area receives the V tile (64 x 128 bf16), copied asynchronously while the
    // Lloyd iterations run, so the final cluster means do not wait on global memory.
    __nv_bfloat16* sV = reinterpret_cast<__nv_bfloat16*>(sP);
    for (int e = tid; e < 64 * 16; e += 256) {
        const int r = e >> 4, c16 = e & 15;
        const bool okr = r < nvalid;
        cp_async16_zfill((uint32_t)__cvta_generic_to_shared(sV + r * HD + c16 * 8),
                         v + ((size_t)(j * 64 + (okr ? r : 0)) * H + h) * HD + c16 * 8, okr ? 16 : 0);
    }
    cp_async_commit();
    __syncthreads();

    // Weighted centroids of the current labels; keep_old: an emptied cluster keeps its centroid. Also the cluster weights
    // and the squared norms of the centroids (two warp partials per cluster in nnp).
    // Thread (token quarter, dim pair) sweeps 16 tokens with the one-hot weights (no branch on the label, every load
    // independent of the arithmetic); thread (cluster, dim pair) then adds the four quarters in a fixed order. The three
    // warp reductions of the second phase (cluster weight, squared norm of the new and of the kept centroid) run side by side.
    float* qpart = dpart;                             // [4 token quarters][4 clusters][128]: dpart and cpart, both dead here
    auto update_centroids = [&](bool keep_old) {
        {
            const int dp = 2 * (tid & 63), tq = tid >> 6;
            float2 sc[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) sc[c] = make_float2(0.f, 0.f);
            // tokens past the valid ones have weight zero
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int t = 16 * tq + i;
                const float4 o = ohw[t];
                const float2 x = *reinterpret_cast<const float2*>(sX + t * XS + dp);
                sc[0].x = fmaf(o.x, x.x, sc[0].x); sc[0].y = fmaf(o.x, x.y, sc[0].y);
                sc[1].x = fmaf(o.y, x.x, sc[1].x); sc[1].y = fmaf(o.y, x.y, sc[1].y);
                sc[2].x = fmaf(o.z, x.x, sc[2].x); sc[2].y = fmaf(o.z, x.y, sc[2].y);
                sc[3].x = fmaf(o.w, x.x, sc[3].x); sc[3].y = fmaf(o.w, x.y, sc[3].y);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) *reinterpret_cast<float2*>(qpart + (tq * 4 + c) * 128 + dp) = sc[c];
        }
        __syncthreads();
        const int c = tid >> 6, d = 2 * (tid & 63);
        // weight of cluster c: every warp of the cluster adds the 64 tokens in the same order
        float ws = reinterpret_cast<const float*>(ohw)[4 * lane + c] + reinterpret_cast<const float*>(ohw)[4 * (lane + 32) + c];
        const float2 p0 = *reinterpret_cast<const float2*>(qpart + (0 * 4 + c) * 128 + d);
        const float2 p1 = *reinterpret_cast<const float2*>(qpart + (1 * 4 + c) * 128 + d);
        const float2 p2 = *reinterpret_cast<const float2*>(qpart + (2 * 4 + c) * 128 + d);
        const float2 p3 = *reinterpret_cast<const float2*>(qpart + (3 * 4 + c) * 128 + d);
        const float2 old = *reinterpret_cast<const float2*>(cen + c * XS + d);
        const float s0 = (p0.x + p1.x) + (p2.x + p3.x), s1 = (p0.y + p1.y) + (p2.y + p3.y);
        float nn_new = s0 * s0 + s1 * s1, nn_old = old.x * old.x + old.y * old.y;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ws += __shfl_xor_sync(0xffffffffu, ws, o);
            nn_new += __shfl_xor_sync(0xffffffffu, nn_new, o);
            nn_old += __shfl_xor_sync(0xffffffffu, nn_old, o);
        }
        float nn;
        if (!keep_old || ws > 0.f) {
            const float inv = 1.0f / fmaxf(ws, 1e-6f);
            *reinterpret_cast<float2*>(cen + c * XS + d) = make_float2(s0 * inv, s1 * inv);
            nn = nn_new * (inv * inv);
        } else {
            nn = nn_old;
        }
        if (lane == 0) nnp[warp] = nn;                // warps 2c, 2c + 1 hold cluster c
        if ((tid & 63) == 0) cw[c] = ws;
        __syncthreads();
    };
    update_centroids(false);
    for (int it = 0; it < iters; ++it) {
        // partial dot products: warp -> (d quarter warp % 4, token half warp / 4), lane -> token; the centroid rows are
        // read as broadcasts, X once; then one thread per token adds the four quarters in a fixed order
        {
            const int dq = warp & 3, tk = 32 * (warp >> 2) + lane;
            float dt[4] = {0.f, 0.f, 0.f, 0.f};
            const float* xr = sX + tk * XS + 32 * dq;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 x = *reinterpret_cast<const float4*>(xr + 4 * i);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float4 y = *reinterpret_cast<const float4*>(cen + c * XS + 32 * dq + 4 * i);
                    dt[c] = fmaf(x.x, y.x, dt[c]); dt[c] = fmaf(x.y, y.y, dt[c]);
                    dt[c] = fmaf(x.z, y.z, dt[c]); dt[c] = fmaf(x.w, y.w, dt[c]);
                }
            }
            *reinterpret_cast<float4*>(dpart + (dq * 64 + tk) * 4) = make_float4(dt[0], dt[1], dt[2], dt[3]);
        }
        __syncthreads();
        int differs = 0;
        if (tid < 64) {                               // one token each
            const float4 d0 = *reinterpret_cast<const float4*>(dpart + (0 * 64 + tid) * 4);
            const float4 d1 = *reinterpret_cast<const float4*>(dpart + (1 * 64 + tid) * 4);
            const float4 d2 = *reinterpret_cast<const float4*>(dpart + (2 * 64 + tid) * 4);
            const float4 d3 = *reinterpret_cast<const float4*>(dpart + (3 * 64 + tid) * 4);
            const float dot[4] = {(d0.x + d1.x) + (d2.x + d3.x), (d0.y + d1.y) + (d2.y + d3.y),
                                  (d0.z + d1.z) + (d2.z + d3.z), (d0.w + d1.w) + (d2.w + d3.w)};
            float bd = INFINITY;
            int best = 0;
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                const float dist = cw[cc] > 0.f ? (nnp[2 * cc] + nnp[2 * cc + 1]) - 2.0f * dot[cc] : INFINITY;
                if (cc == 0 || dist < bd) { bd = dist; best = cc; }
            }
            differs = tid < nvalid && best != lab[tid];
            lab[tid] = best;                          // no other thread reads the labels or the one-hot weights in this phase
            const float wt = w[tid];
            ohw[tid] = make_float4(best == 0 ? wt : 0.f, best == 1 ? wt : 0.f, best == 2 ? wt : 0.f, best == 3 ? wt : 0.f);
        }
        const int changed = __syncthreads_or(differs);
        update_centroids(true);
        if (changed == 0) break;
    }

    // plain means of K and V over the final clusters, and the block means when asked for
    if (warp == 0) {
        const int l0 = lane < nvalid ? lab[lane] : -1, l1 = lane + 32 < nvalid ? lab[lane + 32] : -1;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int n = __popc(__ballot_sync(0xffffffffu, l0 == c)) + __popc(__ballot_sync(0xffffffffu, l1 == c));
            if (lane == c) {
                s_cnt[c] = (float)n;
                c4[(size_t)h * nb4 + j * 4 + c] = n > 0 ? log2f((float)n) : -INFINITY;
            }
        }
        // membership as 0 / 1 in place of the weights (their last readers passed the barrier that ended the iterations)
        ohw[lane] = make_float4(l0 == 0 ? 1.f : 0.f, l0 == 1 ? 1.f : 0.f, l0 == 2 ? 1.f : 0.f, l0 == 3 ? 1.f : 0.f);
        ohw[lane + 32] = make_float4(l1 == 0 ? 1.f : 0.f, l1 == 1 ? 1.f : 0.f, l1 == 2 ? 1.f : 0.f, l1 == 3 ? 1.f : 0.f);
    }
    cp_async_wait<0>();
    __syncthreads();
    {
        // thread (K or V, token half, dim pair): 32 tokens; a multiply-add with the 0 / 1 membership is an exact add
        const int which = tid >> 7, th = (tid >> 6) & 1, dp = 2 * (tid & 63);
        float2 sc[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) sc[c] = make_float2(0.f, 0.f);
        const __nv_bfloat16* src = which ? sV + dp : sK + dp;
        const int stride = which ? HD : KS;
#pragma unroll 8
        for (int i = 0; i < 32; ++i) {
            const int t = 32 * th + i;
            const float4 o = ohw[t];
            const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + t * stride));
            sc[0].x = fmaf(o.x, x.x, sc[0].x); sc[0].y = fmaf(o.x, x.y, sc[0].y);
            sc[1].x = fmaf(o.y, x.x, sc[1].x); sc[1].y = fmaf(o.y, x.y, sc[1].y);
            sc[2].x = fmaf(o.z, x.x, sc[2].x); sc[2].y = fmaf(o.z, x.y, sc[2].y);
            sc[3].x = fmaf(o.w, x.x, sc[3].x); sc[3].y = fmaf(o.w, x.y, sc[3].y);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) *reinterpret_cast<float2*>(qpart + ((which * 2 + th) * 4 + c) * 128 + dp) = sc[c];
    }
    __syncthreads();
    {
        const int which = tid >> 7, d = tid & 127;
        float sacc[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) sacc[c] = qpart[((which * 2 + 0) * 4 + c) * 128 + d] + qpart[((which * 2 + 1) * 4 + c) * 128 + d];
        __nv_bfloat16* o = (which ? v4 : k4) + ((size_t)h * nb4 + j * 4) * HD + d;
#pragma unroll
        for (int c = 0; c < 4; ++c) o[c * HD] = __float2bfloat16_rn(sacc[c] * (1.0f / fmaxf(s_cnt[c], 1.0f)));
        __nv_bfloat16* mo = which ? vm : km;
        if (mo) mo[((size_t)j * H + h) * HD + d] = __float2bfloat16_rn(((sacc[0] + sacc[1]) + (sacc[2] + sacc[3])) / (float)nvalid);
    }
  }
}

}  // namespace es

using namespace es;

// Rows of q per Gram partial, as the reference splits them (representatives.py:160).
static int gram_rows_per_split(int L) { return ((((L + 31) / 32) + 63) / 64) * 64; }

extern "C" int es_reps_gram_splits(int32_t L) {
    if (L <= 0) return 0;
    const int rps = gram_rows_per_split(L);
    return (L + rps - 1) / rps;
}

// q (L, H, 128) bf16 -> metric (H, 128, 128) bf16 (Cholesky factor) and probes (H, 64, 128) bf16.
// gram_parts: scratch of es_reps_gram_splits(L) * H * 128 * 128 floats; gram (H, 128, 128) fp32 receives the
// regularised Gram matrix when not null.
extern "C" int es_reps_metric(const void* q, float* gram_parts, float* gram, void* metric, void* probes, int32_t L,
                              int32_t H, void* stream) {
    if (!q || !gram_parts || !metric || !probes) return set_error(-1, "es_reps_metric: null pointer");
    if (L <= 0 || H <= 0) return set_error(-1, "es_reps_metric: L and H must be positive");
    if ((uintptr_t)q & 15) return set_error(-1, "es_reps_metric: q must be 16-byte aligned");
    const int nb = (L + 63) / 64;
    const int rps = gram_rows_per_split(L), nsplit = (L + rps - 1) / rps;
    cudaStream_t st = (cudaStream_t)stream;
    gram_kernel<<<dim3(H, nsplit), 256, 0, st>>>((const __nv_bfloat16*)q, gram_parts, L, H, rps, nsplit);
    ES_CHECK_LAUNCH("gram");
    const int smem = (2 * HD * 129 + HD) * (int)sizeof(float);
    if (int rc = opt_in_shared_memory((const void*)metric_kernel, smem)) return rc;
    const float scale = 1.0f / sqrtf((float)HD);
    gram_reduce_kernel<<<dim3(H, HD * HD / 1024), 256, 0, st>>>(gram_parts, nsplit, scale * scale / (float)L);
    ES_CHECK_LAUNCH("gram_reduce");
    metric_kernel<<<H, 256, smem, st>>>(gram_parts, (__nv_bfloat16*)metric, gram, nsplit);
    ES_CHECK_LAUNCH("metric");
    probe_kernel<<<dim3(NP, H), HD, 0, st>>>((const __nv_bfloat16*)q, (__nv_bfloat16*)probes, L, H, nb, scale);
    ES_CHECK_LAUNCH("probes");
    return 0;
}

// k, v (L, H, 128) bf16 -> k_rep, v_rep (H, (nb + 1) * 4, 128) bf16 and log_counts (H, (nb + 1) * 4) fp32; block nb of
// the tables is left as the caller initialised it (zeros, -inf). k_mean / v_mean (nb, H, 128) are written when given.
extern "C" int es_reps_kmeans(const void* k, const void* v, const void* metric, const void* probes, void* k_rep,
                              void* v_rep, float* log_counts, void* k_mean, void* v_mean, int32_t L, int32_t H,
                              int32_t iters, void* stream) {
    if (!k || !v || !metric || !probes || !k_rep || !v_rep || !log_counts)
        return set_error(-1, "es_reps_kmeans: null pointer");
    if (L <= 0 || H <= 0) return set_error(-1, "es_reps_kmeans: L and H must be positive");
    if (((uintptr_t)k | (uintptr_t)metric) & 15) return set_error(-1, "es_reps_kmeans: k and metric must be 16-byte aligned");
    if ((k_mean == nullptr) != (v_mean == nullptr)) return set_error(-1, "es_reps_kmeans: give both means or neither");
    const int nb = (L + 63) / 64;
    if (int rc = opt_in_shared_memory((const void*)kmeans_kernel, KM_SMEM)) return rc;
    // kv blocks per CTA: KM_BLOCKS share one load of the head's metric; fewer when that would leave the GPU with only a
    // few waves of CTAs (a handful of heads per GPU), where the last, partly filled wave costs more than the reloads
    int per = KM_BLOCKS;
    while (per > 1 && (long long)((nb + per - 1) / per) * H < 8LL * 2 * 148) per >>= 1;
    kmeans_kernel<<<dim3((nb + per - 1) / per, H), 256, KM_SMEM, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const __nv_bfloat16*)metric, (const __nv_bfloat16*)probes,
        (__nv_bfloat16*)k_rep, (__nv_bfloat16*)v_rep, log_counts, (__nv_bfloat16*)k_mean, (__nv_bfloat16*)v_mean, L, H,
        (nb + 1) * 4, iters, per);
    ES_CHECK_LAUNCH("kmeans");
    return 0;
}

// ------------------------------------------------------------------------------------------------ no-allocation variant
// Scratch for es_reps_metric_static: room for ES_STATIC_GRAM_PARTS partial Gram matrices (128 x 128 floats each), held by
// every GPU that loads this library from load to exit.
#define ES_STATIC_GRAM_PARTS 256
static __device__ __align__(256) float g_static_gram_parts[ES_STATIC_GRAM_PARTS * HD * HD];

// Device address of the scratch array on the current device. In host code the array's name is only a handle for the
// runtime, not an address a kernel could use, so the address is asked for once per device (with that device current).
static float* static_gram_parts() {
    static float* ptrs[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!ptrs[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_gram_parts) != cudaSuccess) return nullptr;
        ptrs[dev] = static_cast<float*>(p);
    }
    return ptrs[dev];
}

extern "C" int es_reps_metric_static_max_heads(void) { return ES_STATIC_GRAM_PARTS; }

extern "C" int es_reps_metric_static(const void* q, float* gram, void* metric, void* probes, int32_t L, int32_t H,
                                     void* stream) {
    if (!q || !metric || !probes) return set_error(-1, "es_reps_metric_static: null pointer");
    if (L <= 0 || H <= 0) return set_error(-1, "es_reps_metric_static: L and H must be positive");
    if ((uintptr_t)q & 15) return set_error(-1, "es_reps_metric_static: q must be 16-byte aligned");
    if (H > ES_STATIC_GRAM_PARTS)
        return set_error(-1, "es_reps_metric_static: more than 256 heads do not fit the built-in scratch; use es_reps_metric");
    float* parts = static_gram_parts();
    if (!parts) return set_error(-2, "es_reps_metric_static: the address of the built-in scratch is not available");
    // as many row splits as the scratch holds for this head count (at most the usual number)
    int nsplit = ES_STATIC_GRAM_PARTS / H;
    const int usual = es_reps_gram_splits(L);
    if (nsplit > usual) nsplit = usual;
    const int rps = (((L + nsplit - 1) / nsplit + 63) / 64) * 64;
    nsplit = (L + rps - 1) / rps;
    const int nb = (L + 63) / 64;
    cudaStream_t st = (cudaStream_t)stream;
    gram_kernel<<<dim3(H, nsplit), 256, 0, st>>>((const __nv_bfloat16*)q, parts, L, H, rps, nsplit);
    ES_CHECK_LAUNCH("gram");
    const int smem = (2 * HD * 129 + HD) * (int)sizeof(float);
    if (int rc = opt_in_shared_memory((const void*)metric_kernel, smem)) return rc;
    const float scale = 1.0f / sqrtf((float)HD);
    gram_reduce_kernel<<<dim3(H, HD * HD / 1024), 256, 0, st>>>(parts, nsplit, scale * scale / (float)L);
    ES_CHECK_LAUNCH("gram_reduce");
    metric_kernel<<<H, 256, smem, st>>>(parts, (__nv_bfloat16*)metric, gram, nsplit);
    ES_CHECK_LAUNCH("metric");
    probe_kernel<<<dim3(NP, H), HD, 0, st>>>((const __nv_bfloat16*)q, (__nv_bfloat16*)probes, L, H, nb, scale);
    ES_CHECK_LAUNCH("probes");
    return 0;
}
