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
// One CTA (8 warps) per (kv block, head), several blocks in turn. Every contraction runs on the tensor cores
// (mma.sync m16n8k16 with float32 sums): the probe scores and X = K M on bf16 inputs (the arithmetic of the reference's
// tl.dot on bf16), the Lloyd iterations on float32 values split into two bf16 halves, x = hi + lo with lo = bf16(x - hi),
// 16 mantissa bits (the reference's tl.dot on float32 inputs runs as TF32 on a GPU, 10 bits; the golden outputs come
// from exact float32):
//   distances   X C^T: the warp's X fragments (hi, lo) stay in registers from the X = K M accumulators; the right operand
//               has the centroids' upper halves in columns 0-3 and their lower halves in columns 4-7, so two MMAs per
//               k-step give all four cross products and no column is padding;
//   centroids   (w X)^T (0 / 1 membership): the token weights are folded into Y = w X once per block, so the membership
//               operand is exact and two products (Y hi, Y lo) suffice; Y is read back by transposing loads;
//   final means (0 / 1 membership)^T K and V, exact products.
constexpr int KS = 136;           // bf16 row stride of the K tile: 272 B, so the 8 rows of an ldmatrix hit distinct banks
constexpr int XB = 136;           // bf16 row stride of the two halves of Y and of the centroids
constexpr int PS = 65;            // float row stride of the probe scores
constexpr int MS = 136;           // bf16 row stride of the metric in shared memory
constexpr int OS = 72;            // bf16 row stride of the (cluster, token) membership matrix
constexpr int KM_BLOCKS = 4;      // kv blocks per CTA: the metric is loaded into shared memory once for all of them
constexpr int VS = 136;           // bf16 row stride of the V tile (it takes the place of the probe scores)
constexpr int KM_SMEM = 128 * MS * 2 + 64 * KS * 2 + 2 * 64 * XB * 2 + 64 * VS * 2 + 8 * XB * 2 + 4 * 64 * 4 + 64 * 4 +
                        64 * 4 + 2 * 64 * 8 * 4 + 8 * OS * 2;
static_assert(64 * VS * 2 >= 64 * PS * 4, "the V tile and the probe scores share one area");

__device__ __forceinline__ void split_bf16(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h2 = __floats2bfloat162_rn(x, y);
    const float2 hf = __bfloat1622float2(h2);
    const __nv_bfloat162 l2 = __floats2bfloat162_rn(x - hf.x, y - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h2);
    lo = *reinterpret_cast<const uint32_t*>(&l2);
}

__global__ void __launch_bounds__(256, 2)
kmeans_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
              const __nv_bfloat16* __restrict__ metric, const __nv_bfloat16* __restrict__ probes,
              __nv_bfloat16* __restrict__ k4, __nv_bfloat16* __restrict__ v4, float* __restrict__ c4,
              __nv_bfloat16* __restrict__ km, __nv_bfloat16* __restrict__ vm, int L, int H, int nb4, int iters,
              int blocks_per_cta) {
    extern __shared__ __align__(16) uint8_t raw[];
    __nv_bfloat16* sM = reinterpret_cast<__nv_bfloat16*>(raw);                     // [128][MS] the head's metric
    __nv_bfloat16* sK = sM + 128 * MS;                                             // [64][KS]
    __nv_bfloat16* sYh = sK + 64 * KS;                                             // [64][XB] Y = w X, upper halves
    __nv_bfloat16* sYl = sYh + 64 * XB;                                            // [64][XB] Y, lower halves
    float* sP = reinterpret_cast<float*>(sYl + 64 * XB);                           // [64 probes][PS]
    __nv_bfloat16* cen = reinterpret_cast<__nv_bfloat16*>(sP) + 64 * VS;           // [8][XB] centroids: rows 0-3 upper, 4-7 lower halves
    float* wpart = reinterpret_cast<float*>(cen + 8 * XB);                         // [4][64]
    float* w = wpart + 4 * 64;                                                     // [64]
    int* lab = reinterpret_cast<int*>(w + 64);                                     // [64]
    float* dpart = reinterpret_cast<float*>(lab + 64);                             // [2 d halves][64 tokens][8 columns]
    __nv_bfloat16* oh = reinterpret_cast<__nv_bfloat16*>(dpart + 2 * 64 * 8);      // [8][OS] (cluster, token) membership, rows 4-7 zero
    __shared__ float cw[4], cwp[4][4], nnp[8][4];
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
    // rows 4-7 of the membership matrix pad the four clusters to the 8 columns of an MMA: zero for good
    for (int e = tid; e < 8 * OS / 2; e += 256) reinterpret_cast<uint32_t*>(oh)[e] = 0u;
    const int mt = warp & 3, nh = warp >> 2;
    const int lj = lane & 7, lm = lane >> 3;
    const __nv_bfloat16 one = __float2bfloat16_rn(1.0f), zero = __float2bfloat16_rn(0.0f);
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
    // this thread's A fragments of the probe scores (probes 16 mt .. +15), requested while the K tile travels
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
    cp_async_wait<0>();
    __syncthreads();
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
        w[tid] = tid < nvalid ? sacc * ((float)nvalid / (float)NP) : 0.f;
    }
    __syncthreads();
    // Warp mt of the first four owns tokens 16 mt .. +15: lane (g, tg) keeps the labels of tokens g and g + 8 and writes
    // cluster tg's column of their rows of the membership matrix; the cluster weights of the 16 tokens are added over the
    // lanes in a fixed order.
    const float w_a = w[16 * mt + g], w_b = w[16 * mt + g + 8];
    int lab_a = mt, lab_b = mt;                       // the initial clusters are the four token quarters
    auto publish = [&]() {
        oh[tg * OS + 16 * mt + g] = lab_a == tg ? one : zero;
        oh[tg * OS + 16 * mt + g + 8] = lab_b == tg ? one : zero;
        if (tg == 0) { lab[16 * mt + g] = lab_a; lab[16 * mt + g + 8] = lab_b; }
        float ws = (lab_a == tg ? w_a : 0.f) + (lab_b == tg ? w_b : 0.f);
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) ws += __shfl_xor_sync(0xffffffffu, ws, o);
        if (g == 0) cwp[mt][tg] = ws;
    };
    if (nh == 0) publish();
    // The probe scores are dead now: their area receives the V tile (64 x 128 bf16), copied asynchronously while the
    // Lloyd iterations run, so the final cluster means do not wait on global memory.
    __nv_bfloat16* sV = reinterpret_cast<__nv_bfloat16*>(sP);
    for (int e = tid; e < 64 * 16; e += 256) {
        const int r = e >> 4, c16 = e & 15;
        const bool okr = r < nvalid;
        cp_async16_zfill((uint32_t)__cvta_generic_to_shared(sV + r * VS + c16 * 8),
                         v + ((size_t)(j * 64 + (okr ? r : 0)) * H + h) * HD + c16 * 8, okr ? 16 : 0);
    }
    cp_async_commit();

    // X = K M: rows 16 mt .. +15, columns 64 nh .. +63. The accumulators of column tiles 2 ks, 2 ks + 1 are, split in two
    // bf16 halves, this warp's A fragment of k-step ks of the distance products (rows = tokens, k = these 64 dims); the
    // rows times their tokens' weights go to shared memory for the centroid sums.
    uint32_t xa_h[4][4], xa_l[4][4];
    {
        float acc[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int x = 0; x < 4; ++x) acc[nt][x] = 0.f;
        const uint32_t a_addr = (uint32_t)__cvta_generic_to_shared(sK + (16 * mt + (lane & 15)) * KS + (lane >> 4) * 8);
        const uint32_t m_addr = (uint32_t)__cvta_generic_to_shared(sM);
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
            uint32_t h0, l0, h1, l1;
            split_bf16(acc[nt][0], acc[nt][1], h0, l0);        // row g
            split_bf16(acc[nt][2], acc[nt][3], h1, l1);        // row g + 8
            xa_h[nt >> 1][(nt & 1) * 2] = h0; xa_h[nt >> 1][(nt & 1) * 2 + 1] = h1;
            xa_l[nt >> 1][(nt & 1) * 2] = l0; xa_l[nt >> 1][(nt & 1) * 2 + 1] = l1;
            split_bf16(acc[nt][0] * w_a, acc[nt][1] * w_a, h0, l0);
            split_bf16(acc[nt][2] * w_b, acc[nt][3] * w_b, h1, l1);
            const int col = 64 * nh + 8 * nt + 2 * tg;
            *reinterpret_cast<uint32_t*>(sYh + (16 * mt + g) * XB + col) = h0;
            *reinterpret_cast<uint32_t*>(sYh + (16 * mt + g + 8) * XB + col) = h1;
            *reinterpret_cast<uint32_t*>(sYl + (16 * mt + g) * XB + col) = l0;
            *reinterpret_cast<uint32_t*>(sYl + (16 * mt + g + 8) * XB + col) = l1;
        }
    }
    __syncthreads();

    // Weighted centroids of the current labels, transposed: rows = this warp's 16 dims, columns = clusters. The warp's
    // fragments of Y^T (all 64 tokens, both halves) are fetched once per block by transposing loads: matrices (tokens lo,
    // dims lo), (tokens lo, dims hi), (tokens hi, dims lo), (tokens hi, dims hi). keep_old: an emptied cluster keeps its
    // centroid (and its squared norm).
    uint32_t ya_h[4][4], ya_l[4][4];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
        const uint32_t off = (uint32_t)((16 * ks + lj + (lm >> 1) * 8) * XB + 16 * warp + (lm & 1) * 8) * 2;
        ldmatrix_x4_trans((uint32_t)__cvta_generic_to_shared(sYh) + off, ya_h[ks][0], ya_h[ks][1], ya_h[ks][2], ya_h[ks][3]);
        ldmatrix_x4_trans((uint32_t)__cvta_generic_to_shared(sYl) + off, ya_l[ks][0], ya_l[ks][1], ya_l[ks][2], ya_l[ks][3]);
    }
    auto update_centroids = [&](bool keep_old) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(oh + g * OS + 16 * ks + 2 * tg);
            const uint32_t b1 = *reinterpret_cast<const uint32_t*>(oh + g * OS + 16 * ks + 8 + 2 * tg);
            mma16816(acc, ya_h[ks][0], ya_h[ks][1], ya_h[ks][2], ya_h[ks][3], b0, b1);
            mma16816(acc, ya_l[ks][0], ya_l[ks][1], ya_l[ks][2], ya_l[ks][3], b0, b1);
        }
        // lanes with tg < 2: dims 16 warp + g and + 8 of clusters 2 tg and 2 tg + 1
        const int ca = (2 * tg) & 3, cb = ca + 1;
        const float wa = (cwp[0][ca] + cwp[1][ca]) + (cwp[2][ca] + cwp[3][ca]);
        const float wb = (cwp[0][cb] + cwp[1][cb]) + (cwp[2][cb] + cwp[3][cb]);
        const bool wr_a = tg < 2 && (!keep_old || wa > 0.f), wr_b = tg < 2 && (!keep_old || wb > 0.f);
        const float ia = 1.0f / fmaxf(wa, 1e-6f), ib = 1.0f / fmaxf(wb, 1e-6f);
        uint32_t ha, la, hb, lb;
        split_bf16(acc[0] * ia, acc[2] * ia, ha, la);          // cluster a: dims g, g + 8
        split_bf16(acc[1] * ib, acc[3] * ib, hb, lb);          // cluster b
        const int d = 16 * warp + g;
        float na = 0.f, nb2 = 0.f;
        if (wr_a) {
            cen[ca * XB + d] = __ushort_as_bfloat16((unsigned short)(ha & 0xFFFFu));
            cen[ca * XB + d + 8] = __ushort_as_bfloat16((unsigned short)(ha >> 16));
            cen[(4 + ca) * XB + d] = __ushort_as_bfloat16((unsigned short)(la & 0xFFFFu));
            cen[(4 + ca) * XB + d + 8] = __ushort_as_bfloat16((unsigned short)(la >> 16));
            const float c0 = bf_lo(ha) + bf_lo(la), c1 = bf_hi(ha) + bf_hi(la);
            na = c0 * c0 + c1 * c1;
        }
        if (wr_b) {
            cen[cb * XB + d] = __ushort_as_bfloat16((unsigned short)(hb & 0xFFFFu));
            cen[cb * XB + d + 8] = __ushort_as_bfloat16((unsigned short)(hb >> 16));
            cen[(4 + cb) * XB + d] = __ushort_as_bfloat16((unsigned short)(lb & 0xFFFFu));
            cen[(4 + cb) * XB + d + 8] = __ushort_as_bfloat16((unsigned short)(lb >> 16));
            const float c0 = bf_lo(hb) + bf_lo(lb), c1 = bf_hi(hb) + bf_hi(lb);
            nb2 = c0 * c0 + c1 * c1;
        }
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            na += __shfl_xor_sync(0xffffffffu, na, o);
            nb2 += __shfl_xor_sync(0xffffffffu, nb2, o);
        }
        if (g == 0) {                                  // the squared norms' shares of these 16 dims
            if (wr_a) nnp[warp][ca] = na;
            if (wr_b) nnp[warp][cb] = nb2;
        }
        if (warp == 0 && g == 0 && tg < 2) { cw[ca] = wa; cw[cb] = wb; }
        __syncthreads();
    };
    update_centroids(false);
    for (int it = 0; it < iters; ++it) {
        // the warp's 16 tokens against the four centroids over its 64 dims: columns 0-3 x . c_hi, columns 4-7 x . c_lo
        {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const int d = 64 * nh + 16 * ks + 2 * tg;
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(cen + g * XB + d);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(cen + g * XB + d + 8);
                mma16816(acc, xa_h[ks][0], xa_h[ks][1], xa_h[ks][2], xa_h[ks][3], b0, b1);
                mma16816(acc, xa_l[ks][0], xa_l[ks][1], xa_l[ks][2], xa_l[ks][3], b0, b1);
            }
            float* mine = dpart + (nh * 64 + 16 * mt + g) * 8 + 2 * tg;
            *reinterpret_cast<float2*>(mine) = make_float2(acc[0], acc[1]);
            *reinterpret_cast<float2*>(mine + 64) = make_float2(acc[2], acc[3]);
        }
        __syncthreads();
        int differs = 0;
        if (nh == 0) {
            // this warp's 16 tokens: both d halves, then upper + lower centroid halves (lanes tg and tg ^ 2), then the
            // smaller distance of the lane's two clusters against that of lane tg ^ 1 (ties to the smaller cluster)
            const float* p0 = dpart + (16 * mt + g) * 8 + 2 * tg;
            const float2 a0 = *reinterpret_cast<const float2*>(p0), a1 = *reinterpret_cast<const float2*>(p0 + 64 * 8);
            const float2 b0 = *reinterpret_cast<const float2*>(p0 + 64), b1 = *reinterpret_cast<const float2*>(p0 + 64 * 8 + 64);
            float da[2] = {a0.x + a1.x, a0.y + a1.y}, db[2] = {b0.x + b1.x, b0.y + b1.y};
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                da[e] += __shfl_xor_sync(0xffffffffu, da[e], 2);
                db[e] += __shfl_xor_sync(0xffffffffu, db[e], 2);
            }
            const int c0 = (2 * tg) & 3;              // lanes tg and tg ^ 2 hold clusters c0, c0 + 1
            float dist_a[2], dist_b[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int cc = c0 + e;
                const float nn = ((nnp[0][cc] + nnp[1][cc]) + (nnp[2][cc] + nnp[3][cc])) +
                                 ((nnp[4][cc] + nnp[5][cc]) + (nnp[6][cc] + nnp[7][cc]));
                const bool live = cw[cc] > 0.f;
                dist_a[e] = live ? nn - 2.0f * da[e] : INFINITY;
                dist_b[e] = live ? nn - 2.0f * db[e] : INFINITY;
            }
            auto pick = [&](const float (&d)[2]) -> int {
                float bd = d[0];
                int bi = c0;
                if (d[1] < bd) { bd = d[1]; bi = c0 + 1; }
                const float od = __shfl_xor_sync(0xffffffffu, bd, 1);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, 1);
                return (od < bd || (od == bd && oi < bi)) ? oi : bi;
            };
            const int na = pick(dist_a), nb_ = pick(dist_b);
            differs = (16 * mt + g < nvalid && na != lab_a) || (16 * mt + g + 8 < nvalid && nb_ != lab_b);
            lab_a = na; lab_b = nb_;
            publish();
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
            // membership of the valid tokens only (the last readers passed the barrier that ended the iterations)
            oh[c * OS + lane] = l0 == c ? one : zero;
            oh[c * OS + lane + 32] = l1 == c ? one : zero;
        }
    }
    cp_async_wait<0>();
    __syncthreads();
#pragma unroll
    for (int which = 0; which < 2; ++which) {
        // (membership)^T K and (membership)^T V: rows = clusters (4 of 16), columns = this warp's 16 dims; products with
        // 0 / 1 are exact, the sums are float32
        float acc[2][4];
#pragma unroll
        for (int jj = 0; jj < 2; ++jj)
#pragma unroll
            for (int x = 0; x < 4; ++x) acc[jj][x] = 0.f;
        const uint32_t src = (uint32_t)__cvta_generic_to_shared(which ? sV : sK);
        const int stride = which ? VS : KS;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const uint32_t a0 = *reinterpret_cast<const uint32_t*>(oh + g * OS + 16 * ks + 2 * tg);
            const uint32_t a2 = *reinterpret_cast<const uint32_t*>(oh + g * OS + 16 * ks + 8 + 2 * tg);
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(src + (uint32_t)((16 * ks + lj + (lm & 1) * 8) * stride + 16 * warp + (lm >> 1) * 8) * 2, b0, b1, b2, b3);
            mma16816(acc[0], a0, 0u, a2, 0u, b0, b1);
            mma16816(acc[1], a0, 0u, a2, 0u, b2, b3);
        }
        const float inv = g < 4 ? 1.0f / fmaxf(s_cnt[g], 1.0f) : 0.f;
        __nv_bfloat16* o = (which ? v4 : k4) + ((size_t)h * nb4 + j * 4 + (g & 3)) * HD + 16 * warp + 2 * tg;
        __nv_bfloat16* mo = which ? vm : km;
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
            if (g < 4) *reinterpret_cast<__nv_bfloat162*>(o + 8 * jj) = __floats2bfloat162_rn(acc[jj][0] * inv, acc[jj][1] * inv);
            // block mean: the four clusters' sums, (0 + 1) + (2 + 3), held by lanes 4 c + tg
            float t0 = acc[jj][0], t1 = acc[jj][1];
            t0 += __shfl_xor_sync(0xffffffffu, t0, 4); t1 += __shfl_xor_sync(0xffffffffu, t1, 4);
            t0 += __shfl_xor_sync(0xffffffffu, t0, 8); t1 += __shfl_xor_sync(0xffffffffu, t1, 8);
            if (mo && g == 0)
                *reinterpret_cast<__nv_bfloat162*>(mo + ((size_t)j * H + h) * HD + 16 * warp + 8 * jj + 2 * tg) =
                    __floats2bfloat162_rn(t0 / (float)nvalid, t1 / (float)nvalid);
        }
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
