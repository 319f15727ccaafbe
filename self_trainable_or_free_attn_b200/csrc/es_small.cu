// The memory-bound kernels around the attention kernel: block means, per-tile scales, mass estimates of the skipped
// blocks (the block-mean compensation of fallback tiles is a mode of the attention kernel). Vectorised 16-byte loads, warp shuffles, mma.sync for the
// one small contraction (16 sampled query rows x block-mean keys).
#include "es_api_internal.h"
#include "es_vsa_mma.cuh"

#include <cuda_bf16.h>
#include <math.h>

namespace es {

constexpr int HD = 128;
constexpr float LOG2E_F = 1.4426950408889634f;

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// ------------------------------------------------------------------------------------------------ block means
// Mean key and value of every 64-token block, (L, H, 128) -> (nb, H, 128); the tail block divides by its real length
// (echosparse/kernels/triton_ops.py:21-40). One CTA per (block, head): thread = (row group of 4 rows, 16-byte column).
__global__ void __launch_bounds__(256)
block_mean_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                  __nv_bfloat16* __restrict__ km, __nv_bfloat16* __restrict__ vm, int L, int H) {
    __shared__ float part[2][16][HD];
    const int j = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int rg = tid >> 4, c16 = tid & 15;
    float ak[8] = {0, 0, 0, 0, 0, 0, 0, 0}, av[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = j * 64 + i * 16 + rg;
        if (row < L) {
            const size_t off = ((size_t)row * H + h) * HD + c16 * 8;
            const uint4 a = *reinterpret_cast<const uint4*>(k + off);
            const uint4 b = *reinterpret_cast<const uint4*>(v + off);
            ak[0] += bf16_lo(a.x); ak[1] += bf16_hi(a.x); ak[2] += bf16_lo(a.y); ak[3] += bf16_hi(a.y);
            ak[4] += bf16_lo(a.z); ak[5] += bf16_hi(a.z); ak[6] += bf16_lo(a.w); ak[7] += bf16_hi(a.w);
            av[0] += bf16_lo(b.x); av[1] += bf16_hi(b.x); av[2] += bf16_lo(b.y); av[3] += bf16_hi(b.y);
            av[4] += bf16_lo(b.z); av[5] += bf16_hi(b.z); av[6] += bf16_lo(b.w); av[7] += bf16_hi(b.w);
        }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        part[0][rg][c16 * 8 + e] = ak[e];
        part[1][rg][c16 * 8 + e] = av[e];
    }
    __syncthreads();
    const int which = tid >> 7, d = tid & 127;
    float s = 0.f;
#pragma unroll
    for (int g = 0; g < 16; ++g) s += part[which][g][d];
    const float n = (float)min(L - j * 64, 64);
    (which ? vm : km)[((size_t)j * H + h) * HD + d] = __float2bfloat16_rn(s / n);
}

// ------------------------------------------------------------------------------------------------ full-step scales
// After a step that computed every block (triton_ops.py:180-199): scale_exact = mean_rows 2^clamp(m - lse) / rows,
// scale_skip = 1, and the padding rows of lse go back to 1e30.
__global__ void __launch_bounds__(128)
full_scale_kernel(const float* __restrict__ m, float* __restrict__ lse, float* __restrict__ scale_exact,
                  float* __restrict__ scale_skip, int L, int H, int nq) {
    __shared__ float part[4];
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int row = t * 128 + tid;
    const bool rv = row < L;
    const float nrows = (float)min(L - t * 128, 128);
    const float ls = lse[(size_t)row * H + h];
    if (!rv) lse[(size_t)row * H + h] = 1e30f;
    float f = rv ? exp2f(fminf(fmaxf(m[(size_t)row * H + h] - ls, -100.f), 100.f)) : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) f += __shfl_xor_sync(0xffffffffu, f, o);
    if ((tid & 31) == 0) part[tid >> 5] = f;
    __syncthreads();
    if (tid == 0) {
        const float s = (part[0] + part[1]) + (part[2] + part[3]);
        scale_exact[h * nq + t] = s / nrows / nrows;
        scale_skip[h * nq + t] = 1.0f;
    }
}

// ------------------------------------------------------------------------------------------------ estimates
// Mass estimates of the skipped blocks for the next selection, and the per-tile scales (triton_ops.py:122-177):
//   est[t, b] = mean over 16 sampled rows r = 128 t + 8 s of 2^min(c q_r.kmean_b - m_r + log2 len_b, 100), written into
//   the map for blocks that were not kept; f = mean_rows 2^clamp(m - m_new); scale_exact = f / rows;
//   scale_skip = f * clamp((sum_kept mass / rows) / sum_kept est, 1, 64).
// One CTA per (8 consecutive tiles, head), one warp per tile. The block-mean keys travel through shared memory in tiles of
// 64 blocks (cp.async, two stages, 16-byte chunks XOR-swizzled by the row) that all eight warps consume with ldmatrix:
// S(16 sampled rows x 64 blocks) by mma.sync m16n8k16 over d. Reading the keys once per eight tiles with 16-byte accesses,
// instead of once per tile with 4-byte ones, is what the kernel's time depends on (the keys of a head are 300 KB).
constexpr int EST_TILES = 8;
__global__ void __launch_bounds__(256)
estimate_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ km,
                const uint8_t* __restrict__ keep, const float* __restrict__ m, const float* __restrict__ mnew,
                float* __restrict__ map, float* __restrict__ scale_exact, float* __restrict__ scale_skip,
                float scale_log2, int L, int nb, float lb_last, int H, int nq) {
    using namespace es::vsa;
    __shared__ __align__(128) uint8_t tiles[2][64 * HD * 2];
    const int h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t = blockIdx.x * EST_TILES + warp;
    const bool tv = t < nq;                                   // warps past the last tile still help with the copies
    const int g = lane >> 2, tg = lane & 3;
    // A fragments of the 16 sampled rows (row s -> query row 128 t + 8 s), all 8 k-steps
    uint32_t afr[8][4];
    const int r0 = t * 128 + 8 * g, r1 = t * 128 + 8 * (g + 8);
    const bool v0 = tv && r0 < L, v1 = tv && r1 < L;
    const __nv_bfloat16* q0 = q + ((size_t)(v0 ? r0 : 0) * H + h) * HD;
    const __nv_bfloat16* q1 = q + ((size_t)(v1 ? r1 : 0) * H + h) * HD;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
        const int d = ks * 16 + tg * 2;
        afr[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + d) : 0u;
        afr[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + d) : 0u;
        afr[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + d + 8) : 0u;
        afr[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + d + 8) : 0u;
    }
    const float m0 = v0 ? m[(size_t)r0 * H + h] : 0.f, m1 = v1 ? m[(size_t)r1 * H + h] : 0.f;
    int nsv = 0;
    for (int s = 0; s < 16; ++s) nsv += tv && (t * 128 + 8 * s) < L;
    const float inv_ns = 1.0f / fmaxf((float)nsv, 1.0f);
    const size_t mbase = ((size_t)h * nq + (tv ? t : 0)) * nb;
    const int nct = (nb + 63) / 64;
    auto load_keys = [&](int stage, int ct) {
        const uint32_t dst = smem_addr(tiles[stage]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {                         // 64 rows x 16 chunks of 16 bytes over 256 threads
            const int idx = i * 256 + tid, row = idx >> 4, ch = idx & 15;
            const int blk = min(ct * 64 + row, nb - 1);       // rows past the last block repeat it; their columns are masked
            cp16(dst + tile_off<HD>(row, ch), km + ((size_t)blk * H + h) * HD + ch * 8);
        }
    };
    load_keys(0, 0);
    cp_commit();
    float num = 0.f, den = 0.f;
    for (int ct = 0; ct < nct; ++ct) {
        if (ct + 1 < nct) load_keys((ct + 1) & 1, ct + 1);
        cp_commit();
        cp_wait<1>();
        __syncthreads();
        const uint32_t tile = smem_addr(tiles[ct & 1]);
        // Lane l owns blocks 64 ct + 2 l, + 1 of the chunk in the map: their keep bytes and masses are requested here, before
        // the products, so that the loads have landed when the estimates are ready (asked for one by one after the
        // products, behind the branch on the keep byte, they were a chain of dependent round trips to L2).
        const int c0 = ct * 64 + 2 * lane;
        const bool in0 = tv && c0 < nb, in1 = tv && c0 + 1 < nb;
        const uint8_t kp0 = in0 ? keep[mbase + c0] : (uint8_t)0, kp1 = in1 ? keep[mbase + c0 + 1] : (uint8_t)0;
        const float old0 = in0 ? map[mbase + c0] : 0.f, old1 = in1 ? map[mbase + c0 + 1] : 0.f;
        float acc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b[4];
                load_b_nk<HD>(tile, np, ks, lane, b);
                Elt<__nv_bfloat16>::mma(acc[2 * np], afr[ks], b[0], b[1]);
                Elt<__nv_bfloat16>::mma(acc[2 * np + 1], afr[ks], b[2], b[3]);
            }
        // acc[i][0], acc[i][1]: row g, blocks 64 ct + 8 i + 2 tg, + 1; acc[i][2], acc[i][3]: row g + 8. After the sums over
        // the 16 rows (the lanes with the same tg) every lane holds the estimates of blocks 8 i + 2 tg, + 1 for all i;
        // the pair with i == g is the one this lane owns: 8 g + 2 tg = 2 lane.
        float est0 = 0.f, est1 = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float e[2];
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                const int cc = ct * 64 + i * 8 + 2 * tg + x;
                const float lb = (cc == nb - 1) ? lb_last : 6.0f;
                const float e0 = v0 ? exp2f(fminf(acc[i][x] * scale_log2 - m0 + lb, 100.f)) : 0.f;
                const float e1 = v1 ? exp2f(fminf(acc[i][2 + x] * scale_log2 - m1 + lb, 100.f)) : 0.f;
                float s2 = e0 + e1;
                s2 += __shfl_xor_sync(0xffffffffu, s2, 4);
                s2 += __shfl_xor_sync(0xffffffffu, s2, 8);
                s2 += __shfl_xor_sync(0xffffffffu, s2, 16);
                e[x] = s2 * inv_ns;
            }
            if (i == g) { est0 = e[0]; est1 = e[1]; }
        }
        // kept blocks: their exact masses calibrate the estimates; the others receive their estimate
        if (in0) {
            if (kp0 != 0) { num += old0; den += est0; } else map[mbase + c0] = est0;
        }
        if (in1) {
            if (kp1 != 0) { num += old1; den += est1; } else map[mbase + c0 + 1] = est1;
        }
        __syncthreads();
    }
    cp_wait<0>();
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        num += __shfl_xor_sync(0xffffffffu, num, o);
        den += __shfl_xor_sync(0xffffffffu, den, o);
    }
    if (!tv) return;
    // f over the tile's rows: four per lane, summed in a fixed order
    float f = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = t * 128 + 32 * i + lane;
        if (row < L) {
            const float a = m[(size_t)row * H + h], b = mnew[(size_t)row * H + h];
            f += exp2f(fminf(fmaxf(a - b, -100.f), 100.f));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) f += __shfl_xor_sync(0xffffffffu, f, o);
    if (lane == 0) {
        const float nrows = (float)min(L - t * 128, 128);
        const float ff = f / nrows;
        scale_exact[h * nq + t] = ff / nrows;
        // The block-mean estimate underestimates block mass (Jensen): calibrate it on the blocks computed exactly.
        const float nn = num / nrows;
        const float c = den > 0.f ? fminf(fmaxf(nn / fmaxf(den, 1e-30f), 1.0f), 64.0f) : 1.0f;
        scale_skip[h * nq + t] = ff * c;
    }
}

}  // namespace es

using namespace es;

extern "C" int es_block_means(const void* k, const void* v, void* k_mean, void* v_mean, int32_t L, int32_t H,
                              void* stream) {
    if (!k || !v || !k_mean || !v_mean) return set_error(-1, "es_block_means: null pointer");
    if (L <= 0 || H <= 0) return set_error(-1, "es_block_means: L and H must be positive");
    if (((uintptr_t)k | (uintptr_t)v) & 15) return set_error(-1, "es_block_means: k and v must be 16-byte aligned");
    const int nb = (L + 63) / 64;
    block_mean_kernel<<<dim3(nb, H), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)k_mean, (__nv_bfloat16*)v_mean, L, H);
    ES_CHECK_LAUNCH("block_means");
    return 0;
}

extern "C" int es_full_step_scales(const float* offset, float* lse, float* scale_exact, float* scale_skip, int32_t L,
                                   int32_t H, void* stream) {
    if (!offset || !lse || !scale_exact || !scale_skip) return set_error(-1, "es_full_step_scales: null pointer");
    if (L <= 0 || H <= 0) return set_error(-1, "es_full_step_scales: L and H must be positive");
    const int nq = (L + 127) / 128;
    full_scale_kernel<<<dim3(nq, H), 128, 0, (cudaStream_t)stream>>>(offset, lse, scale_exact, scale_skip, L, H, nq);
    ES_CHECK_LAUNCH("full_step_scales");
    return 0;
}

extern "C" int es_estimate_skipped(const void* q, const void* k_mean, const uint8_t* keep, const float* offset,
                                   const float* lse, float* mass, float* scale_exact, float* scale_skip, int32_t L,
                                   int32_t H, void* stream) {
    if (!q || !k_mean || !keep || !offset || !lse || !mass || !scale_exact || !scale_skip)
        return set_error(-1, "es_estimate_skipped: null pointer");
    if (L <= 0 || H <= 0) return set_error(-1, "es_estimate_skipped: L and H must be positive");
    const int nq = (L + 127) / 128, nb = (L + 63) / 64;
    const int tail = L - (nb - 1) * 64;
    estimate_kernel<<<dim3((nq + EST_TILES - 1) / EST_TILES, H), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_mean, keep, offset, lse, mass, scale_exact, scale_skip,
        LOG2E_F / sqrtf((float)HD), L, nb, log2f((float)tail), H, nq);
    ES_CHECK_LAUNCH("estimate_skipped");
    return 0;
}
