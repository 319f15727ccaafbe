// Fixed-offset block-sparse attention for sm_100a: one CTA per (128-row query tile, head).
//
// What it computes (reference: echosparse/kernels/block_attention.py:206-303, sparse_attention.py:1-13, 430-575,
// and the same formula in echosparse/kernels/sm120.py:27-96): for query row r with offset m_r (the previous step's
// log2 LSE), over three kinds of columns,
//     p = 2^(c * q_r.k_j - m_r + bias_j),   l_r = sum p,   O_r = sum bf16(p) v_j / l_r,   lse_r = m_r + log2 l_r
//   exact:  the tokens of the listed 64-token blocks (bias 0, tail tokens past L masked),
//   mean:   one column per block whose bit in skip_bits is clear: the block's mean key / value, bias log2(len),
//   refine: four representatives of every block of the tile's refine list, bias log2(cluster size).
// mass[h, tile, b] = sum over the tile's rows of the exact block b's p; flag[tile, h] = some valid row has
// log2 l_r outside [-th, th].  There is no running maximum and no rescaling.
//
// FALLBACK = true is the online-softmax recomputation of flagged tiles (triton_ops.py:203-234): a first sweep of QK
// MMAs finds every row's maximum logit, then the same fixed-offset pipeline runs with that maximum as the offset,
// which is the online-softmax result without rescaling steps.
//
// Pipeline: warps 0-3 softmax (thread = query row), warp 4 issues tcgen05 MMAs, warp 5 issues TMA loads / gathers.
// An iteration covers 128 columns as two 64-column halves, each with its own K slot, V slot, S/P columns in tensor
// memory and barriers, so PV of one half and QK of the next iteration overlap the softmax of the other half.
// Tensor memory: columns [0,128) S (fp32) with P (bf16 pairs) written over it, [128,256) O. Two CTAs fit an SM.
#include "es_ptx.cuh"
#include "es_api_internal.h"

namespace es {

constexpr int BM = 128;       // query rows per tile
constexpr int BK = 64;        // tokens per kv block
constexpr int HD = 128;       // head dim
constexpr int NTHREADS = 192;
constexpr uint32_t TMEM_COLS = 256;
constexpr uint32_t O_COL = 128;
constexpr int NSLOT = 5;      // K/V tiles in flight per CTA (two CTAs share an SM's shared memory)

constexpr uint32_t Q_BYTES = BM * HD * 2;        // 32 KB: [d half][128 rows][64 d] 128B-swizzled
constexpr uint32_t KV_BYTES = BK * HD * 2;       // 16 KB: [d half][64 rows][64 d]
constexpr uint32_t SMEM_Q = 0;
constexpr uint32_t SMEM_RING = SMEM_Q + Q_BYTES;                 // NSLOT tiles, K or V
constexpr uint32_t SMEM_CTL = SMEM_RING + NSLOT * KV_BYTES;      // barriers and small scratch
constexpr uint32_t SMEM_ALLOC = SMEM_CTL + 512;

struct Ctl {
    uint64_t qfull;
    uint64_t full[NSLOT], empty[NSLOT];
    uint64_t sfull[2], pfull[2];
    uint64_t ofull, drain;
    uint64_t massbar, flagbar;     // softmax warps' lane 0 -> the thread that adds their partial results
    uint32_t tmem_base;
    int abort;
    int flag_part[4];
    float mass_part[2][2][4];      // [iteration parity][half][warp]
};
static_assert(sizeof(Ctl) <= 512, "control block");

struct AttnArgs {
    __nv_bfloat16* out;
    const int* counts;           // (nq, H)
    const int* blocks;           // (nq, H, nk) ascending block ids
    int nk;
    const float* offset;         // (nq*128, H) log2
    float* lse;                  // (nq*128, H) log2
    int* flags;                  // (nq, H)
    float* mass;                 // (H, nq, nb) or null
    const int* skip_bits;        // (H, nq, nw)
    int nw;
    const int* refine;           // (nq, H, rw) padded with nb
    int rw;
    const __nv_bfloat16* k_rep;  // (H, nb4, 128)
    const __nv_bfloat16* v_rep;
    const float* log_counts;     // (H, nb4)
    int nb4;
    int L, H, nq, nb;
    float scale_log2, th;
    int tail_valid;              // tokens of the last block
    float tail_log2;             // log2(tail_valid)
    int nvirt, nref;             // mean iterations (128 blocks each), refine iterations (32 list entries each)
    int* status;
    uint32_t* trace;             // optional clock trace of the first CTAs (null: off); see es_debug_set_trace
};

// Clock trace for pipeline debugging: CTAs 0 .. TRACE_CTAS-1, softmax thread 0 (role 0) and the MMA thread (role 1),
// the first TRACE_ITERS iterations, both halves, 8 time stamps each (clock cycles since the CTA started).
constexpr int TRACE_CTAS = 8, TRACE_ITERS = 64;
__device__ __forceinline__ void trace_put(uint32_t* tr, int role, int i, int x, int k, long long t0) {
    if (tr != nullptr && blockIdx.x < TRACE_CTAS && i < TRACE_ITERS)
        tr[((((size_t)blockIdx.x * 2 + role) * TRACE_ITERS + i) * 2 + x) * 8 + k] = (uint32_t)(clock64() - t0);
}

// K-major operand tile [d half][rows][64]: 8-row groups 1024 B apart; k step ks (16 elements) of the MMA.
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t base, uint32_t half_bytes, int ks) {
    return umma_desc_sw128(base + (uint32_t)(ks >> 2) * half_bytes + (uint32_t)(ks & 3) * 32, 16, 1024);
}
// MN-major B tile (V): [d half][key rows][64 d]; N chunks of 64 d are `half_bytes` apart, 8-key groups 1024 B apart;
// k step ks covers 16 keys.
__device__ __forceinline__ uint64_t mnmajor_desc(uint32_t base, uint32_t half_bytes, int ks) {
    return umma_desc_sw128(base + (uint32_t)ks * 2048, half_bytes, 1024);
}

// 64 rows x 256 B gathered into one 128B-swizzled slot by the 32 lanes of a warp: list entry e (block `my` of lane
// 16*half + e) supplies rows 4e .. 4e+3, which are contiguous in the representative table.
__device__ __forceinline__ void gather_slot(uint32_t slot, const __nv_bfloat16* table, int my, int half, int lane,
                                            uint32_t bar) {
    const int c16 = lane & 15, kh = c16 >> 3, cc = c16 & 7;
#pragma unroll 8
    for (int it = 0; it < 32; ++it) {
        const int b = __shfl_sync(0xffffffffu, my, 16 * half + (it >> 1));
        const int row = 2 * it + (lane >> 4);
        const uint32_t dst = slot + (uint32_t)kh * (KV_BYTES / 2) + (uint32_t)row * 128 + (uint32_t)((cc ^ (row & 7)) << 4);
        const char* src = reinterpret_cast<const char*>(table) + ((size_t)(4 * b + (row & 3))) * 256 + c16 * 16;
        cp_async16(dst, src);
    }
    cp_async_mbar_arrive(bar);
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}

// p = 2^x for a pair of columns. MUFU computes 16 exponentials per clock and SM, as many clocks as the tensor cores need
// for the same tile, so a share of the pairs (EMU) is computed on the FMA pipe instead: x = n + f with n = floor(x),
// 2^f by a degree-4 polynomial (relative error 3e-6, far below the bf16 rounding of P), n added to the exponent field.
__device__ __forceinline__ float2 exp2_pair_mufu(float2 x) { return make_float2(ex2_approx(x.x), ex2_approx(x.y)); }
__device__ __forceinline__ float2 exp2_pair_fma(float2 x) {
    const float M = 12582912.0f;                               // 2^23 + 2^22: the integer part lands in the low mantissa bits
    x.x = fmaxf(x.x, -126.0f);
    x.y = fmaxf(x.y, -126.0f);
    const float2 t = __fadd2_rd(x, make_float2(M, M));         // rounded down: f stays in [0, 1)
    const float2 n = __fadd2_rn(t, make_float2(-M, -M));
    const float2 f = __fadd2_rn(x, make_float2(-n.x, -n.y));
    float2 p = make_float2(0.013426586054265499f, 0.013426586054265499f);
    p = __ffma2_rn(p, f, make_float2(0.05224263295531273f, 0.05224263295531273f));
    p = __ffma2_rn(p, f, make_float2(0.24128012359142303f, 0.24128012359142303f));
    p = __ffma2_rn(p, f, make_float2(0.6930448412895203f, 0.6930448412895203f));
    p = __ffma2_rn(p, f, make_float2(1.0f, 1.0f));
    p.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
    p.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
    return p;
}
// Pair j (columns 2j, 2j+1) of a 64-column half goes to the FMA pipe when bit (j & 3) of EMU_PATTERN is set.
#ifndef ES_EMU_PATTERN
#define ES_EMU_PATTERN 0x5
#endif
__device__ __forceinline__ constexpr bool emulate_pair(int j) { return (ES_EMU_PATTERN >> (j & 3)) & 1; }

template <bool FALLBACK>
__global__ void __launch_bounds__(NTHREADS, 2)
attention_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmKm,
                 const __grid_constant__ CUtensorMap tmVm, const AttnArgs a) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long long t_start = clock64();
    // adjacent CTAs are adjacent query tiles of one head: their kv lists overlap in L2
    const int qb = blockIdx.x % a.nq, h = blockIdx.x / a.nq;
    const int th_idx = qb * a.H + h;
    if (FALLBACK) {
        if (a.flags[th_idx] == 0) return;          // uniform over the CTA, before anything is allocated
    }

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + SMEM_CTL);
    const uint32_t sQ = base + SMEM_Q, sRing = base + SMEM_RING;
    volatile int* abort_flag = &ctl->abort;

    if (tid == 0) {
        if (base & 1023u) atomicCAS(a.status, 0, 901);   // the swizzled tiles need a 1024-byte aligned base
        mbar_init(smem_u32(&ctl->qfull), 1);
        for (int i = 0; i < NSLOT; ++i) {
            mbar_init(smem_u32(&ctl->full[i]), 1);
            mbar_init(smem_u32(&ctl->empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&ctl->sfull[i]), 1);
            mbar_init(smem_u32(&ctl->pfull[i]), 128);
        }
        mbar_init(smem_u32(&ctl->ofull), 1);
        mbar_init(smem_u32(&ctl->drain), 1);
        mbar_init(smem_u32(&ctl->massbar), 4);
        mbar_init(smem_u32(&ctl->flagbar), 4);
        ctl->abort = (base & 1023u) ? 1 : 0;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == 4) {
        tmem_alloc(smem_u32(&ctl->tmem_base), TMEM_COLS);
        tmem_relinquish();
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctl->tmem_base;

    const int n64 = a.counts[th_idx];
    const int n = (n64 + 1) >> 1;                     // exact iterations: pairs of 64-token blocks
    const int nvirt = FALLBACK ? 0 : a.nvirt;
    const int nref = FALLBACK ? 0 : a.nref;
    const int nt = n + nvirt + nref;
    const int* list = a.blocks + (size_t)th_idx * a.nk;

    // K and V tiles travel through one ring of NSLOT slots in the order the MMA warp consumes them:
    //   [fallback sweep: Ka(0) Kb(0) Ka(1) Kb(1) ...]  Ka(0) Kb(0)  { Va(i) Ka(i+1) Vb(i) Kb(i+1) } for i = 0 .. nt-1
    // tile number `seq` lives in slot seq % NSLOT; its barriers are in phase (seq / NSLOT) & 1.
    uint32_t pseq = 0;                                // producer: tiles issued (used again at teardown)

    if (warp == 5) {
        // ------------------------------------------------------------ loads (all lanes walk the sequence together)
        bool ok = true;
        if (lane == 0) {
            tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
            mbar_arrive_expect_tx(smem_u32(&ctl->qfull), Q_BYTES);
            tma_load_3d(sQ, &tmQ, smem_u32(&ctl->qfull), 0, qb * BM, h);
            tma_load_3d(sQ + Q_BYTES / 2, &tmQ, smem_u32(&ctl->qfull), 64, qb * BM, h);
        }
        const __nv_bfloat16* krep = a.k_rep + (size_t)h * a.nb4 * HD;
        const __nv_bfloat16* vrep = a.v_rep + (size_t)h * a.nb4 * HD;
        const int* rl = a.refine + (size_t)th_idx * a.rw;
        // tile of iteration i, half x: K (is_v = false) or V
        auto put = [&](int i, int x, bool is_v) {
            if (!ok) return;
            const uint32_t slot = pseq % NSLOT, par = ((pseq / NSLOT) & 1) ^ 1;
            if (lane == 0) ok = mbar_wait(smem_u32(&ctl->empty[slot]), par, abort_flag, a.status, 101);
            ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;     // the other lanes sleep at the shuffle instead of polling
            if (!ok) return;
            const uint32_t dst = sRing + slot * KV_BYTES, bar = smem_u32(&ctl->full[slot]);
            if (i < n + nvirt) {
                if (lane == 0) {
                    int row;
                    const CUtensorMap* m;
                    if (i < n) {
                        const int e = 2 * i + x;
                        row = list[e < n64 ? e : e - 1] * BK;           // odd list: block a again, masked in the softmax
                        m = is_v ? &tmV : &tmK;
                    } else {
                        row = (i - n) * 128 + 64 * x;                   // rows of the block-mean tables
                        m = is_v ? &tmVm : &tmKm;
                    }
                    mbar_arrive_expect_tx(bar, KV_BYTES);
                    tma_load_3d(dst, m, bar, 0, row, h);
                    tma_load_3d(dst + KV_BYTES / 2, m, bar, 64, row, h);
                }
            } else {
                // refine iteration: list entry 32 c + e fills columns 4e .. 4e+3 of the 128-column tile
                const int my = rl[32 * (i - n - nvirt) + lane];
                gather_slot(dst, is_v ? vrep : krep, my, x, lane, bar);
            }
            ++pseq;
        };
        if (FALLBACK) {
            for (int i = 0; i < n; ++i) { put(i, 0, false); put(i, 1, false); }
        }
        if (nt > 0) { put(0, 0, false); put(0, 1, false); }
        for (int i = 0; i < nt; ++i) {
            put(i, 0, true);
            if (i + 1 < nt) put(i + 1, 0, false);
            put(i, 1, true);
            if (i + 1 < nt) put(i + 1, 1, false);
        }
    } else if (warp == 4) {
        // ------------------------------------------------------------ MMAs: the warp runs uniformly, one elected lane issues
        {
            constexpr uint32_t IDESC_QK = umma_idesc_bf16(BM, BK, 0);
            constexpr uint32_t IDESC_PV = umma_idesc_bf16(BM, HD, 1);
            // Shared-memory descriptors: everything but the start address is a constant of the layout, so the words are
            // built once and an MMA costs one add. K-major (Q, K): LBO 16, SBO 1024; MN-major (V): LBO = half tile, SBO 1024.
            const uint64_t dk0 = umma_desc_sw128(0, 16, 1024), dv0 = umma_desc_sw128(0, KV_BYTES / 2, 1024);
            const uint32_t k_hi = (uint32_t)(dk0 >> 32), k_lo0 = (uint32_t)dk0;
            const uint32_t v_hi = (uint32_t)(dv0 >> 32), v_lo0 = (uint32_t)dv0;
            uint32_t q_lo[HD / 16];
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks)
                q_lo[ks] = k_lo0 + ((sQ + (uint32_t)(ks >> 2) * (Q_BYTES / 2) + (uint32_t)(ks & 3) * 32) >> 4);
            uint32_t cseq = 0, nQK[2] = {0, 0}, wP[2] = {0, 0};
            bool ok = mbar_wait(smem_u32(&ctl->qfull), 0, abort_flag, a.status, 201);
            auto take = [&](bool gathered) -> uint32_t {
                const uint32_t slot = cseq % NSLOT;
                ok = ok && mbar_wait(smem_u32(&ctl->full[slot]), (cseq / NSLOT) & 1, abort_flag, a.status, 202);
                ++cseq;
                if (gathered) fence_proxy_async_smem();    // cp.async gathers are generic-proxy writes
                return slot;
            };
            // S of half x <- Q K_x^T. The S columns also hold the previous P of that half: every earlier use must have
            // been handed back by the softmax warps (pfull) before they are overwritten.
            auto issue_qk = [&](int x, bool gathered) {
                const uint32_t slot = take(gathered);
                while (ok && wP[x] < nQK[x]) {
                    ok = mbar_wait(smem_u32(&ctl->pfull[x]), wP[x] & 1, abort_flag, a.status, 203);
                    ++wP[x];
                }
                if (!ok) return;
                tc_fence_after();
                const uint32_t d = tmem + (uint32_t)x * BK;
                const uint32_t kb_lo = k_lo0 + ((sRing + slot * KV_BYTES) >> 4);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)
                    if (elect_one()) umma_ss_lohi(d, q_lo[ks], k_hi, kb_lo + (uint32_t)(((ks >> 2) * (KV_BYTES / 2) + (ks & 3) * 32) >> 4), k_hi,
                                 IDESC_QK, ks > 0);
                if (elect_one()) umma_commit(smem_u32(&ctl->sfull[x]));
                if (elect_one()) umma_commit(smem_u32(&ctl->empty[slot]));
                ++nQK[x];
            };
            if (FALLBACK) {
                for (int i = 0; i < n && ok; ++i) { issue_qk(0, false); issue_qk(1, false); }
            }
            if (nt > 0) {
                issue_qk(0, n + nvirt == 0);
                issue_qk(1, n + nvirt == 0);
            }
            for (int i = 0; i < nt && ok; ++i) {
                const bool gat = i >= n + nvirt, nxg = i + 1 >= n + nvirt;
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    if (!ok) break;
                    if (lane == 0) trace_put(a.trace, 1, i, x, 0, t_start);
                    const uint32_t slot = take(gat);
                    if (lane == 0) trace_put(a.trace, 1, i, x, 1, t_start);
                    ok = ok && mbar_wait(smem_u32(&ctl->pfull[x]), wP[x] & 1, abort_flag, a.status, 205);   // P_x(i) stored
                    if (lane == 0) trace_put(a.trace, 1, i, x, 2, t_start);
                    if (!ok) break;
                    ++wP[x];
                    tc_fence_after();
                    const uint32_t p = tmem + (uint32_t)x * BK;            // bf16 pairs over the first 32 S columns
                    const uint32_t vb_lo = v_lo0 + ((sRing + slot * KV_BYTES) >> 4);
#pragma unroll
                    for (int ks = 0; ks < BK / 16; ++ks)
                        if (elect_one()) umma_ts_lohi(tmem + O_COL, p + ks * 8, vb_lo + (uint32_t)((ks * 2048) >> 4), v_hi, IDESC_PV,
                                     (i > 0 || x > 0 || ks > 0) ? 1u : 0u);
                    if (elect_one()) umma_commit(smem_u32(&ctl->empty[slot]));
                    if (i + 1 == nt && x == 1) if (elect_one()) umma_commit(smem_u32(&ctl->ofull));
                    if (lane == 0) trace_put(a.trace, 1, i, x, 3, t_start);
                    if (i + 1 < nt) {
                        const uint32_t kslot = take(nxg);
                        if (lane == 0) trace_put(a.trace, 1, i, x, 4, t_start);
                        // P_x(i) was waited for above, so S_x is free again
                        const uint32_t d = tmem + (uint32_t)x * BK;
                        const uint32_t kb_lo = k_lo0 + ((sRing + kslot * KV_BYTES) >> 4);
                        if (ok) {
#pragma unroll
                            for (int ks = 0; ks < HD / 16; ++ks)
                                if (elect_one()) umma_ss_lohi(d, q_lo[ks], k_hi,
                                             kb_lo + (uint32_t)(((ks >> 2) * (KV_BYTES / 2) + (ks & 3) * 32) >> 4), k_hi,
                                             IDESC_QK, ks > 0);
                            if (elect_one()) umma_commit(smem_u32(&ctl->sfull[x]));
                            if (elect_one()) umma_commit(smem_u32(&ctl->empty[kslot]));
                            ++nQK[x];
                        }
                    }
                    if (lane == 0) trace_put(a.trace, 1, i, x, 5, t_start);
                }
            }
            // every MMA issued above has finished before tensor memory is freed
            if (elect_one()) umma_commit(smem_u32(&ctl->drain));
            mbar_wait(smem_u32(&ctl->drain), 0, abort_flag, a.status, 206);
        }
    } else {
        // ------------------------------------------------------------ softmax and epilogue: thread t = row t
        const int row = qb * BM + tid;
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        float m = a.offset[(size_t)row * a.H + h];
        uint32_t uS[2] = {0, 0}, uM = 0;
        bool ok = true;
        uint32_t s[64];

        if (FALLBACK) {
            float mx = -INFINITY;
            for (int i = 0; i < n && ok; ++i) {
                const int ba = list[2 * i];
                const bool has_b = 2 * i + 1 < n64;
                const int bb = has_b ? list[2 * i + 1] : ba;
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    ok = ok && mbar_wait(smem_u32(&ctl->sfull[x]), uS[x] & 1, abort_flag, a.status, 301);
                    if (!ok) break;
                    ++uS[x];
                    tc_fence_after();
                    tmem_ld32(lane_base + x * BK, &s[0]);
                    tmem_ld32(lane_base + x * BK + 32, &s[32]);
                    tmem_wait_ld();
                    tc_fence_before();
                    mbar_arrive(smem_u32(&ctl->pfull[x]));
                    const int blk = x == 0 ? ba : bb;
                    int lim = (blk == a.nb - 1) ? a.tail_valid : BK;
                    if (x == 1 && !has_b) lim = 0;
#pragma unroll
                    for (int c = 0; c < 64; ++c)
                        if (c < lim) mx = fmaxf(mx, __uint_as_float(s[c]));
                }
            }
            m = (mx == -INFINITY) ? 0.f : mx * a.scale_log2;
        }

        float2 lsum[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        const int* rl = a.refine + (size_t)th_idx * a.rw;
        const float* lc = a.log_counts + (size_t)h * a.nb4;
        const int* bits = a.skip_bits + ((size_t)h * a.nq + qb) * a.nw;
        const bool want_mass = !FALLBACK && a.mass != nullptr;
        const float2 sc2 = make_float2(a.scale_log2, a.scale_log2);

        // block ids of the exact iteration that comes next, loaded one iteration ahead
        int nba = n > 0 ? list[0] : 0, nbb = n64 > 1 ? list[1] : nba;
        // thread 0 stores the masses of an iteration at the start of the next one: by then the other warps' partial sums
        // have long arrived, so the store never holds back the warp that the other three wait for
        int pend_a = -1, pend_b = -1, pend_buf = 0;
        auto flush_mass = [&]() {
            if (tid == 0 && pend_a >= 0) {
                ok = mbar_wait(smem_u32(&ctl->massbar), uM & 1, abort_flag, a.status, 304);
                ++uM;
                if (ok) {
                    const float* mp = ctl->mass_part[pend_buf][0];
                    float* mrow = a.mass + ((size_t)h * a.nq + qb) * a.nb;
                    mrow[pend_a] = ((mp[0] + mp[1]) + mp[2]) + mp[3];
                    if (pend_b >= 0) mrow[pend_b] = ((mp[4] + mp[5]) + mp[6]) + mp[7];
                }
                pend_a = -1;
            }
        };
        for (int i = 0; i < nt && ok; ++i) {
            const bool exact = i < n, pooled = !exact && i < n + nvirt;
            const int ba = nba, bb = nbb;
            const bool has_b = 2 * i + 1 < n64 || !exact;
            if (i + 1 < n) {
                nba = list[2 * i + 2];
                nbb = 2 * i + 3 < n64 ? list[2 * i + 3] : nba;
            }
            flush_mass();
            float part[2];
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                if (tid == 0) trace_put(a.trace, 0, i, x, 0, t_start);
                ok = ok && mbar_wait(smem_u32(&ctl->sfull[x]), uS[x] & 1, abort_flag, a.status, 302);
                if (!ok) break;
                if (tid == 0) trace_put(a.trace, 0, i, x, 1, t_start);
                ++uS[x];
                tc_fence_after();
                tmem_ld32(lane_base + x * BK, &s[0]);
                tmem_ld32(lane_base + x * BK + 32, &s[32]);
                tmem_wait_ld();
                if (tid == 0) trace_put(a.trace, 0, i, x, 2, t_start);
                float2 acc = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
                uint32_t pk[32];
                if (exact) {
                    const int blk = x == 0 ? ba : bb;
                    int lim = (blk == a.nb - 1) ? a.tail_valid : BK;
                    if (x == 1 && !has_b) lim = 0;
                    const float2 off2 = make_float2(-m, -m);
                    if (lim == BK) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float2 xv = __ffma2_rn(make_float2(__uint_as_float(s[2 * j]), __uint_as_float(s[2 * j + 1])), sc2, off2);
                            const float2 p = emulate_pair(j) ? exp2_pair_fma(xv) : exp2_pair_mufu(xv);
                            if (j & 1) acc1 = __fadd2_rn(acc1, p); else acc = __fadd2_rn(acc, p);
                            pk[j] = pack_bf16x2(p.x, p.y);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float2 xv = __ffma2_rn(make_float2(__uint_as_float(s[2 * j]), __uint_as_float(s[2 * j + 1])), sc2, off2);
                            float2 p = exp2_pair_mufu(xv);
                            p.x = 2 * j < lim ? p.x : 0.f;
                            p.y = 2 * j + 1 < lim ? p.y : 0.f;
                            acc = __fadd2_rn(acc, p);
                            pk[j] = pack_bf16x2(p.x, p.y);
                        }
                    }
                } else if (pooled) {
                    // block-mean columns: column c of this half is block 128 cv + 64 x + c; a set bit masks it
                    const int cv = i - n;
                    const uint32_t w0 = (uint32_t)bits[4 * cv + 2 * x], w1 = (uint32_t)bits[4 * cv + 2 * x + 1];
                    const float2 off2 = make_float2(-m + 6.0f, -m + 6.0f);   // log2(64): a mean stands for its block's tokens
                    const int last_c = (a.nb - 1) - (128 * cv + 64 * x);   // column of the (maybe shorter) last block
                    const float fix = a.tail_log2 - 6.0f;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float2 xv = __ffma2_rn(make_float2(__uint_as_float(s[2 * j]), __uint_as_float(s[2 * j + 1])), sc2, off2);
                        if (2 * j == last_c) xv.x += fix;
                        if (2 * j + 1 == last_c) xv.y += fix;
                        float2 p = exp2_pair_mufu(xv);
                        const uint32_t w = j < 16 ? w0 : w1;
                        p.x = ((w >> ((2 * j) & 31)) & 1u) ? 0.f : p.x;
                        p.y = ((w >> ((2 * j + 1) & 31)) & 1u) ? 0.f : p.y;
                        acc = __fadd2_rn(acc, p);
                        pk[j] = pack_bf16x2(p.x, p.y);
                    }
                } else {
                    // representatives: columns 4e .. 4e+3 of this half belong to list entry 32 cr + 16 x + e
                    const int cr = i - n - nvirt;
                    const int4* ent = reinterpret_cast<const int4*>(rl + 32 * cr + 16 * x);
#pragma unroll
                    for (int e4 = 0; e4 < 4; ++e4) {
                        const int4 bq = __ldg(ent + e4);
                        const int bl[4] = {bq.x, bq.y, bq.z, bq.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float4 b4 = __ldg(reinterpret_cast<const float4*>(lc + 4 * bl[j]));
                            const int c = 16 * e4 + 4 * j;
                            const float2 x0 = __ffma2_rn(make_float2(__uint_as_float(s[c]), __uint_as_float(s[c + 1])), sc2,
                                                         make_float2(b4.x - m, b4.y - m));
                            const float2 x1 = __ffma2_rn(make_float2(__uint_as_float(s[c + 2]), __uint_as_float(s[c + 3])), sc2,
                                                         make_float2(b4.z - m, b4.w - m));
                            const float2 p0 = exp2_pair_mufu(x0), p1 = exp2_pair_mufu(x1);
                            acc = __fadd2_rn(acc, p0);
                            acc1 = __fadd2_rn(acc1, p1);
                            pk[c / 2] = pack_bf16x2(p0.x, p0.y);
                            pk[c / 2 + 1] = pack_bf16x2(p1.x, p1.y);
                        }
                    }
                }
                if (tid == 0) trace_put(a.trace, 0, i, x, 3, t_start);
                tmem_st32(lane_base + x * BK, pk);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(smem_u32(&ctl->pfull[x]));
                if (tid == 0) trace_put(a.trace, 0, i, x, 4, t_start);
                acc = __fadd2_rn(acc, acc1);
                part[x] = acc.x + acc.y;
                lsum[x] = __fadd2_rn(lsum[x], acc);
            }
            if (!ok) break;
            if (want_mass && exact) {
                // per-block mass: 32 rows by shuffle, the four warps' partial sums added in a fixed order by one
                // thread and stored (no atomics: the map is reproducible bit for bit)
                float pa = part[0], pb = part[1];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    pa += __shfl_xor_sync(0xffffffffu, pa, o);
                    pb += __shfl_xor_sync(0xffffffffu, pb, o);
                }
                // The partial sums are double-buffered over iterations: a warp can write those of iteration i + 2
                // only after S(i + 2) exists, which needs thread 0's pfull arrivals of iteration i + 1, made after
                // it has stored the masses of iteration i.
                if (lane == 0) {
                    ctl->mass_part[i & 1][0][warp] = pa;
                    ctl->mass_part[i & 1][1][warp] = pb;
                    mbar_arrive(smem_u32(&ctl->massbar));
                }
                pend_a = ba;
                pend_b = has_b ? bb : -1;
                pend_buf = i & 1;
            }
        }
        if (ok) flush_mass();

        // ---- epilogue
        const float l = (lsum[0].x + lsum[0].y) + (lsum[1].x + lsum[1].y);
        const float lg = log2f(l);
        const bool valid = row < a.L;
        if (nt > 0) ok = ok && mbar_wait(smem_u32(&ctl->ofull), 0, abort_flag, a.status, 303);
        if (ok) {
            tc_fence_after();
            const float inv = 1.0f / l;
            __nv_bfloat16* orow = a.out + ((size_t)row * a.H + h) * HD;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch) {
                uint32_t* o = &s[0];
                if (nt > 0) {
                    tmem_ld32(lane_base + O_COL + ch * 32, o);
                    tmem_wait_ld();
                }
                if (valid) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint4 w;
                        w.x = pack_bf16x2(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
                        w.y = pack_bf16x2(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
                        w.z = pack_bf16x2(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
                        w.w = pack_bf16x2(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
                        if (nt == 0) w = make_uint4(0, 0, 0, 0);
                        *reinterpret_cast<uint4*>(orow + ch * 32 + c) = w;
                    }
                }
            }
            tc_fence_before();
            // rows past L keep the "no offset" value, as echosparse/kernels/sm120.py:96
            a.lse[(size_t)row * a.H + h] = valid ? m + lg : 1e30f;
            if (!FALLBACK) {
                // a tile whose row sums leave 2^[-th, th] is flagged and recomputed with online softmax
                const bool bad = valid && !(lg >= -a.th && lg <= a.th);
                const unsigned ballot = __ballot_sync(0xffffffffu, bad);
                if (lane == 0) {
                    ctl->flag_part[warp] = ballot != 0;
                    mbar_arrive(smem_u32(&ctl->flagbar));
                }
                if (tid == 0 && mbar_wait(smem_u32(&ctl->flagbar), 0, abort_flag, a.status, 305))
                    a.flags[th_idx] = ctl->flag_part[0] | ctl->flag_part[1] | ctl->flag_part[2] | ctl->flag_part[3];
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    __syncwarp();
    if (warp == 5 && lane == 0 && *abort_flag) {
        // a wait gave up somewhere: let the loads already issued land before the CTA's shared memory goes away
        auto settle = [](uint32_t bar, uint32_t parity) {
            for (uint32_t t = 0; t < (1u << 20) && !mbar_try_wait(bar, parity); ++t) {}
        };
        settle(smem_u32(&ctl->qfull), 0);
        for (uint32_t back = 1; back <= NSLOT && back <= pseq; ++back) {
            const uint32_t sq = pseq - back;
            settle(smem_u32(&ctl->full[sq % NSLOT]), (sq / NSLOT) & 1);
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------------- host side
static int make_map(CUtensorMap* m, const void* ptr, int rows, int H, int box_rows) {
    // (rows, H, 128) bf16 viewed as dims {128 d, rows, H}; a box is 64 d x box_rows rows, 128-byte swizzled
    cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)rows, (cuuint64_t)H};
    cuuint64_t strides[2] = {(cuuint64_t)H * HD * 2, (cuuint64_t)HD * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return encode_tensor_map(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                             CU_TENSOR_MAP_SWIZZLE_128B);
}

static uint32_t* g_trace = nullptr;

struct AttnCall {
    const void *q, *k, *v, *k_mean, *v_mean;
    AttnArgs a;
};

static int launch_attention(const AttnCall& c, bool fallback, cudaStream_t stream) {
    const AttnArgs& a = c.a;
    if (a.L <= 0 || a.H <= 0) return set_error(-1, "attention: L and H must be positive");
    if (((uintptr_t)c.q | (uintptr_t)c.k | (uintptr_t)c.v | (uintptr_t)a.out) & 15)
        return set_error(-1, "attention: q, k, v, out must be 16-byte aligned");
    CUtensorMap tq, tk, tv, tkm, tvm;
    int rc;
    if ((rc = make_map(&tq, c.q, a.L, a.H, BM))) return rc;
    if ((rc = make_map(&tk, c.k, a.L, a.H, BK))) return rc;
    if ((rc = make_map(&tv, c.v, a.L, a.H, BK))) return rc;
    if (c.k_mean) {
        if ((rc = make_map(&tkm, c.k_mean, a.nb, a.H, BK))) return rc;
        if ((rc = make_map(&tvm, c.v_mean, a.nb, a.H, BK))) return rc;
    } else {
        tkm = tk; tvm = tv;
    }
    static bool attr_set[2] = {false, false};
    auto kern = fallback ? attention_kernel<true> : attention_kernel<false>;
    if (!attr_set[fallback]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_ALLOC);
        if (e != cudaSuccess) return set_error(-2, cudaGetErrorString(e));
        attr_set[fallback] = true;
    }
    kern<<<a.nq * a.H, NTHREADS, SMEM_ALLOC, stream>>>(tq, tk, tv, tkm, tvm, a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(-2, cudaGetErrorString(e));
    count_launch();
    return 0;
}

static void fill_common(AttnArgs& a, int L, int H, float threshold) {
    a.L = L; a.H = H;
    a.nq = (L + BM - 1) / BM;
    a.nb = (L + BK - 1) / BK;
    a.scale_log2 = 1.4426950408889634f / sqrtf((float)HD);
    a.th = threshold;
    a.tail_valid = L - (a.nb - 1) * BK;
    a.tail_log2 = log2f((float)a.tail_valid);
    a.status = device_status_ptr();
    a.trace = g_trace;
}

}  // namespace es

using namespace es;

extern "C" int es_block_attention(const void* q, const void* k, const void* v, void* out, const int32_t* counts,
                                  const int32_t* blocks, int32_t nk, const float* offset, float* lse, int32_t* flags,
                                  float* mass, int32_t L, int32_t H, float threshold, void* stream) {
    if (!q || !k || !v || !out || !counts || !blocks || !offset || !lse || !flags)
        return set_error(-1, "es_block_attention: null pointer");
    AttnCall c{};
    c.q = q; c.k = k; c.v = v; c.k_mean = nullptr; c.v_mean = nullptr;
    fill_common(c.a, L, H, threshold);
    c.a.out = (__nv_bfloat16*)out; c.a.counts = counts; c.a.blocks = blocks; c.a.nk = nk;
    c.a.offset = offset; c.a.lse = lse; c.a.flags = flags; c.a.mass = mass;
    c.a.nvirt = 0; c.a.nref = 0;
    return launch_attention(c, false, (cudaStream_t)stream);
}

extern "C" int es_sparse_attention(const void* q, const void* k, const void* v, const void* k_mean, const void* v_mean,
                                   const int32_t* skip_bits, int32_t nw, void* out, const int32_t* counts,
                                   const int32_t* blocks, int32_t nk, const float* offset, float* lse, int32_t* flags,
                                   const int32_t* refine, int32_t rw, const void* k_rep, const void* v_rep,
                                   const float* log_counts, float* mass, int32_t L, int32_t H, float threshold,
                                   void* stream) {
    if (!q || !k || !v || !out || !counts || !blocks || !offset || !lse || !flags || !k_mean || !v_mean || !skip_bits)
        return set_error(-1, "es_sparse_attention: null pointer");
    AttnCall c{};
    c.q = q; c.k = k; c.v = v; c.k_mean = k_mean; c.v_mean = v_mean;
    fill_common(c.a, L, H, threshold);
    c.a.out = (__nv_bfloat16*)out; c.a.counts = counts; c.a.blocks = blocks; c.a.nk = nk;
    c.a.offset = offset; c.a.lse = lse; c.a.flags = flags; c.a.mass = mass;
    c.a.skip_bits = skip_bits; c.a.nw = nw;
    c.a.nvirt = (c.a.nb + 127) / 128;
    if (nw < 4 * c.a.nvirt) return set_error(-1, "es_sparse_attention: skip_bits needs 4 * ceil(nb / 128) words per tile");
    if (rw % 32 != 0) return set_error(-1, "es_sparse_attention: refine width must be a multiple of 32");
    if (rw > 0 && (!refine || !k_rep || !v_rep || !log_counts))
        return set_error(-1, "es_sparse_attention: refine list without representative tables");
    if (rw > 0 && ((uintptr_t)refine & 15)) return set_error(-1, "es_sparse_attention: refine must be 16-byte aligned");
    c.a.refine = refine; c.a.rw = rw; c.a.nref = rw / 32;
    c.a.k_rep = (const __nv_bfloat16*)k_rep; c.a.v_rep = (const __nv_bfloat16*)v_rep; c.a.log_counts = log_counts;
    c.a.nb4 = (c.a.nb + 1) * 4;
    return launch_attention(c, false, (cudaStream_t)stream);
}

extern "C" int es_exact_fallback(const void* q, const void* k, const void* v, void* out, const int32_t* counts,
                                 const int32_t* blocks, int32_t nk, float* lse, const int32_t* flags, int32_t L,
                                 int32_t H, void* stream) {
    if (!q || !k || !v || !out || !counts || !blocks || !lse || !flags)
        return set_error(-1, "es_exact_fallback: null pointer");
    AttnCall c{};
    c.q = q; c.k = k; c.v = v; c.k_mean = nullptr; c.v_mean = nullptr;
    fill_common(c.a, L, H, 0.f);
    c.a.out = (__nv_bfloat16*)out; c.a.counts = counts; c.a.blocks = blocks; c.a.nk = nk;
    c.a.offset = lse; c.a.lse = lse; c.a.flags = const_cast<int32_t*>(flags); c.a.mass = nullptr;
    c.a.nvirt = 0; c.a.nref = 0;
    return launch_attention(c, true, (cudaStream_t)stream);
}

// Debugging aid: when `buffer` (device memory, es_debug_trace_words() 32-bit words, zeroed by the caller) is not NULL,
// the attention kernels launched afterwards record clock stamps of their first CTAs' pipeline stages into it.
extern "C" int es_debug_set_trace(void* buffer) {
    es::g_trace = static_cast<uint32_t*>(buffer);
    return 0;
}
extern "C" int es_debug_trace_words(void) { return es::TRACE_CTAS * 2 * es::TRACE_ITERS * 2 * 8; }
