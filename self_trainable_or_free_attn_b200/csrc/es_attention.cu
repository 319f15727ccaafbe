// Fixed-offset block-sparse attention for sm_100a: one CTA per (128-row query tile, head), one CTA per SM.
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
// Pipeline. An iteration covers 128 columns (two 64-token blocks, 128 block means, or 32 refine entries x 4).
//   warps 0-7  softmax: warp w owns rows 32 (w % 4) .. +31 of the tile and columns 64 (w / 4) .. +63 of the iteration
//   warp 8     issues the tcgen05 MMAs (one elected lane); warps 9 and 10 issue the TMA loads of the K and of the V
//              tiles (control code is one dependent chain per tile: two warps halve its length); warp 11 sums and
//              stores the block masses
// Tensor memory (512 columns): S of even iterations [0,128), S of odd iterations [128,256), O [256,384), Q [384,448).
// Q sits in tensor memory as the A operand of QK^T, so the only shared-memory traffic of the MMAs is K and V: with Q in
// shared memory a 128 x 64 x 16 MMA reads 6 KB in the 32 clocks it computes, more than the 128 B/clock an SM delivers.
// P (bf16 pairs) is written over the S columns it came from and is the A operand of PV. Two S buffers let QK of
// iteration i + 1 run while the softmax warps work on iteration i; PV(i) and QK(i + 2) follow as soon as P(i) is stored.
// K and V tiles (32 KB each, [d half][128 rows][128 B], four 8 KB TMA boxes; representative rows: 64 boxes of 512 B)
// travel through a ring of NSLOT shared-memory slots, about three iterations ahead of the MMAs.
#include "es_ptx.cuh"
#include "es_api_internal.h"

namespace es {

constexpr int BM = 128;       // query rows per tile
constexpr int BK = 64;        // tokens per kv block
constexpr int HD = 128;       // head dim
constexpr int NSOFT = 256;    // softmax threads
constexpr int NTHREADS = NSOFT + 128;
constexpr int MMA_WARP = NSOFT / 32, LOADK_WARP = MMA_WARP + 1, LOADV_WARP = MMA_WARP + 2, MASS_WARP = MMA_WARP + 3;
constexpr int NMASS = 8;      // sets of partial block masses in flight between the softmax warps and the mass warp
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t O_COL = 256, Q_COL = 384;
constexpr int NSLOT = 6;      // K / V tiles in flight
constexpr int NBIAS = 8;      // refine iterations whose column biases are staged in shared memory at a time

constexpr uint32_t TILE_BYTES = 128 * HD * 2;    // 32 KB: [d half][128 rows][64 d], 128B-swizzled
constexpr uint32_t HALF_BYTES = TILE_BYTES / 2;  // one d half: 128 rows x 128 B
constexpr uint32_t BLK_BYTES = BK * 128;         // 64 rows of one d half: one TMA box
constexpr uint32_t SMEM_RING = 0;
constexpr uint32_t SMEM_CTL = SMEM_RING + NSLOT * TILE_BYTES;
constexpr uint32_t SMEM_BIAS = SMEM_CTL + 3072;                        // [NBIAS][128] floats
constexpr uint32_t SMEM_MASS = SMEM_BIAS + NBIAS * 128 * 4;            // [NMASS][2 column halves][128 rows] floats
constexpr uint32_t SMEM_ALLOC = SMEM_MASS + NMASS * 2 * BM * 4;        // 211,968 B: one CTA per SM

struct Ctl {
    uint64_t qfull;
    uint64_t full[NSLOT], empty[NSLOT];
    uint64_t sfull[2], pfull[2];
    uint64_t ofull, drain;
    uint64_t massbar[NMASS], flagbar, lbar;   // softmax warps -> the thread(s) that combine their partial results
    uint64_t massfree[NMASS];             // mass warp -> softmax warps: the set's partial sums have been read
    uint64_t sweepbar;                 // K load warp -> V load warp: the fallback sweep's tiles have all been issued
    uint32_t tmem_base;
    int abort;
    int flag_part[4];
    float l_part[2][BM];               // row sums of the two column halves
    float m_part[2][BM];               // row maxima of the two column halves (fallback sweep)
};
static_assert(sizeof(Ctl) <= 3072, "control block");

struct AttnArgs {
    const __nv_bfloat16* q;      // (L, H, 128)
    const uint8_t* keep;         // (H, nq, nb), compensation mode only
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
    const int* tile_list;        // fallback modes: tiles to process (head * nq + tile), ascending, or null: every CTA tests its flag
    const int* tile_count;       // entries of tile_list
    int* status;
};

// p = 2^x for a pair of columns. MUFU computes 16 exponentials per clock and SM, about as many clocks as the tensor
// cores need for the same tile, so a share of the pairs can be computed on the FMA pipe instead: x = n + f with
// n = floor(x), 2^f by a degree-4 polynomial (relative error 3e-6, far below the bf16 rounding of P), n added to the
// exponent field.
__device__ __forceinline__ float2 exp2_pair_mufu(float2 x) { return make_float2(ex2_approx(x.x), ex2_approx(x.y)); }
__device__ __forceinline__ float2 exp2_pair_fma(float2 x) {
    const float M = 12582912.0f;                               // 2^23 + 2^22: the integer part lands in the low mantissa bits
    x.x = fmaxf(x.x, -126.0f);
    x.y = fmaxf(x.y, -126.0f);
    const float2 t = __fadd2_rd(x, make_float2(M, M));         // rounded down: f stays in [0, 1)
    const float2 n = __fadd2_rn(t, make_float2(-M, -M));
    const float2 f = __ffma2_rn(n, make_float2(-1.0f, -1.0f), x);
    float2 p = make_float2(0.013426586054265499f, 0.013426586054265499f);
    p = __ffma2_rn(p, f, make_float2(0.05224263295531273f, 0.05224263295531273f));
    p = __ffma2_rn(p, f, make_float2(0.24128012359142303f, 0.24128012359142303f));
    p = __ffma2_rn(p, f, make_float2(0.6930448412895203f, 0.6930448412895203f));
    p = __ffma2_rn(p, f, make_float2(1.0f, 1.0f));
    p.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
    p.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
    return p;
}
// Pair j (columns 2j, 2j+1) of a thread's 64 columns goes to the FMA pipe when bit (j & 7) of ES_EMU_PATTERN is set.
// Measured on B200 with this kernel: 0x00 (all MUFU) 1.549 ms, 0x11 1.561 ms, 0x55 1.660 ms (Wan-1.3B shape), so the
// default keeps every exponential on MUFU; the FMA path stays available for parts with a different balance.
#ifndef ES_EMU_PATTERN
#define ES_EMU_PATTERN 0x0
#endif
__device__ __forceinline__ constexpr bool emulate_pair(int j) { return (ES_EMU_PATTERN >> (j & 7)) & 1; }

// Order of a tile's iterations. The refine iterations (64 small TMA boxes per tile, slow to fill) are spread evenly among
// the others instead of coming last, so that the ring refills during the cheap iterations in between: iteration i is the
// refine iteration i / p when i % p == p - 1 and i / p < nref (p = nt / nref); the other iterations are the exact ones,
// then the block-mean ones, in their order. kind: 0 exact, 1 block means, 2 refine; idx counts within the kind.
struct Sched {
    int n, nvirt, nref, p;
    __device__ __forceinline__ void decode(int i, int& kind, int& idx) const {
        if (nref > 0) {
            const int q = i / p;
            if (i - q * p == p - 1 && q < nref) { kind = 2; idx = q; return; }
            i -= min(q, nref);
        }
        if (i < n) { kind = 0; idx = i; }
        else { kind = 1; idx = i - n; }
    }
};

// The same order walked one iteration at a time, without the division: ph = i % p, q = i / p, o = iterations before i
// that are not refine iterations.
struct SchedIter {
    int ph = 0, q = 0, o = 0;
    __device__ __forceinline__ void get(const Sched& s, int& kind, int& idx) const {
        if (s.nref > 0 && ph == s.p - 1 && q < s.nref) { kind = 2; idx = q; }
        else if (o < s.n) { kind = 0; idx = o; }
        else { kind = 1; idx = o - s.n; }
    }
    __device__ __forceinline__ void advance(const Sched& s) {
        if (!(s.nref > 0 && ph == s.p - 1 && q < s.nref)) ++o;
        if (++ph == s.p) { ph = 0; ++q; }
    }
};

// One (query tile, head): `tile` = head * nq + query tile. `again`: the CTA has run a tile before (its barriers exist).
template <int MODE>
__device__ __forceinline__ void attention_tile(const CUtensorMap& tmK, const CUtensorMap& tmV, const CUtensorMap& tmKm,
                                               const CUtensorMap& tmVm, const CUtensorMap& tmKr, const CUtensorMap& tmVr,
                                               const AttnArgs& a, const int tile, const bool again) {
    constexpr bool FALLBACK = MODE == 1;       // online-softmax recomputation of flagged tiles
    constexpr bool COMPENSATE = MODE == 2;     // block-mean compensation of flagged tiles, added to out / lse in place
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // adjacent tile numbers are adjacent query tiles of one head: their kv lists overlap in L2
    const int qb = tile % a.nq, h = tile / a.nq;
    const int th_idx = qb * a.H + h;
    if (FALLBACK || COMPENSATE) {
        if (a.flags[th_idx] == 0) return;          // uniform over the CTA, before anything is allocated
    }
    // The tile's first global loads do not depend on one another: the list length, the first window of block ids (load
    // warps) and this thread's half of its Q row (softmax warps) are requested here (in the fallback modes: once the tile
    // is known to be flagged), before the status check, the barrier set-up and the tensor-memory allocation, whose
    // latencies they then share instead of following them.
    const int n64_early = COMPENSATE ? 0 : __ldg(a.counts + th_idx);
    int win_early = 0;
    uint4 q_early[8];
    if (warp == LOADK_WARP || warp == LOADV_WARP) {
        if (!COMPENSATE && lane < a.nk) win_early = __ldg(a.blocks + (size_t)th_idx * a.nk + lane);
    } else if (warp < NSOFT / 32) {
        const int r0 = qb * BM + 32 * (warp & 3) + lane;
        const uint4* src = reinterpret_cast<const uint4*>(a.q + ((size_t)(r0 < a.L ? r0 : 0) * a.H + h) * HD + 64 * (warp >> 2));
#pragma unroll
        for (int i = 0; i < 8; ++i) q_early[i] = r0 < a.L ? __ldg(src + i) : make_uint4(0, 0, 0, 0);
    }
    // a wait has given up earlier (the status word is set until the host reads it): do not start more work
    if (*reinterpret_cast<volatile int*>(a.status) != 0) return;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + SMEM_CTL);
    const uint32_t sRing = base + SMEM_RING;
    volatile int* abort_flag = &ctl->abort;
    float* bias_ring = reinterpret_cast<float*>(smem_raw + SMEM_BIAS);
    float* mass_rows = reinterpret_cast<float*>(smem_raw + SMEM_MASS);

    if (tid == 0) {
        if (base & 1023u) atomicCAS(a.status, 0, 901);   // the swizzled tiles need a 1024-byte aligned base
        if (again) {
            // a CTA that walks a list of tiles makes its barriers anew for every tile
            for (uint64_t* b = &ctl->qfull; b <= &ctl->sweepbar; ++b) mbar_inval(smem_u32(b));
        }
        mbar_init(smem_u32(&ctl->qfull), NSOFT);
        for (int i = 0; i < NSLOT; ++i) {
            mbar_init(smem_u32(&ctl->full[i]), 1);
            mbar_init(smem_u32(&ctl->empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&ctl->sfull[i]), 1);
            mbar_init(smem_u32(&ctl->pfull[i]), NSOFT);
        }
        mbar_init(smem_u32(&ctl->ofull), 1);
        mbar_init(smem_u32(&ctl->drain), 1);
        for (int i = 0; i < NMASS; ++i) {
            mbar_init(smem_u32(&ctl->massbar[i]), 8);
            mbar_init(smem_u32(&ctl->massfree[i]), 1);
        }
        mbar_init(smem_u32(&ctl->flagbar), 4);
        mbar_init(smem_u32(&ctl->lbar), NSOFT);
        mbar_init(smem_u32(&ctl->sweepbar), 1);
        ctl->abort = (base & 1023u) ? 1 : 0;
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&ctl->tmem_base), TMEM_COLS);
        // a CTA that walks a tile list allocates again for its next tile, so it keeps its permit to allocate
        if ((MODE == 0 || a.tile_list == nullptr) && !again) tmem_relinquish();
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctl->tmem_base;

    const int n64 = n64_early;
    const int n = (n64 + 1) >> 1;                     // exact iterations: pairs of 64-token blocks
    const int nvirt = FALLBACK ? 0 : a.nvirt;
    const int nref = (FALLBACK || COMPENSATE) ? 0 : a.nref;
    const int nt = n + nvirt + nref;
    const int* list = a.blocks + (size_t)th_idx * a.nk;
    const Sched sched{n, nvirt, nref, nref > 0 ? max(nt / nref, 1) : 1};

    // K and V tiles travel through one ring of NSLOT slots in the order the MMA warp consumes them:
    //   [fallback sweep: K(0) K(1) ... K(n-1)]  K(0) K(1)  { V(i) K(i+2) } for i = 0 .. nt-1
    // tile number `seq` lives in slot seq % NSLOT; its barriers are in phase (seq / NSLOT) & 1.
    uint32_t pseq = 0;                                // load warps: one past the last tile issued (used again at teardown)

    if (warp == LOADK_WARP || warp == LOADV_WARP) {
        // ------------------------------------------------------------ loads: one warp walks the K tiles, one the V tiles
        const bool is_v = warp == LOADV_WARP;
        bool ok = true;
        const CUtensorMap* map_x = is_v ? &tmV : &tmK;       // exact blocks
        const CUtensorMap* map_m = is_v ? &tmVm : &tmKm;     // block means
        const CUtensorMap* map_r = is_v ? &tmVr : &tmKr;     // representative tables
        if (lane == 0) { tma_prefetch_desc(map_x); tma_prefetch_desc(map_m); tma_prefetch_desc(map_r); }
        const int* rl = a.refine + (size_t)th_idx * a.rw;
        const uint32_t full0 = smem_u32(&ctl->full[0]), empty0 = smem_u32(&ctl->empty[0]);
        const uint32_t box_off = (uint32_t)(lane >> 1) * HALF_BYTES + (uint32_t)(lane & 1) * BLK_BYTES;   // lanes 0..3
        const int box_x = (lane >> 1) * 64;
        // block ids: a 32-entry window of the list held across the lanes, one coalesced load per 16 iterations
        int win = lane < n64 ? win_early : 0, wbase = 0;       // the first window was requested at the top of the kernel
        // tile number `seq` of the ring: K or V tile of iteration i (i < 0: K tile -i-1 of the fallback sweep)
        auto put = [&](uint32_t seq, int i) {
            if (!ok) return;
            int ra = 0, rb = 64;
            const CUtensorMap* m = map_m;
            int kind, idx;
            if (i < 0) { kind = 0; idx = -i - 1; }        // a K tile of the fallback sweep
            else sched.decode(i, kind, idx);
            if (kind == 0) {
                const int e = 2 * idx;
                if ((e & ~31) != wbase) {
                    wbase = e & ~31;
                    win = (wbase + lane < n64) ? list[wbase + lane] : 0;
                }
                ra = __shfl_sync(0xffffffffu, win, e & 31) * BK;
                rb = __shfl_sync(0xffffffffu, win, (e + 1) & 31) * BK;
                if (e + 1 >= n64) rb = ra;                     // odd list: block a again, masked in the softmax
                m = map_x;
            } else {
                ra = idx * 128;                                // rows of the block-mean tables
                rb = ra + 64;
            }
            const uint32_t slot = seq % NSLOT, par = ((seq / NSLOT) & 1) ^ 1;
            if (lane == 0) ok = mbar_wait(empty0 + 8 * slot, par, abort_flag, a.status, 101);
            ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;     // the other lanes sleep at the shuffle instead of polling
            if (!ok) return;
            const uint32_t dst = sRing + slot * TILE_BYTES, bar = full0 + 8 * slot;
            if (kind != 2) {
                if (lane == 0) mbar_arrive_expect_tx(bar, TILE_BYTES);
                __syncwarp();
                if (lane < 4) tma_load_3d(dst + box_off, m, bar, box_x, (lane & 1) ? rb : ra, h);
            } else {
                // refine iteration: list entry 32 c + e (held by lane e) fills rows 4e .. 4e+3 of the tile: the block's four
                // representatives are contiguous rows of the table, one 512-byte TMA box per d half
                const int cr = idx;
                const int my = rl[32 * cr + lane];
                if (!is_v) {
                    // the 128 column biases (log2 cluster sizes) of this iteration, for the softmax warps. Slot cr % NBIAS is
                    // free again: this tile's ring slot was released by QK(i - 3), which was issued after the softmax warps
                    // had handed over iteration i - 5.
                    *reinterpret_cast<float4*>(bias_ring + (cr % NBIAS) * 128 + 4 * lane) =
                        __ldg(reinterpret_cast<const float4*>(a.log_counts + (size_t)h * a.nb4 + 4 * my));
                    __syncwarp();
                }
                if (lane == 0) mbar_arrive_expect_tx(bar, TILE_BYTES);
                __syncwarp();
                tma_load_3d(dst + (uint32_t)lane * 512u, map_r, bar, 0, 4 * my, h);
                tma_load_3d(dst + HALF_BYTES + (uint32_t)lane * 512u, map_r, bar, 64, 4 * my, h);
            }
            pseq = seq + 1;
        };
        uint32_t base = 0;
        if (FALLBACK) {
            // The sweep's K tiles come first in the ring. A wait on a slot's `empty` barrier can only tell two consecutive
            // rounds apart (one parity bit), so the V warp must not start polling while the ring is still rounds behind
            // its first tile: it starts once the K warp has issued the last sweep tile.
            if (!is_v) {
                for (int i = 0; i < n; ++i) put((uint32_t)i, -i - 1);
                if (lane == 0) mbar_arrive(smem_u32(&ctl->sweepbar));
            } else {
                if (lane == 0) ok = mbar_wait(smem_u32(&ctl->sweepbar), 0, abort_flag, a.status, 102);
                ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
            }
            base = (uint32_t)n;
            wbase = -1;
        }
        if (!is_v) {
            // K(0), K(1), then K(i + 2) after every V(i)
            if (nt > 0) put(base, 0);
            if (nt > 1) put(base + 1, 1);
            for (int i = 2; i < nt; ++i) put(base + 2 * i - 1, i);
        } else {
            // V(i) comes after the K tiles 0 .. min(i + 2, nt) - 1 and the V tiles before it
            for (int i = 0; i < nt; ++i) put(base + (uint32_t)(min(i + 2, nt) + i), i);
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------ MMAs: the warp runs uniformly, one elected lane issues
        constexpr uint32_t IDESC = umma_idesc_bf16(BM, 128, 0);        // S = Q K^T: A (Q) from tensor memory, B K-major
        constexpr uint32_t IDESC_PV = umma_idesc_bf16(BM, HD, 1);      // O += P V: A (P) from tensor memory, B MN-major
        // Shared-memory descriptors: everything but the start address is a constant of the layout, so the words are built
        // once and an MMA costs one add. K-major (K): LBO 16, SBO 1024; MN-major (V): LBO = one d half, SBO 1024.
        const uint64_t dk0 = umma_desc_sw128(0, 16, 1024), dv0 = umma_desc_sw128(0, HALF_BYTES, 1024);
        const uint32_t k_hi = (uint32_t)(dk0 >> 32), k_lo0 = (uint32_t)dk0;
        const uint32_t v_hi = (uint32_t)(dv0 >> 32), v_lo0 = (uint32_t)dv0;
        uint32_t cslot = 0, cpar = 0, nQK[2] = {0, 0}, wP[2] = {0, 0};
        const uint32_t full0 = smem_u32(&ctl->full[0]), empty0 = smem_u32(&ctl->empty[0]);
        const uint32_t sfull0 = smem_u32(&ctl->sfull[0]), pfull0 = smem_u32(&ctl->pfull[0]);
        bool ok = mbar_wait_warp(smem_u32(&ctl->qfull), 0, abort_flag, a.status, 201);     // Q is in tensor memory
        // next tile of the ring: returns its slot
        auto take = [&]() -> uint32_t {
            const uint32_t slot = cslot;
            ok = ok && mbar_wait_warp(full0 + 8 * slot, cpar, abort_flag, a.status, 202);
            if (++cslot == NSLOT) { cslot = 0; cpar ^= 1; }
            return slot;
        };
        // S[buf] <- Q K^T. The S columns also hold the previous P of that buffer: every earlier use must have been handed
        // back by the softmax warps (pfull) before they are overwritten; the PV that read it was issued before (in order).
        auto issue_qk = [&](int buf) {
            const uint32_t slot = take();
            while (ok && wP[buf] < nQK[buf]) {
                ok = mbar_wait_warp(pfull0 + 8 * buf, wP[buf] & 1, abort_flag, a.status, 203);
                ++wP[buf];
            }
            if (!ok) return;
            tc_fence_after();
            if (elect_one()) {
                const uint32_t d = tmem + (uint32_t)buf * 128;
                const uint32_t kb_lo = k_lo0 + ((sRing + slot * TILE_BYTES) >> 4);
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)
                    umma_ts_lohi(d, tmem + Q_COL + ks * 8, kb_lo + (uint32_t)(((ks >> 2) * HALF_BYTES + (ks & 3) * 32) >> 4),
                                 k_hi, IDESC, ks > 0);
                umma_commit(sfull0 + 8 * buf);
                umma_commit(empty0 + 8 * slot);
            }
            __syncwarp();
            ++nQK[buf];
        };
        if (FALLBACK) {
            for (int i = 0; i < n && ok; ++i) issue_qk(i & 1);
        }
        if (nt > 0) issue_qk(0);
        if (nt > 1) issue_qk(1);
        for (int i = 0; i < nt && ok; ++i) {
            const int buf = i & 1;
            const uint32_t slot = take();
            ok = ok && mbar_wait_warp(pfull0 + 8 * buf, wP[buf] & 1, abort_flag, a.status, 205);   // P(i) stored
            if (!ok) break;
            ++wP[buf];
            tc_fence_after();
            if (elect_one()) {
                const uint32_t p = tmem + (uint32_t)buf * 128;     // bf16 pairs: keys 0-63 in columns [0,32), 64-127 in [64,96)
                const uint32_t vb_lo = v_lo0 + ((sRing + slot * TILE_BYTES) >> 4);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    umma_ts_lohi(tmem + O_COL, p + (ks < 4 ? ks * 8 : 64 + (ks - 4) * 8),
                                 vb_lo + (uint32_t)((ks * 2048) >> 4), v_hi, IDESC_PV,
                                 (i > 0 || ks > 0) ? 1u : 0u);
                umma_commit(empty0 + 8 * slot);
                if (i + 1 == nt) umma_commit(smem_u32(&ctl->ofull));
            }
            __syncwarp();
            if (i + 2 < nt) issue_qk(buf);
        }
        // every MMA issued above has finished before tensor memory is freed
        if (elect_one()) umma_commit(smem_u32(&ctl->drain));
        __syncwarp();
        mbar_wait(smem_u32(&ctl->drain), 0, abort_flag, a.status, 206);
    } else if (warp == MASS_WARP) {
        // ------------------------------------------------------------ block masses: lane 0 / 1 = first / second block of a pair
        if (!FALLBACK && !COMPENSATE && a.mass != nullptr) {
            float* mrow = a.mass + ((size_t)h * a.nq + qb) * a.nb;
            bool ok = true;
            for (int e = 0; e < n && ok; ++e) {
                const int set = e % NMASS, c = lane & 1;
                const bool mine = lane < 2 && 2 * e + c < n64;
                const int blk = mine ? __ldg(list + 2 * e + c) : 0;           // fetched before the wait
                ok = mbar_wait_warp(smem_u32(&ctl->massbar[set]), (e / NMASS) & 1, abort_flag, a.status, 308);
                if (!ok) break;
                // rows lane, lane + 32, lane + 64, lane + 96 of both column halves, then the 32 lanes: always the same order
                const float* mp = mass_rows + set * 2 * BM;
                float m0 = (mp[lane] + mp[lane + 32]) + (mp[lane + 64] + mp[lane + 96]);
                float m1 = (mp[BM + lane] + mp[BM + lane + 32]) + (mp[BM + lane + 64] + mp[BM + lane + 96]);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    m0 += __shfl_xor_sync(0xffffffffu, m0, o);
                    m1 += __shfl_xor_sync(0xffffffffu, m1, o);
                }
                if (mine) mrow[blk] = c ? m1 : m0;
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctl->massfree[set]));
            }
        }
    } else {
        // ------------------------------------------------------------ softmax and epilogue
        const int rq = warp & 3, ch = warp >> 2;             // row quarter, column half
        const int trow = 32 * rq + lane, row = qb * BM + trow;
        const bool valid = row < a.L;
        const uint32_t lane_base = tmem + ((uint32_t)(32 * rq) << 16);
        uint32_t s[64];
        bool ok = true;

        // this thread's half of its Q row -> tensor memory (bf16 pairs, 32 columns), the A operand of every QK^T
        {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint4 w = q_early[i];
                s[4 * i] = w.x; s[4 * i + 1] = w.y; s[4 * i + 2] = w.z; s[4 * i + 3] = w.w;
            }
            tmem_st32(lane_base + Q_COL + 32 * ch, s);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(smem_u32(&ctl->qfull));
        }
        float m = a.offset[(size_t)row * a.H + h];
        uint32_t uS[2] = {0, 0};

        if (FALLBACK) {
            float mx = -INFINITY;
            for (int i = 0; i < n && ok; ++i) {
                const int buf = i & 1, e = 2 * i + ch;
                const bool has = e < n64;
                const int blk = list[has ? e : e - 1];
                ok = ok && mbar_wait_warp(smem_u32(&ctl->sfull[buf]), uS[buf] & 1, abort_flag, a.status, 301);
                if (!ok) break;
                ++uS[buf];
                tc_fence_after();
                tmem_ld32(lane_base + buf * 128 + 64 * ch, &s[0]);
                tmem_ld32(lane_base + buf * 128 + 64 * ch + 32, &s[32]);
                tmem_wait_ld();
                tc_fence_before();
                mbar_arrive(smem_u32(&ctl->pfull[buf]));
                int lim = (blk == a.nb - 1) ? a.tail_valid : BK;
                if (!has) lim = 0;
#pragma unroll
                for (int c = 0; c < 64; ++c)
                    if (c < lim) mx = fmaxf(mx, __uint_as_float(s[c]));
            }
            // the row maximum over both column halves
            ctl->m_part[ch][trow] = mx;
            mbar_arrive(smem_u32(&ctl->lbar));
            ok = mbar_wait_warp(smem_u32(&ctl->lbar), 0, abort_flag, a.status, 306) && ok;
            mx = fmaxf(ctl->m_part[0][trow], ctl->m_part[1][trow]);
            m = (mx == -INFINITY) ? 0.f : mx * a.scale_log2;
        }

        float2 lsum = make_float2(0.f, 0.f);
        const int* bits = a.skip_bits + ((size_t)h * a.nq + qb) * a.nw;
        const bool want_mass = !FALLBACK && !COMPENSATE && a.mass != nullptr;
        const float2 sc2 = make_float2(a.scale_log2, a.scale_log2);
        // kind, index and block id of an iteration are found one iteration ahead, so that the list entry (a global load)
        // has arrived long before it is needed
        SchedIter walk;
        int kind = 0, idx = 0, blk = 0;
        auto block_of = [&](int kd, int ix) -> int {
            if (kd != 0) return 0;
            const int e = 2 * ix + ch;
            return __ldg(list + (e < n64 ? e : e - 1));
        };
        if (nt > 0) {
            walk.get(sched, kind, idx);
            blk = block_of(kind, idx);
        }
        for (int i = 0; i < nt && ok; ++i) {
            const int buf = i & 1;
            const bool exact = kind == 0, pooled = kind == 1;
            const bool has = !exact || 2 * idx + ch < n64;
            const int cur_idx = idx, cur_blk = blk;
            int nkind = 0, nidx = 0, nblk = 0;
            walk.advance(sched);
            if (i + 1 < nt) {
                walk.get(sched, nkind, nidx);
                nblk = block_of(nkind, nidx);
            }
            // the skip words of a block-mean iteration are fetched before the wait, so that their latency is hidden by it
            uint32_t w0 = 0, w1 = 0;
            if (pooled && !COMPENSATE) {
                w0 = (uint32_t)__ldg(bits + 4 * cur_idx + 2 * ch);
                w1 = (uint32_t)__ldg(bits + 4 * cur_idx + 2 * ch + 1);
            }
            ok = ok && mbar_wait_warp(smem_u32(&ctl->sfull[buf]), uS[buf] & 1, abort_flag, a.status, 302);
            if (!ok) break;
            ++uS[buf];
            tc_fence_after();
            const uint32_t scol = lane_base + buf * 128 + 64 * ch;
            tmem_ld32(scol, &s[0]);
            tmem_ld32(scol + 32, &s[32]);
            tmem_wait_ld();
            float2 acc = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
            uint32_t pk[32];
            if (exact) {
                int lim = (cur_blk == a.nb - 1) ? a.tail_valid : BK;
                if (!has) lim = 0;
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
                // block-mean columns: column c of this half is block 128 cv + 64 ch + c; a set bit masks it
                const int cv = cur_idx;
                if (COMPENSATE) {
                    // every block that was not kept (refined ones included) is compensated: bits from the keep mask
                    const int b0 = 128 * cv + 64 * ch;
                    const uint8_t* kp = a.keep + ((size_t)h * a.nq + qb) * a.nb + b0;
                    w0 = 0; w1 = 0;
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        w0 |= (uint32_t)(b0 + c >= a.nb ? 1 : kp[c] != 0) << c;
                        w1 |= (uint32_t)(b0 + 32 + c >= a.nb ? 1 : kp[32 + c] != 0) << c;
                    }
                }
                const float2 off2 = make_float2(-m + 6.0f, -m + 6.0f);   // log2(64): a mean stands for its block's tokens
                const int last_c = (a.nb - 1) - (128 * cv + 64 * ch);    // column of the (maybe shorter) last block
                const float fix = a.tail_log2 - 6.0f;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    float2 xv = __ffma2_rn(make_float2(__uint_as_float(s[2 * j]), __uint_as_float(s[2 * j + 1])), sc2, off2);
                    if (2 * j == last_c) xv.x += fix;
                    if (2 * j + 1 == last_c) xv.y += fix;
                    if (COMPENSATE) { xv.x = fminf(xv.x, 100.0f); xv.y = fminf(xv.y, 100.0f); }   // triton_ops.py:275
                    float2 p = exp2_pair_mufu(xv);
                    const uint32_t w = j < 16 ? w0 : w1;
                    p.x = ((w >> ((2 * j) & 31)) & 1u) ? 0.f : p.x;
                    p.y = ((w >> ((2 * j + 1) & 31)) & 1u) ? 0.f : p.y;
                    acc = __fadd2_rn(acc, p);
                    pk[j] = pack_bf16x2(p.x, p.y);
                }
            } else {
                // representatives: column c of this half has the bias that the K load warp staged for this iteration
                const int cr = cur_idx;
                const float4* bb = reinterpret_cast<const float4*>(bias_ring + (cr % NBIAS) * 128 + 64 * ch);
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const float4 b4 = bb[e];
                    const int c = 4 * e;
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
            tmem_st32(scol, pk);                       // P over the first 32 of this thread's own 64 S columns
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(smem_u32(&ctl->pfull[buf]));
            acc = __fadd2_rn(acc, acc1);
            lsum = __fadd2_rn(lsum, acc);
            if (want_mass && exact) {
                // per-block mass: every row leaves its sum over the block's columns in shared memory; the mass warp adds
                // the 128 rows in a fixed order and stores the result (no atomics: the map is reproducible bit for bit). A
                // set of row sums is written again NMASS exact iterations later, once the mass warp has handed it back.
                const int set = cur_idx % NMASS, round = cur_idx / NMASS;
                if (round > 0) {
                    ok = mbar_wait_warp(smem_u32(&ctl->massfree[set]), (round - 1) & 1, abort_flag, a.status, 304);
                    if (!ok) break;
                }
                mass_rows[(set * 2 + ch) * BM + trow] = acc.x + acc.y;      // this row's sum over the block's 64 columns
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctl->massbar[set]));
            }
            kind = nkind; idx = nidx; blk = nblk;
        }

        // ---- epilogue: row sums of both column halves, then this thread's 64 columns of O
        ctl->l_part[ch][trow] = lsum.x + lsum.y;
        mbar_arrive(smem_u32(&ctl->lbar));
        ok = mbar_wait_warp(smem_u32(&ctl->lbar), FALLBACK ? 1 : 0, abort_flag, a.status, 307) && ok;
        const float l = ctl->l_part[0][trow] + ctl->l_part[1][trow];
        // compensation: out = (out + sum e v) / (1 + sum e), lse += log2(1 + sum e) (triton_ops.py:280-282)
        const float lg = COMPENSATE ? log2f(1.0f + l) : log2f(l);
        if (nt > 0) ok = mbar_wait_warp(smem_u32(&ctl->ofull), 0, abort_flag, a.status, 303) && ok;
        if (ok) {
            tc_fence_after();
            const float inv = COMPENSATE ? 1.0f / (1.0f + l) : 1.0f / l;
            __nv_bfloat16* orow = a.out + ((size_t)row * a.H + h) * HD + 64 * ch;
#pragma unroll
            for (int part = 0; part < 2; ++part) {
                uint32_t* o = &s[0];
                if (nt > 0) {
                    tmem_ld32(lane_base + O_COL + 64 * ch + 32 * part, o);
                    tmem_wait_ld();
                }
                if (valid) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint4 w;
                        if (COMPENSATE) {
                            const uint4 old = *reinterpret_cast<const uint4*>(orow + 32 * part + c);
                            const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                o[c + 2 * e] = __float_as_uint(__uint_as_float(o[c + 2 * e]) + __uint_as_float(ow[e] << 16));
                                o[c + 2 * e + 1] = __float_as_uint(__uint_as_float(o[c + 2 * e + 1]) + __uint_as_float(ow[e] & 0xFFFF0000u));
                            }
                        }
                        w.x = pack_bf16x2(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
                        w.y = pack_bf16x2(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
                        w.z = pack_bf16x2(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
                        w.w = pack_bf16x2(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
                        if (nt == 0) w = make_uint4(0, 0, 0, 0);
                        *reinterpret_cast<uint4*>(orow + 32 * part + c) = w;
                    }
                }
            }
            tc_fence_before();
            if (ch == 0) {
                // rows past L keep the "no offset" value, as echosparse/kernels/sm120.py:96
                a.lse[(size_t)row * a.H + h] = valid ? m + lg : 1e30f;
                if (!FALLBACK && !COMPENSATE) {
                    // a tile whose row sums leave 2^[-th, th] is flagged and recomputed with online softmax
                    const bool bad = valid && !(lg >= -a.th && lg <= a.th);
                    const unsigned ballot = __ballot_sync(0xffffffffu, bad);
                    if (lane == 0) {
                        ctl->flag_part[rq] = ballot != 0;
                        mbar_arrive(smem_u32(&ctl->flagbar));
                    }
                    if (tid == 0 && mbar_wait(smem_u32(&ctl->flagbar), 0, abort_flag, a.status, 305))
                        a.flags[th_idx] = ctl->flag_part[0] | ctl->flag_part[1] | ctl->flag_part[2] | ctl->flag_part[3];
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    __syncwarp();
    if ((warp == LOADK_WARP || warp == LOADV_WARP) && lane == 0 && *abort_flag) {
        // a wait gave up somewhere: give the loads this warp issued a moment (100 us in all) to land before the CTA's
        // shared memory goes away; a tile that was never issued cannot hold the CTA back
        const uint64_t t_end = global_timer_ns() + 100000ull;
        for (uint32_t back = 1; back <= 2 * NSLOT && back <= pseq; ++back) {
            const uint32_t sq = pseq - back;
            while (!mbar_try_wait(smem_u32(&ctl->full[sq % NSLOT]), (sq / NSLOT) & 1) && global_timer_ns() < t_end) {}
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

template <int MODE>
__global__ void __launch_bounds__(NTHREADS, 1)
attention_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                 const __grid_constant__ CUtensorMap tmKm, const __grid_constant__ CUtensorMap tmVm,
                 const __grid_constant__ CUtensorMap tmKr, const __grid_constant__ CUtensorMap tmVr, const AttnArgs a) {
    if (MODE == 0 || a.tile_list == nullptr) {
        attention_tile<MODE>(tmK, tmV, tmKm, tmVm, tmKr, tmVr, a, (int)blockIdx.x, false);
        return;
    }
    // fallback modes with a tile list: a grid of one CTA per SM walks the flagged tiles, instead of one CTA per tile of
    // which all but a fraction of a percent would find their flag clear and leave
    const int count = *a.tile_count;
    bool again = false;
    for (int e = blockIdx.x; e < count; e += gridDim.x) {
        attention_tile<MODE>(tmK, tmV, tmKm, tmVm, tmKr, tmVr, a, a.tile_list[e], again);
        again = true;
        __syncthreads();
    }
}

// Tiles whose flag is set, in ascending tile number (head * nq + tile): one CTA, ordered compaction by prefix sums. The
// flags are stored tile-major (nq, H); they are copied to shared memory with coalesced loads first (STAGED; 94 KB at 591
// tiles x 40 heads) and walked head-major from there.
template <bool STAGED>
__global__ void __launch_bounds__(1024)
flag_list_kernel(const int* __restrict__ flags, int nq, int H, int* __restrict__ list, int* __restrict__ count) {
    extern __shared__ int staged[];
    __shared__ int warp_sum[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = nq * H, per = (n + 1023) / 1024, b0 = tid * per;
    if (STAGED) {
        for (int i = tid; i < n; i += 1024) staged[i] = flags[i];
        __syncthreads();
    }
    const int* f = STAGED ? staged : flags;
    int mine = 0;
    for (int b = b0; b < min(b0 + per, n); ++b) mine += f[(b % nq) * H + b / nq] != 0;
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) warp_sum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = warp_sum[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += v;
        }
        warp_sum[lane] = w;
    }
    __syncthreads();
    int pos = incl - mine + (warp > 0 ? warp_sum[warp - 1] : 0);
    for (int b = b0; b < min(b0 + per, n); ++b)
        if (f[(b % nq) * H + b / nq] != 0) list[pos++] = b;
    if (tid == 1023) *count = pos;
}

// ---------------------------------------------------------------------------------------------- host side
// Representative tables (H, rows, 128) bf16 viewed as dims {128 d, rows, H}; a box is 64 d x 4 rows (one block's four rows).
static int make_rep_map(CUtensorMap* m, const void* ptr, int rows, int H) {
    cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)rows, (cuuint64_t)H};
    cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)rows * HD * 2};
    cuuint32_t box[3] = {64, 4, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return encode_tensor_map(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                             CU_TENSOR_MAP_SWIZZLE_128B);
}

static int make_map(CUtensorMap* m, const void* ptr, int rows, int H, int box_rows) {
    // (rows, H, 128) bf16 viewed as dims {128 d, rows, H}; a box is 64 d x box_rows rows, 128-byte swizzled
    cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)rows, (cuuint64_t)H};
    cuuint64_t strides[2] = {(cuuint64_t)H * HD * 2, (cuuint64_t)HD * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return encode_tensor_map(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                             CU_TENSOR_MAP_SWIZZLE_128B);
}

struct AttnCall {
    const void *q, *k, *v, *k_mean, *v_mean;
    AttnArgs a;
};

static int launch_attention(const AttnCall& c, int mode, cudaStream_t stream) {
    const AttnArgs& a = c.a;
    if (a.L <= 0 || a.H <= 0) return set_error(-1, "attention: L and H must be positive");
    if (a.status == nullptr) return set_error(-2, "attention: the device status word is not available on this device");
    if (((uintptr_t)c.q | (uintptr_t)c.k | (uintptr_t)c.v | (uintptr_t)a.out) & 15)
        return set_error(-1, "attention: q, k, v, out must be 16-byte aligned");
    CUtensorMap tk, tv, tkm, tvm, tkr, tvr;
    int rc;
    if ((rc = make_map(&tk, c.k, a.L, a.H, BK))) return rc;
    if ((rc = make_map(&tv, c.v, a.L, a.H, BK))) return rc;
    if (c.k_mean) {
        if ((rc = make_map(&tkm, c.k_mean, a.nb, a.H, BK))) return rc;
        if ((rc = make_map(&tvm, c.v_mean, a.nb, a.H, BK))) return rc;
    } else {
        tkm = tk; tvm = tv;
    }
    if (a.nref > 0) {
        if (((uintptr_t)a.k_rep | (uintptr_t)a.v_rep) & 15) return set_error(-1, "attention: k_rep, v_rep must be 16-byte aligned");
        if ((rc = make_rep_map(&tkr, a.k_rep, a.nb4, a.H))) return rc;
        if ((rc = make_rep_map(&tvr, a.v_rep, a.nb4, a.H))) return rc;
    } else {
        tkr = tk; tvr = tv;
    }
    auto kern = mode == 0 ? attention_kernel<0> : mode == 1 ? attention_kernel<1> : attention_kernel<2>;
    if ((rc = opt_in_shared_memory((const void*)kern, (int)SMEM_ALLOC))) return rc;
    int grid = a.nq * a.H;
    if (mode != 0 && a.tile_list != nullptr) {
        // the flagged tiles as a list, then one CTA per SM walking it
        const int flag_bytes = a.nq * a.H * (int)sizeof(int);
        if (flag_bytes <= 200 * 1024) {
            if ((rc = opt_in_shared_memory((const void*)flag_list_kernel<true>, flag_bytes))) return rc;
            flag_list_kernel<true><<<1, 1024, flag_bytes, stream>>>(a.flags, a.nq, a.H, const_cast<int*>(a.tile_list),
                                                                     const_cast<int*>(a.tile_count));
        } else {
            flag_list_kernel<false><<<1, 1024, 0, stream>>>(a.flags, a.nq, a.H, const_cast<int*>(a.tile_list),
                                                             const_cast<int*>(a.tile_count));
        }
        cudaError_t e0 = cudaGetLastError();
        if (e0 != cudaSuccess) return set_error(-2, cudaGetErrorString(e0));
        count_launch();
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return set_error(-2, "attention: cannot read the SM count");
        grid = sms < grid ? sms : grid;
    }
    kern<<<grid, NTHREADS, SMEM_ALLOC, stream>>>(tk, tv, tkm, tvm, tkr, tvr, a);
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
}

static void fill_q(AttnCall& c) { c.a.q = static_cast<const __nv_bfloat16*>(c.q); }

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
    fill_q(c);
    return launch_attention(c, 0, (cudaStream_t)stream);
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
    fill_q(c);
    return launch_attention(c, 0, (cudaStream_t)stream);
}

extern "C" int es_exact_fallback(const void* q, const void* k, const void* v, void* out, const int32_t* counts,
                                 const int32_t* blocks, int32_t nk, float* lse, const int32_t* flags, int32_t L,
                                 int32_t H, int32_t* tile_scratch, void* stream) {
    if (!q || !k || !v || !out || !counts || !blocks || !lse || !flags)
        return set_error(-1, "es_exact_fallback: null pointer");
    AttnCall c{};
    c.q = q; c.k = k; c.v = v; c.k_mean = nullptr; c.v_mean = nullptr;
    fill_common(c.a, L, H, 0.f);
    c.a.out = (__nv_bfloat16*)out; c.a.counts = counts; c.a.blocks = blocks; c.a.nk = nk;
    c.a.offset = lse; c.a.lse = lse; c.a.flags = const_cast<int32_t*>(flags); c.a.mass = nullptr;
    c.a.nvirt = 0; c.a.nref = 0;
    if (tile_scratch) { c.a.tile_count = tile_scratch; c.a.tile_list = tile_scratch + 1; }
    fill_q(c);
    return launch_attention(c, 1, (cudaStream_t)stream);
}

extern "C" int es_compensate_fallback(const void* q, const void* k_mean, const void* v_mean, const uint8_t* keep,
                                      float* lse, void* out, const int32_t* flags, int32_t L, int32_t H,
                                      int32_t* tile_scratch, void* stream) {
    if (!q || !k_mean || !v_mean || !keep || !lse || !out || !flags)
        return set_error(-1, "es_compensate_fallback: null pointer");
    AttnCall c{};
    // no exact blocks in this pass: the K / V maps are only placeholders and point at the mean tables
    c.q = q; c.k = k_mean; c.v = v_mean; c.k_mean = k_mean; c.v_mean = v_mean;
    fill_common(c.a, L, H, 0.f);
    c.a.out = (__nv_bfloat16*)out; c.a.counts = nullptr; c.a.blocks = nullptr; c.a.nk = 0;
    c.a.offset = lse; c.a.lse = lse; c.a.flags = const_cast<int32_t*>(flags); c.a.mass = nullptr;
    c.a.keep = keep;
    c.a.nvirt = (c.a.nb + 127) / 128; c.a.nref = 0;
    if (tile_scratch) { c.a.tile_count = tile_scratch; c.a.tile_list = tile_scratch + 1; }
    fill_q(c);
    return launch_attention(c, 2, (cudaStream_t)stream);
}
