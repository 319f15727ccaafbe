// Block selection and plan bit masks: integer / bit work, one CTA per (query tile, head).
//
// select_blocks follows echosparse/kernels/triton_ops.py:58-105: values = mass x scale, the K-th largest value is
// found exactly on the float bit patterns (the reference bisects; here a 4-pass 8-bit radix select over the same int32
// keys gives the same key), ties at the threshold are all kept, forced blocks are added, the refine list is the R
// largest raw masses among the blocks not kept (ties cut in ascending block order), lists come out ascending.
// pack_plan / rebuild_plan follow echosparse/kernels/sm120.py:259-296.
#include "es_api_internal.h"

#include <math.h>

namespace es {

constexpr int SEL_THREADS = 256;
constexpr int SEL_MAX_ITEMS = 16;           // blocks per thread: nb <= 4096 (kernels are instantiated for 1, 2, 4, 8, 16)

// K-th largest of the non-negative int32 keys held as key[i] = keys of element i * 256 + tid (negative keys never
// count). Returns 0 when fewer than K keys are non-negative, as the reference's bisection does.
template <int ITEMS>
__device__ int kth_largest_key(const int (&key)[ITEMS], int K, int* hist, int* bcast) {
    // hist: two histograms of 256 bins, bcast: two result triples; pass p uses copy p & 1 and clears the other one for pass
    // p + 1, so a pass needs two barriers (after the counting, after the digit is chosen). Both histograms are zero on
    // entry to a pass: the caller's copies start zeroed and every call leaves them zeroed.
    const int tid = threadIdx.x;
    if (K <= 0) return 0x7F800000;            // the bisection converges to its upper end: nothing but +inf passes
    int prefix = 0, need = K;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        int* hs = hist + 256 * (pass & 1);
        int* bc = bcast + 4 * (pass & 1);
        const int himask = pass == 0 ? 0 : (int)(0xFFFFFFFFu << (shift + 8));
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            const int k = key[i];
            if (k >= 0 && (k & himask) == prefix) atomicAdd(&hs[(k >> shift) & 255], 1);
        }
        __syncthreads();
        if (tid < 32) {
            // lane l owns digits 8l .. 8l+7; suffix sums from the top digit down
            int c[8], tot = 0;
            for (int j = 0; j < 8; ++j) { c[j] = hs[8 * tid + j]; hs[8 * tid + j] = 0; tot += c[j]; }
            int above = tot;                                   // inclusive suffix over lanes >= tid
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_down_sync(0xffffffffu, above, o);
                if (tid + o < 32) above += v;
            }
            above -= tot;                                      // keys in digits of higher lanes
            // the wanted digit is in this lane iff above < need <= above + tot
            if (above < need && need <= above + tot) {
                int acc = above, d = 7;
                for (; d >= 0; --d) {
                    if (acc + c[d] >= need) break;
                    acc += c[d];
                }
                bc[0] = 8 * tid + d;
                bc[1] = need - acc;
            }
            if (tid == 0) bc[2] = above + tot;                 // all matching keys
        }
        __syncthreads();
        if (bc[2] < need) return 0;                            // fewer than K non-negative keys (only at pass 0)
        prefix |= bc[0] << shift;
        need = bc[1];
    }
    return prefix;
}

// Ascending compaction of flagged elements in element order i * 256 + tid. Returns the total; `pos` gets each flagged
// element's rank. One barrier pair for all ITEMS rounds: every warp posts its ITEMS ballot counts, then each thread adds
// the counts of the rounds and warps before its own.
template <int ITEMS>
__device__ int compact_positions(const bool (&flag)[ITEMS], int (&pos)[ITEMS], int* warp_cnt) {
    constexpr int NW = SEL_THREADS / 32;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    unsigned b[ITEMS];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        b[i] = __ballot_sync(0xffffffffu, flag[i]);
        if (lane == 0) warp_cnt[i * NW + warp] = __popc(b[i]);
    }
    __syncthreads();
    int base = 0;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        int before = 0, total = 0;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const int c = warp_cnt[i * NW + w];
            if (w < warp) before += c;
            total += c;
        }
        pos[i] = base + before + __popc(b[i] & ((1u << lane) - 1u));
        base += total;
    }
    __syncthreads();
    return base;
}

template <int ITEMS>
__global__ void __launch_bounds__(SEL_THREADS)
select_kernel(const float* __restrict__ map, const uint8_t* __restrict__ keep_prev,
              const float* __restrict__ scale_exact, const float* __restrict__ scale_skip,
              uint8_t* __restrict__ keep_out, int* __restrict__ counts, int* __restrict__ blocks,
              const int* __restrict__ flags, int* __restrict__ bits, int nw, int* __restrict__ refine, int rw, int K,
              int R, int nb, int L, int sink, int H, int nq) {
    __shared__ int hist[512];
    __shared__ int bcast[8];
    __shared__ int warp_cnt[SEL_MAX_ITEMS * (SEL_THREADS / 32)];
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const size_t base = ((size_t)h * nq + t) * nb;
    hist[tid] = 0;
    hist[256 + tid] = 0;
    __syncthreads();
    // the blocks holding the tile's own tokens, one more on each side, and the sink are always computed
    const int lo = (t * 128) / 64 - 1;
    const int hi = (min((t + 1) * 128, L) - 1) / 64 + 1;
    const float se = scale_exact[h * nq + t], ss = scale_skip[h * nq + t];
    const bool fell_back = flags[t * H + h] != 0;

    float raw[ITEMS], val[ITEMS];
    int key[ITEMS];
    bool forced[ITEMS];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const int j = i * SEL_THREADS + tid;
        const bool valid = j < nb;
        raw[i] = valid ? map[base + j] : 0.f;
        const bool kept_before = valid && keep_prev[base + j] != 0;
        forced[i] = valid && ((j >= lo && j <= hi) || j >= sink);
        // a tile that fell back to online softmax has no valid masses: keep its previous blocks first
        float v = kept_before ? (fell_back ? INFINITY : raw[i] * se) : raw[i] * ss;
        v = (v == v) ? v : 0.f;
        v = (j >= sink) ? INFINITY : v;
        v = valid ? v : -1.f;
        val[i] = v;
        key[i] = __float_as_int(v);
    }
    const float thr = __int_as_float(kth_largest_key<ITEMS>(key, K, hist, bcast));
    bool keep[ITEMS];
    int rkey[ITEMS];
    float r2[ITEMS];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const int j = i * SEL_THREADS + tid;
        const bool valid = j < nb;
        keep[i] = valid && (val[i] >= thr || forced[i]);
        // refine candidates: the blocks not kept, by raw mass
        float r = (raw[i] == raw[i]) ? raw[i] : 0.f;
        r = (valid && !keep[i]) ? r : -1.f;
        r2[i] = r;
        rkey[i] = __float_as_int(r);
    }
    const int rthr = kth_largest_key<ITEMS>(rkey, R, hist, bcast);
    bool ref[ITEMS];
    int pos[ITEMS];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) ref[i] = rkey[i] >= rthr && r2[i] >= 0.f;
    compact_positions<ITEMS>(ref, pos, warp_cnt);
    bool ref2[ITEMS];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) ref2[i] = ref[i] && pos[i] < R;       // ties cut in ascending block order
    const int nref = compact_positions<ITEMS>(ref2, pos, warp_cnt);
    int* rlist = refine + ((size_t)t * H + h) * rw;
    for (int j = nref + tid; j < rw; j += SEL_THREADS) rlist[j] = nb;             // padding
#pragma unroll
    for (int i = 0; i < ITEMS; ++i)
        if (ref2[i] && pos[i] < rw) rlist[pos[i]] = i * SEL_THREADS + tid;

    const int nkeep = compact_positions<ITEMS>(keep, pos, warp_cnt);
    int* blist = blocks + ((size_t)t * H + h) * nb;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const int j = i * SEL_THREADS + tid;
        if (keep[i]) blist[pos[i]] = j;
        if (j < nb) keep_out[base + j] = keep[i] ? 1 : 0;
    }
    if (tid == 0) counts[t * H + h] = nkeep;
    // bit set = the block-mean compensation skips the block (exact, refined, or past nb)
    int* words = bits + ((size_t)h * nq + t) * nw;
    const int warp = tid >> 5, lane = tid & 31;
    for (int i = 0; i * (SEL_THREADS / 32) < nw; ++i) {
        const int j = i * SEL_THREADS + tid;
        bool s = true;
        if (i < ITEMS && j < nb) {
            // select the element's flags without dynamic indexing of the register arrays
            bool k = false, r = false;
#pragma unroll
            for (int u = 0; u < ITEMS; ++u)
                if (u == i) { k = keep[u]; r = ref2[u]; }
            s = k || r;
        }
        const unsigned b = __ballot_sync(0xffffffffu, s);
        const int w = i * (SEL_THREADS / 32) + warp;
        if (lane == 0 && w < nw) words[w] = (int)b;
    }
}

__global__ void __launch_bounds__(SEL_THREADS)
pack_kernel(const uint8_t* __restrict__ keep, int* __restrict__ exact_bits, int nw, int nb, int nq) {
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const size_t base = ((size_t)h * nq + t) * nb;
    int* words = exact_bits + ((size_t)h * nq + t) * nw;
    for (int i = 0; i * (SEL_THREADS / 32) < nw; ++i) {
        const int j = i * SEL_THREADS + tid;
        const bool bit = j >= nb || keep[base + j] != 0;
        const unsigned b = __ballot_sync(0xffffffffu, bit);
        const int w = i * (SEL_THREADS / 32) + warp;
        if (lane == 0 && w < nw) words[w] = (int)b;
    }
}

template <int ITEMS>
__global__ void __launch_bounds__(SEL_THREADS)
rebuild_kernel(const int* __restrict__ exact_bits, const int* __restrict__ skip_bits, int nw,
               uint8_t* __restrict__ keep, int* __restrict__ counts, int* __restrict__ blocks,
               int* __restrict__ refine, int rw, int* __restrict__ refine_counts, int* __restrict__ means,
               int* __restrict__ mean_counts, int nb, int nq, int H) {
    __shared__ int warp_cnt[SEL_MAX_ITEMS * (SEL_THREADS / 32)];
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int* ew = exact_bits + ((size_t)h * nq + t) * nw;
    const int* sw = skip_bits + ((size_t)h * nq + t) * nw;
    bool exact[ITEMS], refined[ITEMS], mean[ITEMS];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const int j = i * SEL_THREADS + tid;
        const bool valid = j < nb;
        const bool e = valid && ((ew[j >> 5 < nw ? j >> 5 : 0] >> (j & 31)) & 1);
        const bool s = valid && ((sw[j >> 5 < nw ? j >> 5 : 0] >> (j & 31)) & 1);
        exact[i] = e;
        refined[i] = valid && s && !e;
        mean[i] = valid && !s;
    }
    int pos[ITEMS];
    const size_t lbase = ((size_t)t * H + h) * nb;
    const int nmean = compact_positions<ITEMS>(mean, pos, warp_cnt);
#pragma unroll
    for (int i = 0; i < ITEMS; ++i)
        if (mean[i]) means[lbase + pos[i]] = i * SEL_THREADS + tid;
    const int nexact = compact_positions<ITEMS>(exact, pos, warp_cnt);
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const int j = i * SEL_THREADS + tid;
        if (exact[i]) blocks[lbase + pos[i]] = j;
        if (j < nb) keep[((size_t)h * nq + t) * nb + j] = exact[i] ? 1 : 0;
    }
    const int nref = compact_positions<ITEMS>(refined, pos, warp_cnt);
    int* rlist = refine + ((size_t)t * H + h) * rw;
    for (int j = nref + tid; j < rw; j += SEL_THREADS) rlist[j] = nb;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i)
        if (refined[i] && pos[i] < rw) rlist[pos[i]] = i * SEL_THREADS + tid;
    if (tid == 0) {
        mean_counts[t * H + h] = nmean;
        counts[t * H + h] = nexact;
        refine_counts[t * H + h] = min(nref, rw);
    }
}

// ---------------------------------------------------------------------------------------------- one warp per (tile, head)
// For up to 2048 kv blocks a whole (tile, head) fits the registers of one warp: lane l holds blocks 32 i + l. The K-th
// largest key is then found the way the reference finds it (31 halvings of [0, 0x7F800001) on the int32 bit patterns,
// triton_ops.py:43-54), each step one compare per held key and a warp sum: no shared memory, no atomics, no CTA barrier,
// and every warp of a CTA works on a tile of its own. Word i of a bit mask is simply the ballot of round i.
constexpr int SELW_WARPS = 8;

template <int IPL>
__device__ __forceinline__ int kth_largest_key_warp(const int (&key)[IPL], int K) {
    int lo = 0, hi = 0x7F800001;
#pragma unroll 1
    for (int step = 0; step < 31; ++step) {
        const int mid = lo + (hi - lo) / 2;
        int c = 0;
#pragma unroll
        for (int i = 0; i < IPL; ++i) c += key[i] >= mid;
        c = __reduce_add_sync(0xffffffffu, c);
        if (c >= K) lo = mid; else hi = mid;
    }
    return lo;
}

template <int IPL>
__global__ void __launch_bounds__(SELW_WARPS * 32, IPL <= 40 ? 2 : 1)
select_warp_kernel(const float* __restrict__ map, const uint8_t* __restrict__ keep_prev,
                   const float* __restrict__ scale_exact, const float* __restrict__ scale_skip,
                   uint8_t* __restrict__ keep_out, int* __restrict__ counts, int* __restrict__ blocks,
                   const int* __restrict__ flags, int* __restrict__ bits, int nw, int* __restrict__ refine, int rw, int K,
                   int R, int nb, int L, int sink, int H, int nq) {
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * SELW_WARPS + (threadIdx.x >> 5);       // (head, tile) pairs in the map's order
    if (unit >= nq * H) return;
    const int h = unit / nq, t = unit - h * nq;
    const size_t base = ((size_t)h * nq + t) * nb;
    const int lo = (t * 128) / 64 - 1;
    const int hi = (min((t + 1) * 128, L) - 1) / 64 + 1;
    const float se = scale_exact[h * nq + t], ss = scale_skip[h * nq + t];
    const bool fell_back = flags[t * H + h] != 0;
    const unsigned below = (1u << lane) - 1u;

    float raw[IPL];
    int key[IPL];
#pragma unroll
    for (int i = 0; i < IPL; ++i) {
        const int j = 32 * i + lane;
        const bool valid = j < nb;
        raw[i] = valid ? map[base + j] : 0.f;
        const bool kept_before = valid && keep_prev[base + j] != 0;
        // a tile that fell back to online softmax has no valid masses: keep its previous blocks first
        float v = kept_before ? (fell_back ? INFINITY : raw[i] * se) : raw[i] * ss;
        v = (v == v) ? v : 0.f;
        v = (j >= sink) ? INFINITY : v;
        key[i] = __float_as_int(valid ? v : -1.f);
    }
    const int thr = kth_largest_key_warp<IPL>(key, K);
    // keep = value at or above the K-th largest (ties all kept), or forced: the tile's own blocks, one more on each side,
    // and the sink. From here on key[] holds the refine candidates' keys: raw mass of the blocks not kept, -1 otherwise.
    unsigned mine[(IPL + 31) / 32];          // this lane's keep bits, one per round
#pragma unroll
    for (int w = 0; w < (IPL + 31) / 32; ++w) mine[w] = 0;
    int nkeep = 0;
    int* blist = blocks + ((size_t)t * H + h) * nb;
#pragma unroll
    for (int i = 0; i < IPL; ++i) {
        const int j = 32 * i + lane;
        const bool valid = j < nb;
        // float comparison, as the reference compares values with the threshold value (negative keys are the invalid slots)
        const bool keep = valid && (__int_as_float(key[i]) >= __int_as_float(thr) || (j >= lo && j <= hi) || j >= sink);
        const unsigned b = __ballot_sync(0xffffffffu, keep);
        mine[i >> 5] |= (keep ? 1u : 0u) << (i & 31);
        if (keep) blist[nkeep + __popc(b & below)] = j;
        nkeep += __popc(b);
        if (valid) keep_out[base + j] = keep ? 1 : 0;
        float r = (raw[i] == raw[i]) ? raw[i] : 0.f;
        key[i] = __float_as_int((valid && !keep) ? r : -1.f);
    }
    if (lane == 0) counts[t * H + h] = nkeep;
    const int rthr = kth_largest_key_warp<IPL>(key, R);
    // refine list: candidates at or above the R-th largest raw mass, ties cut in ascending block order
    int* rlist = refine + ((size_t)t * H + h) * rw;
    int* words = bits + ((size_t)h * nq + t) * nw;
    int nref = 0;
#pragma unroll
    for (int i = 0; i < IPL; ++i) {
        const int j = 32 * i + lane;
        const bool cand = key[i] >= rthr && key[i] >= 0;
        const unsigned c = __ballot_sync(0xffffffffu, cand);
        const int pos = nref + __popc(c & below);
        const bool ref = cand && pos < R;
        const unsigned rb = __ballot_sync(0xffffffffu, ref);
        if (ref && pos < rw) rlist[pos] = j;
        nref += __popc(rb);
        // bit set = the block-mean compensation skips the block: exact, refined, or past nb
        const unsigned past = (32 * i + 31 < nb) ? 0u : (32 * i >= nb ? 0xffffffffu : ~((1u << (nb - 32 * i)) - 1u));
        const unsigned kb = __ballot_sync(0xffffffffu, (mine[i >> 5] >> (i & 31)) & 1u);
        if (lane == 0 && i < nw) words[i] = (int)(kb | rb | past);
    }
    for (int j = nref + lane; j < rw; j += 32) rlist[j] = nb;                    // padding
    for (int w = IPL + lane; w < nw; w += 32) words[w] = -1;                      // words past the last block
}

// (exact bits, skip bits) -> keep mask, ascending block list, refine list; lane l expands round i's bit l. `means` may
// be null (the kernels of this library take the block-mean columns from the skip bits, not from a list).
template <int IPL>
__global__ void __launch_bounds__(SELW_WARPS * 32)
rebuild_warp_kernel(const int* __restrict__ exact_bits, const int* __restrict__ skip_bits, int nw,
                    uint8_t* __restrict__ keep, int* __restrict__ counts, int* __restrict__ blocks,
                    int* __restrict__ refine, int rw, int* __restrict__ refine_counts, int* __restrict__ means,
                    int* __restrict__ mean_counts, int nb, int nq, int H) {
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * SELW_WARPS + (threadIdx.x >> 5);
    if (unit >= nq * H) return;
    const int h = unit / nq, t = unit - h * nq;
    const int* ew = exact_bits + ((size_t)h * nq + t) * nw;
    const int* sw = skip_bits + ((size_t)h * nq + t) * nw;
    const size_t lbase = ((size_t)t * H + h) * nb, kbase = ((size_t)h * nq + t) * nb;
    int* rlist = refine + ((size_t)t * H + h) * rw;
    const unsigned below = (1u << lane) - 1u;
    int nexact = 0, nref = 0, nmean = 0;
#pragma unroll
    for (int i = 0; i < IPL; ++i) {
        if (32 * i >= nb) break;
        const int j = 32 * i + lane;
        const unsigned live = (32 * i + 31 < nb) ? 0xffffffffu : ((1u << (nb - 32 * i)) - 1u);
        const unsigned e = (unsigned)ew[i] & live, sk = (unsigned)sw[i] & live;
        const unsigned rf = sk & ~e, mn = ~sk & live;
        if ((e >> lane) & 1u) blocks[lbase + nexact + __popc(e & below)] = j;
        if ((rf >> lane) & 1u) { const int pos = nref + __popc(rf & below); if (pos < rw) rlist[pos] = j; }
        if (means != nullptr && ((mn >> lane) & 1u)) means[lbase + nmean + __popc(mn & below)] = j;
        if ((live >> lane) & 1u) keep[kbase + j] = (e >> lane) & 1u;
        nexact += __popc(e); nref += __popc(rf); nmean += __popc(mn);
    }
    for (int j = min(nref, rw) + lane; j < rw; j += 32) rlist[j] = nb;
    if (lane == 0) {
        counts[t * H + h] = nexact;
        refine_counts[t * H + h] = min(nref, rw);
        if (mean_counts != nullptr) mean_counts[t * H + h] = nmean;
    }
}

}  // namespace es

using namespace es;

extern "C" int es_select_blocks(const float* mass, const uint8_t* keep_prev, const float* scale_exact,
                                const float* scale_skip, uint8_t* keep, int32_t* counts, int32_t* blocks,
                                const int32_t* flags, int32_t* skip_bits, int32_t nw, int32_t* refine, int32_t rw,
                                int32_t k, int32_t r, int32_t L, int32_t H, int32_t sink, void* stream) {
    if (!mass || !keep_prev || !scale_exact || !scale_skip || !keep || !counts || !blocks || !flags || !skip_bits)
        return set_error(-1, "es_select_blocks: null pointer");
    if (L <= 0 || H <= 0) return set_error(-1, "es_select_blocks: L and H must be positive");
    const int nq = (L + 127) / 128, nb = (L + 63) / 64;
    if (nb > SEL_THREADS * SEL_MAX_ITEMS) return set_error(-1, "es_select_blocks: more than 4096 kv blocks");
    if (rw < r) return set_error(-1, "es_select_blocks: refine width smaller than r");
    if (rw > 0 && !refine) return set_error(-1, "es_select_blocks: null refine list");
    if (nw * 32 < nb) return set_error(-1, "es_select_blocks: skip_bits has fewer than nb bits per tile");
    if (nb <= 2048) {
        // one warp per (tile, head), blocks held 32 per round in registers
        const int ipl = (nb + 31) / 32, units = nq * H;
        const dim3 grid((units + SELW_WARPS - 1) / SELW_WARPS);
#define ES_SELECTW_LAUNCH(N)                                                                                          \
    select_warp_kernel<N><<<grid, SELW_WARPS * 32, 0, (cudaStream_t)stream>>>(mass, keep_prev, scale_exact, scale_skip, \
                                                                               keep, counts, blocks, flags, skip_bits,  \
                                                                               nw, refine, rw, k, r, nb, L, sink, H, nq)
        if (ipl <= 8) ES_SELECTW_LAUNCH(8);
        else if (ipl <= 16) ES_SELECTW_LAUNCH(16);
        else if (ipl <= 24) ES_SELECTW_LAUNCH(24);
        else if (ipl <= 32) ES_SELECTW_LAUNCH(32);
        else if (ipl <= 40) ES_SELECTW_LAUNCH(40);
        else if (ipl <= 48) ES_SELECTW_LAUNCH(48);
        else ES_SELECTW_LAUNCH(64);
#undef ES_SELECTW_LAUNCH
        ES_CHECK_LAUNCH("select_blocks");
        return 0;
    }
    const int items = (nb + SEL_THREADS - 1) / SEL_THREADS;
#define ES_SELECT_LAUNCH(N)                                                                                         \
    select_kernel<N><<<dim3(nq, H), SEL_THREADS, 0, (cudaStream_t)stream>>>(mass, keep_prev, scale_exact, scale_skip, \
                                                                             keep, counts, blocks, flags, skip_bits, \
                                                                             nw, refine, rw, k, r, nb, L, sink, H, nq)
    if (items <= 1) ES_SELECT_LAUNCH(1);
    else if (items <= 2) ES_SELECT_LAUNCH(2);
    else if (items <= 4) ES_SELECT_LAUNCH(4);
    else if (items <= 8) ES_SELECT_LAUNCH(8);
    else ES_SELECT_LAUNCH(16);
#undef ES_SELECT_LAUNCH
    ES_CHECK_LAUNCH("select_blocks");
    return 0;
}

extern "C" int es_pack_plan(const uint8_t* keep, int32_t* exact_bits, int32_t nw, int32_t H, int32_t nq, int32_t nb,
                            void* stream) {
    if (!keep || !exact_bits) return set_error(-1, "es_pack_plan: null pointer");
    if (nw * 32 < nb) return set_error(-1, "es_pack_plan: fewer than nb bits per tile");
    pack_kernel<<<dim3(nq, H), SEL_THREADS, 0, (cudaStream_t)stream>>>(keep, exact_bits, nw, nb, nq);
    ES_CHECK_LAUNCH("pack_plan");
    return 0;
}

extern "C" int es_rebuild_plan(const int32_t* exact_bits, const int32_t* skip_bits, int32_t nw, uint8_t* keep,
                               int32_t* counts, int32_t* blocks, int32_t* refine, int32_t rw, int32_t* refine_counts,
                               int32_t* means, int32_t* mean_counts, int32_t H, int32_t nq, int32_t nb, void* stream) {
    if (!exact_bits || !skip_bits || !keep || !counts || !blocks || !refine_counts)
        return set_error(-1, "es_rebuild_plan: null pointer");
    if ((means == nullptr) != (mean_counts == nullptr))
        return set_error(-1, "es_rebuild_plan: give both the mean list and its counts, or neither");
    if (rw > 0 && !refine) return set_error(-1, "es_rebuild_plan: null refine list");
    if (nb > SEL_THREADS * SEL_MAX_ITEMS) return set_error(-1, "es_rebuild_plan: more than 4096 kv blocks");
    if (nw * 32 < nb) return set_error(-1, "es_rebuild_plan: fewer than nb bits per tile");
    if (nb <= 4096) {
        const int ipl = (nb + 31) / 32, units = nq * H;
        const dim3 grid((units + SELW_WARPS - 1) / SELW_WARPS);
#define ES_REBUILDW_LAUNCH(N)                                                                                           \
    rebuild_warp_kernel<N><<<grid, SELW_WARPS * 32, 0, (cudaStream_t)stream>>>(exact_bits, skip_bits, nw, keep, counts,  \
                                                                                blocks, refine, rw, refine_counts,      \
                                                                                means, mean_counts, nb, nq, H)
        if (ipl <= 16) ES_REBUILDW_LAUNCH(16);
        else if (ipl <= 64) ES_REBUILDW_LAUNCH(64);
        else ES_REBUILDW_LAUNCH(128);
#undef ES_REBUILDW_LAUNCH
        ES_CHECK_LAUNCH("rebuild_plan");
        return 0;
    }
    const int items = (nb + SEL_THREADS - 1) / SEL_THREADS;
#define ES_REBUILD_LAUNCH(N)                                                                                          \
    rebuild_kernel<N><<<dim3(nq, H), SEL_THREADS, 0, (cudaStream_t)stream>>>(exact_bits, skip_bits, nw, keep, counts,  \
                                                                              blocks, refine, rw, refine_counts, means, \
                                                                              mean_counts, nb, nq, H)
    if (items <= 1) ES_REBUILD_LAUNCH(1);
    else if (items <= 2) ES_REBUILD_LAUNCH(2);
    else if (items <= 4) ES_REBUILD_LAUNCH(4);
    else if (items <= 8) ES_REBUILD_LAUNCH(8);
    else ES_REBUILD_LAUNCH(16);
#undef ES_REBUILD_LAUNCH
    ES_CHECK_LAUNCH("rebuild_plan");
    return 0;
}
