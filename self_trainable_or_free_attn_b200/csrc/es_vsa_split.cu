// VSA2 split-KV scheduling: the task plan over a CSR list and the merges of the split rows.
//
// Contract (reference: csrc/vsa/split.cu:1-22 and the SplitPlanParams comment of csrc/vsa/vsa2_kernels.h:48-83 of
// shaoshitong/self_trainable_or_free_attn), for the NR = BH * NB rows of a q -> kv list (forward, dQ pass) or a kv -> q
// list (dK / dV pass):
//   a row of n blocks is eligible when n >= thr_h = max(min_len, ceil(tail_frac * W / resident),
//   ceil(rel_mean * nnz_h / NB)), W = all edges of the list, nnz_h = the edges of the row's (b, h); an eligible row has
//   ceil(n / chunk) chunks; with E = the number of eligible rows, row r is split when E <= budget and the running
//   (inclusive) chunk count of the eligible rows up to r stays <= max_slots. Split chunk j of a row covers the edges
//   [beg + j n / c, beg + (j + 1) n / c) and owns slot = its task index; the split chunks come first in the task list (in
//   row order), then one direct task {row, beg, end, -1} per remaining row. merges[m] = {row, first slot, chunks, 0} for the
//   m-th split row. info[8] = tasks, split rows, split slots, NR, E, E <= budget, thr without the per-head term, W.
// Everything stays on the device: one CTA computes the three prefix sums and writes the lists.
//
// Merges, one CTA per split row, chunks combined in their order (reproducible):
//   forward : o = sum_i 2^(lse_i - M) o_i / sum_i 2^(lse_i - M), lse = (M + log2 sum) ln 2; padded rows 0 and -inf
//   backward: out = valid ? sum_i part_i + add[block] / count : 0
#include <string>

#include "es_api_internal.h"
#include "es_vsa_mma.cuh"

namespace es {
namespace vsa {

struct PlanArgs {
    const int* ptr;
    int BH, NB, chunk, max_slots, min_len, resident, budget;
    double rel_mean, tail_frac;
    int *tasks, *merges, *info;
    int* work;            // [3 * NR] chunk counts, their inclusive sums over the eligible rows, split flags
};

__global__ void __launch_bounds__(1024) split_plan_kernel(const PlanArgs a) {
    __shared__ int part[1024];
    __shared__ int s_total;
    const int tid = threadIdx.x, NR = a.BH * a.NB;
    const int per = (NR + 1023) / 1024, lo = min(tid * per, NR), hi = min(lo + per, NR);
    int* cnt = a.work;
    int* incl = a.work + NR;
    int* flag = a.work + 2 * NR;
    auto scan = [&](int v) -> int {          // exclusive prefix over the threads; the total lands in s_total
        part[tid] = v;
        __syncthreads();
        for (int o = 1; o < 1024; o <<= 1) {
            const int x = tid >= o ? part[tid - o] : 0;
            __syncthreads();
            part[tid] += x;
            __syncthreads();
        }
        if (tid == 1023) s_total = part[1023];
        const int r = part[tid] - v;
        __syncthreads();
        return r;
    };
    const long long W = (long long)a.ptr[(size_t)a.BH * (a.NB + 1) - 1] - a.ptr[0];
    int gthr = a.min_len;
    if (a.tail_frac > 0.0) gthr = max(gthr, (int)ceil(a.tail_frac * (double)W / (double)a.resident));
    // chunks of the eligible rows, and how many rows are eligible
    int my_c = 0, my_e = 0;
    for (int r = lo; r < hi; ++r) {
        const int bh = r / a.NB, i = r - bh * a.NB;
        const int* hp = a.ptr + (size_t)bh * (a.NB + 1);
        const int n = hp[i + 1] - hp[i];
        int thr = gthr;
        if (a.rel_mean > 0.0) thr = max(thr, (int)ceil(a.rel_mean * (double)(hp[a.NB] - hp[0]) / (double)a.NB));
        const int c = n >= thr ? (n + a.chunk - 1) / a.chunk : 0;
        cnt[r] = c;
        my_c += c; my_e += n >= thr;
    }
    int run = scan(my_c);
    scan(my_e);
    const int E = s_total;
    const bool within = E <= a.budget;
    // split flags; slots of the split rows; number of direct rows before each row
    int my_slots = 0, my_split = 0, my_direct = 0;
    for (int r = lo; r < hi; ++r) {
        run += cnt[r];
        incl[r] = run;
        const bool split = within && cnt[r] > 0 && run <= a.max_slots;
        flag[r] = split;
        my_slots += split ? cnt[r] : 0; my_split += split; my_direct += !split;
    }
    int slot = scan(my_slots);
    const int t_split = s_total;
    int mrow = scan(my_split);
    const int n_split = s_total;
    int drow = scan(my_direct);
    const int n_direct = s_total;
    int4* tasks = reinterpret_cast<int4*>(a.tasks);
    int4* merges = reinterpret_cast<int4*>(a.merges);
    for (int r = lo; r < hi; ++r) {
        const int bh = r / a.NB, i = r - bh * a.NB;
        const int* rp = a.ptr + (size_t)bh * (a.NB + 1) + i;
        const int beg = rp[0], n = rp[1] - beg;
        if (flag[r]) {
            const int c = cnt[r];
            for (int j = 0; j < c; ++j)
                tasks[slot + j] = make_int4(r, beg + (int)((long long)j * n / c), beg + (int)((long long)(j + 1) * n / c), slot + j);
            merges[mrow++] = make_int4(r, slot, c, 0);
            slot += c;
        } else {
            tasks[t_split + drow++] = make_int4(r, beg, beg + n, -1);
        }
    }
    if (tid == 0) {
        a.info[0] = t_split + n_direct; a.info[1] = n_split; a.info[2] = t_split; a.info[3] = NR;
        a.info[4] = E; a.info[5] = within ? 1 : 0; a.info[6] = gthr; a.info[7] = (int)W;
    }
}

struct MergeArgs {
    const int *merges, *info, *blk_cnt;
    const float *part, *part_lse, *add;
    void* out;
    float *out_f32, *lse;
    int L, NB, add_nb, mask_rows;
};

// FWD: weighted merge of normalised partials; otherwise the plain sum plus the per-block add.
template <typename T, int D, bool FWD>
__global__ void __launch_bounds__(128) split_merge_kernel(const MergeArgs a) {
    if ((int)blockIdx.x >= a.info[1]) return;
    const int4 mg = reinterpret_cast<const int4*>(a.merges)[blockIdx.x];
    const int bh = mg.x / a.NB, blk = mg.x - bh * a.NB, slot0 = mg.y, c = mg.z;
    const int cnt = a.blk_cnt[blk];
    constexpr int CH = D / 4;                       // float4 chunks per row
    for (int e = threadIdx.x; e < TB * CH; e += 128) {
        const int row = e / CH, ch = e % CH;
        const size_t tok = (size_t)bh * a.L + (size_t)blk * TB + row;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float lse = -INFINITY;
        if (FWD) {
            if (row < cnt || !a.mask_rows) {
                float mx = -INFINITY;
                for (int j = 0; j < c; ++j) mx = fmaxf(mx, a.part_lse[(size_t)(slot0 + j) * TB + row]);
                if (mx != -INFINITY) {
                    float sum = 0.f;
                    for (int j = 0; j < c; ++j) {
                        const float w = exp2f(a.part_lse[(size_t)(slot0 + j) * TB + row] - mx);
                        const float4 x = *reinterpret_cast<const float4*>(a.part + ((size_t)(slot0 + j) * TB + row) * D + ch * 4);
                        sum += w;
                        acc.x += w * x.x; acc.y += w * x.y; acc.z += w * x.z; acc.w += w * x.w;
                    }
                    const float inv = 1.f / sum;
                    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
                    lse = (mx + log2f(sum)) * LN2;
                }
            }
            if (ch == 0) a.lse[tok] = lse;
        } else if (row < cnt) {
            for (int j = 0; j < c; ++j) {
                const float4 x = *reinterpret_cast<const float4*>(a.part + ((size_t)(slot0 + j) * TB + row) * D + ch * 4);
                acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
            }
            if (a.add) {
                const float4 ad = *reinterpret_cast<const float4*>(a.add + ((size_t)bh * a.add_nb + blk) * D + ch * 4);
                const float inv = 1.f / (float)cnt;
                acc.x += ad.x * inv; acc.y += ad.y * inv; acc.z += ad.z * inv; acc.w += ad.w * inv;
            }
        }
        if (!FWD && a.out_f32) {
            *reinterpret_cast<float4*>(a.out_f32 + tok * D + ch * 4) = acc;
        } else {
            uint2 w;
            w.x = Elt<T>::pack(acc.x, acc.y);
            w.y = Elt<T>::pack(acc.z, acc.w);
            *reinterpret_cast<uint2*>(static_cast<T*>(a.out) + tok * D + ch * 4) = w;
        }
    }
}

template <bool FWD>
static int launch_merge(const MergeArgs& a, int n_merge_cap, int D, int dtype, cudaStream_t st) {
    if (dtype == 0 && D == 128) split_merge_kernel<__nv_bfloat16, 128, FWD><<<n_merge_cap, 128, 0, st>>>(a);
    else if (dtype == 0) split_merge_kernel<__nv_bfloat16, 64, FWD><<<n_merge_cap, 128, 0, st>>>(a);
    else if (D == 128) split_merge_kernel<__half, 128, FWD><<<n_merge_cap, 128, 0, st>>>(a);
    else split_merge_kernel<__half, 64, FWD><<<n_merge_cap, 128, 0, st>>>(a);
    ES_CHECK_LAUNCH("split_merge_kernel");
    return 0;
}

}  // namespace vsa
}  // namespace es

using namespace es;
using namespace es::vsa;

extern "C" long long es_vsa_split_plan_workspace_bytes(int32_t BH, int32_t NB) {
    return BH > 0 && NB > 0 ? 3LL * BH * NB * 4 : 0;
}

extern "C" int es_vsa_split_plan(const int32_t* ptr, int32_t BH, int32_t NB, int32_t chunk, int32_t max_slots,
                                 int32_t min_len, double rel_mean, double tail_frac, int32_t resident, int32_t budget,
                                 int32_t* tasks, int32_t* merges, int32_t* info, void* workspace, void* stream) {
    if (!ptr || !tasks || !merges || !info || !workspace) return set_error(-1, "es_vsa_split_plan: null pointer");
    if (BH <= 0 || NB <= 0) return set_error(-1, "es_vsa_split_plan: BH and NB must be positive");
    if (chunk < 1 || max_slots < 0) return set_error(-1, "es_vsa_split_plan: chunk >= 1 and max_slots >= 0");
    if (min_len < chunk + 1) return set_error(-1, "es_vsa_split_plan: min_len must be at least chunk + 1");
    if (resident < 1 || budget < 0 || rel_mean < 0.0 || tail_frac < 0.0)
        return set_error(-1, "es_vsa_split_plan: resident >= 1, budget >= 0, rel_mean >= 0, tail_frac >= 0");
    if (((uintptr_t)tasks | (uintptr_t)merges) & 15) return set_error(-1, "es_vsa_split_plan: tasks and merges must be 16-byte aligned");
    PlanArgs a{ptr, BH, NB, chunk, max_slots, min_len, resident, budget, rel_mean, tail_frac, tasks, merges, info,
               static_cast<int*>(workspace)};
    split_plan_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(a);
    ES_CHECK_LAUNCH("split_plan_kernel");
    return 0;
}

extern "C" int es_vsa_split_merge_fwd(const float* part_o, const float* part_lse, const int32_t* merges,
                                      const int32_t* info, int32_t n_merge_cap, const int32_t* blk_cnt, void* o, float* lse,
                                      int32_t L, int32_t D, int32_t mask_rows, int32_t dtype, void* stream) {
    if (!merges || !info || !blk_cnt || !o || !lse) return set_error(-1, "es_vsa_split_merge_fwd: null pointer");
    if (n_merge_cap <= 0) return 0;
    if (!part_o || !part_lse) return set_error(-1, "es_vsa_split_merge_fwd: null partials");
    if (L <= 0 || L % TB != 0 || (D != 64 && D != 128) || (dtype != 0 && dtype != 1))
        return set_error(-1, "es_vsa_split_merge_fwd: bad L, D or dtype");
    MergeArgs a{};
    a.merges = merges; a.info = info; a.blk_cnt = blk_cnt; a.part = part_o; a.part_lse = part_lse; a.out = o; a.lse = lse;
    a.L = L; a.NB = L / TB; a.mask_rows = mask_rows;
    return launch_merge<true>(a, n_merge_cap, D, dtype, (cudaStream_t)stream);
}

extern "C" int es_vsa_split_merge_sum(const float* part, const int32_t* merges, const int32_t* info, int32_t n_merge_cap,
                                      const float* add, int32_t add_nb, const int32_t* blk_cnt, void* out, float* out_f32,
                                      int32_t L, int32_t D, int32_t dtype, void* stream) {
    if (!merges || !info || !blk_cnt || (!out && !out_f32)) return set_error(-1, "es_vsa_split_merge_sum: null pointer");
    if (n_merge_cap <= 0) return 0;
    if (!part) return set_error(-1, "es_vsa_split_merge_sum: null partials");
    if (L <= 0 || L % TB != 0 || (D != 64 && D != 128) || (dtype != 0 && dtype != 1))
        return set_error(-1, "es_vsa_split_merge_sum: bad L, D or dtype");
    if (add && add_nb < L / TB) return set_error(-1, "es_vsa_split_merge_sum: add_nb smaller than the block count");
    MergeArgs a{};
    a.merges = merges; a.info = info; a.blk_cnt = blk_cnt; a.part = part; a.add = add; a.add_nb = add_nb; a.out = out;
    a.out_f32 = out_f32; a.L = L; a.NB = L / TB;
    return launch_merge<false>(a, n_merge_cap, D, dtype, (cudaStream_t)stream);
}
