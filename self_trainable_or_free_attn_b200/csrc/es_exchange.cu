// Sequence <-> head exchange of a sequence-sharded caller as ONE kernel per rank: the layout change and the transfer are
// the same pass. Rank r holds a [rows_total, row_bytes_total] matrix; the slab that peer p needs (a block of columns on
// the way to heads, a block of rows on the way back) is read once from this GPU's memory and stored straight into its final
// place in peer p's receive buffer through a peer mapping (plain 16-byte stores over NVLink / NVSwitch; the local slab is an
// ordinary copy). Nothing waits on another GPU inside the kernel: the caller orders the exchange against the peers' use of
// the buffers with a collective on the same stream (see ulysses.py).
//
// The reference runs this exchange as torch.distributed.all_to_all_single around its attention processor (multi-GPU recipe
// of its README for HunyuanVideo); with NCCL the two layout copies around the all-to-all cost as much HBM time as the
// transfer costs link time.
#include "es_api_internal.h"

namespace es {

constexpr int MAX_PEERS = 16;

struct ExchangeArgs {
    const uint8_t* src;
    uint8_t* dst[MAX_PEERS];          // receive buffer of every rank (this rank's own included), as mapped on this GPU
    long long src_slab_stride;        // bytes between the slabs of consecutive peers in src
    long long src_row_stride;         // bytes between rows of a slab in src
    long long dst_offset;             // where this rank's slab starts in every receive buffer
    long long dst_row_stride;         // bytes between rows in a receive buffer
    long long rows;                   // rows per slab
    int units_per_row;                // 16-byte units per row of a slab
    int peers;
};

__global__ void __launch_bounds__(256)
exchange_kernel(const ExchangeArgs a) {
    const int p = blockIdx.y;
    const uint8_t* __restrict__ src = a.src + (long long)p * a.src_slab_stride;
    uint8_t* __restrict__ dst = a.dst[p] + a.dst_offset;
    const long long total = a.rows * a.units_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / a.units_per_row;
        const int u = (int)(i - row * a.units_per_row);
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + row * a.src_row_stride) + u);
        reinterpret_cast<uint4*>(dst + row * a.dst_row_stride)[u] = v;
    }
}

}  // namespace es

using namespace es;

extern "C" int es_exchange_rows(const void* src, int64_t src_slab_stride, int64_t src_row_stride, void* const* dst_ptrs,
                                int64_t dst_offset, int64_t dst_row_stride, int32_t peers, int64_t rows,
                                int32_t row_bytes, void* stream) {
    if (!src || !dst_ptrs) return set_error(-1, "es_exchange_rows: null pointer");
    if (peers < 1 || peers > MAX_PEERS) return set_error(-1, "es_exchange_rows: 1 .. 16 peers");
    if (rows < 0 || row_bytes <= 0 || row_bytes % 16 != 0) return set_error(-1, "es_exchange_rows: rows of a multiple of 16 bytes");
    if (((uintptr_t)src | (uintptr_t)src_slab_stride | (uintptr_t)src_row_stride | (uintptr_t)dst_offset |
         (uintptr_t)dst_row_stride) & 15)
        return set_error(-1, "es_exchange_rows: pointers, strides and offsets must be multiples of 16 bytes");
    if (src_row_stride < row_bytes || dst_row_stride < row_bytes) return set_error(-1, "es_exchange_rows: a row stride is shorter than a row");
    ExchangeArgs a{};
    a.src = static_cast<const uint8_t*>(src);
    for (int p = 0; p < peers; ++p) {
        if (!dst_ptrs[p] || ((uintptr_t)dst_ptrs[p] & 15)) return set_error(-1, "es_exchange_rows: a receive buffer is null or misaligned");
        a.dst[p] = static_cast<uint8_t*>(dst_ptrs[p]);
    }
    a.src_slab_stride = src_slab_stride; a.src_row_stride = src_row_stride;
    a.dst_offset = dst_offset; a.dst_row_stride = dst_row_stride;
    a.rows = rows; a.units_per_row = row_bytes / 16; a.peers = peers;
    if (rows == 0) return 0;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return set_error(-2, "es_exchange_rows: cannot read the SM count");
    // enough CTAs in flight to cover the link latency: the slabs of all peers together fill the GPU four times
    const long long total = rows * a.units_per_row;
    long long per_peer = (4LL * sms * 2 + peers - 1) / peers;
    const long long need = (total + 255) / 256;
    if (per_peer > need) per_peer = need;
    if (per_peer < 1) per_peer = 1;
    exchange_kernel<<<dim3((unsigned)per_peer, (unsigned)peers), 256, 0, (cudaStream_t)stream>>>(a);
    ES_CHECK_LAUNCH("exchange");
    return 0;
}
