"""B200 (sm_100a) kernel set: the functions `echosparse.attention` calls through `self.K`, same names and argument
meaning as the reference's `echosparse/kernels/sm100.py` (block_attention.py:327, sparse_attention.py:603,
triton_ops.py:37-295, representatives.py:131-166) plus the plan functions of `sm120.py:268-305`.

Every function launches hand-written CUDA through the C ABI on torch's current stream and writes into the tensors the
caller passes. Shapes and dtypes are checked with `assert`, as in the reference; there is no Triton and no CPU path.
"""
import math

import torch

from .. import _native as N

BM = 128
BK = 64
D = 128
NUM_PROBES = 64
LOG2E = 1.4426950408889634


def _cdiv(a, b):
    return -(-a // b)


class KernelTimer:
    """Optional CUDA-event timing of named kernel-set calls on the stream they launch on. Install with
    `set_kernel_timer`; `ms(name)` returns the durations of the recorded calls (synchronises)."""

    def __init__(self, names):
        self.names = set(names)
        self.events = {n: [] for n in names}

    def ms(self, name):
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in self.events[name]]

    def clear(self):
        for v in self.events.values():
            v.clear()


_timer = None


def set_kernel_timer(timer):
    global _timer
    _timer = timer


def _timed(fn):
    name = fn.__name__
    fn = N.device_guard(fn)

    def wrapper(*args, **kwargs):
        t = _timer
        if t is None or name not in t.names:
            return fn(*args, **kwargs)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        out = fn(*args, **kwargs)
        b.record()
        t.events[name].append((a, b))
        return out
    wrapper.__name__, wrapper.__doc__ = name, fn.__doc__
    return wrapper


def _cuda_bf16(*ts):
    for t in ts:
        assert t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous(), "expects contiguous CUDA bf16 tensors"


def _lists(L, H, counts, blocks):
    nq = _cdiv(L, BM)
    assert counts.shape == (nq, H) and counts.dtype == torch.int32 and counts.is_contiguous()
    assert blocks.dtype == torch.int32 and blocks.is_contiguous() and blocks.shape[:2] == (nq, H)


@_timed
def block_attention(q, k, v, out, counts, blocks, offset, lse, flags, mass=None, threshold=60.0):
    """Exact attention over a list of 64-token kv blocks with a fixed offset, plus per-block masses.

    q, k, v, out: (L, H, 128) bf16. counts (nq, H) / blocks (nq, H, nk): sorted block lists. offset, lse: (nq * 128, H)
    float32 log2. flags (nq, H) int32: set where a valid row's sum leaves 2^[-threshold, threshold]. mass (H, nq, nb)
    float32: the listed blocks' entries receive the sum over the tile's rows of 2^(s - offset)."""
    L, H, hd = q.shape
    assert hd == D
    _cuda_bf16(q, k, v, out)
    _lists(L, H, counts, blocks)
    nq = _cdiv(L, BM)
    assert offset.shape == (nq * BM, H) and lse.shape == (nq * BM, H) and offset.dtype == lse.dtype == torch.float32
    assert flags.shape == (nq, H) and flags.dtype == torch.int32
    if mass is not None:
        assert mass.shape == (H, nq, _cdiv(L, BK)) and mass.dtype == torch.float32 and mass.is_contiguous()
    N.check(N.load().es_block_attention(N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(out), N.ptr(counts), N.ptr(blocks),
                                        blocks.shape[-1], N.ptr(offset), N.ptr(lse), N.ptr(flags), N.ptr(mass), L, H,
                                        float(threshold), N.stream_ptr()), "block_attention")
    return out


@_timed
def sparse_attention(q, k, v, k_mean, v_mean, skip_bits, out, counts, blocks, offset, lse, flags, refine, k_rep,
                     v_rep, log_counts, mass=None, threshold=60.0):
    """q, k, v, out: (L, H, 128) bf16. k_mean, v_mean: (nb, H, 128) block means. skip_bits: (H, nq, nw) int32 with
    nw >= 4 * cdiv(nb, 128). counts / blocks: sorted exact block lists. offset, lse: (nq * 128, H) float32 log2.
    refine: (nq, H, 32 * r) int32 refine lists padded with nb. k_rep, v_rep: (H, (nb + 1) * 4, 128) bf16 and
    log_counts (H, (nb + 1) * 4) float32 from `Representatives`. mass: as in `block_attention`, exact blocks only."""
    L, H, hd = q.shape
    assert hd == D
    _cuda_bf16(q, k, v, out, k_mean, v_mean)
    _lists(L, H, counts, blocks)
    nq, nb = _cdiv(L, BM), _cdiv(L, BK)
    nvirt = _cdiv(nb, 128)
    assert k_mean.shape == v_mean.shape == (nb, H, hd)
    assert skip_bits.dtype == torch.int32 and skip_bits.is_contiguous() and skip_bits.shape[:2] == (H, nq)
    assert skip_bits.shape[-1] >= 4 * nvirt
    assert refine.dtype == torch.int32 and refine.shape[:2] == (nq, H) and refine.shape[-1] % 32 == 0
    if refine.shape[-1]:
        assert refine.is_contiguous()
        _cuda_bf16(k_rep, v_rep)
        assert k_rep.shape == v_rep.shape == (H, (nb + 1) * 4, hd)
        assert log_counts.shape == k_rep.shape[:2] and log_counts.dtype == torch.float32 and log_counts.is_contiguous()
    assert offset.shape == (nq * BM, H) and lse.shape == (nq * BM, H)
    if mass is not None:
        assert mass.shape == (H, nq, nb) and mass.dtype == torch.float32 and mass.is_contiguous()
    N.check(N.load().es_sparse_attention(
        N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(k_mean), N.ptr(v_mean), N.ptr(skip_bits), skip_bits.shape[-1], N.ptr(out),
        N.ptr(counts), N.ptr(blocks), blocks.shape[-1], N.ptr(offset), N.ptr(lse), N.ptr(flags), N.ptr(refine),
        refine.shape[-1], N.ptr(k_rep), N.ptr(v_rep), N.ptr(log_counts), N.ptr(mass), L, H, float(threshold),
        N.stream_ptr()), "sparse_attention")
    return out


_tile_scratch = {}


def _tile_list_scratch(flags):
    """Device scratch for the list of flagged tiles (one int32 per tile and one for the count), kept per device and size."""
    key = (flags.device, flags.numel())
    buf = _tile_scratch.get(key)
    if buf is None:
        buf = _tile_scratch[key] = torch.empty(flags.numel() + 1, device=flags.device, dtype=torch.int32)
    return buf


@_timed
def exact_fallback(q, k, v, out, counts, blocks, lse, flags):
    """Online-softmax attention over the block list, for the tiles whose fixed offset was too far off."""
    L, H, hd = q.shape
    assert hd == D
    _cuda_bf16(q, k, v, out)
    _lists(L, H, counts, blocks)
    N.check(N.load().es_exact_fallback(N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(out), N.ptr(counts), N.ptr(blocks),
                                       blocks.shape[-1], N.ptr(lse), N.ptr(flags), L, H,
                                       N.ptr(_tile_list_scratch(flags)), N.stream_ptr()), "exact_fallback")


@_timed
def compensate_fallback(q, k_mean, v_mean, keep, lse, out, flags):
    """Block-mean compensation of the skipped blocks for the fallback tiles, in place on `out` and `lse`."""
    L, H, hd = q.shape
    _cuda_bf16(q, k_mean, v_mean, out)
    nq, nb = _cdiv(L, BM), _cdiv(L, BK)
    assert keep.shape == (H, nq, nb) and keep.dtype == torch.uint8 and keep.is_contiguous()
    N.check(N.load().es_compensate_fallback(N.ptr(q), N.ptr(k_mean), N.ptr(v_mean), N.ptr(keep), N.ptr(lse), N.ptr(out),
                                            N.ptr(flags), L, H, N.ptr(_tile_list_scratch(flags)), N.stream_ptr()),
            "compensate_fallback")


@_timed
def block_means(k, v, k_mean, v_mean):
    """Mean key and value of every 64-token block: (L, H, D) -> (nb, H, D)."""
    L, H, hd = k.shape
    assert hd == D
    _cuda_bf16(k, v, k_mean, v_mean)
    assert k_mean.shape == v_mean.shape == (_cdiv(L, BK), H, hd)
    N.check(N.load().es_block_means(N.ptr(k), N.ptr(v), N.ptr(k_mean), N.ptr(v_mean), L, H, N.stream_ptr()),
            "block_means")


@_timed
def select_blocks(mass, keep_prev, scale_exact, scale_skip, keep, counts, blocks, flags, skip_bits, refine, k, r, L,
                  sink=1 << 30):
    """Top-k blocks of every (query tile, head) by block probability, plus the forced ones.

    Writes the sorted block list (counts, blocks), the keep mask, the refine list (the top-r skipped blocks) and
    the bit mask of blocks the block-mean compensation leaves out. `sink`: first block every tile computes."""
    H, nq, nb = mass.shape
    assert mass.dtype == torch.float32 and mass.is_contiguous() and mass.is_cuda
    assert keep_prev.shape == keep.shape == (H, nq, nb) and keep_prev.dtype == keep.dtype == torch.uint8
    assert blocks.shape == (nq, H, nb) and blocks.dtype == torch.int32 and blocks.is_contiguous()
    assert refine.shape[-1] >= r and refine.dtype == torch.int32
    assert skip_bits.shape[:2] == (H, nq) and skip_bits.dtype == torch.int32 and skip_bits.is_contiguous()
    N.check(N.load().es_select_blocks(N.ptr(mass), N.ptr(keep_prev), N.ptr(scale_exact), N.ptr(scale_skip), N.ptr(keep),
                                      N.ptr(counts), N.ptr(blocks), N.ptr(flags), N.ptr(skip_bits), skip_bits.shape[-1],
                                      N.ptr(refine), refine.shape[-1], int(k), int(r), L, H, min(int(sink), 1 << 30),
                                      N.stream_ptr()), "select_blocks")


@_timed
def estimate_skipped(q, k_mean, keep, offset, lse, mass, scale_exact, scale_skip):
    """Mass estimates of the skipped blocks for the next step's selection, and the per-tile scales."""
    L, H, hd = q.shape
    _cuda_bf16(q, k_mean)
    N.check(N.load().es_estimate_skipped(N.ptr(q), N.ptr(k_mean), N.ptr(keep), N.ptr(offset), N.ptr(lse), N.ptr(mass),
                                         N.ptr(scale_exact), N.ptr(scale_skip), L, H, N.stream_ptr()),
            "estimate_skipped")


@_timed
def full_step_scales(offset, lse, scale_exact, scale_skip, L):
    """Map scales after a step that computed every block; also resets the padding rows of `lse` to 1e30."""
    H, nq = scale_exact.shape
    N.check(N.load().es_full_step_scales(N.ptr(offset), N.ptr(lse), N.ptr(scale_exact), N.ptr(scale_skip), L, H,
                                         N.stream_ptr()), "full_step_scales")


@_timed
def pack_plan(keep, exact_bits):
    """Bit mask of the exactly computed blocks: keep (H, nq, nb) uint8 -> exact_bits (H, nq, NW) int32."""
    H, nq, nb = keep.shape
    assert keep.dtype == torch.uint8 and exact_bits.dtype == torch.int32 and exact_bits.shape[:2] == (H, nq)
    N.check(N.load().es_pack_plan(N.ptr(keep), N.ptr(exact_bits), exact_bits.shape[-1], H, nq, nb, N.stream_ptr()),
            "pack_plan")


@_timed
def rebuild_plan(exact_bits, skip_bits, keep, counts, blocks, refine, refine_counts, means=None, mean_counts=None):
    """keep mask, sorted block list and refine list (padded with nb) with their lengths, from the two bit masks of a plan.
    `means` (shaped as `blocks`) and `mean_counts` receive the sorted list of the blocks left to their means when given;
    this library's fused kernel takes those columns from `skip_bits` itself, so its processor passes None."""
    H, nq, nb = keep.shape
    assert exact_bits.shape == skip_bits.shape and exact_bits.dtype == skip_bits.dtype == torch.int32
    assert blocks.shape == (nq, H, nb) and (means is None or means.shape == blocks.shape)
    assert (means is None) == (mean_counts is None)
    N.check(N.load().es_rebuild_plan(N.ptr(exact_bits), N.ptr(skip_bits), exact_bits.shape[-1], N.ptr(keep),
                                     N.ptr(counts), N.ptr(blocks), N.ptr(refine), refine.shape[-1],
                                     N.ptr(refine_counts), N.ptr(means), N.ptr(mean_counts), H, nq, nb,
                                     N.stream_ptr()), "rebuild_plan")


class Representatives:
    """Builds the representatives of one sequence shape; buffers are reused across calls
    (reference: echosparse/kernels/representatives.py:131-166). Unlike the reference there is no lower limit of 64 kv
    blocks: probes of short sequences simply repeat query blocks."""

    def __init__(self, L, H, D, device, iters=6):
        assert D == 128
        nb = _cdiv(L, BK)
        self.L, self.H, self.D, self.nb, self.iters = L, H, D, nb, iters
        nb4 = (nb + 1) * 4
        self.k = torch.zeros(H, nb4, D, device=device, dtype=torch.bfloat16)
        self.v = torch.zeros(H, nb4, D, device=device, dtype=torch.bfloat16)
        self.log_counts = torch.full((H, nb4), -math.inf, device=device)
        self._gram = torch.empty(H, D, D, device=device)
        self._parts = torch.empty(N.load().es_reps_gram_splits(L), H, D, D, device=device)
        self._probes = torch.empty(H, NUM_PROBES, D, device=device, dtype=torch.bfloat16)
        self._metric = torch.empty(H, D, D, device=device, dtype=torch.bfloat16)

    def build(self, q, k, v, k_mean=None, v_mean=None):
        """Representatives of every block; given k_mean / v_mean (nb, H, D), also the block means."""
        t = _timer
        if t is not None and "reps_build" in t.names:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            self._build(q, k, v, k_mean, v_mean)
            b.record()
            t.events["reps_build"].append((a, b))
        else:
            self._build(q, k, v, k_mean, v_mean)

    @N.device_guard
    def _build(self, q, k, v, k_mean, v_mean):
        _cuda_bf16(q, k, v)
        assert q.shape == k.shape == v.shape == (self.L, self.H, self.D)
        lib = N.load()
        N.check(lib.es_reps_metric(N.ptr(q), N.ptr(self._parts), N.ptr(self._gram), N.ptr(self._metric),
                                   N.ptr(self._probes), self.L, self.H, N.stream_ptr()), "reps_metric")
        N.check(lib.es_reps_kmeans(N.ptr(k), N.ptr(v), N.ptr(self._metric), N.ptr(self._probes), N.ptr(self.k),
                                   N.ptr(self.v), N.ptr(self.log_counts), N.ptr(k_mean), N.ptr(v_mean), self.L, self.H,
                                   self.iters, N.stream_ptr()), "reps_kmeans")
