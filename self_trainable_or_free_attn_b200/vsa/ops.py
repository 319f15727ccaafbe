"""VSA2 operator: autograd wiring around the native kernels (C ABI of include/echosparse_vsa_sm100.h).

Mirrors the public entry points of the reference's `echosparse/vsa/ops.py`: `Selection` (:90-117), `mask_to_selection`
(:107-122), `route` (:216-223), `vsa2_attention` (:534-571) and `fine_block_sparse_attention` (:670-679), with the same
argument meaning, layout contract and error behaviour:

  q, k, v : [B, H, L, D] contiguous, bf16 or fp16, D in {64, 128}, L = NB * 64, tokens block-major, block i holding
            blk_cnt[i] valid tokens first, then padding (finite values; zeros recommended).
  gate    : optional pre-activation, [B, H, L] or [B, H, L, D]. O = O_fine + act(gate) * O_coarse[block].
  blk_cnt : int32 [NB], 1..64.

Every stage is a CUDA kernel of this library; torch is used for allocation and for the shape-only dense CSR of the coarse
branch. The backward has one owner per output row in both passes (kv -> q lists for dK / dV, q -> kv lists for dQ), so
gradients are reproducible bit for bit; the intermediates are released after the first backward (ops.py:520-522 there).
"""
import math
from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native as N

GATE_ACTS = {"tanh": 0, "identity": 1}
ROW_NORMS = {"valid_groups": 0, "paper": 1}
_DTYPES = {torch.bfloat16: 0, torch.float16: 1}


@dataclass
class Selection:
    """Exact block selection, CSR. Absolute offsets into the idx arrays."""
    q2k_ptr: torch.Tensor   # [B, H, NB+1] int32
    q2k_idx: torch.Tensor   # [nnz] int32, kv block ids ascending per row
    k2q_ptr: torch.Tensor   # [B, H, NB+1]
    k2q_idx: torch.Tensor   # [nnz], query block ids ascending per column

    def row_counts(self):
        return (self.q2k_ptr[..., 1:] - self.q2k_ptr[..., :-1]).to(torch.int64)

    def to_mask(self, nb):
        """Dense bool block mask [B, H, NB, NB]."""
        B, H = self.q2k_ptr.shape[:2]
        ptr = self.q2k_ptr.reshape(B * H, nb + 1).to(torch.int64)
        mask = torch.zeros(B * H * nb, nb, dtype=torch.bool, device=ptr.device)
        cnt = (ptr[:, 1:] - ptr[:, :-1]).reshape(-1)
        rows = torch.repeat_interleave(torch.arange(B * H * nb, device=ptr.device), cnt)
        # rows of one (b, h) are contiguous in idx; different (b, h) may leave gaps between their ranges
        offs = torch.arange(int(cnt.sum()), device=ptr.device) - torch.repeat_interleave(torch.cumsum(cnt, 0) - cnt, cnt)
        src = torch.repeat_interleave(ptr[:, :-1].reshape(-1), cnt) + offs
        mask[rows, self.q2k_idx[src].to(torch.int64)] = True
        return mask.reshape(B, H, nb, nb)


def mask_to_selection(mask):
    """Bool block mask [B, H, NB, NB] -> CSR selection (test / diagnostic utility)."""
    assert mask.dim() == 4 and mask.dtype == torch.bool

    def csr(m):
        B, H, n, _ = m.shape
        cnt = m.reshape(-1, n).sum(-1).to(torch.int64)
        incl = torch.cumsum(cnt, 0)
        ptr = torch.cat([(incl - cnt).reshape(B * H, n), incl.reshape(B * H, n)[:, -1:]], dim=1)
        idx = m.reshape(-1, n).nonzero()[:, 1]
        if idx.numel() == 0:
            idx = torch.zeros(1, dtype=torch.int64, device=m.device)
        return ptr.reshape(B, H, n + 1).to(torch.int32).contiguous(), idx.to(torch.int32).contiguous()

    qp, qi = csr(mask)
    kp, ki = csr(mask.transpose(-1, -2).contiguous())
    return Selection(qp, qi, kp, ki)


def _check_tokens(q, k, v):
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor: this operator has no CPU path")
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous [B,H,L,D]")
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise RuntimeError("q, k, v must share the dtype bfloat16 or float16")
    B, H, L, D = q.shape
    if k.shape != q.shape or v.shape != q.shape or L % 64 != 0 or D not in (64, 128):
        raise RuntimeError("q, k, v must be [B, H, NB*64, D] with D in {64, 128}")
    return B, H, L, D


def _pad64(n):
    return -(-n // 64) * 64


@N.device_guard
def pool_fwd(q, k, v, blk_cnt, R):
    """(qr, kr [B,H,Lr_pad,D] router group means; qc, kc, vc [B,H,NBc_pad,D] block means)."""
    B, H, L, D = q.shape
    nb, G = L // 64, 64 // R
    lr_pad, nbc_pad = _pad64(nb * G), _pad64(nb)
    mk = lambda n: torch.empty(B, H, n, D, device=q.device, dtype=q.dtype)
    qr, kr, qc, kc, vc = mk(lr_pad), mk(lr_pad), mk(nbc_pad), mk(nbc_pad), mk(nbc_pad)
    N.check(N.load().es_vsa_pool(N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(qr), N.ptr(kr), None, N.ptr(qc), N.ptr(kc), N.ptr(vc),
                                 N.ptr(blk_cnt), B * H, L, D, R, lr_pad, nbc_pad, _DTYPES[q.dtype], N.stream_ptr()),
            "es_vsa_pool")
    return qr, kr, qc, kc, vc


@N.device_guard
def router_scores(qr, kr, blk_cnt, R, row_norm=1):
    """Block scores [B, H, NB, NB] fp32 of the PSP router (diagnostic; `route` uses the same kernels)."""
    B, H, lr_pad, D = qr.shape
    nb = blk_cnt.numel()
    lse2 = torch.empty(B, H, lr_pad, device=qr.device, dtype=torch.float32)
    lib, dt, st = N.load(), _DTYPES[qr.dtype], N.stream_ptr()
    N.check(lib.es_vsa_router_lse(N.ptr(qr), N.ptr(kr), N.ptr(lse2), N.ptr(blk_cnt), B * H, nb, D, R, lr_pad, dt, st),
            "es_vsa_router_lse")
    scores = torch.empty(B, H, nb, nb, device=qr.device, dtype=torch.float32)
    N.check(lib.es_vsa_router_scores(N.ptr(qr), N.ptr(kr), N.ptr(lse2), N.ptr(scores), N.ptr(blk_cnt), B * H, nb, D, R,
                                     lr_pad, 0, B * H, row_norm, dt, st), "es_vsa_router_scores")
    return scores


@N.device_guard
def global_topk(scores, budget):
    """Exact global top-`budget` of every (b, h) score matrix -> Selection."""
    B, H, nb, _ = scores.shape
    budget = max(0, min(int(budget), nb * nb))
    dev = scores.device
    lib = N.load()
    i32 = dict(device=dev, dtype=torch.int32)
    qp, kp = torch.empty(B, H, nb + 1, **i32), torch.empty(B, H, nb + 1, **i32)
    qi, ki = torch.empty(max(1, B * H * budget), **i32), torch.empty(max(1, B * H * budget), **i32)
    ws = torch.empty(int(lib.es_vsa_topk_workspace_bytes(B * H, nb)), device=dev, dtype=torch.uint8)
    N.check(lib.es_vsa_global_topk(N.ptr(scores.contiguous()), nb, 0, B * H, budget, N.ptr(qp), N.ptr(qi), N.ptr(kp),
                                   N.ptr(ki), N.ptr(ws), N.stream_ptr()), "es_vsa_global_topk")
    return Selection(qp, qi, kp, ki)


# ------------------------------------------------------------------------------------------- backward variant knobs
# The reference has three generic fine-backward variants (0 / 1: dQ added with atomics, 2: a second q -> kv pass without
# atomics; echosparse/vsa/dispatch.py:1-53) and bit options for its ThunderKittens backward (ops.py:171-177). This
# library has one backward, the atomics-free two-pass form (their variant 2), so the knobs are accepted, validated the
# same way and remembered, and change nothing: code written against the reference keeps importing and running.
BWD_VARIANTS = (0, 1, 2)
TK_BWD_OPTS = (0, 1, 2, 3, 16, 17, 18, 19)
_knobs = {"bwd_variant": None, "tk_bwd_opts": None}


def set_bwd_variant(v):
    """Accepted for compatibility (None, 0, 1 or 2; anything else raises ValueError). The backward here is always the
    two-pass, atomics-free one."""
    if v is not None and v not in BWD_VARIANTS:
        raise ValueError(f"set_bwd_variant takes None or one of {BWD_VARIANTS}; got {v!r}")
    _knobs["bwd_variant"] = None if v is None else int(v)


def resolve_bwd_variant(q, call=None):
    """(variant, source) the way the reference reports it: this build always runs variant 2; `source` says whether a
    per-call value, `set_bwd_variant` or nothing ("auto") asked for one."""
    for value, source in ((call, "call"), (_knobs["bwd_variant"], "set_bwd_variant")):
        if value is not None:
            if value not in BWD_VARIANTS:
                raise ValueError(f"{source}: the variant is one of {BWD_VARIANTS}; got {value!r}")
            return 2, source
    return 2, "auto"


def set_tk_bwd_opts(v):
    """Accepted for compatibility (None or one of the reference's option words). There is no ThunderKittens backward
    in this build, so nothing changes."""
    if v is not None and v not in TK_BWD_OPTS:
        raise ValueError(f"set_tk_bwd_opts takes None or one of {TK_BWD_OPTS}; got {v!r}")
    _knobs["tk_bwd_opts"] = v


def budget_from_topk(nb, topk, budget):
    if budget is not None:
        return int(budget)
    if topk is None:
        raise ValueError("pass topk (average kv blocks per query block) or budget")
    return int(nb) * int(topk)


def _route(qr, kr, blk_cnt, R, budget, row_norm):
    return global_topk(router_scores(qr, kr, blk_cnt, R, row_norm), budget)


@N.device_guard
def route(q, k, blk_cnt, R=16, topk=None, budget=None, row_norm="paper"):
    """Standalone VSA2 PSP router + exact global top-k (stop-gradient)."""
    _check_tokens(q, k, k)
    blk_cnt = blk_cnt.to(torch.int32).contiguous()
    qr, kr, _, _, _ = pool_fwd(q, k, k, blk_cnt, R)
    return _route(qr, kr, blk_cnt, R, budget_from_topk(q.shape[2] // 64, topk, budget), ROW_NORMS[row_norm])


# Original VSA only needs the whole-block means of pool_fwd; R = 32 makes its unused router pools smallest.
_ROWS_POOL_R = 32


@N.device_guard
def block_scores(qc, kc, nb):
    """Original-VSA block scores [B, H, NB, NB] in the token dtype from the block means."""
    B, H, nbc_pad, D = qc.shape
    scores = torch.empty(B, H, nb, nb, device=qc.device, dtype=qc.dtype)
    N.check(N.load().es_vsa_block_scores(N.ptr(qc), N.ptr(kc), N.ptr(scores), B * H, nb, D, nbc_pad, 0, B * H,
                                         _DTYPES[qc.dtype], N.stream_ptr()), "es_vsa_block_scores")
    return scores


@N.device_guard
def row_topk(scores, topk):
    """Exactly min(topk, NB) kv blocks per query row of 16-bit scores [B, H, NB, NB] -> Selection."""
    B, H, nb, _ = scores.shape
    K = max(0, min(int(topk), nb))
    lib = N.load()
    i32 = dict(device=scores.device, dtype=torch.int32)
    qp, kp = torch.empty(B, H, nb + 1, **i32), torch.empty(B, H, nb + 1, **i32)
    qi, ki = torch.empty(max(1, B * H * nb * K), **i32), torch.empty(max(1, B * H * nb * K), **i32)
    ws = torch.empty(int(lib.es_vsa_topk_workspace_bytes(B * H, nb)), device=scores.device, dtype=torch.uint8)
    N.check(lib.es_vsa_row_topk(N.ptr(scores.contiguous()), nb, 0, B * H, K, N.ptr(qp), N.ptr(qi), N.ptr(kp), N.ptr(ki),
                                N.ptr(ws), _DTYPES[scores.dtype], N.stream_ptr()), "es_vsa_row_topk")
    return Selection(qp, qi, kp, ki)


@N.device_guard
def route_rows(q, k, blk_cnt, topk):
    """Standalone original-VSA router (stop-gradient): whole-block scores, exactly min(topk, NB) blocks per row."""
    _check_tokens(q, k, k)
    blk_cnt = blk_cnt.to(torch.int32).contiguous()
    _, _, qc, kc, _ = pool_fwd(q, k, k, blk_cnt, _ROWS_POOL_R)
    return row_topk(block_scores(qc, kc, q.shape[2] // 64), topk)


@N.device_guard
def attn_fwd(q, k, v, ptr, idx, cnt):
    """(O, lse) of the list attention; q, k, v [B, H, L, D], lists over L / 64 blocks."""
    B, H, L, D = q.shape
    o = torch.empty_like(q)
    lse = torch.empty(B, H, L, device=q.device, dtype=torch.float32)
    N.check(N.load().es_vsa_attn_fwd(N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(o), N.ptr(lse), N.ptr(ptr), N.ptr(idx),
                                     N.ptr(cnt), B * H, L, D, _DTYPES[q.dtype], N.stream_ptr()), "es_vsa_attn_fwd")
    return o, lse


def _coarse_meta(B, H, nb, nbc_pad, device):
    """Dense CSR over the 64-row tiles of the pooled sequence (shape-only metadata) and the tiles' valid counts."""
    T = nbc_pad // 64
    cnt = torch.clamp(nb - 64 * torch.arange(T, device=device), max=64).to(torch.int32).contiguous()
    bh = torch.arange(B * H, device=device, dtype=torch.int64)
    ptr = (bh[:, None] * (T * T) + torch.arange(T + 1, device=device, dtype=torch.int64)[None, :] * T)
    idx = torch.arange(T, device=device, dtype=torch.int32).repeat(B * H * T).contiguous()
    return cnt, ptr.to(torch.int32).reshape(B, H, T + 1).contiguous(), idx


def _bwd_kv(q, k, v, dout, lse, delta, ptr, idx, cnt, add_dk=None, add_dv=None, f32=False):
    B, H, L, D = q.shape
    mk = (lambda: torch.empty(B, H, L, D, device=q.device, dtype=torch.float32)) if f32 else (lambda: torch.empty_like(q))
    dk, dv = mk(), mk()
    add_nb = add_dk.shape[2] if add_dk is not None else 0
    N.check(N.load().es_vsa_attn_bwd_kv(
        N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(dout), N.ptr(lse), N.ptr(delta), None if f32 else N.ptr(dk),
        None if f32 else N.ptr(dv), N.ptr(dk) if f32 else None, N.ptr(dv) if f32 else None, N.ptr(add_dk), N.ptr(add_dv),
        add_nb, N.ptr(ptr), N.ptr(idx), N.ptr(cnt), B * H, L, D, _DTYPES[q.dtype], N.stream_ptr()), "es_vsa_attn_bwd_kv")
    return dk, dv


def _bwd_q(q, k, v, dout, lse, delta, ptr, idx, cnt, add_dq=None, f32=False):
    B, H, L, D = q.shape
    dq = torch.empty(B, H, L, D, device=q.device, dtype=torch.float32) if f32 else torch.empty_like(q)
    add_nb = add_dq.shape[2] if add_dq is not None else 0
    N.check(N.load().es_vsa_attn_bwd_q(
        N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(dout), N.ptr(lse), N.ptr(delta), None if f32 else N.ptr(dq),
        N.ptr(dq) if f32 else None, N.ptr(add_dq), add_nb, N.ptr(ptr), N.ptr(idx), N.ptr(cnt), B * H, L, D,
        _DTYPES[q.dtype], N.stream_ptr()), "es_vsa_attn_bwd_q")
    return dq


# ------------------------------------------------------------------------------------------- split-KV scheduling
def _want_nonneg_real(owner, field, value):
    """Thresholds: a finite real number >= 0 (bool is not a number here). TypeError / ValueError as the reference raises."""
    if type(value) is bool or not isinstance(value, (int, float)):
        raise TypeError(f"{owner}.{field} takes a real number, not {type(value).__name__}")
    if value != value or value in (math.inf, -math.inf) or value < 0:
        raise ValueError(f"{owner}.{field} = {value!r}: expected a finite value >= 0")


def _want_count(owner, field, value):
    """Counts: a true int >= 1."""
    if type(value) is bool or not isinstance(value, int):
        raise TypeError(f"{owner}.{field} takes an int, not {type(value).__name__}")
    if value < 1:
        raise ValueError(f"{owner}.{field} = {value!r}: expected at least 1")


@dataclass(frozen=True)
class SplitPolicy:
    """Automatic per-direction choice of the lists worth splitting (reference: echosparse/vsa/ops.py:226-262).

    A list of n blocks is eligible when n >= max(min_chunks * chunk, chunk + 1, rel_mean * (mean list length of its
    head), tail_frac * (all edges of that direction) / resident CTAs); if more than waves * resident lists are eligible
    nothing is split in that direction. resident = SMs x CTAs per SM of the consuming kernel, or `resident_ctas`."""
    rel_mean: float = 4.0
    tail_frac: float = 0.05
    min_chunks: int = 2
    fwd_waves: float = 1.0
    bwd_waves: float = 8.0
    max_task_waves: int = 64
    resident_ctas: Optional[int] = None

    def __post_init__(self):
        for field in ("rel_mean", "tail_frac", "fwd_waves", "bwd_waves"):
            _want_nonneg_real("SplitPolicy", field, getattr(self, field))
        _want_count("SplitPolicy", "min_chunks", self.min_chunks)
        _want_count("SplitPolicy", "max_task_waves", self.max_task_waves)
        if self.resident_ctas is not None:
            _want_count("SplitPolicy", "resident_ctas", self.resident_ctas)


@dataclass(frozen=True)
class SplitKV:
    """Balanced split-KV scheduling of the fine attention (reference: echosparse/vsa/ops.py:265-305). A query block
    (forward, dQ pass) or kv block (dK / dV pass) whose list is chosen runs as ceil(n / chunk) balanced chunk tasks; the
    chunks write fp32 partials that are merged per block in chunk order (deterministic). Without `policy` every list
    longer than `chunk` is chosen; with a SplitPolicy (`SplitKV.auto()`) the planner on the GPU picks the clearly long
    ones per direction. Partials are capped at `max_scratch_bytes` per stage (later long lists run unsplit)."""
    chunk: int = 64
    fwd: bool = True
    bwd: bool = True
    max_scratch_bytes: int = 1 << 30
    policy: Optional[SplitPolicy] = None

    def __post_init__(self):
        chunk, cap = int(self.chunk), int(self.max_scratch_bytes)
        if chunk < 1 or chunk > 2 ** 30:
            raise ValueError(f"SplitKV.chunk = {self.chunk}: a chunk holds between 1 and 2**30 blocks")
        if cap < 0:
            raise ValueError(f"SplitKV.max_scratch_bytes = {self.max_scratch_bytes}: a byte count cannot be negative")
        if not (self.policy is None or isinstance(self.policy, SplitPolicy)):
            raise TypeError(f"SplitKV.policy takes a SplitPolicy or None, not {type(self.policy).__name__}")

    @classmethod
    def auto(cls, chunk=64, fwd=True, bwd=True, max_scratch_bytes=64 << 20, policy=None):
        """The planner on the GPU decides per direction which lists to split (default thresholds of `SplitPolicy`);
        forward partials limited to 64 MiB unless told otherwise."""
        if policy is None:
            policy = SplitPolicy()
        return cls(chunk, fwd, bwd, max_scratch_bytes, policy)


def split_slots(nnz, chunk, slot_bytes, max_bytes):
    """Partial slots of a plan: max_bytes // slot_bytes, and never more than a split plan can use (2 * ceil(nnz / chunk))."""
    return max(0, min(int(max_bytes) // int(slot_bytes), 2 * (-(-int(nnz) // int(chunk)))))


# resident CTAs per SM of the kernels that consume a plan (shared memory: 80 KB forward, 97 KB dK / dV, 96 KB dQ at D = 128)
_CTAS_PER_SM = {("fwd", 64): 5, ("fwd", 128): 2, ("bwd_kv", 64): 4, ("bwd_kv", 128): 2, ("bwd_q", 64): 4, ("bwd_q", 128): 2}


def split_resident(q, kind, policy=None):
    if policy is not None and policy.resident_ctas is not None:
        return int(policy.resident_ctas)
    return torch.cuda.get_device_properties(q.device).multi_processor_count * _CTAS_PER_SM[(kind, q.shape[-1])]


@N.device_guard
def split_plan(ptr, chunk, max_slots, min_len=0, rel_mean=0.0, tail_frac=0.0, resident=1, budget=-1):
    """(tasks [NR + max_slots, 4], merges [max(1, min(NR, max_slots // 2)), 4], info [8]) int32 on the device."""
    B, H, n1 = ptr.shape
    nr = B * H * (n1 - 1)
    i32 = dict(device=ptr.device, dtype=torch.int32)
    tasks = torch.empty(nr + max_slots, 4, **i32)
    merges = torch.empty(max(1, min(nr, max_slots // 2)), 4, **i32)
    info = torch.empty(8, **i32)
    lib = N.load()
    ws = torch.empty(int(lib.es_vsa_split_plan_workspace_bytes(B * H, n1 - 1)), device=ptr.device, dtype=torch.uint8)
    N.check(lib.es_vsa_split_plan(N.ptr(ptr), B * H, n1 - 1, int(chunk), int(max_slots), max(int(chunk) + 1, int(min_len)),
                                  float(rel_mean), float(tail_frac), int(resident),
                                  2 ** 31 - 1 if budget < 0 else int(budget), N.ptr(tasks), N.ptr(merges), N.ptr(info),
                                  N.ptr(ws), N.stream_ptr()), "es_vsa_split_plan")
    return tasks, merges, info


def split_plan_for(q, ptr, idx, split, kind, slot_bytes):
    """(tasks, merges, info, slots) of one direction. kind: fwd (q2k), bwd_kv (k2q), bwd_q (q2k)."""
    nnz, nb = idx.numel(), ptr.shape[-1] - 1
    slots = split_slots(nnz, split.chunk, slot_bytes, split.max_scratch_bytes)
    pol = split.policy
    if pol is None:
        return (*split_plan(ptr, split.chunk, slots), slots)
    resident = split_resident(q, kind, pol)
    budget = int((pol.fwd_waves if kind == "fwd" else pol.bwd_waves) * resident)
    slots = min(slots, budget * (-(-nb // split.chunk)), pol.max_task_waves * resident)
    plan = split_plan(ptr, split.chunk, slots, max(split.chunk + 1, pol.min_chunks * split.chunk), pol.rel_mean,
                      pol.tail_frac, resident, budget)
    return (*plan, slots)


def split_fine_fwd(q, k, v, ptr, idx, blk_cnt, split):
    """Balanced fine forward: plan, chunk / direct tasks, merge. Returns (O_f, lse) like attn_fwd."""
    B, H, L, D = q.shape
    tasks, merges, info, slots = split_plan_for(q, ptr, idx, split, "fwd", 64 * (D + 1) * 4)
    part_o = torch.empty(max(slots, 1), 64, D, device=q.device, dtype=torch.float32)
    part_lse = torch.empty(max(slots, 1), 64, device=q.device, dtype=torch.float32)
    o = torch.empty_like(q)
    lse = torch.empty(B, H, L, device=q.device, dtype=torch.float32)
    lib, dt, st = N.load(), _DTYPES[q.dtype], N.stream_ptr()
    N.check(lib.es_vsa_attn_fwd_tasks(N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(o), N.ptr(lse), N.ptr(idx), N.ptr(blk_cnt),
                                      N.ptr(tasks), N.ptr(info), tasks.shape[0], N.ptr(part_o), N.ptr(part_lse), B * H, L,
                                      D, dt, st), "es_vsa_attn_fwd_tasks")
    if slots:
        N.check(lib.es_vsa_split_merge_fwd(N.ptr(part_o), N.ptr(part_lse), N.ptr(merges), N.ptr(info), merges.shape[0],
                                           N.ptr(blk_cnt), N.ptr(o), N.ptr(lse), L, D, 1, dt, st), "es_vsa_split_merge_fwd")
    return o, lse


def _merge_sum(part, merges, info, add, blk_cnt, out, L, D, dt):
    N.check(N.load().es_vsa_split_merge_sum(N.ptr(part), N.ptr(merges), N.ptr(info), merges.shape[0], N.ptr(add),
                                            add.shape[2] if add is not None else 0, N.ptr(blk_cnt), N.ptr(out), None, L, D,
                                            dt, N.stream_ptr()), "es_vsa_split_merge_sum")


def split_fine_bwd(q, k, v, dout, lse, delta, sel, blk_cnt, dqc, dkc, dvc, split):
    """Balanced fine backward: the dK / dV pass over a plan of the kv -> q lists, the dQ pass over one of the q -> kv lists."""
    B, H, L, D = q.shape
    lib, dt, st = N.load(), _DTYPES[q.dtype], N.stream_ptr()
    f32 = dict(device=q.device, dtype=torch.float32)
    add_nb = dkc.shape[2] if dkc is not None else 0
    tasks, merges, info, slots = split_plan_for(q, sel.k2q_ptr, sel.k2q_idx, split, "bwd_kv", 2 * 64 * D * 4)
    part_dk, part_dv = torch.empty(max(slots, 1), 64, D, **f32), torch.empty(max(slots, 1), 64, D, **f32)
    dk, dv = torch.empty_like(q), torch.empty_like(q)
    N.check(lib.es_vsa_attn_bwd_kv_tasks(
        N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(dout), N.ptr(lse), N.ptr(delta), N.ptr(dk), N.ptr(dv), None, None, N.ptr(dkc),
        N.ptr(dvc), add_nb, N.ptr(sel.k2q_idx), N.ptr(blk_cnt), N.ptr(tasks), N.ptr(info), tasks.shape[0], N.ptr(part_dk),
        N.ptr(part_dv), B * H, L, D, dt, st), "es_vsa_attn_bwd_kv_tasks")
    if slots:
        _merge_sum(part_dk, merges, info, dkc, blk_cnt, dk, L, D, dt)
        _merge_sum(part_dv, merges, info, dvc, blk_cnt, dv, L, D, dt)
    del part_dk, part_dv
    tasks, merges, info, slots = split_plan_for(q, sel.q2k_ptr, sel.q2k_idx, split, "bwd_q", 64 * D * 4)
    part_dq = torch.empty(max(slots, 1), 64, D, **f32)
    dq = torch.empty_like(q)
    N.check(lib.es_vsa_attn_bwd_q_tasks(
        N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(dout), N.ptr(lse), N.ptr(delta), N.ptr(dq), None, N.ptr(dqc), add_nb,
        N.ptr(sel.q2k_idx), N.ptr(blk_cnt), N.ptr(tasks), N.ptr(info), tasks.shape[0], N.ptr(part_dq), B * H, L, D, dt, st),
        "es_vsa_attn_bwd_q_tasks")
    if slots:
        _merge_sum(part_dq, merges, info, dqc, blk_cnt, dq, L, D, dt)
    return dq, dk, dv


def _check_split(split):
    if split is None:
        return None
    if isinstance(split, str) and split == "auto":
        return SplitKV.auto()
    if not isinstance(split, SplitKV):
        raise TypeError(f"split_kv must be a SplitKV, 'auto' or None, got {type(split).__name__}")
    return split


def describe_split(q, selection, split):
    """Diagnostic (synchronises): the plans the operator would build for this selection, per direction."""
    out = {}
    D = q.shape[-1]
    dirs = []
    if split.fwd:
        dirs.append(("fwd", selection.q2k_ptr, selection.q2k_idx, 64 * (D + 1) * 4))
    if split.bwd:
        dirs.append(("bwd_kv", selection.k2q_ptr, selection.k2q_idx, 2 * 64 * D * 4))
        dirs.append(("bwd_q", selection.q2k_ptr, selection.q2k_idx, 64 * D * 4))
    names = ["tasks", "split_rows", "split_slots", "rows", "eligible_rows", "within_budget", "global_threshold", "edges"]
    for kind, ptr, idx, sb in dirs:
        _, merges, info, slots = split_plan_for(q, ptr, idx, split, kind, sb)
        out[kind] = dict(info=dict(zip(names, info.tolist())), max_slots=slots,
                         resident=split_resident(q, kind, split.policy) if split.policy else None)
    return out


def _fine_fwd(q, k, v, sel, blk_cnt, split):
    if split is not None and split.fwd:
        return split_fine_fwd(q, k, v, sel.q2k_ptr, sel.q2k_idx, blk_cnt, split)
    return attn_fwd(q, k, v, sel.q2k_ptr, sel.q2k_idx, blk_cnt)


def _fine_bwd(q, k, v, dout, lse, delta, sel, blk_cnt, dqc, dkc, dvc, split):
    if split is not None and split.bwd:
        return split_fine_bwd(q, k, v, dout, lse, delta, sel, blk_cnt, dqc, dkc, dvc, split)
    dk, dv = _bwd_kv(q, k, v, dout, lse, delta, sel.k2q_ptr, sel.k2q_idx, blk_cnt, add_dk=dkc, add_dv=dvc)
    return _bwd_q(q, k, v, dout, lse, delta, sel.q2k_ptr, sel.q2k_idx, blk_cnt, add_dq=dqc), dk, dv


def _gate_mode(gate, q):
    if gate is None:
        return 0
    if gate.shape == q.shape[:3]:
        return 1
    if gate.shape == q.shape:
        return 2
    raise RuntimeError("gate must be [B, H, L] or [B, H, L, D]")


def _fuse_bwd(dout, of, oc, gate, blk_cnt, gate_act):
    B, H, L, D = dout.shape
    nbc_pad = oc.shape[2]
    mode = _gate_mode(gate, dout)
    delta_f = torch.empty(B, H, L, device=dout.device, dtype=torch.float32)
    dout_c = torch.zeros_like(oc)
    delta_c = torch.zeros(B, H, nbc_pad, device=dout.device, dtype=torch.float32)
    dgate = torch.empty_like(gate) if gate is not None else None
    N.check(N.load().es_vsa_fuse_bwd(N.ptr(dout), N.ptr(of), N.ptr(oc), N.ptr(gate), None, N.ptr(delta_f), N.ptr(dout_c),
                                     N.ptr(delta_c), N.ptr(dgate), N.ptr(blk_cnt), B * H, L, D, nbc_pad, mode, gate_act,
                                     _DTYPES[dout.dtype], N.stream_ptr()), "es_vsa_fuse_bwd")
    return delta_f, dout_c, delta_c, dgate


class _Function(torch.autograd.Function):
    @staticmethod
    @N.device_guard
    def forward(ctx, q, k, v, gate, blk_cnt, R, budget, row_norm, gate_act, sel_in, split):
        B, H, L, D = q.shape
        nb = L // 64
        qr, kr, qc, kc, vc = pool_fwd(q, k, v, blk_cnt, R)
        c_cnt, c_ptr, c_idx = _coarse_meta(B, H, nb, qc.shape[2], q.device)
        oc, lse_c = attn_fwd(qc, kc, vc, c_ptr, c_idx, c_cnt)
        if sel_in is not None:
            sel = sel_in
        elif row_norm < 0:                               # original VSA: per-row top-K of the whole-block scores
            sel = row_topk(block_scores(qc, kc, nb), budget)
        else:
            sel = _route(qr, kr, blk_cnt, R, budget, row_norm)
        of, lse_f = _fine_fwd(q, k, v, sel, blk_cnt, split)
        o = torch.empty_like(q)
        N.check(N.load().es_vsa_fuse_fwd(N.ptr(of), N.ptr(oc), N.ptr(gate), N.ptr(o), N.ptr(blk_cnt), B * H, L, D,
                                         oc.shape[2], _gate_mode(gate, q), gate_act, _DTYPES[q.dtype], N.stream_ptr()),
                "es_vsa_fuse_fwd")
        ctx.save_for_backward(q, k, v, gate, blk_cnt)
        # held as attributes, not saved tensors, so that backward can release them after their last use
        ctx.inter = [qc, kc, vc, oc, lse_c, of, lse_f, sel, c_cnt, c_ptr, c_idx]
        ctx.has_gate = gate is not None
        ctx.gate_act = gate_act
        ctx.split = split
        ctx.mark_non_differentiable(sel.q2k_ptr, sel.q2k_idx, sel.k2q_ptr, sel.k2q_idx)
        return o, sel.q2k_ptr, sel.q2k_idx, sel.k2q_ptr, sel.k2q_idx

    @staticmethod
    @N.device_guard
    def backward(ctx, dout, *unused):
        q, k, v, gate, blk_cnt = ctx.saved_tensors
        if ctx.inter is None:
            raise RuntimeError("VSA backward frees its intermediates after the first backward; "
                               "re-run the forward instead of backward(retain_graph=True) twice")
        qc, kc, vc, oc, lse_c, of, lse_f, sel, c_cnt, c_ptr, c_idx = ctx.inter
        dout = dout.contiguous()
        delta_f, dout_c, delta_c, dgate = _fuse_bwd(dout, of, oc, gate if ctx.has_gate else None, blk_cnt, ctx.gate_act)
        ctx.inter[5] = None
        del of
        # coarse branch (dense over the block means) -> fp32 per-block gradients; the dense lists are their own inverse
        dkc, dvc = _bwd_kv(qc, kc, vc, dout_c, lse_c, delta_c, c_ptr, c_idx, c_cnt, f32=True)
        dqc = _bwd_q(qc, kc, vc, dout_c, lse_c, delta_c, c_ptr, c_idx, c_cnt, f32=True)
        # fine branch on the forward's selection, plus the unpooled coarse gradients (block gradient / count per token)
        dq, dk, dv = _fine_bwd(q, k, v, dout, lse_f, delta_f, sel, blk_cnt, dqc, dkc, dvc, ctx.split)
        ctx.inter = None
        return (dq, dk, dv, dgate if ctx.has_gate else None) + (None,) * 7


@N.device_guard
def vsa2_attention(q, k, v, gate, blk_cnt, *, R=16, topk=None, budget=None, row_norm="paper", gate_act="tanh",
                   backend="auto", selection: Optional[Selection] = None, return_selection=False, split_kv=None):
    """Full VSA2 attention: O = O_fine + act(gate) * repeat(O_coarse).

    The router (pool R -> softmax over all pooled keys -> pool to 64-token blocks) and the exact global top-k (budget =
    NB * topk connections per (b, h)) run on every call unless a frozen `selection` is passed (testing). `backend` is kept
    for signature compatibility; there is a single sm_100a backend. `split_kv`: a SplitKV (manual), SplitKV.auto() or
    "auto" (planner on the GPU), None (default) unsplit.
    """
    if backend not in ("auto", "generic"):
        raise ValueError(f"unknown backend {backend!r}: this build has the one sm_100a backend ('auto' or 'generic')")
    _check_tokens(q, k, v)
    nb = q.shape[2] // 64
    blk_cnt = blk_cnt.to(torch.int32).contiguous()
    if blk_cnt.numel() != nb:
        raise RuntimeError("blk_cnt must have one entry per 64-token block")
    if gate is not None:
        gate = gate.contiguous()
        if gate.dtype != q.dtype:
            raise RuntimeError("gate must have the dtype of q")
        _gate_mode(gate, q)
    b = budget_from_topk(nb, topk, budget) if selection is None else 0
    o, qp, qi, kp, ki = _Function.apply(q, k, v, gate, blk_cnt, int(R), b, ROW_NORMS[row_norm], GATE_ACTS[gate_act],
                                        selection, _check_split(split_kv))
    if return_selection:
        return o, Selection(qp, qi, kp, ki)
    return o


@N.device_guard
def vsa_attention(q, k, v, blk_cnt, topk, *, weight=None, backend="auto", selection: Optional[Selection] = None,
                  return_selection=False, split_kv=None):
    """Original VSA attention (64-token blocks): O = O_fine + W * repeat(O_coarse) (reference: echosparse/vsa/ops.py:574-601).

    Router: whole-block means q_c, k_c; S = (q_c @ k_c^T) / sqrt(D) rounded as the original's bf16 / fp16 Torch ops; every
    query block keeps exactly min(topk, NB) kv blocks (score descending, ties to the smaller kv index). `weight` is a full
    [B, H, L, D] direct weight, no activation; None means W = 1. Coarse attention, fine attention, fusion and the backward
    are the kernels shared with VSA2; padded slots are never pooled, output 0 and get zero gradient."""
    if backend not in ("auto", "generic"):
        raise ValueError(f"unknown backend {backend!r}: this build has the one sm_100a backend ('auto' or 'generic')")
    _check_tokens(q, k, v)
    if weight is not None and weight.shape != q.shape:
        raise ValueError(f"weight must be [B, H, L, D] like q, got {tuple(weight.shape)}")
    nb = q.shape[2] // 64
    blk_cnt = blk_cnt.to(torch.int32).contiguous()
    if blk_cnt.numel() != nb:
        raise RuntimeError("blk_cnt must have one entry per 64-token block")
    if weight is not None:
        weight = weight.contiguous()
        if weight.dtype != q.dtype:
            raise RuntimeError("weight must have the dtype of q")
    o, qp, qi, kp, ki = _Function.apply(q, k, v, weight, blk_cnt, _ROWS_POOL_R, int(topk), -1, GATE_ACTS["identity"],
                                        selection, _check_split(split_kv))
    if return_selection:
        return o, Selection(qp, qi, kp, ki)
    return o


class _FineFunction(torch.autograd.Function):
    @staticmethod
    @N.device_guard
    def forward(ctx, q, k, v, blk_cnt, sel, split):
        of, lse = _fine_fwd(q, k, v, sel, blk_cnt, split)
        ctx.split = split
        ctx.save_for_backward(q, k, v, blk_cnt, of, lse, sel.q2k_ptr, sel.q2k_idx, sel.k2q_ptr, sel.k2q_idx)
        ctx.mark_non_differentiable(lse)
        return of, lse

    @staticmethod
    @N.device_guard
    def backward(ctx, dout, dlse):
        q, k, v, blk_cnt, of, lse, qp, qi, kp, ki = ctx.saved_tensors
        B, H, L, D = q.shape
        dout = dout.contiguous()
        oc0 = torch.zeros(B, H, _pad64(L // 64), D, device=q.device, dtype=q.dtype)
        delta_f, _, _, _ = _fuse_bwd(dout, of, oc0, None, blk_cnt, 0)
        dq, dk, dv = _fine_bwd(q, k, v, dout, lse, delta_f, Selection(qp, qi, kp, ki), blk_cnt, None, None, None, ctx.split)
        return dq, dk, dv, None, None, None


@N.device_guard
def fine_block_sparse_attention(q, k, v, blk_cnt, selection: Selection, backend="auto", split_kv=None):
    """Diagnostic fine-only primitive (no coarse branch, no router). Returns (O_f, lse); query blocks without an edge and
    padded rows give O_f = 0 and lse = -inf."""
    _check_tokens(q, k, v)
    return _FineFunction.apply(q, k, v, blk_cnt.to(torch.int32).contiguous(), selection, _check_split(split_kv))
