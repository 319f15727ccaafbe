"""VSA2 with 64 / RM / 1 representative tiers: autograd wiring around the native kernels.

Mirrors the public entry points of the reference's `experiments/vsa2_representative/vsa2_rep/ops.py`: `RepTiers`
(:50-84), `TierSelection` (:87-127), `route_tiers` (:137-146) and the fine operator `rep_fine_attention`. VSA2 routes
every query block to the top-k kv blocks of its PSP router and drops the rest; here the dropped blocks are kept at reduced
resolution: the most important `frac_full` of the (query block, kv block) pairs keep all 64 tokens, the next `frac_mid`
keep `mid_reps` group means per block, every remaining pair keeps the block mean. A representative standing for c tokens
enters the single softmax as one column with + log2(c) on its logit. Routing is VSA2's own router and exact global top-k,
run at two budgets over one score matrix.
"""
import math
from dataclasses import dataclass
from typing import Tuple

import torch

from .. import _native as N
from . import ops

PHASE_A, PHASE_B, PHASE_C = 1, 2, 4
PHASE_ALL = PHASE_A | PHASE_B | PHASE_C
MID_REPS_OK = (2, 4, 8, 16)


@dataclass(frozen=True)
class RepTiers:
    """Three-tier KV budget, as fractions of all NB * NB (query block, kv block) pairs."""
    frac_full: float = 0.10
    frac_mid: float = 0.20
    mid_reps: int = 4

    def __post_init__(self):
        ops._want_nonneg_real("RepTiers", "frac_full", self.frac_full)
        ops._want_nonneg_real("RepTiers", "frac_mid", self.frac_mid)
        both = self.frac_full + self.frac_mid
        if both > 1.0 + 1e-9:
            raise ValueError(f"RepTiers: tiers A and B together take {both} of the pairs; at most 1")
        if self.mid_reps not in MID_REPS_OK:
            raise ValueError(f"RepTiers.mid_reps = {self.mid_reps!r}: a block splits into one of {MID_REPS_OK} groups")

    def budgets(self, nb) -> Tuple[int, int]:
        """Pairs per (b, h) in tier A, and in tiers A and B together; never more than NB * NB, the second never less than
        the first (reference: vsa2_rep/ops.py:76-81)."""
        pairs = nb * nb
        full = min(pairs, int(round(self.frac_full * pairs)))
        full_or_mid = int(round((self.frac_full + self.frac_mid) * pairs))
        return full, min(pairs, max(full, full_or_mid))


@dataclass
class TierSelection:
    """Frozen three-tier assignment: tier A as CSR lists, tiers B and C from the two bitmaps (B = bits_ab & ~bits_a,
    C = ~bits_ab), [B, H, NB, ceil(NB / 32)] int32."""
    q2k_ptr: torch.Tensor
    q2k_idx: torch.Tensor
    k2q_ptr: torch.Tensor
    k2q_idx: torch.Tensor
    bits_a: torch.Tensor
    bits_ab: torch.Tensor

    def tier_masks(self, nb):
        a, ab = unpack_bits(self.bits_a, nb), unpack_bits(self.bits_ab, nb)
        return a, ab & ~a, ~ab


def unpack_bits(bits, nb):
    bit = torch.arange(32, device=bits.device, dtype=torch.int32)
    x = (bits.unsqueeze(-1) >> bit) & 1
    return x.reshape(*bits.shape[:-1], bits.shape[-1] * 32)[..., :nb].to(torch.bool)


def pack_bits(mask):
    """Dense bool [B, H, NB, NB] -> the kernels' [B, H, NB, ceil(NB / 32)] int32 bitmap."""
    B, H, nb, _ = mask.shape
    w = (nb + 31) // 32
    m = torch.zeros(B, H, nb, w * 32, dtype=torch.int64, device=mask.device)
    m[..., :nb] = mask
    packed = (m.reshape(B, H, nb, w, 32) << torch.arange(32, device=mask.device, dtype=torch.int64)).sum(-1)
    return (packed - ((packed >> 31) & 1) * (1 << 32)).to(torch.int32).contiguous()


def selection_from_masks(tier_a, tier_ab):
    """Hand-made tier assignment (tests): bool masks [B, H, NB, NB] of tier A and of tier A or B."""
    s = ops.mask_to_selection(tier_a)
    return TierSelection(s.q2k_ptr, s.q2k_idx, s.k2q_ptr, s.k2q_idx, pack_bits(tier_a), pack_bits(tier_a | tier_ab))


def _topk_with_bits(scores, budget):
    B, H, nb, _ = scores.shape
    budget = max(0, min(int(budget), nb * nb))
    lib = N.load()
    i32 = dict(device=scores.device, dtype=torch.int32)
    qp, kp = torch.empty(B, H, nb + 1, **i32), torch.empty(B, H, nb + 1, **i32)
    qi, ki = torch.empty(max(1, B * H * budget), **i32), torch.empty(max(1, B * H * budget), **i32)
    ws = torch.empty(int(lib.es_vsa_topk_workspace_bytes(B * H, nb)), device=scores.device, dtype=torch.uint8)
    N.check(lib.es_vsa_global_topk(N.ptr(scores), nb, 0, B * H, budget, N.ptr(qp), N.ptr(qi), N.ptr(kp), N.ptr(ki),
                                   N.ptr(ws), N.stream_ptr()), "es_vsa_global_topk")
    off = int(lib.es_vsa_topk_bits_offset(B * H, nb))
    w = (nb + 31) // 32
    bits = ws[off: off + B * H * nb * w * 4].view(torch.int32).reshape(B, H, nb, w).clone()
    return ops.Selection(qp, qi, kp, ki), bits


@N.device_guard
def route_tiers(q, k, blk_cnt, tiers: RepTiers = RepTiers(), *, R=16, row_norm="paper"):
    """VSA2's PSP router + exact global top-k at two budgets (stop-gradient)."""
    ops._check_tokens(q, k, k)
    blk_cnt = blk_cnt.to(torch.int32).contiguous()
    nb = q.shape[2] // 64
    qr, kr, _, _, _ = ops.pool_fwd(q, k, k, blk_cnt, R)
    scores = ops.router_scores(qr, kr, blk_cnt, R, ops.ROW_NORMS[row_norm]).contiguous()
    ba, bab = tiers.budgets(nb)
    sel_a, bits_a = _topk_with_bits(scores, ba)
    _, bits_ab = _topk_with_bits(scores, bab)
    return TierSelection(sel_a.q2k_ptr, sel_a.q2k_idx, sel_a.k2q_ptr, sel_a.k2q_idx, bits_a, bits_ab)


@N.device_guard
def rep_build(k, v, blk_cnt, mid_reps):
    """Representative tables (k_mid, v_mid [B,H,mid_stride,D], k_tail, v_tail [B,H,tail_stride,D]): the group means of the
    64 / mid_reps-token groups and the block means of K and V over their valid tokens, rounded to the token dtype."""
    B, H, L, D = k.shape
    nb = L // 64
    mid_stride, tail_stride = ops._pad64(nb * mid_reps), ops._pad64(nb)
    mk = lambda n: torch.empty(B, H, n, D, device=k.device, dtype=k.dtype)
    k_mid, v_mid, k_tail, v_tail = mk(mid_stride), mk(mid_stride), mk(tail_stride), mk(tail_stride)
    N.check(N.load().es_vsa_pool(None, N.ptr(k), N.ptr(v), None, N.ptr(k_mid), N.ptr(v_mid), None, N.ptr(k_tail),
                                 N.ptr(v_tail), N.ptr(blk_cnt), B * H, L, D, 64 // mid_reps, mid_stride, tail_stride,
                                 ops._DTYPES[k.dtype], N.stream_ptr()), "es_vsa_pool")
    return k_mid, v_mid, k_tail, v_tail


def _tier_fwd(q, k, v, tab, sel, blk_cnt, mid_reps, phases):
    B, H, L, D = q.shape
    o = torch.empty_like(q)
    lse = torch.empty(B, H, L, device=q.device, dtype=torch.float32)
    k_mid, v_mid, k_tail, v_tail = tab
    N.check(N.load().es_vsa_tier_attn_fwd(
        N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(k_mid), N.ptr(v_mid), N.ptr(k_tail), N.ptr(v_tail), N.ptr(o), N.ptr(lse),
        N.ptr(sel.q2k_ptr), N.ptr(sel.q2k_idx), N.ptr(sel.bits_a), N.ptr(sel.bits_ab), N.ptr(blk_cnt), B * H, L, D, mid_reps,
        k_mid.shape[2], k_tail.shape[2], phases, ops._DTYPES[q.dtype], N.stream_ptr()), "es_vsa_tier_attn_fwd")
    return o, lse


def _tier_bwd(q, k, v, tab, dout, lse, delta, sel, blk_cnt, mid_reps, phases, add_dq=None, add_dk=None, add_dv=None):
    """(dq, dk, dv) of the three-tier fine branch; add_* are optional per-block gradients (the coarse branch)."""
    B, H, L, D = q.shape
    lib, dt, st = N.load(), ops._DTYPES[q.dtype], N.stream_ptr()
    k_mid, v_mid, k_tail, v_tail = tab
    f32 = dict(device=q.device, dtype=torch.float32)
    add_nb = add_dq.shape[2] if add_dq is not None else 0
    dq = torch.empty_like(q)
    N.check(lib.es_vsa_tier_attn_bwd_q(
        N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(k_mid), N.ptr(v_mid), N.ptr(k_tail), N.ptr(v_tail), N.ptr(dout), N.ptr(lse),
        N.ptr(delta), N.ptr(dq), N.ptr(add_dq), add_nb, N.ptr(sel.q2k_ptr), N.ptr(sel.q2k_idx), N.ptr(sel.bits_a),
        N.ptr(sel.bits_ab), N.ptr(blk_cnt), B * H, L, D, mid_reps, k_mid.shape[2], k_tail.shape[2], phases, dt, st),
        "es_vsa_tier_attn_bwd_q")
    dk_a = dv_a = None
    if phases & PHASE_A:
        dk_a, dv_a = ops._bwd_kv(q, k, v, dout, lse, delta, sel.k2q_ptr, sel.k2q_idx, blk_cnt, f32=True)
    dk_mid, dv_mid = torch.zeros(k_mid.shape, **f32), torch.zeros(k_mid.shape, **f32)
    dk_tail, dv_tail = torch.zeros(k_tail.shape, **f32), torch.zeros(k_tail.shape, **f32)
    N.check(lib.es_vsa_tier_rep_bwd(
        N.ptr(q), N.ptr(k_mid), N.ptr(v_mid), N.ptr(k_tail), N.ptr(v_tail), N.ptr(dout), N.ptr(lse), N.ptr(delta),
        N.ptr(dk_mid), N.ptr(dv_mid), N.ptr(dk_tail), N.ptr(dv_tail), N.ptr(sel.bits_a), N.ptr(sel.bits_ab), N.ptr(blk_cnt),
        B * H, L, D, mid_reps, k_mid.shape[2], k_tail.shape[2], phases, dt, st), "es_vsa_tier_rep_bwd")
    outs = []
    for tok, mid, tail, add in ((dk_a, dk_mid, dk_tail, add_dk), (dv_a, dv_mid, dv_tail, add_dv)):
        out = torch.empty_like(q)
        N.check(lib.es_vsa_tier_unpool(N.ptr(tok), N.ptr(mid), N.ptr(tail), N.ptr(add), add.shape[2] if add is not None else 0,
                                       N.ptr(out), N.ptr(blk_cnt), B * H, L, D, mid_reps, mid.shape[2], tail.shape[2], dt, st),
                "es_vsa_tier_unpool")
        outs.append(out)
    return dq, outs[0], outs[1]


class _TierFineFunction(torch.autograd.Function):
    @staticmethod
    @N.device_guard
    def forward(ctx, q, k, v, blk_cnt, sel, mid_reps, phases):
        tab = rep_build(k, v, blk_cnt, mid_reps)
        of, lse = _tier_fwd(q, k, v, tab, sel, blk_cnt, mid_reps, phases)
        ctx.save_for_backward(q, k, v, blk_cnt, of, lse, *tab)
        ctx.sel, ctx.mid_reps, ctx.phases = sel, mid_reps, phases
        ctx.mark_non_differentiable(lse)
        return of, lse

    @staticmethod
    @N.device_guard
    def backward(ctx, dout, dlse):
        q, k, v, blk_cnt, of, lse, *tab = ctx.saved_tensors
        B, H, L, D = q.shape
        dout = dout.contiguous()
        oc0 = torch.zeros(B, H, ops._pad64(L // 64), D, device=q.device, dtype=q.dtype)
        delta, _, _, _ = ops._fuse_bwd(dout, of, oc0, None, blk_cnt, 0)
        dq, dk, dv = _tier_bwd(q, k, v, tab, dout, lse, delta, ctx.sel, blk_cnt, ctx.mid_reps, ctx.phases)
        return dq, dk, dv, None, None, None, None


@N.device_guard
def rep_fine_attention(q, k, v, blk_cnt, selection: TierSelection, mid_reps=4, phases=PHASE_ALL):
    """The three-tier fine branch alone (no coarse branch, no router). Returns (O_f, lse natural); padded rows and rows
    without a visible column give 0 and -inf. Gradients flow to the tokens through all three tiers: a representative's
    gradient is spread over the tokens it averaged (1 / count each)."""
    ops._check_tokens(q, k, v)
    if mid_reps not in MID_REPS_OK:
        raise ValueError(f"mid_reps must be one of {MID_REPS_OK}, got {mid_reps!r}")
    return _TierFineFunction.apply(q, k, v, blk_cnt.to(torch.int32).contiguous(), selection, int(mid_reps), int(phases))
