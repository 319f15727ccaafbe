"""Original VSA (whole-block router, exactly K kv blocks per query block, direct weight) on the GPU against the oracle and
the golden vectors of the reference's own oracle. Cases follow the reference's tests/test_vsa.py: exact per-row top-K with
ties and signed zeros, block scores in the original's rounding, frozen and routed operator, weight forms."""
import os

import numpy as np
import pytest
import torch

from golden_util import vsa_case, vsa_mask
from oracle import vsa_ref as R
from test_gpu_vsa import close, make, rand_mask

pytestmark = pytest.mark.gpu
DEV = "cuda"
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "vsa2.npz"))


def vsa():
    from self_trainable_or_free_attn_b200 import vsa as V
    return V


@pytest.mark.parametrize("nb", [1, 7, 33, 130, 300])
@pytest.mark.parametrize("ties", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_row_topk_exact(nb, ties, dtype):
    from self_trainable_or_free_attn_b200.vsa import ops
    rs = np.random.RandomState(nb)
    s = torch.from_numpy(rs.standard_normal((2, 2, nb, nb)).astype(np.float32))
    if ties:
        s = (s * 2).round() / 2
        s[..., ::3] = 0.0
        s[..., 1::6] = -0.0
    s = s.to(dtype)
    for topk in sorted({0, 1, 3, nb // 2, nb, nb + 4}):
        sel = ops.row_topk(s.to(DEV), topk)
        K = min(topk, nb)
        assert torch.equal(sel.to_mask(nb).cpu(), R.row_topk_mask(s, topk)), (nb, ties, topk)
        assert sel.row_counts().eq(K).all()
        inv = ops.Selection(sel.k2q_ptr, sel.k2q_idx, sel.q2k_ptr, sel.q2k_idx).to_mask(nb).transpose(-1, -2)
        assert torch.equal(inv.cpu(), sel.to_mask(nb).cpu())
        if K:
            idx = sel.q2k_idx[: 4 * nb * K].reshape(4 * nb, K).cpu()
            assert (idx[:, 1:] > idx[:, :-1]).all(), "lists ascend"


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_block_scores_and_route_rows(D, dtype):
    V = vsa()
    from self_trainable_or_free_attn_b200.vsa import ops
    B, H, nb = 1, 3, 20
    q, k, v, _, cnt, _ = make(B, H, nb, D, dtype, "mixed", seed=D)
    qd, kd, cd = q.to(DEV), k.to(DEV), cnt.to(DEV)
    _, _, qc, kc, _ = ops.pool_fwd(qd, kd, kd, cd, 32)
    S = ops.block_scores(qc, kc, nb).cpu()
    S_ref = R.vsa_block_scores(q, k, cnt)
    # the block means are rounded to the element type on both sides, from sums taken in different orders: a mean may
    # differ by one rounding step, and so may a score, by a step of the largest scores
    eps = 2 ** -7 if dtype == torch.bfloat16 else 2 ** -10
    assert (S.float() - S_ref.float()).abs().max() <= 2 * eps * S_ref.float().abs().max()
    assert (S == S_ref).float().mean() > 0.9
    sel = V.route_rows(qd, kd, cd, 4)
    assert torch.equal(sel.to_mask(nb).cpu(), R.row_topk_mask(S, 4)), "exactly the per-row top-K of its own scores"


def test_golden_scores_and_operator():
    V = vsa()
    from self_trainable_or_free_attn_b200.vsa import ops
    T = lambda n: torch.from_numpy(G[n].astype(np.float32))
    q, k, _, _, cnt, _ = vsa_case("route")
    _, _, qc, kc, _ = ops.pool_fwd(q.to(DEV), k.to(DEV), k.to(DEV), cnt.to(DEV), 32)
    S = ops.block_scores(qc, kc, cnt.numel()).cpu().float()
    assert (S - T("rows_scores")).abs().max() <= 2 ** -6 * T("rows_scores").abs().max()
    assert (S == T("rows_scores")).float().mean() > 0.9
    q, k, v, gate, cnt, dout = vsa_case("full")
    mask = vsa_mask("full", cnt.numel())
    w = torch.tanh(gate.float())[..., None].expand(-1, -1, -1, q.shape[-1]).to(q.dtype).contiguous()
    leaves = [x.to(DEV).clone().requires_grad_(True) for x in (q, k, v, w)]
    o = V.vsa_attention(*leaves[:3], cnt.to(DEV), 3, weight=leaves[3], selection=V.mask_to_selection(mask.to(DEV)))
    g = torch.autograd.grad(o, leaves, dout.to(DEV))
    close("golden vsa_o", o, T("vsa_o"), 2e-2)
    for n, got in zip(("vsa_dq", "vsa_dk", "vsa_dv", "vsa_dw"), g):
        close("golden " + n, got, T(n), 4e-2)


@pytest.mark.parametrize("weight", ["full", "none"])
@pytest.mark.parametrize("cnt_kind", ["full", "mixed"])
def test_vsa_frozen_and_routed(weight, cnt_kind):
    V = vsa()
    B, H, nb, D = 2, 2, 10, 128
    q, k, v, w, cnt, dout = make(B, H, nb, D, torch.bfloat16, cnt_kind, seed=5, gate_mode="elem" if weight == "full" else "none")
    dout = torch.from_numpy(np.random.RandomState(6).standard_normal(tuple(q.shape)).astype(np.float32)).to(torch.bfloat16)
    for routed in (False, True):
        leaves = [x.to(DEV).clone().requires_grad_(True) for x in (q, k, v)] + ([w.to(DEV).clone().requires_grad_(True)] if w is not None else [])
        kw = {} if routed else dict(selection=V.mask_to_selection(rand_mask(B, H, nb, 3, "random").to(DEV)))
        o, sel = V.vsa_attention(leaves[0], leaves[1], leaves[2], cnt.to(DEV), 3, weight=leaves[3] if w is not None else None,
                                 return_selection=True, **kw)
        grads = torch.autograd.grad(o, leaves, dout.to(DEV))
        mask = sel.to_mask(nb).cpu()
        if routed:
            assert mask.sum(-1).eq(3).all()
        lf = [x.float().clone().requires_grad_(True) for x in (q, k, v)] + ([w.float().clone().requires_grad_(True)] if w is not None else [])
        o_r = R.vsa_output(lf[0], lf[1], lf[2], lf[3] if w is not None else None, cnt, mask)
        close("o", o, o_r, 2e-2)
        for name, g_, gr in zip(["dq", "dk", "dv", "dw"], grads, torch.autograd.grad(o_r, lf, dout.float())):
            close(name, g_, gr, 4e-2)
    with pytest.raises(ValueError, match="weight"):
        V.vsa_attention(q.to(DEV), k.to(DEV), v.to(DEV), cnt.to(DEV), 3, weight=q.to(DEV)[..., :64].contiguous())
