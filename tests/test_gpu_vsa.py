"""VSA2 kernels through the C ABI against the CPU restatement (oracle/vsa_ref.py) and the golden vectors made by the
reference's own torch oracles (tests/golden/vsa2.npz). Cases follow the reference's tests/test_vsa2.py: frozen masks
(full / diagonal / random with an empty row, a full row and a single edge), ragged block counts, both dtypes and head
dims, gate modes, the routed operator, exact top-k with ties. Tolerances as there (check(): max error relative to the
largest reference value): 2e-2 forward, 4e-2 gradients in bf16; half of that in fp16."""
import os

import numpy as np
import pytest
import torch

from golden_util import vsa_case, vsa_counts, vsa_mask
from oracle import vsa_ref as R

pytestmark = pytest.mark.gpu
DEV = "cuda"
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "vsa2.npz"))


def vsa():
    from self_trainable_or_free_attn_b200 import vsa as V
    return V


def close(name, got, exp, rtol):
    got, exp = got.float().cpu(), exp.float().cpu()
    assert torch.isfinite(got).all(), f"{name}: non-finite values"
    scale = exp.abs().max().clamp(min=1e-6).item()
    err = (got - exp).abs().max().item()
    assert err <= rtol * scale + 1e-5, f"{name}: max err {err:.3e} > {rtol} * {scale:.3e}"


def make(B, H, nb, D, dtype, kind, seed, gate_mode="token"):
    rs = np.random.RandomState(seed)
    cnt = vsa_counts(nb, kind, rs)
    L = nb * 64
    valid = R.token_valid(cnt, L)[None, None, :, None]
    mk = lambda: (torch.from_numpy(rs.standard_normal((B, H, L, D)).astype(np.float32)) * valid).to(dtype)
    q, k, v = mk(), mk(), mk()
    if gate_mode == "token":
        gate = torch.from_numpy((rs.standard_normal((B, H, L)) * 1.5).astype(np.float32)).to(dtype)
    elif gate_mode == "elem":
        gate = torch.from_numpy((rs.standard_normal((B, H, L, D)) * 1.5).astype(np.float32)).to(dtype)
    elif gate_mode == "zero":
        gate = torch.zeros(B, H, L, dtype=dtype)
    else:
        gate = None
    dout = (torch.from_numpy(rs.standard_normal((B, H, L, D)).astype(np.float32)) * valid).to(dtype)
    return q, k, v, gate, cnt, dout


def rand_mask(B, H, nb, seed, kind):
    if kind == "full":
        return torch.ones(B, H, nb, nb, dtype=torch.bool)
    if kind == "diag":
        return torch.eye(nb, dtype=torch.bool).expand(B, H, nb, nb).contiguous()
    rs = np.random.RandomState(seed)
    m = torch.from_numpy(rs.random_sample((B, H, nb, nb)) < 0.3)
    m[:, :, 0] = False
    m[:, :, -1] = True
    if nb > 3:
        m[:, :, 2] = False
        m[:, :, 2, 1] = True
    return m


def to_dev(*ts):
    return [None if t is None else t.to(DEV) for t in ts]


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("mask_kind", ["full", "diag", "random"])
@pytest.mark.parametrize("cnt_kind", ["full", "tail", "mixed"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fine_frozen(D, mask_kind, cnt_kind, dtype):
    V = vsa()
    B, H, nb = 1, 2, 9
    q, k, v, _, cnt, dout = make(B, H, nb, D, dtype, cnt_kind, seed=D + 1)
    mask = rand_mask(B, H, nb, 5, mask_kind)
    sel = V.mask_to_selection(mask.to(DEV))
    qq, kk, vv = (x.to(DEV).clone().requires_grad_(True) for x in (q, k, v))
    of, lse = V.fine_block_sparse_attention(qq, kk, vv, cnt.to(DEV), sel)
    dq, dk, dv = torch.autograd.grad(of, (qq, kk, vv), dout.to(DEV))
    leaves = [x.float().clone().requires_grad_(True) for x in (q, k, v)]
    of_r, lse_r = R.fine_attention(*leaves, cnt, mask)
    g_r = torch.autograd.grad(of_r, leaves, dout.float())
    rt = 2e-2 if dtype == torch.bfloat16 else 1e-2
    close("fine_o", of, of_r, rt)
    fin = torch.isfinite(lse_r)
    assert torch.equal(torch.isfinite(lse.cpu()), fin), "lse sentinel mismatch"
    close("fine_lse", torch.where(fin, lse.cpu(), torch.zeros(())), torch.where(fin, lse_r, torch.zeros(())), 1e-2)
    for name, got, exp in zip(("dq", "dk", "dv"), (dq, dk, dv), g_r):
        close("fine_" + name, got, exp, 2 * rt)
    pad = ~R.token_valid(cnt, nb * 64)
    if pad.any():
        for t in (of, dq, dk, dv):
            assert (t[:, :, pad.to(DEV)] == 0).all(), "padded tokens must be zero"


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("gate_mode", ["token", "elem", "zero", "none"])
@pytest.mark.parametrize("cnt_kind", ["full", "mixed"])
def test_full_frozen(D, gate_mode, cnt_kind):
    V = vsa()
    B, H, nb, dtype = 2, 2, 10, torch.bfloat16
    q, k, v, gate, cnt, dout = make(B, H, nb, D, dtype, cnt_kind, seed=2, gate_mode=gate_mode)
    dout = torch.from_numpy(np.random.RandomState(3).standard_normal(tuple(q.shape)).astype(np.float32)).to(dtype)
    mask = rand_mask(B, H, nb, 11, "random")
    sel = V.mask_to_selection(mask.to(DEV))
    leaves = [x.to(DEV).clone().requires_grad_(True) for x in (q, k, v)] + \
             ([gate.to(DEV).clone().requires_grad_(True)] if gate is not None else [])
    o = V.vsa2_attention(leaves[0], leaves[1], leaves[2], leaves[3] if gate is not None else None, cnt.to(DEV), R=16,
                         selection=sel)
    grads = torch.autograd.grad(o, leaves, dout.to(DEV))
    lf = [x.float().clone().requires_grad_(True) for x in (q, k, v)] + \
         ([gate.float().clone().requires_grad_(True)] if gate is not None else [])
    o_r = R.vsa2_output(lf[0], lf[1], lf[2], lf[3] if gate is not None else None, cnt, mask)
    grads_r = torch.autograd.grad(o_r, lf, dout.float())
    close("full_o", o, o_r, 2e-2)
    for name, g_, gr in zip(["dq", "dk", "dv", "dgate"], grads, grads_r):
        close("full_" + name, g_, gr, 4e-2)
    pad = ~R.token_valid(cnt, nb * 64)
    assert (o[:, :, pad.to(DEV)] == 0).all()


def test_golden_fine_and_full():
    V = vsa()
    T = lambda n: torch.from_numpy(G[n].astype(np.float32))
    q, k, v, _, cnt, dout = vsa_case("fine")
    sel = V.mask_to_selection(vsa_mask("fine", cnt.numel()).to(DEV))
    leaves = [x.to(DEV).clone().requires_grad_(True) for x in (q, k, v)]
    of, lse = V.fine_block_sparse_attention(*leaves, cnt.to(DEV), sel)
    g = torch.autograd.grad(of, leaves, dout.to(DEV))
    close("golden fine_o", of, T("fine_o"), 2e-2)
    fin = torch.isfinite(T("fine_lse"))
    assert torch.equal(torch.isfinite(lse.cpu()), fin)
    assert (lse.cpu()[fin] - T("fine_lse")[fin]).abs().max() < 1e-2
    for n, got in zip(("fine_dq", "fine_dk", "fine_dv"), g):
        close("golden " + n, got, T(n), 4e-2)
    q, k, v, gate, cnt, dout = vsa_case("full")
    sel = V.mask_to_selection(vsa_mask("full", cnt.numel()).to(DEV))
    leaves = [x.to(DEV).clone().requires_grad_(True) for x in (q, k, v, gate)]
    o = V.vsa2_attention(*leaves, cnt.to(DEV), R=16, selection=sel)
    g = torch.autograd.grad(o, leaves, dout.to(DEV))
    close("golden full_o", o, T("full_o"), 2e-2)
    for n, got in zip(("full_dq", "full_dk", "full_dv", "full_dgate"), g):
        close("golden " + n, got, T(n), 4e-2)


@pytest.mark.parametrize("norm", ["paper", "valid_groups"])
def test_golden_route(norm):
    """Router scores within 1e-5 of the reference's; the selection equal to the reference's except at near-ties (scores
    within 1e-6 of the cut), and exactly the exact top-k of this library's own scores."""
    V = vsa()
    from self_trainable_or_free_attn_b200.vsa import ops
    q, k, _, _, cnt, _ = vsa_case("route")
    nb = cnt.numel()
    qd, kd, cd = q.to(DEV), k.to(DEV), cnt.to(DEV)
    qr, kr, _, _, _ = ops.pool_fwd(qd, kd, kd, cd, 16)
    S = ops.router_scores(qr, kr, cd, 16, ops.ROW_NORMS[norm]).cpu()
    S_ref = torch.from_numpy(G[f"route_scores_{norm}"])
    assert (S - S_ref).abs().max() < 1e-5
    sel = V.route(qd, kd, cd, R=16, topk=3, row_norm=norm)
    mask = sel.to_mask(nb).cpu()
    assert torch.equal(mask, R.global_topk_mask(S, nb * 3)), "not the exact top-k of its own scores"
    ref_mask = torch.from_numpy(G[f"route_mask_{norm}"])
    diff = mask ^ ref_mask
    if diff.any():
        cut = S_ref[ref_mask].reshape(1, 2, -1).min(-1).values
        assert ((S_ref - cut[:, :, None, None]).abs()[diff] < 1e-6).all()
    # the inverse lists describe the same mask
    inv = ops.Selection(sel.k2q_ptr, sel.k2q_idx, sel.q2k_ptr, sel.q2k_idx).to_mask(nb).transpose(-1, -2).cpu()
    assert torch.equal(inv, mask)


@pytest.mark.parametrize("nb", [1, 7, 33, 130])
@pytest.mark.parametrize("ties", [False, True])
def test_topk_exact(nb, ties):
    from self_trainable_or_free_attn_b200.vsa import ops
    rs = np.random.RandomState(nb)
    s = torch.from_numpy(rs.random_sample((2, 3, nb, nb)).astype(np.float32))
    if ties:
        s = (s * 4).floor() / 4           # many equal scores, zeros included
    for budget in sorted({0, 1, nb, (nb * nb) // 3, nb * nb, nb * nb + 5}):
        sel = ops.global_topk(s.to(DEV), budget)
        got = sel.to_mask(nb).cpu()
        exp = R.global_topk_mask(s, budget)
        assert torch.equal(got, exp), (nb, ties, budget)
        b = min(budget, nb * nb)
        assert sel.row_counts().sum(-1).eq(b).all()
        for ptr in (sel.q2k_ptr, sel.k2q_ptr):
            p = ptr.cpu().reshape(6, nb + 1)
            assert torch.equal(p[:, 0], torch.arange(6, dtype=torch.int32) * b) and (p[:, -1] - p[:, 0]).eq(b).all()


@pytest.mark.parametrize("R_", [8, 16])
@pytest.mark.parametrize("cnt_kind", ["tail", "mixed"])
def test_full_routed(R_, cnt_kind):
    V = vsa()
    B, H, nb, D, topk = 1, 4, 20, 128, 3
    q, k, v, gate, cnt, dout = make(B, H, nb, D, torch.bfloat16, cnt_kind, seed=7)
    leaves = [x.to(DEV).clone().requires_grad_(True) for x in (q, k, v, gate)]
    o, sel = V.vsa2_attention(*leaves, cnt.to(DEV), R=R_, topk=topk, return_selection=True)
    grads = torch.autograd.grad(o, leaves, dout.to(DEV))
    mask = sel.to_mask(nb).cpu()
    assert mask.reshape(B, H, -1).sum(-1).eq(nb * topk).all()
    # the kernel's own selection, frozen, through the oracle
    lf = [x.float().clone().requires_grad_(True) for x in (q, k, v, gate)]
    o_r = R.vsa2_output(*lf, cnt, mask)
    grads_r = torch.autograd.grad(o_r, lf, dout.float())
    close("routed_o", o, o_r, 2e-2)
    for name, g_, gr in zip(["dq", "dk", "dv", "dgate"], grads, grads_r):
        close("routed_" + name, g_, gr, 4e-2)
    # and the selection against the oracle's router: equal except where scores tie within 1e-6
    S = R.psp_scores(q, k, cnt, R_, round_to=q.dtype)
    ref_mask = R.global_topk_mask(S, nb * topk)
    diff = mask ^ ref_mask
    if diff.any():
        cut = S[ref_mask].reshape(B, H, -1).min(-1).values
        assert ((S - cut[:, :, None, None]).abs()[diff] < 1e-5).all()


def test_zero_edges_and_budget_limits():
    V = vsa()
    B, H, nb, D = 1, 2, 6, 128
    q, k, v, gate, cnt, dout = make(B, H, nb, D, torch.bfloat16, "mixed", seed=9)
    qd, kd, vd, gd, cd = to_dev(q, k, v, gate, cnt)
    # no fine edge at all: the output is the gated coarse branch
    sel = V.mask_to_selection(torch.zeros(B, H, nb, nb, dtype=torch.bool, device=DEV))
    o = V.vsa2_attention(qd, kd, vd, gd, cd, selection=sel)
    o_r = R.vsa2_output(q.float(), k.float(), v.float(), gate.float(), cnt, torch.zeros(B, H, nb, nb, dtype=torch.bool))
    close("coarse only", o, o_r, 2e-2)
    # budget 0 through the router, and a budget past NB^2 clamps to the dense mask
    o0, s0 = V.vsa2_attention(qd, kd, vd, gd, cd, budget=0, return_selection=True)
    assert s0.row_counts().sum() == 0
    close("budget 0", o0, o_r, 2e-2)
    o1, s1 = V.vsa2_attention(qd, kd, vd, gd, cd, budget=10 ** 9, return_selection=True)
    assert s1.to_mask(nb).all()
    o_d = R.vsa2_output(q.float(), k.float(), v.float(), gate.float(), cnt, torch.ones(B, H, nb, nb, dtype=torch.bool))
    close("dense", o1, o_d, 2e-2)


def test_deterministic_rerun_stream_and_second_backward():
    V = vsa()
    B, H, nb, D = 1, 3, 12, 128
    q, k, v, gate, cnt, dout = make(B, H, nb, D, torch.bfloat16, "tail", seed=21)
    outs = []
    for rep in range(2):
        leaves = [x.to(DEV).clone().requires_grad_(True) for x in (q, k, v, gate)]
        o = V.vsa2_attention(*leaves, cnt.to(DEV), R=16, topk=4)
        outs.append([o] + list(torch.autograd.grad(o, leaves, dout.to(DEV))))
    for a, b in zip(*outs):
        assert torch.equal(a, b), "two runs differ"
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        leaves = [x.to(DEV).clone().requires_grad_(True) for x in (q, k, v, gate)]
        o = V.vsa2_attention(*leaves, cnt.to(DEV), R=16, topk=4)
        g = torch.autograd.grad(o, leaves, dout.to(DEV), retain_graph=True)
        s.synchronize()
    assert torch.equal(o, outs[0][0]) and torch.equal(g[0], outs[0][1])
    with pytest.raises(RuntimeError, match="frees its intermediates"):
        torch.autograd.grad(o, leaves, dout.to(DEV))


def test_rejected_inputs():
    V = vsa()
    q, k, v, gate, cnt, _ = make(1, 2, 2, 128, torch.bfloat16, "full", seed=1)
    qd, kd, vd, gd, cd = to_dev(q, k, v, gate, cnt)
    with pytest.raises(RuntimeError, match="no CPU path"):
        V.vsa2_attention(q, k, v, gate, cnt, topk=1)
    with pytest.raises(ValueError, match="contiguous"):
        V.vsa2_attention(qd.transpose(1, 2).contiguous().transpose(1, 2), kd, vd, gd, cd, topk=1)
    with pytest.raises(ValueError, match="topk"):
        V.vsa2_attention(qd, kd, vd, gd, cd)
    with pytest.raises(RuntimeError):
        V.vsa2_attention(qd.float(), kd.float(), vd.float(), None, cd, topk=1)
