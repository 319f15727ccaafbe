"""The oracle (oracle/echosparse_ref.py) against the outputs of the reference's own kernels stored in
tests/golden/echosparse_step.npz (made by tests/golden/make_golden.py). Integer and bit results must be identical;
floating-point results within the stated tolerances. Runs on CPU."""
import numpy as np
import pytest
import torch

from oracle import echosparse_ref as R
from golden_util import MG, T, bf16_from_bits, qkv, rel_l2

L, H = MG.L, MG.H
NQ, NB = R.cdiv(L, 128), R.cdiv(L, 64)
ALL_COUNTS = torch.full((NQ, H), NB, dtype=torch.int32)
ALL_BLOCKS = torch.arange(NB, dtype=torch.int32).expand(NQ, H, NB).contiguous()
ROWS = slice(None, None, 9)          # the rows of the outputs that the fixture stores


def test_budget_and_words(golden):
    assert R.budget(MG.DENSITY, NB) == (int(golden["top"]), int(golden["refined"]))
    assert R.plan_words(NB) == int(golden["words"])


def test_full_step(golden):
    q, k, v = qkv(1)
    mass = torch.zeros(H, NQ, NB)
    out, lse, flags = R.fixed_offset_attention(q, k, v, ALL_COUNTS, ALL_BLOCKS, T(golden["offset0"]), mass=mass)
    assert rel_l2(out[ROWS], bf16_from_bits(golden["full_out"])) < 2e-3
    assert (lse[:L] - T(golden["full_lse"])[:L]).abs().max() < 1e-4
    assert torch.equal(flags, T(golden["full_flags"]))
    assert rel_l2(mass, T(golden["full_mass"])) < 1e-5
    lse2, se, ss = R.full_step_scales(T(golden["offset0"]), T(golden["full_lse"]), L)
    assert torch.equal(lse2, T(golden["full_lse_reset"]))
    assert rel_l2(se, T(golden["full_scale_exact"])) < 1e-6 and torch.equal(ss, T(golden["full_scale_skip"]))


def _check_selection(got, golden, prefix, blocks_key=None):
    keep, counts, blocks, bits, refine = got
    assert torch.equal(keep, T(golden[f"{prefix}_keep"]))
    assert torch.equal(counts, T(golden[f"{prefix}_counts"]))
    assert torch.equal(bits, T(golden[f"{prefix}_bits"]))
    assert torch.equal(refine, T(golden[f"{prefix}_refine"]))
    if blocks_key:
        ref = T(golden[blocks_key])
        for t in range(NQ):
            for h in range(H):
                n = int(counts[t, h])
                assert torch.equal(blocks[t, h, :n], ref[t, h, :n])


def test_selection_bit_exact(golden):
    ones = torch.ones(H, NQ, NB, dtype=torch.uint8)
    got = R.select_blocks(T(golden["full_mass"]), ones, T(golden["full_scale_exact"]), T(golden["full_scale_skip"]),
                          T(golden["full_flags"]), int(golden["top"]), int(golden["refined"]), L, int(golden["rw"]))
    _check_selection(got, golden, "sel", "sel_blocks")
    got = R.select_blocks(T(golden["est_mass"]), T(golden["sel_keep"]), T(golden["est_scale_exact"]),
                          T(golden["est_scale_skip"]), T(golden["sparse_flags"]), int(golden["top"]),
                          int(golden["refined"]), L, int(golden["rw"]))
    _check_selection(got, golden, "sel2")


@pytest.mark.parametrize("case", ["c1", "c2", "c3", "c4"])
def test_selection_corner_cases(golden, case):
    """NaN / inf masses, ties, a sink, fell-back tiles, r = 0 and k = nb: the synthetic map of make_golden.py."""
    rng = np.random.Generator(np.random.PCG64(7))
    cm = rng.random((H, NQ, NB), dtype=np.float32)
    cm[:, :, 5] = cm[:, :, 9]
    cm[0, 3, 11] = np.nan
    cm[1, 4, 12] = np.inf
    cm[:, 6, :] = 0.25
    keep_prev = T((rng.random((H, NQ, NB)) < 0.2).astype(np.uint8))
    se = T(rng.random((H, NQ), dtype=np.float32) + 0.5)
    ss = T(rng.random((H, NQ), dtype=np.float32) + 0.5)
    flags = T((rng.random((NQ, H)) < 0.2).astype(np.int32))
    k, r, sink, w = (int(x) for x in golden[f"{case}_args"])
    got = R.select_blocks(T(cm), keep_prev, se, ss, flags, k, r, L, w, sink=sink)
    _check_selection(got, golden, case)


def test_plans_bit_exact(golden):
    keep = T(golden["sel_keep"])
    exact = R.pack_plan(keep)
    assert torch.equal(exact, T(golden["plan_exact"]))
    k2, counts, blocks, refine, rc, means, mc = R.rebuild_plan(exact, T(golden["sel_bits"]), NB, int(golden["rw"]))
    assert torch.equal(k2, keep) and torch.equal(counts, T(golden["sel_counts"]))
    assert torch.equal(refine, T(golden["sel_refine"])) and torch.equal(rc, T(golden["plan_refine_counts"]))
    assert torch.equal(mc, T(golden["plan_mean_counts"]))
    gm = T(golden["plan_means"])
    for t in range(NQ):
        for h in range(H):
            assert torch.equal(means[t, h, :int(mc[t, h])], gm[t, h, :int(mc[t, h])])


def test_block_means(golden):
    _, k, v = qkv(2)
    km, vm = R.block_means(k, v)
    # a mean may land one bf16 step away where the float32 sums differ in their last bit
    assert (km.float() - bf16_from_bits(golden["k_mean"]).float()).abs().max() < 2e-2
    assert rel_l2(km, bf16_from_bits(golden["k_mean"])) < 1e-3 and rel_l2(vm, bf16_from_bits(golden["v_mean"])) < 1e-3


def test_metric_and_probes(golden):
    q, _, _ = qkv(2)
    g, metric, probes = R.query_metric(q)
    g_raw = g - 1e-3 * g.diagonal(dim1=-2, dim2=-1).mean(-1)[:, None, None] * torch.eye(128)
    assert rel_l2(g_raw, T(golden["gram"])) < 1e-4
    assert rel_l2(metric, bf16_from_bits(golden["metric"])) < 5e-3
    assert rel_l2(probes, bf16_from_bits(golden["probes"])) < 1e-3


def test_representatives(golden):
    """With the reference's own metric and probes the clustering must reproduce the reference's cluster sizes on
    (almost) every block: labels are decided by float32 comparisons, so a near-tie can move a token."""
    q, k, v = qkv(2)
    kr, vr, lc, _ = R.representatives(q, k, v, int(golden["iters"]), bf16_from_bits(golden["metric"]),
                                      bf16_from_bits(golden["probes"]))
    glc = T(golden["log_counts"])
    same = ((lc == glc) | ((lc - glc).abs() < 1e-6)).view(H, NB + 1, 4).all(-1)
    assert same.float().mean() > 0.97
    gk, gv = bf16_from_bits(golden["k_rep"]).view(H, NB + 1, 4, 128), bf16_from_bits(golden["v_rep"]).view(H, NB + 1, 4, 128)
    assert rel_l2(kr.view(H, NB + 1, 4, 128)[same], gk[same]) < 2e-3
    assert rel_l2(vr.view(H, NB + 1, 4, 128)[same], gv[same]) < 2e-3
    # invariants the reference tests (tests/test_sm120.py:65-83): sizes add up to the block, size x mean = block sum
    cnt = torch.exp2(lc[:, :NB * 4]).view(H, NB, 4)
    assert torch.equal(cnt.sum(-1).round().long(), R.block_len(L, NB).long().expand(H, NB))


def test_sparse_step(golden):
    q, k, v = qkv(2)
    mass = torch.zeros(H, NQ, NB)
    out, lse, flags = R.fixed_offset_attention(
        q, k, v, T(golden["sel_counts"]), T(golden["sel_blocks"]), T(golden["full_lse_reset"]), mass=mass,
        k_mean=bf16_from_bits(golden["k_mean"]), v_mean=bf16_from_bits(golden["v_mean"]), skip_bits=T(golden["sel_bits"]),
        refine=T(golden["sel_refine"]), k_rep=bf16_from_bits(golden["k_rep"]), v_rep=bf16_from_bits(golden["v_rep"]),
        log_counts=T(golden["log_counts"]))
    assert rel_l2(out[ROWS], bf16_from_bits(golden["sparse_out"])) < 2e-3
    assert (lse[:L] - T(golden["sparse_lse"])[:L]).abs().max() < 1e-4
    assert torch.equal(flags, T(golden["sparse_flags"]))
    assert rel_l2(mass, T(golden["sparse_mass"])) < 1e-5


def test_estimates(golden):
    q, _, _ = qkv(2)
    mass, se, ss = R.estimate_skipped(q, bf16_from_bits(golden["k_mean"]), T(golden["sel_keep"]),
                                      T(golden["full_lse_reset"]), T(golden["sparse_lse"]), T(golden["sparse_mass"]))
    assert rel_l2(mass, T(golden["est_mass"])) < 1e-5
    assert rel_l2(se, T(golden["est_scale_exact"])) < 1e-5 and rel_l2(ss, T(golden["est_scale_skip"])) < 1e-4


def test_fallback(golden):
    q, k, v = qkv(2)
    assert int(golden["fb_flags"].sum()) == NQ * H           # the +200 offset flags every tile
    flags = T(golden["fb_flags"])
    out = torch.zeros(L, H, 128, dtype=torch.bfloat16)
    lse = torch.full((NQ * 128, H), 1e30)
    R.exact_fallback(q, k, v, out, T(golden["sel_counts"]), T(golden["sel_blocks"]), lse, flags)
    assert rel_l2(out[ROWS], bf16_from_bits(golden["fb_exact_out"])) < 2e-3
    assert (lse[:L] - T(golden["fb_exact_lse"])[:L]).abs().max() < 1e-4
    R.compensate_fallback(q, bf16_from_bits(golden["k_mean"]), bf16_from_bits(golden["v_mean"]), T(golden["sel_keep"]),
                          lse, out, flags)
    assert rel_l2(out[ROWS], bf16_from_bits(golden["fb_comp_out"])) < 2e-3
    assert (lse[:L] - T(golden["fb_comp_lse"])[:L]).abs().max() < 1e-4
