"""Parity of every CUDA kernel, called through the C ABI, with (a) the golden outputs of the reference's own kernels and
(b) the oracle on seeded inputs at other shapes (empty / ragged tails, nb < 32, odd list lengths).

Tolerances (bf16 path): outputs relative L2 <= 1e-2 and max-abs <= 3e-2; LSE and other float32 results <= 1e-4;
selections, lists and bit masks identical."""
import pytest
import torch

from oracle import echosparse_ref as R
from golden_util import MG, T, bf16_from_bits, qkv, rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def K():
    from self_trainable_or_free_attn_b200 import _native, backends
    mod = backends.kernels(backends.resolve("auto", DEV))
    yield mod
    assert _native.device_status() == 0, "a bounded wait inside a kernel gave up"


def _all_lists(L, H):
    nq, nb = R.cdiv(L, 128), R.cdiv(L, 64)
    return (torch.full((nq, H), nb, device=DEV, dtype=torch.int32),
            torch.arange(nb, device=DEV, dtype=torch.int32).expand(nq, H, nb).contiguous())


def _outputs(L, H, like):
    nq = R.cdiv(L, 128)
    return (torch.full_like(like, 7.0), torch.zeros(nq * 128, H, device=DEV),
            torch.full((nq, H), -1, device=DEV, dtype=torch.int32))


def _close_out(got, want):
    assert rel_l2(got, want) <= 1e-2
    assert (got.float() - want.float()).abs().max() <= 3e-2


# ------------------------------------------------------------------------------------------------ golden (reference)
L, H = MG.L, MG.H
NQ, NB = R.cdiv(L, 128), R.cdiv(L, 64)
ROWS = slice(None, None, 9)


def test_full_step_matches_reference(K, golden):
    q, k, v = qkv(1, DEV)
    counts, blocks = _all_lists(L, H)
    out, lse, flags = _outputs(L, H, q)
    mass = torch.zeros(H, NQ, NB, device=DEV)
    K.block_attention(q, k, v, out, counts, blocks, T(golden["offset0"], DEV), lse, flags, mass=mass)
    _close_out(out[ROWS], bf16_from_bits(golden["full_out"], DEV))
    assert (lse[:L] - T(golden["full_lse"], DEV)[:L]).abs().max() <= 1e-4
    assert torch.equal(flags, T(golden["full_flags"], DEV))
    assert rel_l2(mass, T(golden["full_mass"], DEV)) <= 1e-4
    se, ss = torch.empty(H, NQ, device=DEV), torch.empty(H, NQ, device=DEV)
    lse_ref = T(golden["full_lse"], DEV).clone()
    K.full_step_scales(T(golden["offset0"], DEV), lse_ref, se, ss, L)
    assert torch.equal(lse_ref, T(golden["full_lse_reset"], DEV))
    assert rel_l2(se, T(golden["full_scale_exact"], DEV)) <= 1e-5 and torch.equal(ss, T(golden["full_scale_skip"], DEV))


def _select(K, mass, keep_prev, se, ss, flags, k, r, L, H, rw, sink=1 << 30):
    nq, nb = R.cdiv(L, 128), R.cdiv(L, 64)
    keep = torch.full((H, nq, nb), 9, device=DEV, dtype=torch.uint8)
    counts = torch.full((nq, H), -1, device=DEV, dtype=torch.int32)
    blocks = torch.zeros(nq, H, nb, device=DEV, dtype=torch.int32)
    bits = torch.full((H, nq, R.plan_words(nb)), -1, device=DEV, dtype=torch.int32)
    refine = torch.full((nq, H, rw), -5, device=DEV, dtype=torch.int32)
    K.select_blocks(mass, keep_prev, se, ss, keep, counts, blocks, flags, bits, refine, k, r, L, sink=sink)
    return keep, counts, blocks, bits, refine


def _same_selection(got, want):
    keep, counts, blocks, bits, refine = got
    wkeep, wcounts, wblocks, wbits, wrefine = (x.to(DEV) for x in want)
    assert torch.equal(keep, wkeep) and torch.equal(counts, wcounts)
    assert torch.equal(bits, wbits) and torch.equal(refine, wrefine)
    if wblocks is not None:
        col = torch.arange(blocks.shape[-1], device=DEV)[None, None, :]
        live = col < counts[:, :, None]
        assert torch.equal(blocks[live], wblocks[live])


def test_selection_matches_reference_bit_for_bit(K, golden):
    ones = torch.ones(H, NQ, NB, device=DEV, dtype=torch.uint8)
    got = _select(K, T(golden["full_mass"], DEV), ones, T(golden["full_scale_exact"], DEV),
                  T(golden["full_scale_skip"], DEV), T(golden["full_flags"], DEV), int(golden["top"]),
                  int(golden["refined"]), L, H, int(golden["rw"]))
    _same_selection(got, [T(golden[f"sel_{n}"]) for n in ("keep", "counts", "blocks", "bits", "refine")])
    got = _select(K, T(golden["est_mass"], DEV), T(golden["sel_keep"], DEV), T(golden["est_scale_exact"], DEV),
                  T(golden["est_scale_skip"], DEV), T(golden["sparse_flags"], DEV), int(golden["top"]),
                  int(golden["refined"]), L, H, int(golden["rw"]))
    want = [T(golden[f"sel2_{n}"]) for n in ("keep", "counts")] + [None] + [T(golden["sel2_bits"]), T(golden["sel2_refine"])]
    keep, counts, blocks, bits, refine = got
    assert torch.equal(keep, want[0].to(DEV)) and torch.equal(counts, want[1].to(DEV))
    assert torch.equal(bits, want[3].to(DEV)) and torch.equal(refine, want[4].to(DEV))


@pytest.mark.parametrize("case", ["c1", "c2", "c3", "c4"])
def test_selection_corner_cases_match_reference(K, golden, case):
    import numpy as np
    rng = np.random.Generator(np.random.PCG64(7))
    cm = rng.random((H, NQ, NB), dtype=np.float32)
    cm[:, :, 5] = cm[:, :, 9]
    cm[0, 3, 11] = np.nan
    cm[1, 4, 12] = np.inf
    cm[:, 6, :] = 0.25
    keep_prev = T((rng.random((H, NQ, NB)) < 0.2).astype(np.uint8), DEV)
    se = T(rng.random((H, NQ), dtype=np.float32) + 0.5, DEV)
    ss = T(rng.random((H, NQ), dtype=np.float32) + 0.5, DEV)
    flags = T((rng.random((NQ, H)) < 0.2).astype(np.int32), DEV)
    k, r, sink, w = (int(x) for x in golden[f"{case}_args"])
    keep, counts, blocks, bits, refine = _select(K, T(cm, DEV), keep_prev, se, ss, flags, k, r, L, H, w, sink=sink)
    assert torch.equal(keep, T(golden[f"{case}_keep"], DEV)) and torch.equal(counts, T(golden[f"{case}_counts"], DEV))
    assert torch.equal(bits, T(golden[f"{case}_bits"], DEV)) and torch.equal(refine, T(golden[f"{case}_refine"], DEV))


def test_plans_match_reference_bit_for_bit(K, golden):
    keep = T(golden["sel_keep"], DEV)
    exact = torch.zeros(H, NQ, int(golden["words"]), device=DEV, dtype=torch.int32)
    K.pack_plan(keep, exact)
    assert torch.equal(exact, T(golden["plan_exact"], DEV))
    rw = int(golden["rw"])
    keep2 = torch.full_like(keep, 9)
    counts = torch.zeros(NQ, H, device=DEV, dtype=torch.int32)
    blocks = torch.zeros(NQ, H, NB, device=DEV, dtype=torch.int32)
    refine = torch.zeros(NQ, H, rw, device=DEV, dtype=torch.int32)
    rc, mc = torch.zeros_like(counts), torch.zeros_like(counts)
    means = torch.zeros_like(blocks)
    K.rebuild_plan(exact, T(golden["sel_bits"], DEV), keep2, counts, blocks, refine, rc, means, mc)
    assert torch.equal(keep2, keep) and torch.equal(counts, T(golden["sel_counts"], DEV))
    assert torch.equal(refine, T(golden["sel_refine"], DEV)) and torch.equal(rc, T(golden["plan_refine_counts"], DEV))
    assert torch.equal(mc, T(golden["plan_mean_counts"], DEV))
    col = torch.arange(NB, device=DEV)[None, None, :]
    assert torch.equal(blocks[col < counts[:, :, None]], T(golden["sel_blocks"], DEV)[col < counts[:, :, None]])
    assert torch.equal(means[col < mc[:, :, None]], T(golden["plan_means"], DEV)[col < mc[:, :, None]])


def test_block_means_match_reference(K, golden):
    _, k, v = qkv(2, DEV)
    km = torch.empty(NB, H, 128, device=DEV, dtype=torch.bfloat16)
    vm = torch.empty_like(km)
    K.block_means(k, v, km, vm)
    assert rel_l2(km, bf16_from_bits(golden["k_mean"], DEV)) <= 1e-3
    assert rel_l2(vm, bf16_from_bits(golden["v_mean"], DEV)) <= 1e-3


def test_representatives_match_reference(K, golden):
    q, k, v = qkv(2, DEV)
    reps = K.Representatives(L, H, 128, DEV, iters=int(golden["iters"]))
    reps.build(q, k, v)
    assert rel_l2(reps._metric, bf16_from_bits(golden["metric"], DEV)) <= 5e-3
    assert rel_l2(reps._probes, bf16_from_bits(golden["probes"], DEV)) <= 1e-3
    glc = T(golden["log_counts"], DEV)
    same = ((reps.log_counts == glc) | ((reps.log_counts - glc).abs() < 1e-6)).view(H, NB + 1, 4).all(-1)
    assert same.float().mean() > 0.95            # near-ties in float32 distances may move single tokens
    gk = bf16_from_bits(golden["k_rep"], DEV).view(H, NB + 1, 4, 128)
    gv = bf16_from_bits(golden["v_rep"], DEV).view(H, NB + 1, 4, 128)
    assert rel_l2(reps.k.view(H, NB + 1, 4, 128)[same], gk[same]) <= 5e-3
    assert rel_l2(reps.v.view(H, NB + 1, 4, 128)[same], gv[same]) <= 5e-3
    # the invariants of the reference's tests/test_sm120.py:65-83
    cnt = torch.exp2(reps.log_counts[:, :NB * 4]).view(H, NB, 4)
    assert torch.equal(cnt.sum(-1).round().long().cpu(), R.block_len(L, NB).long().expand(H, NB))
    pad = torch.zeros((NB + 1) * 64 - L, H, 128, device=DEV)
    sums = torch.cat([k.float(), pad]).view(NB + 1, 64, H, 128).sum(1).permute(1, 0, 2)[:, :NB]
    got = (cnt[..., None] * reps.k.float().view(H, NB + 1, 4, 128)[:, :NB]).sum(2)
    assert rel_l2(got, sums) <= 1e-2
    assert torch.isinf(reps.log_counts[:, NB * 4:]).all() and (reps.k[:, NB * 4:] == 0).all()


def test_sparse_step_matches_reference(K, golden):
    q, k, v = qkv(2, DEV)
    out, lse, flags = _outputs(L, H, q)
    mass = torch.zeros(H, NQ, NB, device=DEV)
    K.sparse_attention(q, k, v, bf16_from_bits(golden["k_mean"], DEV), bf16_from_bits(golden["v_mean"], DEV),
                       T(golden["sel_bits"], DEV), out, T(golden["sel_counts"], DEV), T(golden["sel_blocks"], DEV),
                       T(golden["full_lse_reset"], DEV), lse, flags, T(golden["sel_refine"], DEV),
                       bf16_from_bits(golden["k_rep"], DEV), bf16_from_bits(golden["v_rep"], DEV),
                       T(golden["log_counts"], DEV), mass=mass)
    _close_out(out[ROWS], bf16_from_bits(golden["sparse_out"], DEV))
    assert (lse[:L] - T(golden["sparse_lse"], DEV)[:L]).abs().max() <= 1e-4
    assert (lse[L:] == 1e30).all()
    assert torch.equal(flags, T(golden["sparse_flags"], DEV))
    assert rel_l2(mass, T(golden["sparse_mass"], DEV)) <= 1e-4
    mass3 = T(golden["sparse_mass"], DEV).clone()
    se, ss = torch.empty(H, NQ, device=DEV), torch.empty(H, NQ, device=DEV)
    K.estimate_skipped(q, bf16_from_bits(golden["k_mean"], DEV), T(golden["sel_keep"], DEV),
                       T(golden["full_lse_reset"], DEV), T(golden["sparse_lse"], DEV), mass3, se, ss)
    assert rel_l2(mass3, T(golden["est_mass"], DEV)) <= 1e-4
    assert rel_l2(se, T(golden["est_scale_exact"], DEV)) <= 1e-4 and rel_l2(ss, T(golden["est_scale_skip"], DEV)) <= 1e-4


def test_fallback_matches_reference(K, golden):
    """A far-off offset flags every tile; online softmax over the list, then block-mean compensation."""
    q, k, v = qkv(2, DEV)
    bad = T(golden["full_lse_reset"], DEV).clone()
    bad[:L] += 200.0
    out, lse, flags = _outputs(L, H, q)
    K.sparse_attention(q, k, v, bf16_from_bits(golden["k_mean"], DEV), bf16_from_bits(golden["v_mean"], DEV),
                       T(golden["sel_bits"], DEV), out, T(golden["sel_counts"], DEV), T(golden["sel_blocks"], DEV), bad, lse,
                       flags, T(golden["sel_refine"], DEV), bf16_from_bits(golden["k_rep"], DEV),
                       bf16_from_bits(golden["v_rep"], DEV), T(golden["log_counts"], DEV))
    assert torch.equal(flags, T(golden["fb_flags"], DEV)) and int(flags.sum()) == NQ * H
    K.exact_fallback(q, k, v, out, T(golden["sel_counts"], DEV), T(golden["sel_blocks"], DEV), lse, flags)
    _close_out(out[ROWS], bf16_from_bits(golden["fb_exact_out"], DEV))
    assert (lse[:L] - T(golden["fb_exact_lse"], DEV)[:L]).abs().max() <= 1e-4
    K.compensate_fallback(q, bf16_from_bits(golden["k_mean"], DEV), bf16_from_bits(golden["v_mean"], DEV),
                          T(golden["sel_keep"], DEV), lse, out, flags)
    _close_out(out[ROWS], bf16_from_bits(golden["fb_comp_out"], DEV))
    assert (lse[:L] - T(golden["fb_comp_lse"], DEV)[:L]).abs().max() <= 1e-4
    assert (lse[L:] == 1e30).all()


# ------------------------------------------------------------------------------------------------ oracle, other shapes
def _inputs(L, H, seed):
    g = torch.Generator().manual_seed(seed)
    pos = torch.arange(L, dtype=torch.float32)[:, None, None] / 300.0
    freq = torch.randn(1, H, 128, generator=g)
    base = [torch.sin(pos * freq + torch.randn(1, H, 128, generator=g)) * 3.0 for _ in range(3)]
    return [(b + 0.05 * torch.randn(b.shape, generator=g)).to(torch.bfloat16).to(DEV) for b in base]


# 512: the 8-block CPU configuration (nb < 32); 200: a single ragged tile; 4096 + 192: three heads, even tail;
# 8256: 129 blocks, two 128-block chunks of mean columns with one live column in the second
@pytest.mark.parametrize("L,H,density", [(512, 2, 0.25), (200, 1, 0.3), (4288, 3, 0.1), (8256, 1, 0.1), (1000, 2, 1.0)])
def test_pipeline_matches_oracle(K, L, H, density):
    nq, nb = R.cdiv(L, 128), R.cdiv(L, 64)
    q, k, v = _inputs(L, H, seed=L)
    _, lse_d = R.dense_attention(q, k, v)
    offset = torch.full((nq * 128, H), 1e30, device=DEV)
    offset[:L] = lse_d + 0.3 * torch.randn(L, H, generator=torch.Generator().manual_seed(1)).to(DEV)
    counts, blocks = _all_lists(L, H)
    out, lse, flags = _outputs(L, H, q)
    mass = torch.zeros(H, nq, nb, device=DEV)
    K.block_attention(q, k, v, out, counts, blocks, offset, lse, flags, mass=mass)
    mass_r = torch.zeros_like(mass)
    out_r, lse_r, flags_r = R.fixed_offset_attention(q, k, v, counts, blocks, offset, mass=mass_r)
    _close_out(out, out_r)
    assert (lse - lse_r).abs()[:L].max() <= 1e-4 and torch.equal(flags, flags_r) and rel_l2(mass, mass_r) <= 1e-4
    se, ss = torch.empty(H, nq, device=DEV), torch.empty(H, nq, device=DEV)
    K.full_step_scales(offset, lse, se, ss, L)
    top, refined = R.budget(density, nb)
    rw = -(-refined // 32) * 32
    ones = torch.ones(H, nq, nb, device=DEV, dtype=torch.uint8)
    zero_flags = torch.zeros(nq, H, device=DEV, dtype=torch.int32)
    sel = _select(K, mass, ones, se, ss, zero_flags, top, refined, L, H, rw)
    _same_selection(sel, R.select_blocks(mass, ones, se, ss, zero_flags, top, refined, L, rw))
    keep, cnt, blk, bits, refine = sel
    km = torch.empty(nb, H, 128, device=DEV, dtype=torch.bfloat16)
    vm = torch.empty_like(km)
    K.block_means(k, v, km, vm)
    km_r, vm_r = R.block_means(k, v)
    assert rel_l2(km, km_r) <= 1e-3 and rel_l2(vm, vm_r) <= 1e-3
    reps = K.Representatives(L, H, 128, DEV, iters=10)
    reps.build(q, k, v)
    kr, vr, lc, _ = R.representatives(q, k, v, 10, reps._metric, reps._probes)
    same = ((lc == reps.log_counts) | ((lc - reps.log_counts).abs() < 1e-6)).view(H, nb + 1, 4).all(-1)
    # cluster labels are decided by float32 comparisons: a near-tie may move a token in a few blocks
    differing = int((~same).sum())
    assert differing <= max(1, same.numel() // 10), (differing, torch.exp2(lc).view(H, nb + 1, 4)[~same],
                                                      torch.exp2(reps.log_counts).view(H, nb + 1, 4)[~same])
    assert rel_l2(reps.k.view(H, nb + 1, 4, 128)[same], kr.view(H, nb + 1, 4, 128)[same]) <= 5e-3
    out2, lse2, flags2 = _outputs(L, H, q)
    mass2 = torch.zeros(H, nq, nb, device=DEV)
    K.sparse_attention(q, k, v, km, vm, bits, out2, cnt, blk, lse, lse2, flags2, refine, reps.k, reps.v, reps.log_counts,
                       mass=mass2)
    mass2_r = torch.zeros_like(mass2)
    o_r, l_r, f_r = R.fixed_offset_attention(q, k, v, cnt, blk, lse, mass=mass2_r, k_mean=km, v_mean=vm, skip_bits=bits,
                                             refine=refine, k_rep=reps.k, v_rep=reps.v, log_counts=reps.log_counts)
    _close_out(out2, o_r)
    assert (lse2 - l_r).abs()[:L].max() <= 1e-4 and torch.equal(flags2, f_r) and rel_l2(mass2, mass2_r) <= 1e-4
    mass3, se3, ss3 = mass2.clone(), torch.empty_like(se), torch.empty_like(ss)
    K.estimate_skipped(q, km, keep, lse, lse2, mass3, se3, ss3)
    m3_r, se3_r, ss3_r = R.estimate_skipped(q, km, keep, lse, lse2, mass2)
    assert rel_l2(mass3, m3_r) <= 1e-4 and rel_l2(se3, se3_r) <= 1e-4 and rel_l2(ss3, ss3_r) <= 1e-4
    # flag half of the tiles by hand and recompute them
    flags3 = (torch.arange(nq * H, device=DEV).view(nq, H) % 2).to(torch.int32)
    out3, lse3 = out2.clone(), lse2.clone()
    K.exact_fallback(q, k, v, out3, cnt, blk, lse3, flags3)
    K.compensate_fallback(q, km, vm, keep, lse3, out3, flags3)
    out3_r, lse3_r = o_r.clone(), l_r.clone()
    R.exact_fallback(q, k, v, out3_r, cnt, blk, lse3_r, flags3)
    R.compensate_fallback(q, km, vm, keep, lse3_r, out3_r, flags3)
    _close_out(out3, out3_r)
    assert (lse3 - lse3_r).abs()[:L].max() <= 1e-4


def test_odd_and_single_block_lists(K):
    """Lists of 1, 2 and 3 blocks (an odd count leaves the second half of the last iteration empty), the tail block
    alone, and a list that is only the forced blocks."""
    L, H = 1000, 2
    nq, nb = R.cdiv(L, 128), R.cdiv(L, 64)
    q, k, v = _inputs(L, H, seed=3)
    counts = torch.tensor([[1, 2], [3, 1], [2, 3], [1, 1], [3, 3], [16, 15], [1, 2], [5, 1]], device=DEV, dtype=torch.int32)
    blocks = torch.zeros(nq, H, nb, device=DEV, dtype=torch.int32)
    g = torch.Generator().manual_seed(5)
    for t in range(nq):
        for h in range(H):
            n = int(counts[t, h])
            ids = torch.randperm(nb, generator=g)[:n].sort().values
            if (t, h) == (3, 0):
                ids = torch.tensor([nb - 1])                       # the 40-token tail block alone
            blocks[t, h, :n] = ids.to(DEV)
    offset = torch.full((nq * 128, H), 1e30, device=DEV)
    offset[:L] = 3.0
    out, lse, flags = _outputs(L, H, q)
    mass = torch.zeros(H, nq, nb, device=DEV)
    K.block_attention(q, k, v, out, counts, blocks, offset, lse, flags, mass=mass)
    mass_r = torch.zeros_like(mass)
    out_r, lse_r, flags_r = R.fixed_offset_attention(q, k, v, counts, blocks, offset, mass=mass_r)
    _close_out(out, out_r)
    assert (lse - lse_r).abs()[:L].max() <= 1e-4 and torch.equal(flags, flags_r) and rel_l2(mass, mass_r) <= 1e-4


def test_mass_map_is_reproducible(K):
    """Masses are stored by one thread in a fixed order, so two runs give the same bits."""
    L, H = 4152, 2
    q, k, v = _inputs(L, H, seed=9)
    nq, nb = R.cdiv(L, 128), R.cdiv(L, 64)
    counts, blocks = _all_lists(L, H)
    offset = torch.full((nq * 128, H), 1e30, device=DEV)
    offset[:L] = 5.0
    runs = []
    for _ in range(2):
        out, lse, flags = _outputs(L, H, q)
        mass = torch.zeros(H, nq, nb, device=DEV)
        K.block_attention(q, k, v, out, counts, blocks, offset, lse, flags, mass=mass)
        runs.append((out.clone(), lse.clone(), mass.clone()))
    assert all(torch.equal(a, b) for a, b in zip(*runs))


def test_fallback_over_a_tile_list_equals_one_cta_per_tile(K):
    """The recomputation and compensation kernels walk a list of the flagged tiles when given scratch for it (the kernel-set
    module always gives it); without scratch every tile's CTA tests its own flag. Same bits either way, for no, some and
    all tiles flagged; 195 tiles, so that with every tile flagged the CTAs of the list walk (one per SM) run several tiles."""
    from self_trainable_or_free_attn_b200 import _native as N
    L, H = 8256, 3
    nq, nb = R.cdiv(L, 128), R.cdiv(L, 64)
    q, k, v = _inputs(L, H, seed=21)
    counts, blocks = _all_lists(L, H)
    km = torch.empty(nb, H, 128, device=DEV, dtype=torch.bfloat16)
    vm = torch.empty_like(km)
    K.block_means(k, v, km, vm)
    keep = (torch.rand(H, nq, nb, device=DEV) < 0.3).to(torch.uint8)
    lib = N.load()
    for pattern in ("none", "some", "all"):
        flags = {"none": torch.zeros(nq, H), "some": (torch.arange(nq * H).view(nq, H) % 5 == 1).float(),
                 "all": torch.ones(nq, H)}[pattern].to(DEV).to(torch.int32)
        base_out = torch.randn(L, H, 128, device=DEV).to(torch.bfloat16)
        base_lse = torch.full((nq * 128, H), 3.0, device=DEV)
        got = []
        for scratch in (True, False):
            out, lse = base_out.clone(), base_lse.clone()
            if scratch:
                K.exact_fallback(q, k, v, out, counts, blocks, lse, flags)
                K.compensate_fallback(q, km, vm, keep, lse, out, flags)
            else:
                N.check(lib.es_exact_fallback(N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(out), N.ptr(counts), N.ptr(blocks), nb,
                                              N.ptr(lse), N.ptr(flags), L, H, None, N.stream_ptr()), "exact_fallback")
                N.check(lib.es_compensate_fallback(N.ptr(q), N.ptr(km), N.ptr(vm), N.ptr(keep), N.ptr(lse), N.ptr(out),
                                                   N.ptr(flags), L, H, None, N.stream_ptr()), "compensate_fallback")
            got.append((out, lse))
        assert torch.equal(got[0][0], got[1][0]) and torch.equal(got[0][1], got[1][1]), pattern
        if pattern == "none":
            assert torch.equal(got[0][0], base_out) and torch.equal(got[0][1], base_lse)
