"""The sampled long-sequence VSA2 oracle (oracle/vsa_sampled.py) equals autograd through the dense oracle
(oracle/vsa_ref.py, itself pinned against the reference's tests/vsa_reference.py) on every block of small problems:
ragged block counts, rows without any selected block, kv blocks nobody selected, with and without a gate."""
import pytest
import torch

from oracle import vsa_ref as R
from oracle.vsa_sampled import SampledVSA2, lists_from_csr


def _problem(nb, seed, empty_row=True):
    g = torch.Generator().manual_seed(seed)
    cnt = torch.randint(1, 65, (nb,), generator=g).to(torch.int32)
    cnt[0] = 64
    L, D = nb * 64, 128
    valid = R.token_valid(cnt, L)[:, None]
    q, k, v, dout = ((torch.randn(L, D, generator=g) * valid).to(torch.bfloat16) for _ in range(4))
    gate = torch.randn(L, generator=g).to(torch.bfloat16)
    mask = torch.rand(nb, nb, generator=g) < 0.4
    if empty_row:
        mask[2] = False          # a query block with no kv block
        mask[:, 3] = False       # a kv block nobody selected
    return q, k, v, gate, dout, cnt, mask


@pytest.mark.parametrize("nb,seed,with_gate", [(6, 0, True), (9, 1, False), (5, 2, True)])
def test_sampled_oracle_equals_autograd_through_the_dense_oracle(nb, seed, with_gate):
    q, k, v, gate, dout, cnt, mask = _problem(nb, seed)
    leaves = [x.float()[None, None].requires_grad_(True) for x in (q, k, v)]
    gl = gate.float()[None, None].requires_grad_(True) if with_gate else None
    o_ref = R.vsa2_output(*leaves, gl, cnt, mask[None, None], round_pooled=False)
    grads = torch.autograd.grad(o_ref, leaves + ([gl] if with_gate else []), dout.float()[None, None])
    _, lse_ref = R.fine_attention(q.float()[None, None], k.float()[None, None], v.float()[None, None], cnt, mask[None, None])
    q2k = [mask[i].nonzero().flatten().tolist() for i in range(nb)]
    k2q = [mask[:, j].nonzero().flatten().tolist() for j in range(nb)]
    s = SampledVSA2(q, k, v, gate if with_gate else None, dout, cnt, q2k, k2q, round_to=None)
    tol = lambda ref: 2e-5 * float(ref.abs().max()) + 1e-6
    for i in range(nb):
        sl = slice(64 * i, 64 * (i + 1))
        o, lse, dq, dgate = s.query_block(i)
        assert (o - o_ref[0, 0, sl]).abs().max() <= tol(o_ref)
        both_inf = torch.isinf(lse) & torch.isinf(lse_ref[0, 0, sl])
        assert (torch.where(both_inf, torch.zeros_like(lse), lse - lse_ref[0, 0, sl])).abs().max() <= 1e-5
        assert (dq - grads[0][0, 0, sl]).abs().max() <= tol(grads[0])
        if with_gate:
            assert (dgate - grads[3][0, 0, sl]).abs().max() <= tol(grads[3])
        dk, dv = s.kv_block(i)
        assert (dk - grads[1][0, 0, sl]).abs().max() <= tol(grads[1])
        assert (dv - grads[2][0, 0, sl]).abs().max() <= tol(grads[2])


def test_sampled_oracle_rounds_the_block_means_like_the_kernels():
    q, k, v, gate, dout, cnt, mask = _problem(4, 3, empty_row=False)
    nb = 4
    q2k = [mask[i].nonzero().flatten().tolist() for i in range(nb)]
    k2q = [mask[:, j].nonzero().flatten().tolist() for j in range(nb)]
    s = SampledVSA2(q, k, v, gate, dout, cnt, q2k, k2q)
    oc = R.coarse_attention(q.float()[None, None], k.float()[None, None], v.float()[None, None], cnt, torch.bfloat16)[0, 0]
    assert torch.allclose(s.oc, oc, rtol=1e-6, atol=1e-7)


def test_lists_from_csr():
    mask = torch.tensor([[1, 0, 1], [0, 0, 0], [1, 1, 1]], dtype=torch.bool)[None, None]
    qp, qi, kp, ki = R.mask_to_csr(mask)
    assert lists_from_csr(qp[0, 0], qi, 3) == [[0, 2], [], [0, 1, 2]]
    assert lists_from_csr(kp[0, 0], ki, 3) == [[0, 2], [2], [0, 2]]


@pytest.mark.parametrize("nb,seed,rm", [(6, 0, 4), (8, 1, 8), (5, 2, 2)])
def test_sampled_tier_oracle_equals_autograd_through_the_dense_tier_oracle(nb, seed, rm):
    from oracle.vsa_sampled import SampledTiers
    q, k, v, _, dout, cnt, mask = _problem(nb, seed, empty_row=False)
    g = torch.Generator().manual_seed(seed + 10)
    tier_a = mask
    tier_ab = mask | (torch.rand(nb, nb, generator=g) < 0.3)
    tier_a[2] = False                                      # a query block that sees no kv block in full
    # float32 leaves: the dense oracle rounds its tables to the leaves' dtype, so neither side rounds to bf16 here
    leaves = [x.float()[None, None].requires_grad_(True) for x in (q, k, v)]
    o_ref, lse_ref = R.tier_fine_attention(*leaves, cnt, tier_a[None, None], tier_ab[None, None], mid_reps=rm,
                                           dtype=torch.float64)
    grads = torch.autograd.grad(o_ref, leaves, dout.double()[None, None])
    s = SampledTiers(q, k, v, dout, cnt, tier_a, tier_ab, mid_reps=rm, round_to=None)
    dk, dv = s.kv_gradients()
    tol = lambda ref: 5e-5 * float(ref.detach().abs().max()) + 1e-6
    for i in range(nb):
        sl = slice(64 * i, 64 * (i + 1))
        o, lse, dq = s.query_block(i)
        assert (o - o_ref[0, 0, sl].detach()).abs().max() <= tol(o_ref)
        lr = lse_ref[0, 0, sl].detach().float()
        assert torch.equal(torch.isinf(lse), torch.isinf(lr))                   # padded rows: -inf on both sides
        assert torch.where(torch.isinf(lr), torch.zeros_like(lr), lse - lr).abs().max() <= 1e-4
        assert (dq - grads[0][0, 0, sl].float()).abs().max() <= tol(grads[0].float())
    assert (dk - grads[1][0, 0].float()).abs().max() <= tol(grads[1].float())
    assert (dv - grads[2][0, 0].float()).abs().max() <= tol(grads[2].float())
