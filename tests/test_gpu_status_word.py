"""A bounded wait inside a kernel that runs out ends as an error the host sees, never as a hang or as silent garbage:
the kernel returns, the device status word holds the wait's code, attention launches return at once until the word has
been read, the attention processor raises when it reads it, and everything works again afterwards. The wait that runs out
here is a barrier nobody arrives on (the library's self test); no kernel faults, traps or spins without a limit."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_a_wait_that_runs_out_is_reported_and_cleared():
    from self_trainable_or_free_attn_b200 import _native as N, backends
    from self_trainable_or_free_attn_b200.attention import EchoSparseAttention
    K = backends.kernels(backends.resolve("auto", DEV))
    lib = N.load()
    assert N.device_status() == 0
    L, H = 1024, 2
    g = torch.Generator(device=DEV).manual_seed(0)
    q, k, v = (torch.randn(L, H, 128, device=DEV, generator=g).to(torch.bfloat16) for _ in range(3))
    nq, nb = L // 128, L // 64
    counts = torch.full((nq, H), nb, device=DEV, dtype=torch.int32)
    blocks = torch.arange(nb, device=DEV, dtype=torch.int32).expand(nq, H, nb).contiguous()
    ones = torch.ones(nq, H, device=DEV, dtype=torch.int32)

    def dense():
        out = torch.full_like(q, 7.0)
        lse = torch.zeros(nq * 128, H, device=DEV)
        K.exact_fallback(q, k, v, out, counts, blocks, lse, ones)
        torch.cuda.synchronize()
        return out

    good = dense()
    assert not bool((good == 7.0).all())
    # a wait of 2 ms that nothing ends: the kernel comes back, the word holds the code
    N.check(lib.es_selftest_wait_timeout(2000, N.stream_ptr()), "selftest")
    torch.cuda.synchronize()
    # the attention kernels are switched off until the word has been read: the launch returns without touching `out`
    assert bool((dense() == 7.0).all())
    attn = EchoSparseAttention(dense_steps=2, dense_layers=(), min_blocks=1)
    attn._bind(torch.device(DEV, torch.cuda.current_device()))
    with pytest.raises(N.NativeError, match="status 777"):
        attn.check_status()
    # reading cleared it
    assert N.device_status() == 0
    assert torch.equal(dense(), good)
    attn.reset()                                     # the per-video check passes again


def test_self_test_rejects_limits_out_of_range():
    from self_trainable_or_free_attn_b200 import _native as N
    lib = N.load()
    assert lib.es_selftest_wait_timeout(0, None) < 0 and "limit" in N.last_error()
    assert lib.es_selftest_wait_timeout(10 ** 6, None) < 0
    assert N.device_status() == 0
