"""es_reps_metric_static: the entry point for callers that cannot allocate device scratch (a plugin inside another
framework's memory pool, code in a no-allocation region). It must give what es_reps_metric gives, on consecutive calls
that share the library's built-in scratch array. This file is collected last on purpose."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _metric(lib, N, q, static):
    L, H, D = q.shape
    gram = torch.empty(H, D, D, device="cuda")
    metric = torch.empty(H, D, D, device="cuda", dtype=torch.bfloat16)
    probes = torch.empty(H, 64, D, device="cuda", dtype=torch.bfloat16)
    if static:
        rc = lib.es_reps_metric_static(N.ptr(q), N.ptr(gram), N.ptr(metric), N.ptr(probes), L, H, N.stream_ptr())
    else:
        parts = torch.empty(lib.es_reps_gram_splits(L), H, D, D, device="cuda")
        rc = lib.es_reps_metric(N.ptr(q), N.ptr(parts), N.ptr(gram), N.ptr(metric), N.ptr(probes), L, H, N.stream_ptr())
    N.check(rc, "reps metric")
    torch.cuda.synchronize()
    return gram, metric, probes


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


def test_static_scratch_matches_caller_scratch_on_two_calls_in_a_row():
    from self_trainable_or_free_attn_b200 import _native as N
    lib = N.load()
    g = torch.Generator(device="cuda").manual_seed(11)
    # two different problems back to back: the second call finds the first one's partial sums in the shared array
    for L, H in ((4152, 2), (9000, 40)):
        q = (torch.randn(L, H, 128, device="cuda", generator=g) * 1.5).to(torch.bfloat16)
        want = _metric(lib, N, q, static=False)
        got = _metric(lib, N, q, static=True)
        assert _rel(got[0], want[0]) <= 1e-5            # Gram matrix (float32 sums in a different split)
        assert _rel(got[1], want[1]) <= 5e-3            # Cholesky factor in bf16
        assert torch.equal(got[2], want[2])             # probes do not use the scratch
    assert N.device_status() == 0


def test_sizes_beyond_the_built_in_scratch_are_rejected():
    from self_trainable_or_free_attn_b200 import _native as N
    lib = N.load()
    H = lib.es_reps_metric_static_max_heads() + 1
    q = torch.zeros(64, H, 128, device="cuda", dtype=torch.bfloat16)
    metric = torch.empty(H, 128, 128, device="cuda", dtype=torch.bfloat16)
    probes = torch.empty(H, 64, 128, device="cuda", dtype=torch.bfloat16)
    before = N.launch_count()
    assert lib.es_reps_metric_static(N.ptr(q), None, N.ptr(metric), N.ptr(probes), 64, H, N.stream_ptr()) < 0
    assert "256 heads" in N.last_error() and N.launch_count() == before
