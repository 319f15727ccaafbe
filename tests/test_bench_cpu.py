"""bench.py's host-side pieces, without a GPU: the roofline object, the configuration both arms print, the seeded fallback
injection and the VSA2 workload description."""
import importlib.util
import os
from types import SimpleNamespace

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _args(**kw):
    base = dict(workload="wan_14b_720p", heads=0, threshold=60.0, ulysses=False, nccl_exchange=False, skew="uniform",
                split="none", gpus=1)
    base.update(kw)
    return SimpleNamespace(**base)


def test_roofline_object_has_the_three_fractions():
    b = _bench()
    peaks = {"burst": 1700.0, "sustained": 1400.0, "hbm_gbs": 6500.0, "sm_max_mhz": 1965.0, "source": "measured"}
    r = b.tensor_roofline("k", 850.0, 17.0, 20, {"sm_mhz": 1572.0}, peaks, traffic=3.0e9)
    assert r["bound"] == "tensor" and r["unit"] == "TFLOP/s" and r["peak"] == 1700.0 and r["achieved"] == 850.0
    assert abs(r["frac"] - 0.5) < 1e-12 and abs(r["frac_of_sustained"] - 850.0 / 1400.0) < 1e-12
    assert abs(r["pipe_peak_at_sampled_clock"] - 2250.0 * 0.8) < 1e-9 and abs(r["frac_of_pipe_at_sampled_clock"] - 850.0 / 1800.0) < 1e-12
    assert r["ms_per_launch"] == 17.0 and r["launches_timed"] == 20 and r["traffic"] == 3.0e9
    assert "burst" in r["peak_source"] and "measured" in r["peak_source"]
    no_clock = b.tensor_roofline("k", 850.0, 17.0, 20, {}, peaks)
    assert no_clock["pipe_peak_at_sampled_clock"] == 2250.0


def test_both_arms_print_the_same_config():
    b = _bench()
    ours, ref = b.workload_config(_args(), 1), b.workload_config(_args(gpus=1), 1)
    assert ours == ref and ours["tokens"] == 75600 and ours["heads"] == 40 and ours["branches"] == 2 and ours["density"] == 0.1
    assert b.workload_config(_args(heads=5), 8)["heads"] == 5
    hy = b.workload_config(_args(workload="hunyuan_720p", ulysses=True), 8)
    assert hy["tokens"] == 119056 and "exchange kernel over peer memory" in hy["partition"]
    assert "all_to_all_single" in b.workload_config(_args(workload="hunyuan_720p", ulysses=True, nccl_exchange=True), 8)["partition"]
    assert "Ulysses" not in b.workload_config(_args(workload="hunyuan_720p", ulysses=True), 1)["partition"]
    assert b.sink_of("hunyuan_720p") == 1856 and b.sink_of("wan_14b_720p") is None
    v = b.vsa2_config(_args(workload="vsa2_train", skew="tenth_x4", split="auto"), 2)
    assert v["workload"] == "vsa2_train" and v["tokens"] == 32768 and v["heads"] == 12 and v["selection"] == "tenth_x4"
    assert v["split_kv"] == "auto"


def test_fallback_injection_is_seeded_and_scales_whole_tiles():
    b = _bench()
    q = torch.ones(1, 128 * 40 + 5, 3, 4)
    n = b.inject_fallback(q, 0.25, 3.0, seed=11)
    q2 = torch.ones(1, 128 * 40 + 5, 3, 4)
    assert b.inject_fallback(q2, 0.25, 3.0, seed=11) == n and torch.equal(q, q2) and 0 < n < 41 * 3
    tiles = q[0, :, :, 0].split(128, dim=0)
    assert all(bool(((t == 1) | (t == 3)).all()) and bool((t == t[0]).all()) for t in tiles)
    assert sum(int((t[0] == 3).sum()) for t in tiles) == n


def test_measured_peaks_fall_back_when_the_file_is_absent(monkeypatch):
    b = _bench()
    monkeypatch.setattr(b, "ROOT", "/nonexistent")
    p = b.measured_peaks()
    assert p["source"] == "fallback" and p["burst"] == 1590.0 and p["hbm_gbs"] == 6650.0
