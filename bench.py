"""Benchmark of the two hot paths on B200: the EchoSparse sparse-step attention layer and the VSA2 training layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

EchoSparse workloads (default `wan_14b_720p`: 2 CFG branches x 40 heads x 75,600 tokens, 10 % of the blocks kept, ~0.5 % of
the tiles pushed into the online-softmax fallback): a step is one sparse-step attention layer, both CFG branches through
`EchoSparseAttention.__call__` (plan -> lists, block means, representatives, fused sparse attention, fallback, estimates,
next plan). With N GPUs the heads are sharded (both branches of a head on one GPU), no collective in the data path.
`--heads H` keeps only the first H heads (a small case for a profiler).

`--workload vsa2_train` (B = 1, 12 heads, 32,768 tokens of a 16 x 32 x 64 grid, top-k 32): a step is one forward + backward
of `vsa2_attention` on a frozen selection; `--skew CASE` picks the shape of the selection (`tenth_x4`: 10 % of the query
blocks select 4 x more kv blocks), `--split none|auto|manual` the split-KV scheduling.

Rank 0 prints one JSON line. Inputs are seeded synthetic activations (`synthetic.py`, `vsa/workloads.py`).
`--impl reference` times the CPU restatement of the same step (oracle/) on the host cores, on a bounded sample of the same
workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from self_trainable_or_free_attn_b200 import synthetic  # noqa: E402

CONFIG_IDS = {"cpu_small": 0, "wan_1_3b_480p": 1, "wan_14b_720p": 2, "hunyuan_720p": 3}
FALLBACK_RATE = 0.005        # share of (tile, head) pairs whose Q is scaled by 3x
FALLBACK_Q_SCALE = 3.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"burst": float(d["bf16_tflops"]), "sustained": float(d["bf16_tflops_sustained"]),
                "hbm_gbs": float(d["hbm_gbs"]), "sm_max_mhz": float(d.get("sm_max_mhz", 1965.0)), "source": "measured"}
    return {"burst": 1590.0, "sustained": 1400.0, "hbm_gbs": 6650.0, "sm_max_mhz": 1965.0, "source": "fallback"}


NOMINAL_BF16_TFLOPS = 2250.0      # dense bf16 at the maximum SM clock


def tensor_roofline(kernel, achieved, ms, launches, clocks, peaks, **more):
    """The roofline object of a tensor-core-bound kernel. `frac` is against the burst peak (a cuBLAS GEMM timed alone, the
    comparable figure for a kernel that runs tens of milliseconds at full clocks); the sustained-peak fraction and the
    fraction of the nominal pipe rate at the SM clock sampled during the run stand beside it."""
    sm = clocks.get("sm_mhz") or peaks["sm_max_mhz"]
    pipe = NOMINAL_BF16_TFLOPS * sm / peaks["sm_max_mhz"]
    out = {"bound": "tensor", "kernel": kernel, "achieved": achieved, "peak": peaks["burst"], "unit": "TFLOP/s",
           "frac": achieved / peaks["burst"], "peak_source": f"bf16_tflops (burst) of {peaks['source']}",
           "frac_of_sustained": achieved / peaks["sustained"], "peak_sustained": peaks["sustained"],
           "frac_of_pipe_at_sampled_clock": achieved / pipe, "pipe_peak_at_sampled_clock": pipe,
           "ms_per_launch": ms, "launches_timed": launches}
    out.update(more)
    return out


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def count(self):
        return len(self.lines) if self.proc is not None else 1 << 30

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6 or not parts[0].isdigit():
                continue
            sm.append(int(parts[0]))
            mx.append(int(parts[1]))
            reasons.update(n for n, v in zip(self.NAMES, parts[2:]) if v == "Active")
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def bind_host_to_gpu_node(device_index):
    """Runs the calling thread on the CPUs of the NUMA node the GPU hangs off, so that the pinned host buffers it allocates
    afterwards (first touch) sit on that node and the copies do not cross the socket link. Returns the node, or None when the
    machine does not say (one node, no sysfs entry): host-side placement only, nothing of the GPU is changed."""
    try:
        bus = torch.cuda.get_device_properties(device_index).pci_bus_id
        dev = torch.cuda.get_device_properties(device_index).pci_device_id
        dom = torch.cuda.get_device_properties(device_index).pci_domain_id
        path = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev:02x}.0/numa_node"
        node = int(open(path).read())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return node
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None


def inject_fallback(q, rate, scale, seed):
    """Scales Q by `scale` on a seeded random share of (tile, head) pairs, in place. Returns the number chosen."""
    _, L, H, _ = q.shape
    nq = -(-L // 128)
    g = torch.Generator().manual_seed(seed)
    pick = (torch.rand(nq, H, generator=g) < rate).nonzero().tolist()
    for t, h in pick:
        q[0, 128 * t:128 * (t + 1), h] *= scale
    return len(pick)


def workload_config(args, world=1):
    """The keys both arms print under `config`: what the workload is, not how an arm runs it."""
    grid, heads_all, branches, density, text = synthetic.WORKLOADS[args.workload]
    heads = min(args.heads, heads_all) if args.heads else heads_all
    return {"workload": args.workload, "tokens": synthetic.grid_tokens(grid) + text, "heads": heads, "branches": branches,
            "density": density, "head_dim": 128, "flag_threshold_log2": args.threshold,
            "partition": (f"heads over {world} GPU(s), both CFG branches of a head together"
                          + ("; sequence-sharded caller (Ulysses): q, k, v and the output cross the ranks every step, by "
                             + ("all_to_all_single between two layout copies" if getattr(args, "nccl_exchange", False)
                                else "this library's exchange kernel over peer memory")
                             if args.ulysses and world > 1 else "")),
            "l2": "inputs (q, k, v of a branch >> 126 MB) exceed L2 between iterations",
            "step": "one sparse-step attention layer, both CFG branches: plan -> lists, block means, representatives, fused "
                    "sparse attention, fallback of flagged tiles, estimates, next plan"}


def sink_of(workload):
    """First kv block of the text tokens (always computed), or None: hunyuan_video.py:66 of the reference."""
    grid, _, _, _, text = synthetic.WORKLOADS[workload]
    return synthetic.grid_tokens(grid) // 64 if text else None


def build_job(args, rank, world, device):
    """Inputs of this rank's head shard, and an attention processor taken through the dense and the full step on the
    previous step's (perturbed) inputs, so that the next call is a sparse step."""
    from self_trainable_or_free_attn_b200.attention import EchoSparseAttention
    grid, heads_all, branches, density, text = synthetic.WORKLOADS[args.workload]
    cid = CONFIG_IDS[args.workload]
    heads = synthetic.shard_heads(min(args.heads, heads_all) if args.heads else heads_all, rank, world)
    attn = EchoSparseAttention(density=density, dense_steps=2, dense_layers=(), refine_iters=6,
                               threshold=args.threshold, min_blocks=1, state=args.state)
    for b in range(branches):
        qp, kp, vp = synthetic.branch_qkv(grid, cid, b, heads, device, text, prev=True)
        attn(qp, kp, vp, 0, b, layer=1, sink=sink_of(args.workload))    # dense: log2 LSE of the perturbed inputs -> offset
        attn(qp, kp, vp, 1, b, layer=1, sink=sink_of(args.workload))    # full step: first mass map, exact LSE
        del qp, kp, vp
    # Two versions of every branch's Q that differ on a seeded 0.5 % of the (tile, head) pairs (Q scaled by 3 there).
    # Steps alternate between them, so every step meets that share of tiles with an offset that is far off (in one
    # direction or the other) and sends them through the online-softmax fallback.
    inputs, injected = [], 0
    for b in range(branches):
        q, k, v = synthetic.branch_qkv(grid, cid, b, heads, device, text)
        q2 = q.clone()
        injected += inject_fallback(q2, FALLBACK_RATE, FALLBACK_Q_SCALE, seed=977 * cid + 31 * b + rank)
        inputs.append(((q, q2), k, v))
    return attn, inputs, heads, injected


def run_steps(attn, inputs, first_step, n, sink=None):
    outs = None
    for i in range(n):
        outs = [attn(q[(first_step + i) & 1], k, v, first_step + i, b, layer=1, sink=sink)
                for b, (q, k, v) in enumerate(inputs)]
    return outs


def layer_flops(attn, inputs, L):
    """Algorithmic FLOP of one step on this rank (L tokens, this rank's heads): every branch uses branch 0's selection."""
    st = attn._states[(0, 1)]
    return len(inputs) * synthetic.step_flops(L, st.counts, st.blocks, st.refine, st.skip_bits)


def cpu_sample(workload, budget_s, threads, repeats=1):
    """Times the CPU restatement of the fused step (oracle/cpu_step.py) on a sample of query tiles of one head and one
    branch of the workload, sized to about `budget_s` seconds. Returns ([TFLOP/s per repeat], description, seconds)."""
    from oracle import cpu_step
    cid = CONFIG_IDS[workload]
    job = cpu_step.build_sample(workload, cid, 4)
    per_tile = cpu_step.time_sample(job, threads) / len(job["tiles"])
    n = max(4, min(job["nq"], int(budget_s / max(per_tile, 1e-4))))
    if n != len(job["tiles"]):
        job = cpu_step.build_sample(workload, cid, n)
    secs = [cpu_step.time_sample(job, threads) for _ in range(repeats)]
    desc = (f"{len(job['tiles'])} of {job['nq']} query tiles of one head of one branch, fused sparse step "
            f"(oracle/echosparse_ref.py) with lists, means and representatives built on the CPU")
    return [job["flop"] / s / 1e12 for s in secs], desc, sum(secs)


def reference_arm(args, threads):
    """The CPU restatement of the step on the host cores: every step is one pass over a bounded sample of query tiles;
    throughput in the same unit, the layer time extrapolated from it."""
    grid, heads_all, branches, density, text = synthetic.WORKLOADS[args.workload]
    n = args.warmup + args.steps
    vals, sample, _ = cpu_sample(args.workload, args.cpu_seconds / 2, threads, repeats=n)
    vals = vals[args.warmup:]
    value = statistics.median(vals)
    nominal = {"wan_14b_720p": 29.98e12, "wan_1_3b_480p": 2.33e12, "hunyuan_720p": 25.67e12}.get(args.workload)
    line = {"impl": "reference", "metric": "sparse_attn_effective_tflops", "value": value, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": nominal / (value * 1e12) * 1e3 if nominal else None, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, args.gpus),
            "how": "fused sparse step of a sample of query tiles on the host cores; ms_per_step extrapolates the sample's "
                   "throughput to the layer's nominal algorithmic FLOP",
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------ VSA2
VSA2_SHAPE = dict(grid=(16, 32, 64), heads=12, topk=32)


def vsa2_config(args, world=1):
    sh = VSA2_SHAPE
    heads = min(args.heads, sh["heads"]) if args.heads else sh["heads"]
    g = sh["grid"]
    return {"workload": "vsa2_train", "tokens": g[0] * g[1] * g[2], "heads": heads, "head_dim": 128, "tile": 64,
            "topk": sh["topk"], "selection": args.skew, "split_kv": args.split,
            "step": "forward + backward of vsa2_attention (fine block-sparse + coarse block-mean attention, tanh gate) on a "
                    "frozen selection: O, dQ, dK, dV, dgate",
            "partition": f"heads over {world} GPU(s), no collective (every kernel is per head)",
            "l2": "q, k, v, dO, O and the gradients of one step (>= 0.8 GB at 12 heads) exceed L2 between iterations"}


def vsa2_reference_arm(args, threads):
    """The sampled float32 CPU oracle (oracle/vsa_sampled.py) on the host cores: per step, forward and gradients of a
    sample of query blocks and kv blocks of one head; throughput on the algorithmic FLOP of what it evaluated."""
    from oracle.vsa_sampled import SampledVSA2
    from self_trainable_or_free_attn_b200.vsa import workloads
    sh = VSA2_SHAPE
    torch.set_num_threads(threads)
    q, k, v, gate, dout, lay = workloads.train_inputs(sh["grid"], 1, device="cpu")
    mask = workloads.selection_mask(args.skew, sh["grid"], 1, sh["topk"])[0, 0]
    nb = mask.shape[0]
    q2k = [mask[i].nonzero().flatten().tolist() for i in range(nb)]
    k2q = [mask[:, j].nonzero().flatten().tolist() for j in range(nb)]
    blocks = list(range(0, nb, 4))                         # a quarter of the query blocks and of the kv blocks

    def one_pass():
        ora = SampledVSA2(q[0, 0], k[0, 0], v[0, 0], gate[0, 0], dout[0, 0], lay.blk_cnt, q2k, k2q)
        t0 = time.perf_counter()
        rows = set()
        for i in blocks:
            ora.query_block(i)
            rows.add(i)
        pairs_kv = 0
        for j in blocks:
            ora.kv_block(j)
            rows.update(k2q[j])
            pairs_kv += len(k2q[j])
        dt = time.perf_counter() - t0
        # forward of every row touched (2 products per pair), dQ of the sampled rows (3), dK / dV of the sampled blocks (4)
        pairs_fwd = sum(len(q2k[i]) for i in rows)
        pairs_q = sum(len(q2k[i]) for i in blocks)
        flop = 2.0 * 64 * 64 * 128 * (2 * pairs_fwd + 3 * pairs_q + 4 * pairs_kv)
        return flop / dt / 1e12, dt

    vals = [one_pass()[0] for _ in range(args.warmup + args.steps)][args.warmup:]
    value = statistics.median(vals)
    nominal = 3.5 * 4.0 * 64 * 64 * 128 * nb * sh["topk"] * sh["heads"]
    sample = (f"{len(blocks)} of {nb} query blocks (O, LSE, dQ, dgate) and {len(blocks)} of {nb} kv blocks (dK, dV) of one head, "
              f"closed-form float32 (oracle/vsa_sampled.py), selection {args.skew}")
    line = {"impl": "reference", "metric": "vsa2_fwd_bwd_effective_tflops", "value": value, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": nominal / (value * 1e12) * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": vsa2_config(args, args.gpus),
            "how": "sampled blocks on the host cores; ms_per_step extrapolates the sample's throughput to the layer's "
                   "algorithmic FLOP",
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def vsa2_abba(args, local):
    """One arm against the default in ABBA order inside one process (default, arm, arm, default), the way the reference's
    benchmarks/vsa2_native_bench.py orders its four runs: ratios only come from inside one run, because separate runs
    drift. Arms are the split-KV schedules. Per leg: CUDA-event medians of the forward and of forward + backward, and
    SHA-256 digests of O, dQ, dK, dV, dgate. Verdict, worst first: FAIL (a non-finite value or a non-zero padded slot),
    NONDETERMINISTIC (the two default legs differ: every kernel here has one owner per output row, so they must not),
    OVER_TOL (an output of the arm is further from the default than --abba-tol in relative L2), WITHIN_TOL, IDENTICAL."""
    import hashlib
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    from self_trainable_or_free_attn_b200 import _native, vsa
    from self_trainable_or_free_attn_b200.vsa import ops, workloads
    sh = VSA2_SHAPE
    heads = min(args.heads, sh["heads"]) if args.heads else sh["heads"]
    q, k, v, gate, dout, lay = workloads.train_inputs(sh["grid"], heads, device=device)
    cnt = lay.blk_cnt.to(device)
    sel, nb = workloads.selection(args.skew, sh["grid"], heads, sh["topk"], device)
    arms = {"baseline": None, "split_auto": vsa.SplitKV.auto(), "split_manual": vsa.SplitKV(chunk=64)}
    valid = (torch.arange(q.shape[2], device=device) % 64 < cnt.repeat_interleave(64))[None, None, :, None]

    def leg(split):
        def fwd():
            with torch.no_grad():
                return vsa.vsa2_attention(q, k, v, gate, cnt, R=16, selection=sel, split_kv=split)

        def both():
            leaves = [x.detach().requires_grad_(True) for x in (q, k, v, gate)]
            o = vsa.vsa2_attention(*leaves, cnt, R=16, selection=sel, split_kv=split)
            return (o.detach(),) + torch.autograd.grad(o, leaves, dout)

        def median_ms(fn):
            for _ in range(args.warmup):
                fn()
            ts = []
            for _ in range(args.steps):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(b))
            return statistics.median(ts), (max(ts) - min(ts))
        f_ms, f_spread = median_ms(fwd)
        fb_ms, fb_spread = median_ms(both)
        outs = both()
        torch.cuda.synchronize()
        finite = all(bool(torch.isfinite(t.float()).all()) for t in outs)
        padding = all(bool((t.float() * (~valid if t.dim() == 4 else ~valid[..., 0]) == 0).all()) for t in outs)
        digests = [hashlib.sha256(t.contiguous().cpu().view(torch.uint8).numpy().tobytes()).hexdigest()[:16] for t in outs]
        return {"fwd_ms": f_ms, "fwd_spread_ms": f_spread, "f_plus_b_ms": fb_ms, "f_plus_b_spread_ms": fb_spread,
                "b_estimate_ms": fb_ms - f_ms, "finite": finite, "padding_zero": padding, "digests": digests}, outs

    order = ("default", "arm", "arm", "default")
    legs, tensors = [], []
    for name in order:
        r, outs = leg(None if name == "default" else arms[args.abba])
        legs.append(dict(r, leg=name))
        tensors.append([t.float().cpu() for t in outs])
    names = ("o", "dq", "dk", "dv", "dgate")
    rel = lambda a, b: float((a - b).norm() / b.norm().clamp(min=1e-30))
    arm_vs_default = {n: max(rel(tensors[1][i], tensors[0][i]), rel(tensors[2][i], tensors[3][i])) for i, n in enumerate(names)}
    aa = {n: rel(tensors[0][i], tensors[3][i]) for i, n in enumerate(names)}
    if not all(l["finite"] and l["padding_zero"] for l in legs):
        verdict = "FAIL"
    elif legs[0]["digests"] != legs[3]["digests"]:
        verdict = "NONDETERMINISTIC"
    elif max(arm_vs_default.values()) > args.abba_tol:
        verdict = "OVER_TOL"
    elif legs[1]["digests"] == legs[0]["digests"] and legs[2]["digests"] == legs[0]["digests"]:
        verdict = "IDENTICAL"
    else:
        verdict = "WITHIN_TOL"
    d_f = statistics.mean([legs[0]["fwd_ms"], legs[3]["fwd_ms"]])
    d_fb = statistics.mean([legs[0]["f_plus_b_ms"], legs[3]["f_plus_b_ms"]])
    a_f = statistics.mean([legs[1]["fwd_ms"], legs[2]["fwd_ms"]])
    a_fb = statistics.mean([legs[1]["f_plus_b_ms"], legs[2]["f_plus_b_ms"]])
    print(json.dumps({"schema": "vsa2-abba/1", "note": "measurement only: medians, spreads, ratios and errors",
                      "arm": args.abba, "config": vsa2_config(args), "order": order, "legs": legs,
                      "ratio_arm_over_default": {"fwd": a_f / d_f, "f_plus_b": a_fb / d_fb},
                      "rel_l2_arm_vs_default": arm_vs_default, "rel_l2_default_vs_default": aa, "tolerance": args.abba_tol,
                      "verdict": verdict, "device_status": _native.device_status()}), flush=True)


def vsa2_arm(args, rank, world, local, threads):
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU; there is no CPU fallback of the product path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    from self_trainable_or_free_attn_b200 import _native, vsa
    from self_trainable_or_free_attn_b200.vsa import ops, workloads
    sh = VSA2_SHAPE
    heads_all = min(args.heads, sh["heads"]) if args.heads else sh["heads"]
    mine = synthetic.shard_heads(heads_all, rank, world)
    if not mine:
        raise SystemExit(f"{world} ranks for {heads_all} heads: a rank without a head")
    q, k, v, gate, dout, lay = workloads.train_inputs(sh["grid"], heads_all, device="cpu")
    q, k, v, gate, dout = (x[:, mine].contiguous().to(device) for x in (q, k, v, gate, dout))
    cnt = lay.blk_cnt.to(device)
    mask = workloads.selection_mask(args.skew, sh["grid"], heads_all, sh["topk"])[:, mine]
    sel = ops.mask_to_selection(mask.to(device))
    split = {"none": None, "auto": vsa.SplitKV.auto(), "manual": vsa.SplitKV(chunk=64)}[args.split]
    fwd_flop, bwd_flop, pairs = workloads.fine_flops(sel)
    rows = sel.row_counts().reshape(-1)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def step(qq, kk, vv, gg, dd):
        leaves = [x.detach().requires_grad_(True) for x in (qq, kk, vv, gg)]
        o = vsa.vsa2_attention(*leaves, cnt, R=16, selection=sel, split_kv=split)
        return (o.detach(),) + torch.autograd.grad(o, leaves, dd)

    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(args.warmup):
        step(q, k, v, gate, dout)
    launches0 = _native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step(q, k, v, gate, dout)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = _native.launch_count() - launches0
    # the fine kernels alone (CUDA events on the launching stream), same inputs
    def timed(fn, n=5):
        """Median of n separately timed calls after one untimed call (one stall of the allocator does not move it)."""
        fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(n):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts), out
    ms_f, (of, lse) = timed(lambda: ops.attn_fwd(q, k, v, sel.q2k_ptr, sel.q2k_idx, cnt))
    delta = (dout.float() * of.float()).sum(-1)
    ms_kv, _ = timed(lambda: ops._bwd_kv(q, k, v, dout, lse, delta, sel.k2q_ptr, sel.k2q_idx, cnt))
    ms_q, _ = timed(lambda: ops._bwd_q(q, k, v, dout, lse, delta, sel.q2k_ptr, sel.q2k_idx, cnt))
    # the three-tier fine branch (64 tokens / 4 group means / 1 block mean per kv block): tier A = this selection, tier B the
    # next 20 % of the pairs by the same local score, tier C the rest; forward alone and forward + backward
    tiers_line = None
    if world == 1:
        from self_trainable_or_free_attn_b200.vsa import tiers as T
        nb = mask.shape[-1]
        scores = workloads.local_scores(sh["grid"], heads_all)[:, mine]
        rest = torch.where(mask, torch.full_like(scores, -1.0), scores).reshape(len(mine), nb * nb)
        n_b = int(round(0.20 * nb * nb))
        pick = torch.sort(rest, dim=1, descending=True, stable=True).indices[:, :n_b]
        tier_ab = mask.clone().reshape(len(mine), nb * nb).scatter_(1, pick, True).reshape(mask.shape)
        tsel = T.selection_from_masks(mask.to(device), tier_ab.to(device))
        cols = 64.0 * int(mask.sum()) + 4.0 * n_b * len(mine) + 1.0 * int((~tier_ab).sum())
        t_flop = 4.0 * 64 * 128 * cols

        def tier_fwd():
            with torch.no_grad():
                return T.rep_fine_attention(q, k, v, cnt, tsel, mid_reps=4)

        def tier_both():
            leaves = [x.detach().requires_grad_(True) for x in (q, k, v)]
            o, _ = T.rep_fine_attention(*leaves, cnt, tsel, mid_reps=4)
            return torch.autograd.grad(o, leaves, dout)
        ms_tf, _ = timed(tier_fwd, 3)
        ms_tfb, _ = timed(tier_both, 3)
        tiers_line = {"forward_ms": round(ms_tf, 4), "backward_ms": round(ms_tfb - ms_tf, 4),
                      "columns_per_query_row_mean": cols / (len(mine) * nb),
                      "forward_tflops": t_flop / ms_tf / 1e9, "backward_tflops": 2.5 * t_flop / (ms_tfb - ms_tf) / 1e9,
                      "frac_of_burst_peak_forward": t_flop / ms_tf / 1e9 / measured_peaks()["burst"],
                      "flop_rule": "4*64*D per (query block, column): 64 columns per tier-A block, 4 per tier-B block, 1 per "
                                   "tier-C block; backward 2.5 x"}
    extra = 0
    while sampler.count() < 3 and extra < 200:
        step(q, k, v, gate, dout)
        torch.cuda.synchronize()
        extra += 1
    clocks = sampler.stop()
    clocks["window"] = "warm-up + timed steps + kernel timings" + (f" + {extra} more steps" if extra else "")
    # ---- end to end: host buffers in, results out, every step
    ms_e2e, h2d, d2h = float("nan"), 0, 0
    if not args.no_e2e:
        host = [x.cpu().pin_memory() for x in (q, k, v, gate, dout)]
        dev = [torch.empty_like(x) for x in (q, k, v, gate, dout)]
        back = [torch.empty(x.shape, dtype=x.dtype).pin_memory() for x in (q, q, k, v, gate)]

        def e2e_step():
            for d, h in zip(dev, host):
                d.copy_(h, non_blocking=True)
            for b, r in zip(back, step(*dev)):
                b.copy_(r, non_blocking=True)
        e2e_step()
        barrier()
        e0.record()
        for _ in range(args.steps):
            e2e_step()
        e1.record()
        barrier()
        ms_e2e = e0.elapsed_time(e1)
        h2d = sum(x.numel() * x.element_size() for x in host)
        d2h = sum(x.numel() * x.element_size() for x in back)
    status = _native.device_status()
    stats = torch.tensor([ms, ms_e2e, fwd_flop + bwd_flop, float(launches), float(h2d), float(d2h), float(status), ms_f,
                          ms_kv + ms_q], device=device, dtype=torch.float64)
    flop_rank = fwd_flop + bwd_flop
    if dist is not None:
        mx, sm = stats.clone(), stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, ms_e2e, status = float(mx[0]), float(mx[1]), int(mx[6])
        flop_all, launches, h2d, d2h = float(sm[2]), int(sm[3]), int(sm[4]), int(sm[5])
    else:
        flop_all = flop_rank
    if rank != 0:
        dist.destroy_process_group()
        return
    if status != 0:
        raise SystemExit(f"a kernel reported status {status}; the numbers are void")
    peaks = measured_peaks()
    ms_step = ms / args.steps
    fwd_tf, bwd_tf = fwd_flop / ms_f / 1e9, bwd_flop / (ms_kv + ms_q) / 1e9
    line = {
        "metric": "vsa2_fwd_bwd_effective_tflops", "value": flop_all / ms_step / 1e9, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": vsa2_config(args, world),
        "run": {"pairs_per_rank": pairs, "list_length_mean": float(rows.float().mean()), "list_length_max": int(rows.max()),
                "algorithmic_tflop_per_step": flop_all / 1e12,
                "flop_rule": "fine branch only: forward 4*64*64*D per selected pair, backward 2.5 x (five products per pair)"},
        "clocks": clocks,
        "e2e": None if args.no_e2e else {"value": flop_all / (ms_e2e / args.steps) / 1e9, "unit": "TFLOP/s",
                                         "ms_per_step": ms_e2e / args.steps, "h2d_bytes_per_step": h2d,
                                         "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "kernel_ms": {"fine_forward": round(ms_f, 4), "fine_backward_kv": round(ms_kv, 4), "fine_backward_q": round(ms_q, 4)},
        "three_tier_fine_branch": tiers_line,
        "roofline": tensor_roofline("fine forward kernel (es_vsa_attn_fwd)", fwd_tf, ms_f, 5, clocks, peaks, traffic=None),
        "roofline_backward": tensor_roofline("fine backward kernels (es_vsa_attn_bwd_kv + es_vsa_attn_bwd_q)", bwd_tf,
                                             ms_kv + ms_q, 5, clocks, peaks, traffic=None),
    }
    if world == 1 and not args.no_cpu_baseline:
        from types import SimpleNamespace
        import contextlib
        import io
        buf = io.StringIO()
        with contextlib.redirect_stdout(buf):
            vsa2_reference_arm(SimpleNamespace(skew=args.skew, split=args.split, heads=args.heads, gpus=1, steps=1, warmup=0),
                               threads)
        line["cpu_baseline"] = json.loads(buf.getvalue())["cpu_baseline"]
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()



def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="wan_14b_720p", choices=sorted(synthetic.WORKLOADS) + ["vsa2_train"])
    ap.add_argument("--heads", type=int, default=0, help="use only the first N heads of the workload (0 = all)")
    ap.add_argument("--state", default="compact", choices=["compact", "layer"], help="what a layer keeps between steps")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer (end to end) measurement")
    ap.add_argument("--skew", default="uniform", help="vsa2_train: shape of the selection (vsa/workloads.py CASES)")
    ap.add_argument("--split", default="none", choices=["none", "auto", "manual"], help="vsa2_train: split-KV scheduling")
    ap.add_argument("--abba", default=None, choices=["baseline", "split_auto", "split_manual"],
                    help="vsa2_train: time this arm against the default in ABBA order and compare their outputs")
    ap.add_argument("--abba-tol", type=float, default=1e-2, help="relative L2 an arm's outputs may differ from the default's")
    ap.add_argument("--threshold", type=float, default=60.0, help="flag threshold on |log2 row sum| (reference: 60)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ulysses", action="store_true",
                    help="N > 1 only: the caller is sequence-sharded; q, k, v and the output cross the ranks inside the timed "
                         "region (this library's exchange kernel over peer memory), the attention itself stays head-sharded")
    ap.add_argument("--nccl-exchange", action="store_true",
                    help="--ulysses: run the exchanges as all_to_all_single between two layout copies instead")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference" and rank != 0:
        return
    threads = os.cpu_count() or 1
    if args.workload == "vsa2_train" and args.abba:
        return vsa2_abba(args, local) if rank == 0 else None
    if args.workload == "vsa2_train":
        return vsa2_reference_arm(args, threads) if args.impl == "reference" else vsa2_arm(args, rank, world, local, threads)
    grid, heads_all, branches, density, text = synthetic.WORKLOADS[args.workload]
    if args.impl == "reference":
        return reference_arm(args, threads)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU; there is no CPU fallback of the product path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    from self_trainable_or_free_attn_b200 import _native
    from self_trainable_or_free_attn_b200.kernels import sm100 as K

    attn, inputs, heads, injected = build_job(args, rank, world, device)
    L = inputs[0][1].shape[1]

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sink = sink_of(args.workload)
    if args.ulysses and dist is not None:
        # the caller's layout: this rank's tokens of every head. The exchange back to heads is part of every step.
        from self_trainable_or_free_attn_b200 import ulysses
        if L % world or heads_all % world:
            raise SystemExit(f"--ulysses needs tokens ({L}) and heads ({heads_all}) divisible by the ranks ({world})")
        inputs = [(tuple(ulysses.heads_to_seq(t) for t in q), ulysses.heads_to_seq(k), ulysses.heads_to_seq(v))
                  for q, k, v in inputs]
        attn_call = ulysses.UlyssesAttention(attn, peer_memory=not args.nccl_exchange)
        if attn_call.peer is not None:
            # the peer-memory exchange against the all-to-all between two layout copies, both directions, once
            q0 = inputs[0][1]
            a, b = attn_call.peer.seq_to_heads(q0, "check_in"), ulysses.seq_to_heads(q0)
            c, d = attn_call.peer.heads_to_seq(b, "check_out"), ulysses.heads_to_seq(b)
            torch.cuda.synchronize()
            if not (torch.equal(a, b) and torch.equal(c, d) and torch.equal(c, q0)):
                raise SystemExit("the peer-memory exchange differs from all_to_all_single")
    else:
        attn_call = attn

    # ---- warm-up, then the device-resident timed region. The clock sampler runs from the warm-up on (the same load), so
    # that a timed region of a few tens of milliseconds (many GPUs, few steps) still has samples.
    sampler = ClockSampler(local)
    sampler.start()
    run_steps(attn_call, inputs, 2, args.warmup, sink)
    names = ["sparse_attention", "block_attention", "exact_fallback", "compensate_fallback", "block_means", "select_blocks",
             "estimate_skipped", "full_step_scales", "reps_build", "pack_plan", "rebuild_plan"]
    timer = K.KernelTimer(names)
    barrier()
    K.set_kernel_timer(timer)
    launches0 = _native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    run_steps(attn_call, inputs, 2 + args.warmup, args.steps, sink)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = _native.launch_count() - launches0
    K.set_kernel_timer(None)
    def some_rank_wants_more():
        """The same answer on every rank (the steps of a sequence-sharded caller contain collectives, so every rank must
        run the same number of them)."""
        want = torch.tensor([1 if sampler.count() < 3 else 0], device=device, dtype=torch.int32)
        if dist is not None:
            dist.all_reduce(want, op=dist.ReduceOp.MAX)
        return bool(int(want[0]))

    extra = 0
    while extra < 40 and some_rank_wants_more():       # nvidia-smi needs ~0.3 s for its first lines: keep the load on
        run_steps(attn_call, inputs, 2 + args.warmup + args.steps + extra, 2, sink)
        torch.cuda.synchronize()
        extra += 2
    clocks = sampler.stop()
    clocks["window"] = "warm-up + timed steps" + (f" + {extra} more steps of the same load" if extra else "")
    kernel_ms = timer.ms("sparse_attention")
    flops_rank = layer_flops(attn, inputs, L)
    flagged = int(attn._states[(0, 1)].flags.sum())          # last call of the timed steps (the last branch)

    # ---- end to end: host buffers, H2D of q, k, v and D2H of the output inside the timed region, double-buffered
    host_node, host_in, host_out, dev_in = None, None, None, None
    if not args.no_e2e:
        host_node = bind_host_to_gpu_node(device.index if device.index is not None else torch.cuda.current_device())
        host_in = [[[t.cpu().pin_memory() for t in q], k.cpu().pin_memory(), v.cpu().pin_memory()] for q, k, v in inputs]
        host_out = [torch.empty(k.shape, dtype=torch.bfloat16).pin_memory() for _, k, _ in inputs]
        dev_in = [[torch.empty_like(inputs[0][1]) for _ in range(3)] for _ in range(2)]
    copy_stream = torch.cuda.Stream()           # host -> device
    back_stream = torch.cuda.Stream()           # device -> host: its own stream, PCIe carries both directions at once
    main_stream = torch.cuda.current_stream()

    def e2e_steps(first_step, n):
        seq = [(first_step + i, b) for i in range(n) for b in range(branches)]
        ready = [torch.cuda.Event() for _ in seq]
        freed = [torch.cuda.Event() for _ in seq]
        for j, (step, b) in enumerate(seq):
            slot = j % 2
            with torch.cuda.stream(copy_stream):
                if j >= 2:
                    copy_stream.wait_event(freed[j - 2])         # the slot's previous user has finished
                hq, hk, hv = host_in[b]
                for d, s in zip(dev_in[slot], (hq[step & 1], hk, hv)):
                    d.copy_(s, non_blocking=True)
                ready[j].record(copy_stream)
            main_stream.wait_event(ready[j])
            out = attn_call(*dev_in[slot], step, b, layer=1, sink=sink)
            freed[j].record(main_stream)
            done = torch.cuda.Event()
            done.record(main_stream)
            with torch.cuda.stream(back_stream):
                back_stream.wait_event(done)
                host_out[b].copy_(out, non_blocking=True)
                out.record_stream(back_stream)
        main_stream.wait_stream(copy_stream)
        main_stream.wait_stream(back_stream)

    ms_e2e = float("nan")
    if not args.no_e2e:
        e2e_steps(2 + args.warmup + args.steps, 1)
        barrier()
        e0.record()
        e2e_steps(3 + args.warmup + args.steps, args.steps)
        e1.record()
        barrier()
        ms_e2e = e0.elapsed_time(e1)
    # the exchanges of a sequence-sharded caller alone: q, k, v in and the output back, both branches, as in one step
    exchange = None
    if args.ulysses and dist is not None:
        from self_trainable_or_free_attn_b200 import ulysses
        outs = [torch.empty(1, L, len(heads), 128, device=device, dtype=torch.bfloat16) for _ in inputs]

        def exchanges():
            for (q, k, v), o in zip(inputs, outs):
                if attn_call.peer is not None:
                    for t, role in ((q[0], "q"), (k, "k"), (v, "v")):
                        attn_call.peer.seq_to_heads(t, role)
                    attn_call.peer.heads_to_seq(o, "out")
                else:
                    for t in (q[0], k, v):
                        ulysses.seq_to_heads(t)
                    ulysses.heads_to_seq(o)
        exchanges()
        barrier()
        e0.record()
        for _ in range(5):
            exchanges()
        e1.record()
        barrier()
        ms_x = e0.elapsed_time(e1) / 5
        sent = sum(4 * k.numel() * 2 for _, k, _ in inputs) * (world - 1) // world      # bytes this rank sends to its peers
        xs = torch.tensor([ms_x], device=device, dtype=torch.float64)
        dist.all_reduce(xs, op=dist.ReduceOp.MAX)
        exchange = {"path": "all_to_all_single between two layout copies (NCCL)" if attn_call.peer is None else
                            "es_exchange_rows into the peers' receive buffers (peer memory) + a 4-byte all-reduce",
                    "exchanges_per_step": 4 * len(inputs), "ms_per_step": float(xs[0]),
                    "bytes_sent_per_rank_per_step": sent, "gb_per_s_per_rank_per_direction": sent / float(xs[0]) / 1e6,
                    "how": "the exchanges of a step (q, k, v in, the output back, every branch) timed alone, max over ranks"}
    # dense steps of branch 0: the first of a video (online softmax over every block) and one that follows it (the previous
    # step's LSE as a fixed offset over every block, flagged tiles recomputed)
    attn.reset()
    q0, k0, v0 = inputs[0]
    attn_call(q0[0], k0, v0, 0, 0, layer=1, sink=sink)
    attn.reset()
    torch.cuda.synchronize()
    e0.record()
    attn_call(q0[0], k0, v0, 0, 0, layer=1, sink=sink)
    e1.record()
    torch.cuda.synchronize()
    ms_dense_first = e0.elapsed_time(e1)
    e0.record()
    attn_call(q0[0], k0, v0, 0, 0, layer=1, sink=sink)
    e1.record()
    torch.cuda.synchronize()
    ms_dense = e0.elapsed_time(e1)
    status = _native.device_status()
    h2d = sum(3 * k.numel() * 2 for _, k, _ in inputs)
    d2h = sum(k.numel() * 2 for _, k, _ in inputs)

    # ---- whole-job numbers: max time over ranks, sum of work
    stats = torch.tensor([ms, ms_e2e, flops_rank, float(launches), float(h2d), float(d2h), float(status),
                          float(flagged), float(injected)], device=device, dtype=torch.float64)
    if dist is not None:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, ms_e2e, status = float(mx[0]), float(mx[1]), int(mx[6])
        flops_all, launches, h2d, d2h = float(sm[2]), int(sm[3]), int(sm[4]), int(sm[5])
        flagged, injected = int(sm[7]), int(sm[8])
    else:
        flops_all = flops_rank
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    if status != 0:
        raise SystemExit(f"a kernel reported status {status}: a bounded wait gave up; the numbers are void")

    peaks = measured_peaks()
    ms_step = ms / args.steps
    value = flops_all / (ms_step * 1e-3) / 1e12
    k_ms = statistics.mean(kernel_ms)
    k_flops = flops_rank / len(inputs)
    achieved = k_flops / (k_ms * 1e-3) / 1e12
    # DRAM bytes of one launch: Nsight Compute measured 332.97 MB read + 95.17 MB written on the 32,760-token, 12-head
    # case (1.06 x the compulsory q, k, v, out bytes); the traffic grows with tokens x heads
    traffic = 428.14e6 * (L * len(heads)) / (32760 * 12)
    line = {
        "metric": "sparse_attn_effective_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, world),
        "run": {"state": args.state, "algorithmic_tflop_per_step": flops_all / 1e12, "fallback_tiles_injected": injected,
                "fallback_tiles_flagged_last_call": flagged},
        "clocks": clocks,
        "e2e": None if args.no_e2e else {
            "value": flops_all / (ms_e2e / args.steps * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e / args.steps,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "host_numa_node": host_node},
        "gpu_launches": launches,
        "kernel_ms_per_step": {n: round(sum(timer.ms(n)) / args.steps, 3) for n in names if timer.events[n]},
        "dense_step_ms_per_branch": round(ms_dense, 3),
        "dense_first_step_ms_per_branch": round(ms_dense_first, 3),
        "ulysses_exchange": exchange,
        "roofline": tensor_roofline(
            "attention_kernel<0> (es_sparse_attention)", achieved, k_ms, len(kernel_ms), clocks, peaks, traffic=traffic,
            traffic_source="dram__bytes_read.sum + dram__bytes_write.sum of one launch captured at the Wan-1.3B shape "
                           "(428.1 MB), scaled by tokens x heads (q, k, v read once, out written once)"),
    }
    if world == 1 and not args.no_cpu_baseline:
        tf, sample, dt = cpu_sample(args.workload, args.cpu_seconds, threads)
        line["cpu_baseline"] = {"value": tf[0], "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample,
                                "seconds": dt}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
