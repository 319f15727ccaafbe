"""Benchmark of the EchoSparse sparse-step attention layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A step is one sparse-step attention layer: both CFG branches through `EchoSparseAttention.__call__` (select, block
means, representatives, fused sparse attention, fallback, estimates). Default workload: the Wan2.1-14B 720p shape
(2 branches x 40 heads x 75,600 tokens, 10 % of the blocks kept, ~0.5 % of the tiles pushed into the online-softmax
fallback). With N GPUs the heads are sharded (both branches of a head on one GPU), no collective in the data path.
Rank 0 prints one JSON line. Inputs are seeded synthetic activations (see `synthetic.py`).

`--impl reference` times the CPU restatement of the same step (oracle/echosparse_ref.py) on the host cores, on a bounded
sample of query tiles of the same workload.
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
        return {"tflops": float(d["bf16_tflops_sustained"]), "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


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
    heads = synthetic.shard_heads(heads_all, rank, world)
    attn = EchoSparseAttention(density=density, dense_steps=2, dense_layers=(), refine_iters=6,
                               threshold=args.threshold, min_blocks=1)
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
            "config": {"workload": args.workload, "tokens": synthetic.grid_tokens(grid) + text, "heads": heads_all,
                       "branches": branches, "density": density,
                       "step": "fused sparse step on host cores; ms_per_step extrapolates the sample's throughput to the "
                               "layer's nominal algorithmic FLOP"},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="wan_14b_720p", choices=sorted(synthetic.WORKLOADS))
    ap.add_argument("--threshold", type=float, default=60.0, help="flag threshold on |log2 row sum| (reference: 60)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ulysses", action="store_true",
                    help="N > 1 only: the caller is sequence-sharded; q, k, v and the output cross the ranks by all-to-all "
                         "(NCCL) inside the timed region, the attention itself stays head-sharded")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference" and rank != 0:
        return
    grid, heads_all, branches, density, text = synthetic.WORKLOADS[args.workload]
    threads = os.cpu_count() or 1
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
        attn_call = ulysses.UlyssesAttention(attn)
    else:
        attn_call = attn

    # ---- warm-up, then the device-resident timed region. The clock sampler runs from the warm-up on (the same load), so
    # that a timed region of a few tens of milliseconds (many GPUs, few steps) still has samples.
    sampler = ClockSampler(local)
    sampler.start()
    run_steps(attn_call, inputs, 2, args.warmup, sink)
    names = ["sparse_attention", "block_attention", "exact_fallback", "compensate_fallback", "block_means", "select_blocks",
             "estimate_skipped", "full_step_scales", "reps_build"]
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
    extra = 0
    while sampler.count() < 3 and extra < 40:          # nvidia-smi needs ~0.3 s for its first lines: keep the load on
        run_steps(attn_call, inputs, 2 + args.warmup + args.steps + extra, 2, sink)
        torch.cuda.synchronize()
        extra += 2
    clocks = sampler.stop()
    clocks["window"] = "warm-up + timed steps" + (f" + {extra} more steps of the same load" if extra else "")
    kernel_ms = timer.ms("sparse_attention")
    status = _native.device_status()
    flops_rank = layer_flops(attn, inputs, L)
    flagged = int(attn._states[(0, 1)].flags.sum())          # branch 0, last timed step

    # ---- end to end: host buffers, H2D of q, k, v and D2H of the output inside the timed region, double-buffered
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

    e2e_steps(2 + args.warmup + args.steps, 1)
    barrier()
    e0.record()
    e2e_steps(3 + args.warmup + args.steps, args.steps)
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
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
        "config": {"workload": args.workload, "tokens": L, "heads": heads_all, "branches": branches, "density": density,
                   "partition": (f"heads over {world} GPU(s), both CFG branches of a head together"
                                 + ("; sequence-sharded caller: q, k, v and the output cross the ranks by NCCL all-to-all every "
                                    "step (Ulysses)" if args.ulysses and world > 1 else "")),
                   "step": "select + block means + representatives + fused sparse attention + fallback + estimates, "
                           "both branches", "algorithmic_tflop_per_step": flops_all / 1e12,
                   "l2": "inputs (q, k, v of a branch >> 126 MB) exceed L2 between iterations",
                   "fallback_tiles_injected": injected, "fallback_tiles_flagged_last_step_branch0": flagged,
                   "flag_threshold_log2": args.threshold},
        "clocks": clocks,
        "e2e": {"value": flops_all / (ms_e2e / args.steps * 1e-3) / 1e12, "unit": "TFLOP/s",
                "ms_per_step": ms_e2e / args.steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "host_numa_node": host_node},
        "gpu_launches": launches,
        "kernel_ms_per_step": {n: round(sum(timer.ms(n)) / args.steps, 3) for n in names if timer.events[n]},
        "roofline": {"bound": "tensor", "kernel": "attention_kernel<0> (es_sparse_attention)", "achieved": achieved,
                     "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["tflops"],
                     "peak_source": f"bf16_tflops_sustained of {peaks['source']}", "ms_per_launch": k_ms,
                     "launches_timed": len(kernel_ms), "traffic": traffic,
                     "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch captured at the "
                                       "Wan-1.3B shape (428.1 MB), scaled by tokens x heads (q, k, v read once, out "
                                       "written once)"},
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
