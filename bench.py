"""Benchmark of the quantized-weight hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (config.workload "ffn_matvec_set_b1"): the Q4_K_M FFN matvec set at
batch 1 -- gate and up [12288 x 4096] in Q4_K and down [4096 x 12288] in Q6_K,
weights N(0, 0.02) before quantization, activations N(0, 1), f32 -- one "step"
being the three matvecs over ONE of several distinct resident weight
instances, so that every step streams its weights from HBM rather than L2.
The three products of a step are submitted as one list (lev_matvec_chain):
one launch of the persistent kernel.

Metric: algorithmic bytes (GGUF block bytes of the three tensors plus the f32
vectors) per second.  `value` is timed with the activations already on the
device (a CUDA graph of K steps, CUDA events); `e2e` is timed through the
C-ABI host-pointer calls with pinned host buffers, copies inside the timed
region.  `--impl reference` times the CPU restatement of the reference's own
matvec loops on the host cores for the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

HIDDEN, FFN = 4096, 12288
Q4_K, Q6_K = 12, 14
GATE_BYTES = FFN * (HIDDEN // 256) * 144      # 28,311,552
DOWN_BYTES = HIDDEN * (FFN // 256) * 210      # 41,287,680
VEC_BYTES = 4 * (HIDDEN + 2 * FFN + FFN + HIDDEN)  # x, gate out, up out, down in, down out
STEP_BYTES = 2 * GATE_BYTES + DOWN_BYTES + VEC_BYTES  # 98,091,008
SEED = 0x4C455649
# dram__bytes_read + dram__bytes_write of one launch of the persistent kernel over the three tensors of a
# step, from the ncu capture summarised in profiles/k_chain_ffn_set_full_capture.txt (None: not captured)
CHAIN_DRAM_TRAFFIC = 101_772_800


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples during the timed region."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.proc, self.lines = device, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.device)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [s.strip() for s in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_inputs():
    from leviathan_b200 import quant as Q

    x = Q.normal(SEED ^ 0x100, (HIDDEN,), 1.0)
    a = Q.normal(SEED ^ 0x101, (FFN,), 1.0)
    return x, a


def tensor_seed(instance: int, j: int) -> int:
    """Seed of tensor j (0 gate, 1 up, 2 down) of weight instance `instance`: 0x4C455649 ^ tensor index."""
    return SEED ^ (16 * instance + j)


def make_instance(i: int, device: str):
    """Quantized gate/up/down of weight instance i (uint8 tensors on `device`): N(0, 0.02) from
    SplitMix64(tensor_seed) by Box-Muller, the same generator on both arms (numpy on the host,
    the identical integer arithmetic in torch on the GPU)."""
    import torch

    from leviathan_b200 import quant as Q

    out = []
    for j, (t, rows, cols) in enumerate(((Q4_K, FFN, HIDDEN), (Q4_K, FFN, HIDDEN), (Q6_K, HIDDEN, FFN))):
        if device == "cpu":
            w = torch.from_numpy(Q.normal(tensor_seed(i, j), (rows, cols), 0.02))
        else:
            w = Q.normal_torch(tensor_seed(i, j), (rows, cols), 0.02, device=device)
        out.append(Q.quantize(t, w))
        del w
    return out


# ---------------------------------------------------------------------------
# CPU arm: the oracle's threaded matvec (the reference's own CPU loops)
# ---------------------------------------------------------------------------

def cpu_step_timer(threads: int | None, steps: int, warmup: int, tensors=None):
    from oracle import oracle as O

    native = None
    try:
        native = O.build(native_out=os.path.join(tempfile.gettempdir(), "lev_oracle_native"))
    except Exception:
        native = None
    threads = threads or O.hardware_threads()
    gate, up, down = tensors if tensors is not None else [t.numpy() for t in make_instance(0, "cpu")]
    x, a = make_inputs()

    def step():
        O.matvec_threaded(Q4_K, gate, FFN, HIDDEN, x, threads, lib_path=native)
        O.matvec_threaded(Q4_K, up, FFN, HIDDEN, x, threads, lib_path=native)
        O.matvec_threaded(Q6_K, down, HIDDEN, FFN, a, threads, lib_path=native)

    for _ in range(warmup):
        step()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    return times, threads, ("native" if native else "portable")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 20))
    times, threads, build = cpu_step_timer(None, steps, max(1, min(args.warmup, 3)))
    ms = 1000.0 * sum(times) / len(times)
    value = STEP_BYTES / (ms * 1e-3) / 1e9
    line = {
        "impl": "reference", "metric": "Q4/Q6 matvec HBM GB/s", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "ffn_matvec_set_b1", "gate_up": "Q4_K 12288x4096 x2", "down": "Q6_K 4096x12288",
                   "columns": 1, "bytes_per_step": STEP_BYTES},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"{steps} full steps of the same three matvecs, oracle C port ({build} build), "
                                   "row chunks over all host threads"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------

def run_gpu(args):
    import torch
    import torch.distributed as dist

    import leviathan_b200 as lev

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    ctx = lev.Context(local)

    # One GPU: whole tensors.  Several GPUs: the output rows of every tensor are split over the ranks
    # (each rank holds rows [rank * R / N, (rank + 1) * R / N) of the SAME instances), a step is the same
    # three products, and every rank ends the step with the whole outputs: the slices travel as peer
    # stores over NVLink (lev_matvec_chain_rowsplit).  Strong scaling: the work of a step is fixed.
    from leviathan_b200 import dist as D

    if world > 1:
        D.init_from_torch(ctx)
    n_inst = args.instances
    inst = []
    for i in range(n_inst):
        g, u, d = make_instance(i, dev)
        if world > 1:
            r0, nr = D.row_shard(FFN, rank, world)
            d0, dn_ = D.row_shard(HIDDEN, rank, world)
            g = D.slice_blocks(g, Q4_K, FFN, HIDDEN, r0, nr).clone()
            u = D.slice_blocks(u, Q4_K, FFN, HIDDEN, r0, nr).clone()
            d = D.slice_blocks(d, Q6_K, HIDDEN, FFN, d0, dn_).clone()
            inst.append((ctx.upload(g, Q4_K, nr, HIDDEN), ctx.upload(u, Q4_K, nr, HIDDEN), ctx.upload(d, Q6_K, dn_, FFN)))
        else:
            inst.append((ctx.upload(g, Q4_K, FFN, HIDDEN), ctx.upload(u, Q4_K, FFN, HIDDEN),
                         ctx.upload(d, Q6_K, HIDDEN, FFN)))
        del g, u, d
    torch.cuda.empty_cache()
    x_h, a_h = make_inputs()
    x = torch.from_numpy(x_h).to(dev)
    a = torch.from_numpy(a_h).to(dev)
    yg = torch.empty(FFN, device=dev)
    yu = torch.empty(FFN, device=dev)
    yd = torch.empty(HIDDEN, device=dev)

    def step(i):
        wg, wu, wd = inst[i % n_inst]
        ops = [dict(w=wg, x=x, out=yg), dict(w=wu, x=x, out=yu), dict(w=wd, x=a, out=yd)]
        if world > 1:
            ctx.matvec_chain_rowsplit(ops)
        else:
            ctx.matvec_chain(ops)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # warm-up (also sizes every scratch buffer before capture)
    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    l0 = ctx.launch_count()
    step(0)
    launches_per_step = ctx.launch_count() - l0
    chain_kernel = ctx.last_evidence()["kernel_name"]
    torch.cuda.synchronize()
    yg_step0, yd_step0 = yg[:64].cpu().numpy(), yd[:64].cpu().numpy()  # for the parity spot check below

    # K steps as one CUDA graph on a side stream; timed with events on that stream
    s = torch.cuda.Stream(device=dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        with torch.cuda.graph(graph, stream=s):
            for i in range(args.steps):
                step(i)
    with torch.cuda.stream(s):
        for _ in range(max(args.warmup, 3)):
            graph.replay()
    torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    reps = args.reps
    e0 = [torch.cuda.Event(enable_timing=True) for _ in range(reps)]
    e1 = [torch.cuda.Event(enable_timing=True) for _ in range(reps)]
    barrier()
    with torch.cuda.stream(s):
        for r in range(reps):
            e0[r].record(s)
            graph.replay()
            e1[r].record(s)
    barrier()
    rep_ms = [a_.elapsed_time(b_) for a_, b_ in zip(e0, e1)]
    ms_per_step = statistics.median(rep_ms) / args.steps
    ms_per_step_min = min(rep_ms) / args.steps

    # per-kernel launch durations for the roofline: separate graphs of one kernel type
    def time_kernel(which):
        g2 = torch.cuda.CUDAGraph()
        n = 4 * n_inst
        with torch.cuda.stream(s):
            with torch.cuda.graph(g2, stream=s):
                for i in range(n):
                    wg, wu, wd = inst[i % n_inst]
                    if which == "q4_k":
                        ctx.matvec(wg if i % 2 == 0 else wu, x, out=yg.view(1, -1))
                    else:
                        ctx.matvec(wd, a, out=yd.view(1, -1))
            for _ in range(3):
                g2.replay()
            ts = []
            for _ in range(7):
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record(s)
                g2.replay()
                a1.record(s)
                a1.synchronize()
                ts.append(a0.elapsed_time(a1) / n)
        return statistics.median(ts)

    k_q4k_ms = time_kernel("q4_k")
    k_q6k_ms = time_kernel("q6_k")
    clocks = sampler.stop() if rank == 0 else None

    # e2e: host buffers through the C-ABI host-pointer path, weights resident
    xp = torch.from_numpy(x_h).pin_memory()
    ap = torch.from_numpy(a_h).pin_memory()
    ygp = torch.empty(1, FFN).pin_memory()
    yup = torch.empty(1, FFN).pin_memory()
    ydp = torch.empty(1, HIDDEN).pin_memory()

    xpn, apn, ygn, yun, ydn = xp.numpy(), ap.numpy(), ygp.numpy().reshape(-1), yup.numpy().reshape(-1), ydp.numpy().reshape(-1)

    # the lev_chain_op arrays of the host-buffer lists, one per weight instance, built once: the timed call is the
    # C entry point itself, as a Swift or C host makes it, not this file's argument marshalling
    host_lists = [ctx.chain_prepare([dict(w=wg, x=xpn, out=ygn), dict(w=wu, x=xpn, out=yun), dict(w=wd, x=apn, out=ydn)])
                  for wg, wu, wd in inst] if world == 1 else None

    def e2e_step(i):
        wg, wu, wd = inst[i % n_inst]
        if world == 1:
            # the same list through the host-buffer form of the C ABI: inputs copied in, one launch,
            # outputs copied back, one synchronisation
            ctx.chain_submit(host_lists[i % n_inst])
        else:
            # several GPUs: pinned host inputs to the device, the row-split list, whole outputs back
            x.copy_(xp, non_blocking=True)
            a.copy_(ap, non_blocking=True)
            step(i)
            ygp.view(-1).copy_(yg, non_blocking=True)
            yup.view(-1).copy_(yu, non_blocking=True)
            ydp.view(-1).copy_(yd, non_blocking=True)
            torch.cuda.synchronize()

    # like the device-side figure: the median of `reps` rounds of exactly K steps each, wall clock around a round
    for i in range(max(3, args.warmup)):
        e2e_step(i)
    rounds = []
    for _ in range(args.reps):
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            e2e_step(i)
        barrier()
        rounds.append(1000.0 * (time.perf_counter() - t0) / args.steps)
    e2e_ms = statistics.median(rounds)

    if world > 1:
        t = torch.tensor([ms_per_step, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_per_step, e2e_ms = t.tolist()

    # parity spot check of what was timed (sampled rows against the oracle)
    parity = None
    if rank == 0 and not args.no_check:
        from oracle import oracle as O

        g_bytes = make_instance(0, dev)
        # the host form of the generator gives the same bytes as the device form the GPU arm uses
        from leviathan_b200 import quant as Q

        head = Q.quantize(Q4_K, torch.from_numpy(Q.normal(tensor_seed(0, 0), (64, HIDDEN), 0.02)))
        generator_match = bool(torch.equal(head, g_bytes[0][: head.numel()].cpu()))
        rows = 64
        sub = g_bytes[0][: rows * (HIDDEN // 256) * 144].cpu().numpy()
        ref = O.q4_k_matvec_f64(sub, rows, HIDDEN, x_h)
        subd = g_bytes[2][: rows * (FFN // 256) * 210].cpu().numpy()
        refd = O.q6_k_matvec_f64(subd, rows, FFN, a_h)
        parity = {"host_and_device_generators_give_the_same_bytes": generator_match,
                  "q4_k_max_rel_err_64_rows": O.max_rel_err(yg_step0, ref),
                  "q6_k_max_rel_err_64_rows": O.max_rel_err(yd_step0, refd)}

    if rank == 0:
        peaks, peak_kind = _peaks()
        value = STEP_BYTES / (ms_per_step * 1e-3) / 1e9  # one step is the whole job at every N
        q4k_bytes = GATE_BYTES + 4 * (HIDDEN + FFN)
        q6k_bytes = DOWN_BYTES + 4 * (HIDDEN + FFN)
        ach = STEP_BYTES / (ms_per_step * 1e-3) / 1e9
        line = {
            "metric": "Q4/Q6 matvec HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "ms_per_step_min": ms_per_step_min,
            "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "ffn_matvec_set_b1", "gate_up": "Q4_K 12288x4096 x2", "down": "Q6_K 4096x12288",
                       "columns": 1, "bytes_per_step": STEP_BYTES, "weight_instances_per_gpu": n_inst,
                       "l2": f"inputs larger than L2: {n_inst} distinct instances = {n_inst * STEP_BYTES / 1e6:.0f} MB "
                             "cycled, one per step", "timing": f"median of {reps} replays of a {args.steps}-step CUDA graph",
                       "generator": "SplitMix64 + Box-Muller, seed 0x4C455649 ^ (16 * instance + tensor); x seed ^ 0x100, "
                                    "down input seed ^ 0x101",
                       "sharding": "one GPU" if world == 1 else
                                   f"output rows of every tensor split over {world} ranks; every rank ends a step with the whole "
                                   f"outputs (slices pushed as peer stores over NVLink, bounded flag waits; "
                                   f"peer memory mapped: {bool(ctx.lib.lev_dist_peer_memory(ctx.handle))})"},
            # the dominant kernel is the one launch of a step: the persistent kernel over the three tensors
            "roofline": {"bound": "hbm", "kernel": chain_kernel + ":k_chain(gate, up, down)",
                         "achieved": ach, "peak": peaks["hbm_gbs"], "peak_source": peak_kind, "unit": "GB/s",
                         "frac": ach / peaks["hbm_gbs"], "traffic": CHAIN_DRAM_TRAFFIC, "us_per_launch": ms_per_step * 1e3,
                         "algorithmic_bytes_per_launch": STEP_BYTES,
                         "single_tensor_launches": {
                             "q4_k": {"achieved": q4k_bytes / (k_q4k_ms * 1e-3) / 1e9, "us_per_launch": k_q4k_ms * 1e3,
                                      "frac": q4k_bytes / (k_q4k_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                      "algorithmic_bytes_per_launch": q4k_bytes},
                             "q6_k": {"achieved": q6k_bytes / (k_q6k_ms * 1e-3) / 1e9, "us_per_launch": k_q6k_ms * 1e3,
                                      "frac": q6k_bytes / (k_q6k_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                      "algorithmic_bytes_per_launch": q6k_bytes}}},
            "e2e": {"value": STEP_BYTES / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": 4 * (HIDDEN + HIDDEN + FFN), "d2h_bytes_per_step": 4 * (FFN + FFN + HIDDEN)},
            "gpu_launches": launches_per_step * args.steps * reps,
            "clocks": clocks, "parity": parity,
        }
        if not args.no_cpu and world == 1:
            # instance 0 as the GPU arm generated it (the same bytes as the host generator gives)
            times, threads, build = cpu_step_timer(None, 11, 3, [t.cpu().numpy() for t in make_instance(0, dev)])
            cms = statistics.median(times)
            line["cpu_baseline"] = {"value": STEP_BYTES / cms / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                                    "sample": f"11 full steps (median) of the same three matvecs, oracle C port "
                                              f"({build} build), row chunks over all host threads"}
    # Side measurements come last and under a watchdog: if they fail or stall on any rank (they use
    # collectives), the headline line is still printed and every rank leaves.
    line_ref = line if rank == 0 else None

    def emit(extras):
        if rank == 0:
            line_ref["extras"] = extras
            print(json.dumps(line_ref), flush=True)

    if args.no_extras:
        emit(None)
    else:
        def bail():
            emit({"error": "side measurements did not finish within 240 s"})
            os._exit(0)

        timer = threading.Timer(240.0, bail)
        timer.daemon = True
        timer.start()
        try:
            extras = run_extras(ctx, inst[0][0], dev, s, world, rank)
        except Exception as exc:  # noqa: BLE001 -- reported in the JSON line
            extras = {"error": repr(exc)[:300]}
        timer.cancel()
        emit(extras)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
# side measurements (not part of `value`): prefill dequant-GEMM and the routed MoE layer
# ---------------------------------------------------------------------------

MOE_EXPERTS, MOE_HIDDEN, MOE_INTER, MOE_TOPK = 128, 2816, 704, 8
MOE_EXPERT_BYTES = (2 * MOE_INTER * (MOE_HIDDEN // 32) + MOE_HIDDEN * (MOE_INTER // 32)) * 18  # 3,345,408
MOE_ROUTER_BYTES = MOE_EXPERTS * MOE_HIDDEN * 4


def _graph_time(torch, stream, fn, iters, reps=7):
    """Median milliseconds per call of fn(i), i = 0..iters-1 captured as one CUDA graph."""
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        for i in range(min(iters, 3)):
            fn(i)
        stream.synchronize()
        with torch.cuda.graph(g, stream=stream):
            for i in range(iters):
                fn(i)
        for _ in range(3):
            g.replay()
        ts = []
        for _ in range(reps):
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record(stream)
            g.replay()
            a1.record(stream)
            a1.synchronize()
            ts.append(a0.elapsed_time(a1) / iters)
    return statistics.median(ts)


def run_extras(ctx, w_gate, dev, stream, world, rank):
    """Prefill GEMM (512 tokens x the Q4_K gate tensor) and the 128-expert top-8 MoE layer at
    1 / 32 / 512 tokens; with more than one rank the experts are sharded and the layer runs
    expert-parallel.  Every rank takes part, rank 0 reports."""
    import torch

    from leviathan_b200 import quant as Q

    peaks, _ = _peaks()
    out = {}
    if world == 1:
        g = torch.Generator(device=dev).manual_seed(SEED ^ 0x300)
        xs = [torch.randn((512, HIDDEN), generator=g, device=dev).to(torch.bfloat16) for _ in range(4)]
        y = torch.empty((512, FFN), device=dev)
        ms = _graph_time(torch, stream, lambda i: ctx.gemm_prefill(w_gate, xs[i % 4], out=y), 8)
        flop = 2.0 * 512 * HIDDEN * FFN
        out["prefill_gemm"] = {"workload": "X bf16 [512x4096] x Q4_K [12288x4096]", "ms": ms,
                               "tflops": flop / ms / 1e9, "peak_tflops_sustained": peaks["bf16_tflops_sustained"],
                               "tensor_frac": flop / ms / 1e9 / peaks["bf16_tflops_sustained"]}
    if world == 1:
        # cfg1: one Q4_0 [4096 x 4096] matvec, 64 distinct instances (604 MB) cycled in one graph
        c1 = []
        for i in range(64):
            wf = Q.normal_torch(SEED ^ (0x2000 + i), (4096, 4096), 0.02, device=dev)
            c1.append(ctx.upload(Q.quantize(2, wf), 2, 4096, 4096))
        del wf
        x1 = torch.from_numpy(Q.normal(SEED ^ 0x200, (1, 4096), 1.0)).to(dev)
        y1 = torch.empty((1, 4096), device=dev)
        y64 = torch.empty((64, 4096), device=dev)
        # the same 64 products submitted as four lists of sixteen (one launch each)
        ms16 = _graph_time(torch, stream, lambda i: ctx.matvec_chain(
            [dict(w=c1[(16 * i + j) % 64], x=x1[0], out=y64[(16 * i + j) % 64]) for j in range(16)]), 4, reps=11) / 16
        g1 = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            for i in range(3):
                ctx.matvec(c1[i], x1, out=y1)
            stream.synchronize()
            with torch.cuda.graph(g1, stream=stream):
                for i in range(64):
                    ctx.matvec(c1[i], x1, out=y1)
            for _ in range(3):
                g1.replay()
            ts = []
            for _ in range(11):
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record(stream)
                g1.replay()
                a1.record(stream)
                a1.synchronize()
                ts.append(a0.elapsed_time(a1) / 64)
            # one launch on an idle stream
            singles = []
            for i in range(8):
                stream.synchronize()
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record(stream)
                ctx.matvec(c1[8 + i], x1, out=y1)
                a1.record(stream)
                a1.synchronize()
                singles.append(a0.elapsed_time(a1))
        b1 = 4096 * 128 * 18 + 2 * 4096 * 4
        med, mn = statistics.median(ts), min(ts)
        out["cfg1_q4_0_matvec"] = {"workload": "Q4_0 [4096x4096], batch 1, 64 instances cycled", "us_median": med * 1e3,
                                   "us_min": mn * 1e3, "gbs": b1 / med / 1e6, "hbm_frac": b1 / med / 1e6 / peaks["hbm_gbs"],
                                   "single_launch_us": statistics.median(singles) * 1e3,
                                   "us_in_lists_of_16": ms16 * 1e3, "gbs_in_lists_of_16": b1 / ms16 / 1e6,
                                   "hbm_frac_in_lists_of_16": b1 / ms16 / 1e6 / peaks["hbm_gbs"]}
        for w1 in c1:
            w1.free()
        # the same FFN set with gate and up row-concatenated into one resident tensor: two launches
        # per step instead of three (a packing choice of the host, same bytes and arithmetic)
        fused = []
        for i in range(4):
            gq, uq, dq = make_instance(100 + i, dev)
            fused.append((ctx.upload(torch.cat([gq, uq]), Q4_K, 2 * FFN, HIDDEN), ctx.upload(dq, Q6_K, HIDDEN, FFN)))
            del gq, uq, dq
        x_h, a_h = make_inputs()
        xd, ad = torch.from_numpy(x_h).to(dev), torch.from_numpy(a_h).to(dev)
        ygu, ydn = torch.empty((1, 2 * FFN), device=dev), torch.empty((1, HIDDEN), device=dev)

        def fused_step(i):
            wgu, wd = fused[i % 4]
            ctx.matvec(wgu, xd, out=ygu)
            ctx.matvec(wd, ad, out=ydn)

        ms = _graph_time(torch, stream, fused_step, 16)
        out["ffn_gate_up_concatenated"] = {"launches_per_step": 2, "ms_per_step": ms, "gbs": STEP_BYTES / ms / 1e6,
                                           "hbm_frac": STEP_BYTES / ms / 1e6 / peaks["hbm_gbs"]}
        # the set through lev_matvec_multi: gate and up stay separate resident tensors, one launch
        sep = []
        for i in range(4):
            gq, uq, dq = make_instance(200 + i, dev)
            sep.append((ctx.upload(gq, Q4_K, FFN, HIDDEN), ctx.upload(uq, Q4_K, FFN, HIDDEN), ctx.upload(dq, Q6_K, HIDDEN, FFN)))
            del gq, uq, dq
        yg2, yu2 = torch.empty((1, FFN), device=dev), torch.empty((1, FFN), device=dev)

        def multi_step(i):
            wg, wu, wd = sep[i % 4]
            ctx.matvec_multi([wg, wu], xd, outs=[yg2, yu2])
            ctx.matvec(wd, ad, out=ydn)

        ms = _graph_time(torch, stream, multi_step, 16)
        xp, ap_ = torch.from_numpy(x_h).pin_memory(), torch.from_numpy(a_h).pin_memory()
        ygp, yup, ydp = (torch.empty(1, FFN).pin_memory(), torch.empty(1, FFN).pin_memory(), torch.empty(1, HIDDEN).pin_memory())

        def multi_host_step(i):
            wg, wu, wd = sep[i % 4]
            ctx.matvec_multi([wg, wu], xp.numpy(), outs=[ygp.numpy(), yup.numpy()])
            ctx.matvec(wd, ap_.numpy(), out=ydp.numpy())

        for i in range(3):
            multi_host_step(i)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(32):
            multi_host_step(i)
        torch.cuda.synchronize()
        e2e_ms = 1000.0 * (time.perf_counter() - t0) / 32
        out["ffn_matvec_multi"] = {"calls_per_step": 2, "ms_per_step": ms, "gbs": STEP_BYTES / ms / 1e6,
                                   "hbm_frac": STEP_BYTES / ms / 1e6 / peaks["hbm_gbs"],
                                   "e2e_ms_per_step": e2e_ms, "e2e_gbs": STEP_BYTES / e2e_ms / 1e6}
        # the whole FFN block of a decode layer: norm -> gate, up -> gelu(gate) * up -> down -> residual
        # (Sources/LeviathanCore/Gemma4.swift:3741-3753), as five launches and as two fused ones
        nw = torch.ones(HIDDEN, device=dev) + 0.1 * torch.randn(HIDDEN, generator=g, device=dev)
        hbuf, gubuf = torch.empty((1, HIDDEN), device=dev), torch.empty((1, 2 * FFN), device=dev)
        actbuf, xo = torch.empty((1, FFN), device=dev), torch.empty((1, HIDDEN), device=dev)
        halves = [gubuf[:, :FFN], gubuf[:, FFN:]]

        def block_unfused(i):
            wg, wu, wd = sep[i % 4]
            ctx.rmsnorm(xd, nw, 1e-6, out=hbuf)
            ctx.matvec_multi([wg, wu], hbuf, outs=halves)
            ctx.gelu_up(gubuf, out=actbuf)
            ctx.matvec(wd, actbuf, out=ydn)
            ctx.axpy(1.0, ydn, xd, out=xo)

        def block_fused(i):
            wg, wu, wd = sep[i % 4]
            ctx.matvec_multi_fused([wg, wu], xd, "rmsnorm", nw, 1e-6, outs=halves)
            ctx.matvec_fused(wd, gubuf, "gelu_up", residual=xd, alpha=1.0, out=xo)

        ms_u = _graph_time(torch, stream, block_unfused, 16)
        ref_out = xo.clone()
        ms_f = _graph_time(torch, stream, block_fused, 16)
        agree = float((xo - ref_out).abs().max() / ref_out.abs().max().clamp_min(1.0))
        out["ffn_block"] = {"workload": "rmsnorm -> Q4_K gate, up -> gelu_up -> Q6_K down -> residual, batch 1",
                            "unfused": {"launches": 5, "ms_per_step": ms_u, "gbs": STEP_BYTES / ms_u / 1e6},
                            "fused": {"launches": 2, "ms_per_step": ms_f, "gbs": STEP_BYTES / ms_f / 1e6,
                                      "hbm_frac": STEP_BYTES / ms_f / 1e6 / peaks["hbm_gbs"]},
                            "max_abs_diff_over_max": agree}
        for ws_ in sep:
            for w_ in ws_:
                w_.free()
        # the same set at n = 2, 4, 8 activation columns (weights are streamed once per launch)
        cols = {}
        for n in (2, 4, 8):
            xn = torch.randn((n, HIDDEN), generator=g, device=dev)
            an = torch.randn((n, FFN), generator=g, device=dev)
            ygun, ydnn = torch.empty((n, 2 * FFN), device=dev), torch.empty((n, HIDDEN), device=dev)

            def col_step(i, xn=xn, an=an, ygun=ygun, ydnn=ydnn):
                wgu, wd = fused[i % 4]
                ctx.matvec(wgu, xn, out=ygun)
                ctx.matvec(wd, an, out=ydnn)

            msn = _graph_time(torch, stream, col_step, 16)
            byts = 2 * GATE_BYTES + DOWN_BYTES + n * VEC_BYTES
            cols[f"n{n}"] = {"ms_per_step": msn, "gbs": byts / msn / 1e6, "hbm_frac": byts / msn / 1e6 / peaks["hbm_gbs"]}
        out["ffn_columns"] = {"workload": "gate/up concatenated + down, n activation columns", **cols}
        # decode attention over an fp16 paged KV cache: 16 query heads, 8 KV heads, head dimension 256,
        # 4096 cached positions (33.5 MB of K and V per layer and sequence); six layers' caches are cycled
        # so that each launch reads from HBM, blocks handed out in a shuffled order
        import leviathan_b200 as lev_pkg
        import random as _random

        QH, KVH, HD, TOK, PAGE = 16, 8, 256, 4096, 16
        caches = []
        for li in range(6):
            c = lev_pkg.PagedKV(TOK // PAGE + 1, PAGE, KVH, HD, slots=1, max_blocks=TOK // PAGE, dtype="f16", device=dev)
            _random.Random(li).shuffle(c.free)
            for p_ in range(0, TOK, PAGE):
                c.ensure(0, p_)
            c.k.copy_((torch.randn(c.k.shape, generator=g, device=dev) * 0.25).to(torch.float16))
            c.v.copy_(torch.randn(c.v.shape, generator=g, device=dev).to(torch.float16))
            caches.append(c)
        qa = torch.randn((1, QH, HD), generator=g, device=dev)
        oa = torch.empty_like(qa)
        slot_a = torch.zeros(1, dtype=torch.int32, device=dev)
        pos_a = torch.full((1,), TOK - 1, dtype=torch.int32, device=dev)

        def attn_step(i):
            ctx.attn_decode(caches[i % 6], slot_a, pos_a, qa, 0, 1.0, out=oa)

        ms = _graph_time(torch, stream, attn_step, 24)
        kv_bytes = 2 * TOK * KVH * HD * 2
        out["attn_decode"] = {"workload": "16 q heads / 8 KV heads / head_dim 256 / 4096 positions, fp16 paged cache (page 16), batch 1",
                              "launches_per_step": 2, "us_per_step": ms * 1e3, "kv_bytes": kv_bytes, "gbs": kv_bytes / ms / 1e6,
                              "hbm_frac": kv_bytes / ms / 1e6 / peaks["hbm_gbs"]}
        del caches
        # the same shape at 32 sequences in one call (1.07 GB of K and V): the per-call fixed part amortised
        NB = 32
        cb = lev_pkg.PagedKV(NB * (TOK // PAGE) + 1, PAGE, KVH, HD, slots=NB, max_blocks=TOK // PAGE, dtype="f16", device=dev)
        _random.Random(99).shuffle(cb.free)
        for s_ in range(NB):
            cb.ensure(s_, TOK - 1)
        cb.k.copy_((torch.randn(cb.k.shape, generator=g, device=dev) * 0.25).to(torch.float16))
        cb.v.copy_(torch.randn(cb.v.shape, generator=g, device=dev).to(torch.float16))
        qb32 = torch.randn((NB, QH, HD), generator=g, device=dev)
        ob32 = torch.empty_like(qb32)
        slot_b = torch.arange(NB, dtype=torch.int32, device=dev)
        pos_b = torch.full((NB,), TOK - 1, dtype=torch.int32, device=dev)
        l0 = ctx.launch_count()
        ctx.attn_decode(cb, slot_b, pos_b, qb32, 0, 1.0, out=ob32)
        n_launch = ctx.launch_count() - l0
        ms = _graph_time(torch, stream, lambda i: ctx.attn_decode(cb, slot_b, pos_b, qb32, 0, 1.0, out=ob32), 8)
        out["attn_decode_b32"] = {"workload": "the same heads and context, 32 sequences in one call (fp16 paged cache, 1.07 GB of K and V)",
                                  "launches_per_step": int(n_launch), "us_per_step": ms * 1e3, "kv_bytes": NB * kv_bytes,
                                  "gbs": NB * kv_bytes / ms / 1e6, "hbm_frac": NB * kv_bytes / ms / 1e6 / peaks["hbm_gbs"],
                                  "tokens_per_s": NB / (ms * 1e-3)}
        del cb
        for wgu, wd in fused:
            wgu.free()
            wd.free()
    if world > 1:
        from leviathan_b200 import dist as lev_dist
        from leviathan_b200 import quant as Qd

        peer = bool(ctx.lib.lev_dist_peer_memory(ctx.handle))
        out["peer_memory_mapped"] = peer
        # dense row-split: every rank holds rows [r*R/G, (r+1)*R/G) of the same Q4_K tensor, activations
        # are replicated, every rank ends with the whole output (peer stores; NCCL all-gather as fallback).
        # With peer memory the calls are our own kernels only and are timed inside a CUDA graph.
        first, per = lev_dist.row_shard(FFN, rank, world)
        gw = torch.Generator(device=dev).manual_seed(SEED ^ 0x500)
        wq = Qd.quantize(Q4_K, torch.randn((FFN, HIDDEN), generator=gw, device=dev) * 0.02)
        row_bytes = (HIDDEN // 256) * 144
        w_loc = ctx.upload(wq[first * row_bytes:(first + per) * row_bytes].contiguous(), Q4_K, per, HIDDEN)
        del wq
        xb = torch.randn((512, HIDDEN), generator=gw, device=dev).to(torch.bfloat16)
        xv = torch.randn((1, HIDDEN), generator=gw, device=dev)
        yb, yv = torch.empty((512, FFN), device=dev), torch.empty((1, FFN), device=dev)

        def eager_ms(fn, iters=16):
            import torch.distributed as dist
            if peer:
                ms_ = _graph_time(torch, stream, lambda i: fn(), iters)
            else:
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record()
                for _ in range(iters):
                    fn()
                a1.record()
                a1.synchronize()
                ms_ = a0.elapsed_time(a1) / iters
            t = torch.tensor([ms_], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item()

        ms = eager_ms(lambda: ctx.gemm_prefill_rowsplit_allgather(w_loc, xb, world, out=yb))
        flop = 2.0 * 512 * HIDDEN * FFN
        out["prefill_gemm_rowsplit"] = {"workload": "X bf16 [512x4096] x Q4_K [12288x4096], rows split, all-gather of Y",
                                        "ms": ms, "tflops": flop / ms / 1e9}
        ms = eager_ms(lambda: ctx.matvec_rowsplit_allgather(w_loc, xv, world, out=yv))
        out["matvec_rowsplit"] = {"workload": "Q4_K [12288x4096] matvec, rows split, all-gather of y", "ms": ms,
                                  "gbs": (GATE_BYTES + 4 * (HIDDEN + FFN)) / ms / 1e6}
        w_loc.free()
    # MoE layer
    g = torch.Generator(device=dev).manual_seed(SEED ^ 0x400)
    first, count = (0, MOE_EXPERTS) if world == 1 else (rank * (MOE_EXPERTS // world), MOE_EXPERTS // world)
    gu, dn = [], []
    for e in range(MOE_EXPERTS):  # every rank draws all experts so that shards agree, keeps its own
        wgu = torch.randn((2 * MOE_INTER, MOE_HIDDEN), generator=g, device=dev) * 0.02
        wdn = torch.randn((MOE_HIDDEN, MOE_INTER), generator=g, device=dev) * 0.02
        if first <= e < first + count:
            gu.append(Q.quantize(2, wgu))
            dn.append(Q.quantize(2, wdn))
    router = torch.randn((MOE_EXPERTS, MOE_HIDDEN), generator=g, device=dev) * 0.02
    mw = ctx.moe_upload(router, torch.cat(gu), torch.cat(dn), MOE_EXPERTS, MOE_HIDDEN, MOE_INTER, first, count)
    del gu, dn
    moe = {}
    for batch in (1, 32, 512):
        # expert-parallel ranks each bring tokens: the batch is split across ranks when it divides
        # (same global batch as one GPU), a single token cannot be split and runs one per rank
        split = world > 1 and batch % world == 0
        tokens = batch // world if split else batch
        global_tokens = batch if (split or world == 1) else batch * world
        xt = [torch.randn((tokens, MOE_HIDDEN), generator=g, device=dev) for _ in range(8)]
        yo = torch.empty((tokens, MOE_HIDDEN), device=dev)
        if world > 1:
            import torch.distributed as dist
            fn = lambda i: ctx.moe_layer(mw, xt[i % 8], MOE_TOPK, out=yo, expert_parallel=True)  # noqa: E731
            if bool(ctx.lib.lev_dist_peer_memory(ctx.handle)):
                ms = _graph_time(torch, stream, fn, 8)
            else:
                # NCCL collectives are not captured: time eager calls with events
                for i in range(3):
                    fn(i)
                torch.cuda.synchronize()
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record()
                for i in range(16):
                    fn(i)
                a1.record()
                a1.synchronize()
                ms = a0.elapsed_time(a1) / 16
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        else:
            ms = _graph_time(torch, stream, lambda i: ctx.moe_layer(mw, xt[i % 8], MOE_TOPK, out=yo), 8)
        idx = ctx.moe_route(mw, xt[0], MOE_TOPK)[0]
        distinct = int(torch.unique(idx).numel())
        byts = MOE_ROUTER_BYTES + distinct * MOE_EXPERT_BYTES
        entry = {"ms_per_layer": ms, "global_tokens": global_tokens, "tokens_per_s": global_tokens / (ms * 1e-3)}
        if world == 1:
            entry.update({"distinct_experts": distinct, "algorithmic_bytes": byts, "gbs": byts / ms / 1e6,
                          "hbm_frac": byts / ms / 1e6 / peaks["hbm_gbs"]})
        moe[f"T{batch}"] = entry
    out["moe_layer"] = {"workload": "128 experts Q4_0 (GU 1408x2816, DN 2816x704), top-8, hidden 2816",
                        "parallelism": "single GPU" if world == 1 else f"expert-parallel over {world} GPUs", **moe}
    mw.free()
    if world == 1:
        for b in (1, 32):
            try:
                out[f"decode_step_batch_{b}"] = _decode_step(ctx, dev, stream, peaks, b)
            except Exception as e:  # a side measurement never takes the headline down
                out[f"decode_step_batch_{b}"] = {"error": repr(e)}
    elif bool(ctx.lib.lev_dist_peer_memory(ctx.handle)):
        # every rank decodes its own sequences, the experts are sharded: one sequence per rank, and 32 in all
        for per_rank in sorted({1, max(1, 32 // world)}):
            out[f"decode_step_batch_{per_rank * world}"] = _decode_step(ctx, dev, stream, peaks, per_rank, rank, world)
    return out if rank == 0 else None


def _decode_step(ctx, dev, stream, peaks, batch, rank=0, world=1):
    """The synthetic 30-layer MoE decode step (leviathan_b200/decoder.py: the token loop of
    Sources/LeviathanCore/Gemma4.swift:3611-3905 without its host round trips) as ONE CUDA graph: embedding row ->
    30 x [norm, q/k/v, head norms + rotary + cache append, attention over 4096 cached positions, output
    projection, norm, 128-expert top-8 MoE] -> norm -> Q6_K [262144 x 2816] head -> softcap -> argmax.  A replay
    decodes one token per sequence and leaves the next token ids on the device."""
    import torch

    from leviathan_b200.decoder import DecoderConfig, SyntheticDecoder

    cfg = DecoderConfig()
    with torch.cuda.stream(stream):
        t0 = time.time()
        dec = SyntheticDecoder(ctx, cfg, batch=batch, device=dev, rank=rank, world=world)
        torch.cuda.synchronize()
        build_s = time.time() - t0
        l0 = ctx.launch_count()
        dec.step()
        ctx.synchronize()
        launches = ctx.launch_count() - l0
        finite = bool(torch.isfinite(dec.logits).all())
        agree = bool((dec.tok.long() == torch.argmax(dec.logits, dim=1)).all())
        dec.capture()
        for _ in range(3):
            dec.replay()
        ts = []
        for _ in range(9):
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record(stream)
            dec.replay()
            a1.record(stream)
            a1.synchronize()
            ts.append(a0.elapsed_time(a1))
        ms = statistics.median(ts)
        if world > 1:  # the slowest rank's median
            import torch.distributed as dist

            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()

        def head(i):
            dec.head_step()

        ms_head = _graph_time(torch, stream, head, 4)
    bt = cfg.bytes_per_token()
    # weights are read once per step whatever the batch; every sequence reads its own cache; the experts a
    # step touches: all top-8 at one sequence, the expected distinct count of a uniform routing otherwise
    gbatch = batch * world
    distinct = cfg.top_k if gbatch == 1 else cfg.experts * (1.0 - (1.0 - cfg.top_k / cfg.experts) ** gbatch)
    # per GPU: its own sequences' caches, the replicated attention weights, router and head, its share of the experts
    step_bytes = cfg.layers * (bt["attention_weights"] + bt["router"] + distinct / world * bt["expert"] + batch * bt["kv_per_sequence"]) + bt["head"]
    bound_ms = step_bytes / (peaks["hbm_gbs"] * 1e6)
    dec.free()
    del dec
    torch.cuda.empty_cache()
    how = "" if world == 1 else f" over {world} GPUs ({batch} per GPU; attention and head local, experts sharded, expert-parallel MoE)"
    return {"workload": f"30 layers, hidden 2816, Q4_0 q/k/v/o (16 q heads, 8 KV heads, head_dim 256), fp16 paged cache at 4096 "
                        f"positions, 128-expert Q4_0 MoE top-8, tied Q6_K head 262144, softcap 30, argmax; batch {gbatch}{how}",
            "projections": "prefill dequant-GEMM, bf16 activations" if batch >= 16 else "decode matvec, f32 activations",
            "one_cuda_graph": True, "launches_per_step": int(launches), "ms_per_step": ms, "tokens_per_s": gbatch / ms * 1e3,
            "algorithmic_bytes_per_step_per_gpu": int(step_bytes), "hbm_bound_ms": bound_ms, "hbm_frac": bound_ms / ms,
            "us_head_softcap_argmax": ms_head * 1e3, "head_gbs": bt["head"] / ms_head / 1e6,
            "outputs_finite": finite, "argmax_matches_torch": agree, "build_seconds": build_s}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--reps", type=int, default=31)
    ap.add_argument("--instances", type=int, default=8)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-check", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the prefill GEMM and MoE layer side measurements")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
