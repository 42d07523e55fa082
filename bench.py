#!/usr/bin/env python
"""Benchmark of the MoE-block hot path (router -> permutation -> grouped gate_up GEMM + SiLU*mul ->
grouped down GEMM + weighted combine -> tensor-parallel all-reduce) on synthetic Qwen3-MoE-shaped inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode|prefill|<name>] [--impl reference]

One step = one forward of the block over one batch. With N > 1 (launched by torch.distributed.run, one
rank per GPU) the intermediate dimension is sharded over the ranks exactly as the reference's tensor
parallelism does and the partial sums are all-reduced over NVLink peer memory: total work is fixed, so
scaling is "strong". Rank 0 prints one JSON line.

  value        whole-block TFLOP/s (2*T*k*3*H*I per step / device time), inputs resident in HBM; the K-step
               region is timed for several rounds (`timed_rounds`) and the median round is reported
  prefill      (default run only) the same legs for the T=8192 layered-prefill batch: the other half of the metric
  parity       first step's output: bit-identical on all ranks, and against the CPU oracle (a failed bound exits 3)
  kernels      both grouped GEMM kernels timed alone; `roofline` is the gate_up kernel's
  reference_gpu  (1 GPU) the reference's own Triton path from oracle/_ref timed on the same tensors, when staged
  e2e          same metric through the public API with pinned host buffers: H2D of hidden states and
               router logits and D2H of the result inside the timed region, every step
  roofline     the dominant kernel (grouped gate_up GEMM) timed alone with CUDA events against the
               measured peak of the box (HBM copy bandwidth for decode, bf16 tensor throughput for prefill)
  cpu_baseline the CPU restatement of the reference's path (oracle/, torch per-expert loop) on the host cores
  --impl reference   times only that CPU path, as the reference arm
Weights rotate over several distinct copies so that no step finds its weights in L2.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

ALIASES = {"decode": "qwen3-30b-a3b-decode-t64", "prefill": "qwen3-30b-a3b-prefill-t8192",
           "t256": "qwen3-30b-a3b-t256", "mixed": "qwen3-30b-a3b-mixed-iteration"}
# config 4: one layered-prefill iteration of a 48-layer stack with 16 layer groups: 256 decode tokens go
# through every layer, 8192 prefill tokens join them in the 3 layers of the designated group
MIXED_LAYERS, MIXED_GROUP, MIXED_DECODE_T, MIXED_PREFILL_T = 48, 3, 256, 8192


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    except Exception:  # noqa: BLE001
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def recorded_traffic(workload_name: str):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, if there is one."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            return json.load(f).get(workload_name, {}).get("grouped_gemm_gate_up_bytes_per_launch")
    except Exception:  # noqa: BLE001
        return None


class ClockSampler:
    """Samples SM clock, power and clock-event reasons through NVML (read-only) while the GPU works."""

    def __init__(self, index: int, period_s: float = 0.01):
        self.samples = []
        self.period = period_s
        self._stop = threading.Event()
        self._thread = None
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[index]) if visible else index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:  # noqa: BLE001
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), float(mhz), int(reasons)))
            except Exception:  # noqa: BLE001
                pass
            time.sleep(self.period)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self, t0: float, t1: float):
        if self.nv is None or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml_unavailable"], "samples": 0}
        nv = self.nv
        window = [s for s in self.samples if t0 <= s[0] <= t1]
        label = "timed_region"
        if not window:  # region shorter than the sampling period: fall back to the whole loaded run
            window, label = self.samples, "whole_run"
        mhz = sorted(s[1] for s in window)
        bits = 0
        for s in window:
            bits |= s[2]
        names = {
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
            "applications_clocks_setting": getattr(nv, "nvmlClocksEventReasonApplicationsClocksSetting", 0x2),
        }
        reasons = [n for n, b in names.items() if bits & b]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons, "samples": len(window),
                "window": label}


def build_parser():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--workload", default="decode")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--weight-sets", type=int, default=4, help="distinct weight copies rotated through (L2 defeat)")
    ap.add_argument("--tokens", type=int, default=None, help="override the workload's token count (profiling)")
    ap.add_argument("--fp8", action="store_true",
                    help="e4m3 block-scaled weights (scales ~ U(0.5, 2) / 448 per 128 x 128 block) and per-token-group "
                         "activation quantisation instead of bf16; 1 GPU")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every step eagerly (default: decode-sized steps replay a captured CUDA graph, as the "
                         "reference does for batches up to 1024 tokens)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-prefill", action="store_true",
                    help="default decode run only: skip the second record (the T=8192 layered-prefill batch)")
    ap.add_argument("--no-reference-gpu", action="store_true",
                    help="skip timing the reference's own Triton path from oracle/_ref (1 GPU)")
    ap.add_argument("--rounds", type=int, default=None,
                    help="how many times the K-step region is timed (default 25); the median round is reported")
    ap.add_argument("--only-steps", action="store_true",
                    help="stop after the timed steps (no e2e, roofline or comparison legs): for ncu launch lists")
    return ap


def config_dict(wl, gpus: int, n_sets: int, fp8: bool = False):
    """The `config` object of the JSON line; both arms print the same one for the same command line."""
    ip = wl.I // max(1, gpus)
    return {"workload": wl.name + ("-fp8" if fp8 else ""), "T": wl.T, "H": wl.H, "E": wl.E, "top_k": wl.top_k, "I": wl.I,
            "tensor_parallel": gpus, "I_per_rank": ip,
            "l2": f"weights rotate over {n_sets} distinct copies ({n_sets * 3 * wl.E * wl.H * ip * (1 if fp8 else 2) / 1e6:.0f} MB per rank) so no step finds them in L2",
            "all_reduce": "fused k-slot sum + peer-memory all-reduce" if gpus > 1 else "none (1 GPU)"}


def cpu_block_time(wl, inputs, tokens: int, repeats: int, threads: int):
    """Seconds per pass of the CPU restatement over the first `tokens` tokens (best of `repeats`)."""
    from oracle import moe_oracle as O
    torch.set_num_threads(threads)
    x = inputs["x"][:tokens].contiguous()
    lg = inputs["router_logits"][:tokens].contiguous()
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        O.moe_block(x, lg, inputs["w13"], inputs["w2"], wl.top_k, True)
        best = min(best, time.perf_counter() - t0)
    return best


def run_reference(args, wl, rank: int):
    """Reference arm: the reference's algorithm for this path on the host CPU cores (oracle port; the
    reference's own GEMM is a Triton GPU kernel and its tree is not available where this runs)."""
    if rank != 0:
        return
    from layered_prefill_b200 import workload as W
    from oracle import moe_oracle as O
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    steps = args.steps if args.steps is not None else 5
    warmup = args.warmup if args.warmup is not None else 1
    inputs = W.make_inputs(wl, seed=0)
    # size the sample so that the whole run stays within about two minutes
    probe_tokens = min(wl.T, 64)
    t_probe = cpu_block_time(wl, inputs, probe_tokens, 1, threads)
    budget = 120.0
    per_step = budget / max(1, steps + warmup)
    tokens = wl.T if t_probe * (wl.T / probe_tokens) <= per_step else max(1, int(probe_tokens * per_step / t_probe))
    tokens = min(tokens, wl.T)
    x = inputs["x"][:tokens].contiguous()
    lg = inputs["router_logits"][:tokens].contiguous()
    for _ in range(warmup):
        O.moe_block(x, lg, inputs["w13"], inputs["w2"], wl.top_k, True)
    t0 = time.perf_counter()
    for _ in range(steps):
        O.moe_block(x, lg, inputs["w13"], inputs["w2"], wl.top_k, True)
    dt = (time.perf_counter() - t0) / max(1, steps)
    flops = 2 * tokens * wl.top_k * 3 * wl.H * wl.I
    val = flops / dt / 1e12
    sample = f"{tokens} of {wl.T} tokens per step, full expert weights, torch fp32 per-expert loop"
    line = {
        "impl": "reference", "metric": "moe_block_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config_dict(wl, args.gpus, max(1, args.weight_sets)), "sampled_tokens": tokens,
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "us_per_layer": dt * 1e6, "tokens_per_s": tokens / dt,
    }
    print(json.dumps(line), flush=True)


class Ctx:
    """Process-wide state of one benchmark run: ranks, device, communicator, weight sets."""

    def __init__(self, args, world, rank, dev, comm):
        self.args, self.world, self.rank, self.dev, self.comm = args, world, rank, dev, comm
        self.sets = []          # per weight set: (w13, w2) of this rank, or (q13, q2, s13, s2) for fp8
        self.set0_cpu = None    # rank 0: the unsharded bf16 weights of set 0 on the host (parity check, CPU baseline)
        self.sets_shape = None

    def barrier(self):
        import torch.distributed as dist
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def check_status(self, where: str):
        """Device status word of every rank (non-zero: a bounded device-side wait ran out). All ranks learn the
        worst value and leave together, so nobody is left waiting in a collective for a rank that quit."""
        from layered_prefill_b200 import ops
        status = ops.read_status(self.dev)
        worst = int(self.max_over_ranks(float(status)))
        if worst != 0:
            if self.rank == 0:
                print(json.dumps({"error": f"device-side wait timed out {where}", "status": worst}), file=sys.stderr, flush=True)
            raise SystemExit(4)

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        import torch.distributed as dist
        t = torch.tensor([v], device=self.dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def make_weight_sets(self, wl):
        """n_sets distinct weight copies drawn on the GPU (seed 1000 + set), sharded over I as the reference's
        weight_loader does. Every rank draws the same full tensors, so the shards belong to one model."""
        shape = (wl.E, wl.H, wl.I, bool(self.args.fp8))
        if self.sets_shape == shape:
            return
        self.sets, self.set0_cpu, self.sets_shape = [], None, shape
        dev, tp, rank = self.dev, self.world, self.rank
        ip = wl.I // tp
        for s in range(max(1, self.args.weight_sets)):
            g = torch.Generator(device=dev)
            g.manual_seed(1000 + s)
            w13_full = (torch.randn(wl.E, 2 * wl.I, wl.H, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
            w2_full = (torch.randn(wl.E, wl.H, wl.I, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
            if s == 0 and rank == 0 and not self.args.fp8:
                self.set0_cpu = (w13_full.cpu(), w2_full.cpu())
            if self.args.fp8:
                def quantise(w):  # masters quantised with drawn scales, as the benchmark config describes
                    e, n, k = w.shape
                    sc = (torch.rand(e, n // 128, k // 128, generator=g, device=dev) * 1.5 + 0.5) / 448.0
                    blocks = w.float().view(e, n // 128, 128, k // 128, 128) / sc[:, :, None, :, None]
                    return blocks.clamp(-448, 448).to(torch.float8_e4m3fn).view(e, n, k).contiguous(), sc
                q13, s13 = quantise(w13_full)
                q2, s2 = quantise(w2_full)
                del w13_full, w2_full
                if tp > 1:  # this rank's slice of I; the scales stay those of the unsharded weights
                    lo, hi = rank * ip, (rank + 1) * ip
                    b13, b2 = q13.view(torch.uint8), q2.view(torch.uint8)
                    q13 = torch.cat([b13[:, lo:hi], b13[:, wl.I + lo:wl.I + hi]], dim=1).contiguous().view(torch.float8_e4m3fn)
                    q2 = b2[:, :, lo:hi].contiguous().view(torch.float8_e4m3fn)
                    del b13, b2
                self.sets.append((q13, q2, s13, s2))
            elif tp == 1:
                self.sets.append((w13_full, w2_full))
            else:
                lo, hi = rank * ip, (rank + 1) * ip
                w13_r = torch.cat([w13_full[:, lo:hi], w13_full[:, wl.I + lo:wl.I + hi]], dim=1).contiguous()
                self.sets.append((w13_r, w2_full[:, :, lo:hi].contiguous()))
                del w13_full, w2_full
        torch.cuda.synchronize()


def event_time_ms(fn, iters: int, warm: int = 3) -> float:
    """Mean milliseconds per call of fn(i), CUDA events on the current stream, after `warm` untimed calls."""
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def capture_graph(dev, fn):
    """fn() captured into a CUDA graph on a side stream (after one eager call there)."""
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        fn()
        with torch.cuda.graph(g, stream=side):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    return g


def run_workload(ctx: Ctx, wl, steps: int, warmup: int, primary: bool, mixed: bool = False):
    """All legs for one workload on the current process group. Returns the record (rank 0 prints it)."""
    import torch.distributed as dist
    from layered_prefill_b200 import fused_moe, ops, workload as W
    from layered_prefill_b200._lib import lib
    args, dev, world, rank, comm = ctx.args, ctx.dev, ctx.world, ctx.rank, ctx.comm
    prefill = wl.T >= 2048
    tp = world
    ip = wl.I // tp
    ctx.make_weight_sets(wl)
    sets, n_sets = ctx.sets, len(ctx.sets)

    # x / logits from the CPU generator (identical on every rank); the expert weights are the GPU-drawn sets
    small = W.make_inputs(W.MoeWorkload("x-only", wl.T, wl.H, wl.E, wl.top_k, 16, wl.logit_bias_std), seed=0)
    x_cpu, lg_cpu = small["x"], small["router_logits"]
    x, logits = x_cpu.to(dev), lg_cpu.to(dev)
    out = torch.empty_like(x)

    def block(i, xin, lgin, dst):
        if args.fp8:
            q13, q2, s13, s2 = sets[i % n_sets]
            if tp == 1:
                return fused_moe.fused_moe_forward_fp8(xin, lgin, q13, s13, q2, s2, wl.top_k, True, out=dst)
            tw_, ti_, _ = fused_moe.fused_topk(xin, lgin, wl.top_k, True)
            return fused_moe.fused_experts_fp8_shard(xin, q13, s13, q2, s2, tw_, ti_, rank * ip, wl.I, out=dst, comm=comm)
        w13, w2 = sets[i % n_sets]
        return fused_moe.fused_moe_forward(xin, lgin, w13, w2, wl.top_k, True, "silu", inplace=False, comm=comm,
                                           out=dst)

    if mixed:
        # decode tokens = the last MIXED_DECODE_T rows; layers of the designated group see all rows
        x_dec, lg_dec = x[MIXED_PREFILL_T:].contiguous(), logits[MIXED_PREFILL_T:].contiguous()
        out_dec = torch.empty_like(x_dec)
        group0 = MIXED_LAYERS // 2

        def step(i, xin=x, lgin=logits):
            o = None
            for layer in range(MIXED_LAYERS):
                if group0 <= layer < group0 + MIXED_GROUP:
                    o = block(i * MIXED_LAYERS + layer, xin, lgin, out)
                else:
                    block(i * MIXED_LAYERS + layer, x_dec, lg_dec, out_dec)
            return o
    else:
        def step(i, xin=x, lgin=logits):
            return block(i, xin, lgin, out)

    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    # the ranks start together: the peer-memory reduction waits for a peer for a bounded time only, and rank 0
    # has just spent longer than that copying a weight set to the host
    ctx.barrier()
    for i in range(warmup):
        step(i)
    ctx.barrier()
    ctx.check_status("during warm-up")

    # ---- parity of the first step's output (outside every timed region): the ranks hold identical bits, and rank 0
    # checks them against the CPU oracle on the same inputs (all tokens up to 256, a spread sample of 96 beyond)
    parity = None
    if not args.fp8:
        first = block(0, x, logits, torch.empty_like(x))
        torch.cuda.synchronize()
        identical = True
        if world > 1:
            gathered = [torch.empty_like(first) for _ in range(world)]
            dist.all_gather(gathered, first)
            identical = all(torch.equal(gathered[0], t) for t in gathered[1:])
        if rank == 0:
            from oracle import moe_oracle as O
            torch.set_num_threads(os.cpu_count() or 1)
            idx = torch.arange(wl.T) if wl.T <= 256 else torch.arange(0, wl.T, wl.T // 96)[:96]
            w13c, w2c = ctx.set0_cpu
            if world == 1:
                want = O.moe_block(x_cpu[idx], lg_cpu[idx], w13c, w2c, wl.top_k, True)
            else:
                want = O.moe_block_tp(x_cpu[idx], lg_cpu[idx], w13c, w2c, wl.top_k, world)
            got = first.cpu()[idx]
            parity = {"rel_l2": O.rel_l2(got, want), "max_abs": O.max_abs(got, want), "ranks_bit_identical": identical,
                      "tokens_checked": int(idx.numel()), "bounds": {"rel_l2": 5e-3, "max_abs": 2e-2},
                      "checker": "CPU oracle, reference rounding points" + (f", {world} rank shards summed in rank order" if world > 1 else "")}
            ok = identical and parity["rel_l2"] <= 5e-3 and parity["max_abs"] <= 2e-2
            parity["ok"] = bool(ok)
        flag = torch.tensor([1 if (rank != 0 or parity["ok"]) else 0], device=dev)
        if world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0 or not identical:
            if rank == 0:
                print(json.dumps({"error": "parity check failed", "workload": wl.name, "parity": parity}), file=sys.stderr, flush=True)
            raise SystemExit(3)
        ctx.barrier()

    # ---- decode-sized batches: one captured graph per weight set (the reference replays its decode layers
    # from CUDA graphs up to 1024 tokens, nanovllm/models/qwen3_moe.py:648-763); larger batches stay eager
    use_graph = (not args.no_graph) and (not mixed) and wl.T <= 1024
    launches_per_graph = 0
    if use_graph:
        graphs = []
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for s_idx in range(n_sets):
                l0 = lib.moe_b200_launch_count()
                gph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gph, stream=side):
                    block(s_idx, x, logits, out)
                launches_per_graph = int(lib.moe_b200_launch_count() - l0)
                graphs.append(gph)
        torch.cuda.current_stream().wait_stream(side)
        eager_step = step

        def step(i, xin=x, lgin=logits):  # noqa: F811
            if xin is x and lgin is logits:
                graphs[i % n_sets].replay()
                return out
            return eager_step(i, xin, lgin)
        for i in range(max(3, n_sets)):
            step(i)
        ctx.barrier()
    ctx.check_status("during graph warm-up")

    # ---- timed region: exactly `steps` steps between CUDA events on the launching stream, barrier and
    # synchronize on both sides, max over ranks; repeated for `rounds` rounds, the median round is reported
    def one_round():
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx.barrier()
        ev0.record()
        for i in range(steps):
            step(i)
        ev1.record()
        ctx.barrier()
        return ctx.max_over_ranks(ev0.elapsed_time(ev1))

    launches0 = lib.moe_b200_launch_count()
    t_wall0 = time.perf_counter()
    round_ms = [one_round()]
    launches = int(lib.moe_b200_launch_count() - launches0)
    if use_graph:
        launches = launches_per_graph * steps  # replayed kernels are not seen by the library's launch counter
    rounds = args.rounds if args.rounds else 25
    for _ in range(rounds - 1):
        round_ms.append(one_round())
    t_wall1 = time.perf_counter()
    srt = sorted(round_ms)
    ms_total = srt[len(srt) // 2]
    ms_per_step = ms_total / steps
    clocks = sampler.summary(t_wall0, t_wall1)
    ctx.check_status("in the timed region")
    timed_rounds = {"rounds": rounds, "steps_per_round": steps, "median_ms": ms_total, "min_ms": srt[0], "max_ms": srt[-1],
                    "reported": "median round"}

    flops = wl.flops()
    if mixed:
        per_token = 2 * wl.top_k * 3 * wl.H * wl.I
        flops = per_token * (MIXED_GROUP * wl.T + (MIXED_LAYERS - MIXED_GROUP) * MIXED_DECODE_T)
    value = flops / (ms_per_step * 1e-3) / 1e12
    rec = {"workload": wl.name, "value": value, "ms_per_step": ms_per_step, "steps": steps, "warmup": warmup,
           "timed_rounds": timed_rounds, "gpu_launches": launches, "clocks": clocks, "parity": parity,
           "use_graph": use_graph, "n_sets": n_sets, "flops": flops}
    if args.only_steps:
        sampler.stop()
        return rec
    state = {"x": x, "logits": logits, "x_cpu": x_cpu, "lg_cpu": lg_cpu, "out": out, "block": block, "step": step,
             "sampler": sampler, "prefill": prefill, "ip": ip, "mixed": mixed}
    finish_workload(ctx, wl, rec, state, primary)
    return rec


def e2e_leg(ctx: Ctx, wl, rec, st):
    """The same metric through the public API with pinned host buffers: every step uploads its hidden states and
    router logits and downloads its result; three buffer sets and two copy streams let step i's upload, step i-1's
    compute and step i-2's download overlap, as a serving loop does."""
    dev, n_sets, steps = ctx.dev, rec["n_sets"], rec["steps"]
    x, logits, block, step, mixed = st["x"], st["logits"], st["block"], st["step"], st["mixed"]
    xh, lh = st["x_cpu"].clone().pin_memory(), st["lg_cpu"].clone().pin_memory()
    nb = 3
    xd = [torch.empty_like(x) for _ in range(nb)]
    ld = [torch.empty_like(logits) for _ in range(nb)]
    od = [torch.empty_like(x) for _ in range(nb)]
    oh = [torch.empty_like(st["x_cpu"]).pin_memory() for _ in range(nb)]
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    cur = torch.cuda.current_stream()
    in_done = [torch.cuda.Event() for _ in range(nb)]
    comp_done = [torch.cuda.Event() for _ in range(nb)]
    out_done = [torch.cuda.Event() for _ in range(nb)]
    e2e_graphs = None
    if rec["use_graph"]:  # one captured graph per (buffer set, weight set), as the device-timed region replays
        e2e_graphs = [[None] * n_sets for _ in range(nb)]
        side_e = torch.cuda.Stream(device=dev)
        side_e.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side_e):
            for b in range(nb):
                for s_idx in range(n_sets):
                    gph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gph, stream=side_e):
                        block(s_idx, xd[b], ld[b], od[b])
                    e2e_graphs[b][s_idx] = gph
        torch.cuda.current_stream().wait_stream(side_e)
        ctx.barrier()

    def e2e_step(i):
        b = i % nb
        with torch.cuda.stream(s_in):
            s_in.wait_event(comp_done[b])      # the compute that last read xd[b] / ld[b]
            xd[b].copy_(xh, non_blocking=True)
            ld[b].copy_(lh, non_blocking=True)
            in_done[b].record(s_in)
        cur.wait_event(in_done[b])
        cur.wait_event(out_done[b])            # the download that last read od[b]
        if mixed:
            o = step(i, xd[b], ld[b])
            od[b].copy_(o, non_blocking=True)
        elif e2e_graphs is not None:
            e2e_graphs[b][i % n_sets].replay()
        else:
            block(i, xd[b], ld[b], od[b])
        comp_done[b].record(cur)
        with torch.cuda.stream(s_out):
            s_out.wait_event(comp_done[b])
            oh[b].copy_(od[b], non_blocking=True)
            out_done[b].record(s_out)

    for ev in comp_done + out_done:
        ev.record(cur)
    for i in range(min(rec["warmup"], 10)):
        e2e_step(i)
    for ev in out_done:
        cur.wait_event(ev)
    e_steps = max(steps, 200) if wl.T <= 1024 else steps
    ctx.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    s_in.wait_event(e0)
    s_out.wait_event(e0)
    for i in range(e_steps):
        e2e_step(i)
    for ev in out_done:
        cur.wait_event(ev)
    e1.record()
    ctx.barrier()
    e_ms = ctx.max_over_ranks(e0.elapsed_time(e1)) / e_steps
    return {"value": rec["flops"] / (e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "h2d_bytes_per_step": xh.numel() * 2 + lh.numel() * 2, "d2h_bytes_per_step": oh[0].numel() * 2,
            "overlap": "uploads, compute and downloads of consecutive steps overlap (3 buffer sets, 2 copy streams)",
            "steps": e_steps, "ms_per_step": e_ms, "us_per_layer": e_ms * 1e3, "tokens_per_s": wl.T / (e_ms * 1e-3)}


def kernel_rooflines(ctx: Ctx, wl, rec, st):
    """The two grouped GEMM kernels timed alone (CUDA events on the launching stream, weights rotating over the
    sets) against the measured peak of the box: HBM copy bandwidth for decode-sized batches, bf16 tensor
    throughput for prefill-sized ones. Returns (roofline of the dominant kernel, per-kernel details, n_active)."""
    from layered_prefill_b200 import fused_moe, ops
    from layered_prefill_b200._lib import lib
    dev, world, sets, n_sets = ctx.dev, ctx.world, ctx.sets, rec["n_sets"]
    x, logits, prefill, ip = st["x"], st["logits"], st["prefill"], st["ip"]
    peaks = measured_peaks()
    tw, ti, _ = fused_moe.fused_topk(x, logits, wl.top_k, True)
    n_active = int(torch.unique(ti).numel())
    bm = lib.moe_b200_block_m()
    s_ids, e_ids, post = fused_moe.moe_align_block_size(ti, bm, wl.E)
    rows_cap = (s_ids.numel() + bm - 1) // bm * bm
    s_pad = torch.full((rows_cap,), wl.T * wl.top_k, dtype=torch.int32, device=dev)
    s_pad[:s_ids.numel()] = s_ids
    h_sorted = torch.empty(rows_cap, ip, dtype=torch.bfloat16, device=dev)
    c3 = torch.empty(wl.T * wl.top_k, wl.H, dtype=torch.bfloat16, device=dev)
    stw = ops.status_word(dev).data_ptr()
    stream = torch.cuda.current_stream().cuda_stream

    def gate_up(i):
        rc = lib.moe_b200_grouped_gemm_gate_up(x.data_ptr(), sets[i % n_sets][0].data_ptr(), 0, s_pad.data_ptr(),
                                               e_ids.data_ptr(), post.data_ptr(), h_sorted.data_ptr(), rows_cap, wl.T,
                                               wl.E, wl.top_k, wl.H, ip, 0, stw, stream)
        if rc != 0:
            raise SystemExit("gate_up launch failed: " + lib.moe_b200_last_error().decode())

    def down(i):
        rc = lib.moe_b200_grouped_gemm_down(h_sorted.data_ptr(), rows_cap, sets[i % n_sets][1].data_ptr(), 0,
                                            tw.data_ptr(), s_pad.data_ptr(), e_ids.data_ptr(), post.data_ptr(),
                                            c3.data_ptr(), wl.T, wl.E, wl.top_k, wl.H, ip, stw, stream)
        if rc != 0:
            raise SystemExit("down launch failed: " + lib.moe_b200_last_error().decode())

    k_iters = 20 if prefill else 200
    gu_ms = max(event_time_ms(gate_up, k_iters, 5), 1e-6)
    dn_ms = max(event_time_ms(down, k_iters, 5), 1e-6)
    traffic = recorded_traffic(wl.name)
    traffic_note = "ncu capture at 1 GPU"
    if traffic is not None and world > 1:
        traffic, traffic_note = traffic / world, f"1-GPU ncu capture divided by {world}: a rank streams 1/{world} of the weights"
    kernels = {}
    if prefill:
        for name, ms, fl in (("gate_up", gu_ms, 2 * wl.T * wl.top_k * 2 * ip * wl.H), ("down", dn_ms, 2 * wl.T * wl.top_k * wl.H * ip)):
            ach = fl / (ms * 1e-3) / 1e12
            kernels[name] = {"us_per_launch": ms * 1e3, "flops_per_launch": fl, "achieved_tflops": ach,
                             "frac_of_burst": ach / peaks["bf16_tflops"], "frac_of_sustained": ach / peaks["bf16_tflops_sustained"]}
        roofline = {"bound": "tensor", "achieved": kernels["gate_up"]["achieved_tflops"], "peak": peaks["bf16_tflops"],
                    "unit": "TFLOP/s", "frac": kernels["gate_up"]["frac_of_burst"], "traffic": traffic}
    else:
        by = {"gate_up": n_active * 2 * ip * wl.H * 2 + wl.T * wl.H * 2 + wl.T * wl.top_k * ip * 2,
              "down": n_active * wl.H * ip * 2 + wl.T * wl.top_k * ip * 2 + wl.T * wl.top_k * wl.H * 2}
        for name, ms in (("gate_up", gu_ms), ("down", dn_ms)):
            ach = by[name] / (ms * 1e-3) / 1e9
            kernels[name] = {"us_per_launch": ms * 1e3, "bytes_per_launch": by[name], "achieved_gbs": ach,
                             "frac_of_measured_hbm": ach / peaks["hbm_gbs"]}
        roofline = {"bound": "hbm", "achieved": kernels["gate_up"]["achieved_gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": kernels["gate_up"]["frac_of_measured_hbm"], "traffic": traffic}
    roofline.update({"kernel": "grouped_gemm_kernel<1> (gate_up + SiLU*mul)", "us_per_launch": gu_ms * 1e3,
                     "peak_source": f"of {peaks['source']}", "launches_timed": k_iters, "traffic_note": traffic_note})
    return roofline, kernels, n_active, (tw, ti)


def reference_gpu_leg(ctx: Ctx, wl, rec, st):
    """The reference's own GPU path for the block (its routing op + Triton fused_moe_kernel twice + activation op +
    moe_sum; nanovllm/layers/for_moe/fused_moe.py:393-633) from the staged copy under oracle/_ref/, on the same
    tensors with the same rotation of weight sets, event-timed. A comparison line, not the reference arm."""
    try:
        from oracle.build_ref import load_reference_package
        pkg = load_reference_package()
    except Exception as e:  # noqa: BLE001
        pkg, err = None, str(e)
    else:
        err = "oracle/_ref/nanovllm is not staged on this machine (built where the reference tree is mounted)"
    if pkg is None:
        return {"unavailable": err}
    import nanovllm.layers.for_moe.fused_moe as rfm
    x, logits, sets, n_sets = st["x"], st["logits"], ctx.sets, rec["n_sets"]
    try:
        def ref_block(i):
            w13, w2 = sets[i % n_sets]
            tw, ti, _ = rfm.fused_topk(x, logits, wl.top_k, True)
            return rfm.fused_experts(x, w13, w2, None, None, tw, ti, inplace=False)

        ref_out = ref_block(0)
        torch.cuda.synchronize()
        ours = st["block"](0, x, logits, torch.empty_like(x))
        d = (ours.float() - ref_out.float())
        parity = {"rel_l2_vs_ours": float(d.norm() / ref_out.float().norm().clamp_min(1e-30)), "max_abs_vs_ours": float(d.abs().max())}
        launch = "eager launches"
        run = ref_block
        if rec["use_graph"]:  # the reference replays decode-sized batches from CUDA graphs too
            try:
                graphs = [capture_graph(ctx.dev, lambda s=s: ref_block(s)) for s in range(n_sets)]
                run, launch = (lambda i: graphs[i % n_sets].replay()), "cuda graph replay per step"
            except Exception as e:  # noqa: BLE001
                launch = f"eager launches (graph capture failed: {str(e)[:80]})"
        iters = 20 if st["prefill"] else 200
        ms = event_time_ms(run, iters, 5)
        return {"us_per_layer": ms * 1e3, "tflops": rec["flops"] / (ms * 1e-3) / 1e12, "launch": launch, "steps": iters,
                "path": "reference fused_topk + fused_experts (Triton fused_moe_kernel, untuned default tiles on this GPU)",
                **parity}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"the reference path raised: {type(e).__name__}: {str(e)[:200]}"}


def all_reduce_legs(ctx: Ctx, wl, rec, st):
    """N > 1: the reductions alone. Decode-sized tensors are timed from a replayed CUDA graph (device time, not
    launch overhead), large ones eagerly with NCCL on the same tensor beside them."""
    import torch.distributed as dist
    from layered_prefill_b200 import ops
    from layered_prefill_b200._lib import check, lib
    dev, comm, rank = ctx.dev, ctx.comm, ctx.rank
    outd = {}
    sizes = sorted({wl.T, MIXED_DECODE_T} if st["mixed"] else {wl.T})
    for t_ar in sizes:
        buf = torch.randn(t_ar, wl.H, device=dev).to(torch.bfloat16)
        res = torch.empty_like(buf)
        c3 = torch.randn(t_ar * wl.top_k, wl.H, device=dev).to(torch.bfloat16) if t_ar <= 1024 else None
        stw = ops.status_word(dev).data_ptr()

        def plain(i=0):
            comm.all_reduce(buf, out=res)

        def fused(i=0):
            check(lib.moe_b200_ar_moe_sum_all_reduce(comm._ptr, c3.data_ptr(), res.data_ptr(), t_ar, wl.top_k, wl.H,
                                                     comm.buffer_ptrs[rank], comm.max_size, 0, stw,
                                                     torch.cuda.current_stream().cuda_stream))
        def fused_barriers(i=0):  # algo 3: the same reduction kept off the flag-in-data path
            check(lib.moe_b200_ar_moe_sum_all_reduce(comm._ptr, c3.data_ptr(), res.data_ptr(), t_ar, wl.top_k, wl.H,
                                                     comm.buffer_ptrs[rank], comm.max_size, 3, stw,
                                                     torch.cuda.current_stream().cuda_stream))
        legs = {"all_reduce_staged": plain}
        if c3 is not None:
            legs["k_slot_sum_all_reduce"] = fused
            legs["k_slot_sum_all_reduce_with_barriers"] = fused_barriers
        entry = {}
        for label, fn in legs.items():
            run, how = fn, "eager"
            if t_ar <= 1024:
                ctx.barrier()
                g = capture_graph(dev, fn)
                run, how = (lambda i=0, g=g: g.replay()), "graph replay"
            reps = 200 if t_ar <= 1024 else 30
            for _ in range(5):
                run()
            ctx.barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(reps):
                run()
            a1.record()
            ctx.barrier()
            entry[label + "_us"] = ctx.max_over_ranks(a0.elapsed_time(a1)) / reps * 1e3
            entry["timed_by"] = how
        if t_ar > 1024:  # the reference sends this size to NCCL (custom_all_reduce.py:253,364)
            for _ in range(3):
                dist.all_reduce(buf)
            ctx.barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(20):
                dist.all_reduce(buf)
            a1.record()
            ctx.barrier()
            entry["nccl_all_reduce_us"] = ctx.max_over_ranks(a0.elapsed_time(a1)) / 20 * 1e3
            n = ctx.world
            entry["bytes"] = t_ar * wl.H * 2
            entry["two_shot_link_bytes_per_direction"] = 2 * (n - 1) / n * t_ar * wl.H * 2
            entry["frac_of_770_gbs_per_direction"] = entry["two_shot_link_bytes_per_direction"] / (entry["all_reduce_staged_us"] * 1e-6) / 770e9
        outd[f"T{t_ar}"] = entry
    return outd


def finish_workload(ctx: Ctx, wl, rec, st, primary: bool):
    """Everything after the device-timed rounds: end to end, kernel rooflines, comparisons, CPU baseline."""
    import torch.nn.functional as F
    from layered_prefill_b200 import fused_moe, ops
    args, dev, world, rank = ctx.args, ctx.dev, ctx.world, ctx.rank
    x, logits, block, prefill, ip, mixed = st["x"], st["logits"], st["block"], st["prefill"], st["ip"], st["mixed"]
    n_sets, ms_per_step, value = rec["n_sets"], rec["ms_per_step"], rec["value"]
    peaks = measured_peaks()
    if primary and not args.no_e2e:
        rec["e2e"] = e2e_leg(ctx, wl, rec, st)
    st["sampler"].stop()

    if args.fp8:
        tw, ti, _ = fused_moe.fused_topk(x, logits, wl.top_k, True)
        n_active = int(torch.unique(ti).numel())
        # the fp8 kernels have no stand-alone entry point: the whole block against the HBM stream of its fp8 bytes
        f8_bytes = (n_active * 3 * wl.H * ip * (1 + 4 / 16384) + wl.T * wl.H * (2 + 1 + 2)
                    + wl.T * wl.top_k * (ip * (2 + 2 + 1 + 1) + wl.H * 4))
        achieved = f8_bytes / (ms_per_step * 1e-3) / 1e9
        rec["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                           "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                           "kernel": "whole fp8 block (quantise x, permute, gate_up, quantise h, down, k-slot sum)",
                           "us_per_launch": ms_per_step * 1e3, "peak_source": f"of {peaks['source']}",
                           "launches_timed": rec["steps"], "algorithmic_bytes": f8_bytes}
        blk_bytes = f8_bytes
    else:
        rec["roofline"], rec["kernels"], n_active, (tw, ti) = kernel_rooflines(ctx, wl, rec, st)
        blk_bytes = wl.algorithmic_bytes(n_active, world)
    rec["block"] = {"hbm_gbs": blk_bytes / (ms_per_step * 1e-3) / 1e9,
                    "hbm_frac_of_measured": blk_bytes / (ms_per_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
                    "tflops_per_gpu": value / world,
                    "tensor_frac_of_measured_burst": value / world / peaks["bf16_tflops"],
                    "tensor_frac_of_measured_sustained": value / world / peaks["bf16_tflops_sustained"],
                    "algorithmic_bytes_per_rank": blk_bytes, "n_active_experts": n_active}

    # ---- the same tokens as 16 sequential chunks of 512 (what chunked prefill does): expert-reload bytes saved
    if prefill and not mixed and not args.fp8 and wl.T % 512 == 0 and wl.T >= 1024:
        n_chunks = wl.T // 512
        xs = [x[c * 512:(c + 1) * 512].contiguous() for c in range(n_chunks)]
        ls = [logits[c * 512:(c + 1) * 512].contiguous() for c in range(n_chunks)]
        oc = torch.empty_like(xs[0])
        act_chunks = [int(torch.unique(ti[c * 512:(c + 1) * 512]).numel()) for c in range(n_chunks)]

        def chunked(i):
            for c in range(n_chunks):
                block(i, xs[c], ls[c], oc)

        for i in range(3):
            chunked(i)
        ctx.barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        c0.record()
        for i in range(reps):
            chunked(i)
        c1.record()
        ctx.barrier()
        c_ms = ctx.max_over_ranks(c0.elapsed_time(c1)) / reps
        per_expert = 3 * wl.H * ip * 2
        rec["chunked_prefill"] = {
            "chunks": n_chunks, "chunk_tokens": 512, "us_all_chunks": c_ms * 1e3, "us_single_pass": ms_per_step * 1e3,
            "speedup_single_pass": c_ms / ms_per_step,
            "weight_bytes_chunked": sum(act_chunks) * per_expert, "weight_bytes_single_pass": n_active * per_expert,
            "expert_reload_bytes_saved": (sum(act_chunks) - n_active) * per_expert}

    # ---- the steps in front of the block (add + RMSNorm, gate projection, top-k): one library call against the
    # reference's sequence of three ops (its norm kernel's twin, a cuBLAS linear, the routing kernel)
    if primary and not mixed and not args.fp8 and world == 1:
        gpre = torch.Generator(device=dev)
        gpre.manual_seed(7)
        attn = torch.randn(wl.T, wl.H, generator=gpre, device=dev).to(torch.bfloat16)
        resid = torch.randn(wl.T, wl.H, generator=gpre, device=dev).to(torch.bfloat16)
        nw = torch.ones(wl.H, device=dev, dtype=torch.bfloat16)
        wg = (torch.randn(wl.E, wl.H, generator=gpre, device=dev) * 0.02).to(torch.bfloat16)
        normed_buf = torch.empty_like(attn)

        def fused_pre(i=0):
            fused_moe.pre_moe(attn, resid, nw, 1e-6, wg, wl.top_k, True)

        def three_ops(i=0):
            ops.add_rms_norm(normed_buf, resid, attn, nw, 1e-6)
            fused_moe.fused_topk(normed_buf, F.linear(normed_buf, wg), wl.top_k, True)

        pre = {}
        for label, fn in (("one_call_us", fused_pre), ("three_ops_us", three_ops)):
            run = fn
            if not prefill:  # device time, not Python call overhead: replay a captured graph
                gq = capture_graph(dev, fn)
                run = lambda i=0, gq=gq: gq.replay()  # noqa: E731
            pre[label] = event_time_ms(run, 50 if prefill else 300, 5) * 1e3
        pre["note"] = ("graph replay" if not prefill else "eager launches") + \
            "; inputs L2-resident across repetitions; three_ops = add_rms_norm + torch linear (cuBLAS) + routing kernel"
        rec["pre_moe"] = pre

    if world > 1 and not args.fp8:
        rec["all_reduce"] = all_reduce_legs(ctx, wl, rec, st)
        comm = ctx.comm
        if primary and not mixed and wl.T <= 1024:  # all-reduce followed by the next layer's add + RMSNorm
            buf = torch.randn(wl.T, wl.H, device=dev).to(torch.bfloat16)
            resid = torch.randn(wl.T, wl.H, device=dev).to(torch.bfloat16)
            nw = torch.ones(wl.H, device=dev, dtype=torch.bfloat16)
            nout = torch.empty_like(buf)
            tail = {}
            for label, fn in (("all_reduce_then_add_rms_norm_us", lambda i=0: ops.add_rms_norm(nout, resid, comm.all_reduce(buf), nw, 1e-6)),
                              ("one_call_us", lambda i=0: comm.all_reduce_add_rms_norm(buf, resid, nw, 1e-6))):
                ctx.barrier()
                g = capture_graph(dev, fn)
                for _ in range(5):
                    g.replay()
                ctx.barrier()
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record()
                for _ in range(200):
                    g.replay()
                a1.record()
                ctx.barrier()
                tail[label] = ctx.max_over_ranks(a0.elapsed_time(a1)) / 200 * 1e3
            tail["timed_by"] = "graph replay"
            rec["all_reduce_add_rms_norm"] = tail
    if mixed:
        rec["mixed_iteration"] = {"layers": MIXED_LAYERS, "group_layers": MIXED_GROUP, "decode_tokens": MIXED_DECODE_T,
                                  "prefill_tokens": MIXED_PREFILL_T, "moe_path_us_per_iteration": ms_per_step * 1e3}

    if world == 1 and not args.fp8 and not mixed and not args.no_reference_gpu:
        rec["reference_gpu"] = reference_gpu_leg(ctx, wl, rec, st)

    if primary and rank == 0 and world == 1 and not args.no_cpu_baseline and ctx.set0_cpu is not None:
        threads = os.cpu_count() or 1
        tokens = wl.T if wl.T <= 256 else 256
        inputs = {"x": st["x_cpu"], "router_logits": st["lg_cpu"], "w13": ctx.set0_cpu[0], "w2": ctx.set0_cpu[1]}
        sec = cpu_block_time(wl, inputs, tokens, 3 if tokens <= 64 else 2, threads)
        cpu_flops = 2 * tokens * wl.top_k * 3 * wl.H * wl.I
        rec["cpu_baseline"] = {"value": cpu_flops / sec / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                               "sample": f"{tokens} of {wl.T} tokens, all {wl.E} experts' weights, torch fp32 per-expert loop, "
                                         f"best of {3 if tokens <= 64 else 2} passes", "us_per_layer": sec * 1e6}


def main():
    args = build_parser().parse_args()
    from layered_prefill_b200 import workload as W
    name = ALIASES.get(args.workload, args.workload)
    if name not in W.WORKLOADS and name != "qwen3-30b-a3b-mixed-iteration":
        raise SystemExit(f"unknown workload {args.workload}; known: {sorted(W.WORKLOADS)} or {sorted(ALIASES)}")
    mixed = name == "qwen3-30b-a3b-mixed-iteration"
    if mixed:
        wl = W.with_tokens(W.WORKLOADS["qwen3-30b-a3b-prefill-t8192"], MIXED_PREFILL_T + MIXED_DECODE_T)
        wl = W.MoeWorkload(name, wl.T, wl.H, wl.E, wl.top_k, wl.I, wl.logit_bias_std)
    else:
        wl = W.WORKLOADS[name]
    if args.tokens is not None:
        wl = W.with_tokens(wl, args.tokens)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, wl, rank)
        return
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 needs `python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...`")
        raise SystemExit(f"WORLD_SIZE={world} does not match --gpus {args.gpus}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    if args.fp8 and mixed:
        raise SystemExit("--fp8 runs the single block workloads only")

    import torch.distributed as dist
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    comm = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL announces its version on stdout while it initialises; stdout carries the one JSON line only,
        # so file descriptor 1 points at stderr until the communicators exist.
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            # short collective timeouts: a rank that dropped out ends the run in minutes, not in half an hour
            from datetime import timedelta
            dist.init_process_group("nccl", device_id=dev, timeout=timedelta(seconds=180))
            from layered_prefill_b200.custom_all_reduce import CustomAllreduce
            comm = CustomAllreduce(group=dist.new_group(backend="gloo", timeout=timedelta(seconds=180)), device=dev)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
        if comm.disabled:
            raise SystemExit("peer-memory all-reduce could not be initialised on this box")
        from layered_prefill_b200._lib import check as _check, lib as _lib
        _check(_lib.moe_b200_ar_set_wait_limit_ns(comm._ptr, 20_000_000_000))  # ranks of a benchmark may drift by seconds
    ctx = Ctx(args, world, rank, dev, comm)

    prefill = wl.T >= 2048
    steps = args.steps if args.steps is not None else (20 if mixed else 50 if prefill else 200)
    warmup = max(args.warmup if args.warmup is not None else (3 if mixed else 10 if prefill else 50), 3)
    rec = run_workload(ctx, wl, steps, warmup, primary=True, mixed=mixed)

    # the other half of the headline metric: the layered-prefill batch (T=8192, skewed routing) next to the decode
    # batch, in the same run, on the same weight sets
    second = None
    if (not args.only_steps and not args.no_prefill and not mixed and not args.fp8 and args.tokens is None
            and wl.name == "qwen3-30b-a3b-decode-t64"):
        second = run_workload(ctx, W.WORKLOADS["qwen3-30b-a3b-prefill-t8192"], 20, 5, primary=False)

    if rank == 0:
        tp, ip = world, wl.I // world
        n_sets = rec["n_sets"]
        if args.only_steps:
            line = {"metric": "moe_block_tflops", "value": rec["value"], "unit": "TFLOP/s", "n_gpus": world,
                    "steps": steps, "warmup": warmup, "ms_per_step": rec["ms_per_step"],
                    "config": {"workload": wl.name}, "gpu_launches": rec["gpu_launches"], "only_steps": True}
        else:
            line = {
                "metric": "moe_block_tflops", "value": rec["value"], "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
                "warmup": warmup, "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "fp8_e4m3 (w8a8, block scales, fp32 accumulation)" if args.fp8 else "bf16",
                "data": "synthetic",
                "config": config_dict(wl, world, n_sets, args.fp8),
                "launch": "cuda graph replay per step" if rec["use_graph"] else "eager launches",
                "us_per_layer": rec["ms_per_step"] * 1e3, "tokens_per_s": wl.T / (rec["ms_per_step"] * 1e-3),
                "timed_rounds": rec["timed_rounds"], "roofline": rec.get("roofline"), "kernels": rec.get("kernels"),
                "block": rec.get("block"), "parity": rec["parity"], "cpu_baseline": rec.get("cpu_baseline"),
                "e2e": rec.get("e2e"), "gpu_launches": rec["gpu_launches"], "clocks": rec["clocks"],
            }
            for key in ("chunked_prefill", "pre_moe", "all_reduce", "all_reduce_add_rms_norm", "mixed_iteration", "reference_gpu"):
                if key in rec:
                    line[key] = rec[key]
            if second is not None:
                line["prefill"] = {
                    "workload": second["workload"], "T": 8192, "us_per_layer": second["ms_per_step"] * 1e3,
                    "tflops": second["value"], "tokens_per_s": 8192 / (second["ms_per_step"] * 1e-3),
                    "steps": second["steps"], "warmup": second["warmup"], "launch": "eager launches",
                    "timed_rounds": second["timed_rounds"], "roofline": second.get("roofline"),
                    "kernels": second.get("kernels"), "block": second.get("block"), "parity": second["parity"],
                    "clocks": second["clocks"], "gpu_launches": second["gpu_launches"],
                    "note": "sw_power_cap is expected on a dense GEMM at the 1 kW limit and is kept",
                }
                for key in ("chunked_prefill", "all_reduce", "reference_gpu"):
                    if key in second:
                        line["prefill"][key] = second[key]
        print(json.dumps(line), flush=True)
    if world > 1:
        ctx.barrier()
        comm.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
