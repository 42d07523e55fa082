#!/usr/bin/env python
"""Benchmark of the MoE-block hot path (router -> permutation -> grouped gate_up GEMM + SiLU*mul ->
grouped down GEMM + weighted combine -> tensor-parallel all-reduce) on synthetic Qwen3-MoE-shaped inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode|prefill|<name>] [--impl reference]

One step = one forward of the block over one batch. With N > 1 (launched by torch.distributed.run, one
rank per GPU) the intermediate dimension is sharded over the ranks exactly as the reference's tensor
parallelism does and the partial sums are all-reduced over NVLink peer memory: total work is fixed, so
scaling is "strong". Rank 0 prints one JSON line.

  value        whole-block TFLOP/s (2*T*k*3*H*I per step / device time), inputs resident in HBM
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

    def __init__(self, index: int, period_s: float = 0.02):
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
    ap.add_argument("--only-steps", action="store_true",
                    help="stop after the timed steps (no e2e, roofline or comparison legs): for ncu launch lists")
    return ap


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
        "config": {"workload": wl.name, "T": wl.T, "H": wl.H, "E": wl.E, "top_k": wl.top_k, "I": wl.I,
                   "sampled_tokens": tokens},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "us_per_layer": dt * 1e6, "tokens_per_s": tokens / dt,
    }
    print(json.dumps(line), flush=True)


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

    import torch.distributed as dist
    from layered_prefill_b200 import fused_moe, ops
    from layered_prefill_b200._lib import lib

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
            dist.init_process_group("nccl", device_id=dev)
            from layered_prefill_b200.custom_all_reduce import CustomAllreduce
            comm = CustomAllreduce(group=dist.new_group(backend="gloo"), device=dev)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
        if comm.disabled:
            raise SystemExit("peer-memory all-reduce could not be initialised on this box")

    if args.fp8 and mixed:
        raise SystemExit("--fp8 runs the single block workloads only")
    prefill = wl.T >= 2048
    steps = args.steps if args.steps is not None else (20 if mixed else 200 if prefill else 2000)
    warmup = args.warmup if args.warmup is not None else (3 if mixed else 10 if prefill else 50)
    warmup = max(warmup, 3)
    tp = world
    ip = wl.I // tp

    # ---- inputs: x / logits from the CPU generator (identical on every rank), weights per set on the GPU
    cpu_inputs = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_inputs = W.make_inputs(wl, seed=0)
        x_cpu, lg_cpu = cpu_inputs["x"], cpu_inputs["router_logits"]
    else:
        small = W.make_inputs(W.MoeWorkload("x-only", wl.T, wl.H, wl.E, wl.top_k, 16, wl.logit_bias_std), seed=0)
        x_cpu, lg_cpu = small["x"], small["router_logits"]
    x = x_cpu.to(dev)
    logits = lg_cpu.to(dev)
    n_sets = max(1, args.weight_sets)
    sets = []
    for s in range(n_sets):
        g = torch.Generator(device=dev)
        g.manual_seed(1000 + s)
        w13_full = (torch.randn(wl.E, 2 * wl.I, wl.H, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        w2_full = (torch.randn(wl.E, wl.H, wl.I, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        if args.fp8:
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
            sets.append((q13, q2, s13, s2))
        elif tp == 1:
            sets.append((w13_full, w2_full))
        else:
            lo, hi = rank * ip, (rank + 1) * ip
            w13_r = torch.cat([w13_full[:, lo:hi], w13_full[:, wl.I + lo:wl.I + hi]], dim=1).contiguous()
            sets.append((w13_r, w2_full[:, :, lo:hi].contiguous()))
            del w13_full, w2_full
    torch.cuda.synchronize()
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

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local_rank)
    sampler.start()
    for i in range(warmup):
        step(i)
    barrier()
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
        barrier()
    if ops.read_status(dev) != 0:
        raise SystemExit("device-side wait timed out during warm-up")

    # ---- timed region: exactly `steps` steps, CUDA events on the launching stream
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = lib.moe_b200_launch_count()
    t_wall0 = time.perf_counter()
    ev0.record()
    for i in range(steps):
        step(i)
    ev1.record()
    barrier()
    t_wall1 = time.perf_counter()
    launches = int(lib.moe_b200_launch_count() - launches0)
    if use_graph:
        launches = launches_per_graph * steps  # replayed kernels are not seen by the library's launch counter
    ms_total = max_over_ranks(ev0.elapsed_time(ev1))
    ms_per_step = ms_total / steps
    clocks = sampler.summary(t_wall0, t_wall1)
    status = ops.read_status(dev)
    if status != 0:
        raise SystemExit(f"device-side wait timed out (status {status})")

    flops = wl.flops()
    if mixed:
        per_token = 2 * wl.top_k * 3 * wl.H * wl.I
        flops = per_token * (MIXED_GROUP * wl.T + (MIXED_LAYERS - MIXED_GROUP) * MIXED_DECODE_T)
    value = flops / (ms_per_step * 1e-3) / 1e12

    if args.only_steps:
        sampler.stop()
        if rank == 0:
            print(json.dumps({"metric": "moe_block_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
                              "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step,
                              "config": {"workload": wl.name}, "gpu_launches": launches, "only_steps": True}), flush=True)
        if world > 1:
            barrier()
            comm.close()
            dist.destroy_process_group()
        return

    # ---- end to end: pinned host inputs in, result out, every step
    e2e = None
    if not args.no_e2e:
        xh = x_cpu.clone().pin_memory()
        lh = lg_cpu.clone().pin_memory()
        # Three buffer sets and two copy streams: step i's upload, step i-1's compute and step i-2's download
        # overlap, as a serving loop does; every step still moves its own inputs in and its own result out.
        nb = 3
        xd = [torch.empty_like(x) for _ in range(nb)]
        ld = [torch.empty_like(logits) for _ in range(nb)]
        od = [torch.empty_like(x) for _ in range(nb)]
        oh = [torch.empty_like(x_cpu).pin_memory() for _ in range(nb)]
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        cur = torch.cuda.current_stream()
        in_done = [torch.cuda.Event() for _ in range(nb)]
        comp_done = [torch.cuda.Event() for _ in range(nb)]
        out_done = [torch.cuda.Event() for _ in range(nb)]

        # decode-sized batches replay one captured graph per (buffer set, weight set), as the timed region above does:
        # at N = 8 a step's kernels take less time than its eager launches
        e2e_graphs = None
        if use_graph:
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
            barrier()

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

        e_steps = steps
        for ev in comp_done + out_done:
            ev.record(cur)
        for i in range(min(warmup, 10)):
            e2e_step(i)
        for ev in out_done:
            cur.wait_event(ev)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        s_in.wait_event(e0)
        s_out.wait_event(e0)
        for i in range(e_steps):
            e2e_step(i)
        for ev in out_done:
            cur.wait_event(ev)
        e1.record()
        barrier()
        e_ms = max_over_ranks(e0.elapsed_time(e1)) / e_steps
        e2e = {"value": flops / (e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": xh.numel() * 2 + lh.numel() * 2, "d2h_bytes_per_step": oh[0].numel() * 2,
               "overlap": "uploads, compute and downloads of consecutive steps overlap (3 buffer sets, 2 copy streams)",
               "ms_per_step": e_ms, "us_per_layer": e_ms * 1e3, "tokens_per_s": wl.T / (e_ms * 1e-3)}
    sampler.stop()

    # ---- roofline of the dominant kernel (grouped gate_up GEMM), timed alone
    peaks = measured_peaks()
    tw, ti, _ = fused_moe.fused_topk(x, logits, wl.top_k, True)
    n_active = int(torch.unique(ti).numel())
    bm = lib.moe_b200_block_m()
    s_ids, e_ids, post = fused_moe.moe_align_block_size(ti, bm, wl.E)
    rows_cap = (s_ids.numel() + bm - 1) // bm * bm
    s_pad = torch.full((rows_cap,), wl.T * wl.top_k, dtype=torch.int32, device=dev)
    s_pad[:s_ids.numel()] = s_ids
    h_sorted = torch.empty(rows_cap, ip, dtype=torch.bfloat16, device=dev)
    stw = ops.status_word(dev).data_ptr()
    stream = torch.cuda.current_stream().cuda_stream

    def gate_up(i):
        if args.fp8:
            return
        w13, _ = sets[i % n_sets]
        rc = lib.moe_b200_grouped_gemm_gate_up(x.data_ptr(), w13.data_ptr(), 0, s_pad.data_ptr(), e_ids.data_ptr(),
                                               post.data_ptr(), h_sorted.data_ptr(), rows_cap, wl.T, wl.E, wl.top_k,
                                               wl.H, ip, 0, stw, stream)
        if rc != 0:
            raise SystemExit("gate_up launch failed: " + lib.moe_b200_last_error().decode())

    k_iters = 20 if prefill else 200
    for i in range(5):
        gate_up(i)
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for i in range(k_iters):
        gate_up(i)
    k1.record()
    torch.cuda.synchronize()
    k_ms = max(k0.elapsed_time(k1) / k_iters, 1e-6)
    if prefill:
        k_flops = 2 * wl.T * wl.top_k * 2 * ip * wl.H
        achieved = k_flops / (k_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["bf16_tflops"], "traffic": recorded_traffic(wl.name)}
    else:
        k_bytes = n_active * 2 * ip * wl.H * 2 + wl.T * wl.H * 2 + wl.T * wl.top_k * ip * 2
        achieved = k_bytes / (k_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": recorded_traffic(wl.name)}
    roofline.update({"kernel": "grouped_gemm_kernel<1> (gate_up + SiLU*mul)", "us_per_launch": k_ms * 1e3,
                     "peak_source": f"of {peaks['source']}", "launches_timed": k_iters})
    if args.fp8:
        # the fp8 kernels have no stand-alone entry point: the whole block against the HBM stream of its fp8 bytes
        f8_bytes = (n_active * 3 * wl.H * ip * (1 + 4 / 16384) + wl.T * wl.H * (2 + 1 + 2)
                    + wl.T * wl.top_k * (ip * (2 + 2 + 1 + 1) + wl.H * 4))
        achieved = f8_bytes / (ms_per_step * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                    "kernel": "whole fp8 block (quantise x, permute, gate_up, quantise h, down, k-slot sum)",
                    "us_per_launch": ms_per_step * 1e3, "peak_source": f"of {peaks['source']}", "launches_timed": steps,
                    "algorithmic_bytes": f8_bytes}

    # whole-block fractions of both rooflines, for the record
    blk_bytes = roofline["algorithmic_bytes"] if args.fp8 else wl.algorithmic_bytes(n_active, tp)
    block_stats = {"hbm_gbs": blk_bytes / (ms_per_step * 1e-3) / 1e9,
             "hbm_frac_of_measured": blk_bytes / (ms_per_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
             "tflops_per_gpu": value / tp, "tensor_frac_of_measured_sustained": value / tp / peaks["bf16_tflops_sustained"],
             "algorithmic_bytes_per_rank": blk_bytes, "n_active_experts": n_active}

    extras = {}
    # ---- config 2's comparison: the same tokens as 16 sequential chunks of 512 (what chunked prefill does)
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
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        c0.record()
        for i in range(reps):
            chunked(i)
        c1.record()
        barrier()
        c_ms = max_over_ranks(c0.elapsed_time(c1)) / reps
        per_expert = 3 * wl.H * ip * 2
        extras["chunked_prefill"] = {
            "chunks": n_chunks, "chunk_tokens": 512, "us_all_chunks": c_ms * 1e3, "us_single_pass": ms_per_step * 1e3,
            "speedup_single_pass": c_ms / ms_per_step,
            "weight_bytes_chunked": sum(act_chunks) * per_expert, "weight_bytes_single_pass": n_active * per_expert,
            "expert_reload_bytes_saved": (sum(act_chunks) - n_active) * per_expert}
    # ---- the steps in front of the block (add + RMSNorm, gate projection, top-k): one library call against the
    # reference's sequence of three ops (its norm kernel's twin, a cuBLAS linear, the routing kernel)
    if not mixed and not args.fp8 and world == 1:
        import torch.nn.functional as F
        gpre = torch.Generator(device=dev)
        gpre.manual_seed(7)
        attn = torch.randn(wl.T, wl.H, generator=gpre, device=dev).to(torch.bfloat16)
        resid = torch.randn(wl.T, wl.H, generator=gpre, device=dev).to(torch.bfloat16)
        nw = torch.ones(wl.H, device=dev, dtype=torch.bfloat16)
        wg = (torch.randn(wl.E, wl.H, generator=gpre, device=dev) * 0.02).to(torch.bfloat16)
        normed_buf = torch.empty_like(attn)

        def fused_pre(i):
            fused_moe.pre_moe(attn, resid, nw, 1e-6, wg, wl.top_k, True)

        def three_ops(i):
            ops.add_rms_norm(normed_buf, resid, attn, nw, 1e-6)
            fused_moe.fused_topk(normed_buf, F.linear(normed_buf, wg), wl.top_k, True)

        pre = {}
        for label, fn in (("one_call_us", fused_pre), ("three_ops_us", three_ops)):
            for i in range(5):
                fn(i)
            torch.cuda.synchronize()
            run = fn
            if not prefill:  # device time, not Python call overhead: replay a captured graph
                side2 = torch.cuda.Stream(device=dev)
                side2.wait_stream(torch.cuda.current_stream())
                gq = torch.cuda.CUDAGraph()
                with torch.cuda.stream(side2):
                    fn(0)
                    with torch.cuda.graph(gq, stream=side2):
                        fn(0)
                torch.cuda.current_stream().wait_stream(side2)
                run = lambda i, gq=gq: gq.replay()  # noqa: E731
                run(0)
                torch.cuda.synchronize()
            p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 50 if prefill else 300
            p0.record()
            for i in range(reps):
                run(i)
            p1.record()
            torch.cuda.synchronize()
            pre[label] = p0.elapsed_time(p1) / reps * 1e3
        pre["note"] = ("graph replay" if not prefill else "eager launches") + \
            "; inputs L2-resident across repetitions; three_ops = add_rms_norm + torch linear (cuBLAS) + routing kernel"
        extras["pre_moe"] = pre
    # ---- all-reduce alone (N > 1): the [T, H] bf16 reduction of this workload's batch sizes
    if world > 1:
        ar = {}
        for t_ar in sorted({wl.T, MIXED_DECODE_T} if mixed else {wl.T}):
            buf = torch.randn(t_ar, wl.H, device=dev).to(torch.bfloat16)
            for _ in range(5):
                comm.all_reduce(buf)
            barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 50
            a0.record()
            for _ in range(reps):
                comm.all_reduce(buf)
            a1.record()
            barrier()
            ar[f"T{t_ar}"] = max_over_ranks(a0.elapsed_time(a1)) / reps * 1e3
        extras["all_reduce_us_staged"] = ar
        # the all-reduce followed by the next layer's residual add + RMSNorm: one call vs the two steps
        if not mixed and wl.T <= 1024:
            buf = torch.randn(wl.T, wl.H, device=dev).to(torch.bfloat16)
            resid = torch.randn(wl.T, wl.H, device=dev).to(torch.bfloat16)
            nw = torch.ones(wl.H, device=dev, dtype=torch.bfloat16)
            nout = torch.empty_like(buf)

            def two_steps():
                ops.add_rms_norm(nout, resid, comm.all_reduce(buf), nw, 1e-6)

            def one_call():
                comm.all_reduce_add_rms_norm(buf, resid, nw, 1e-6)

            tail = {}
            for label, fn in (("all_reduce_then_add_rms_norm_us", two_steps), ("one_call_us", one_call)):
                for _ in range(5):
                    fn()
                barrier()
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = 100
                a0.record()
                for _ in range(reps):
                    fn()
                a1.record()
                barrier()
                tail[label] = max_over_ranks(a0.elapsed_time(a1)) / reps * 1e3
            extras["all_reduce_add_rms_norm"] = tail
    if mixed:
        extras["mixed_iteration"] = {"layers": MIXED_LAYERS, "group_layers": MIXED_GROUP, "decode_tokens": MIXED_DECODE_T,
                                     "prefill_tokens": MIXED_PREFILL_T, "moe_path_us_per_iteration": ms_per_step * 1e3}

    cpu_baseline = None
    if rank == 0 and world == 1 and cpu_inputs is not None:
        threads = os.cpu_count() or 1
        tokens = wl.T if wl.T <= 256 else 256
        sec = cpu_block_time(wl, cpu_inputs, tokens, 3 if tokens <= 64 else 2, threads)
        cpu_flops = 2 * tokens * wl.top_k * 3 * wl.H * wl.I
        cpu_baseline = {"value": cpu_flops / sec / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                        "sample": f"{tokens} of {wl.T} tokens, all {wl.E} experts' weights, torch fp32 per-expert loop, "
                                  f"best of {3 if tokens <= 64 else 2} passes", "us_per_layer": sec * 1e6}

    if rank == 0:
        line = {
            "metric": "moe_block_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3 (w8a8, block scales, fp32 accumulation)" if args.fp8 else "bf16",
            "data": "synthetic",
            "config": {"workload": wl.name + ("-fp8" if args.fp8 else ""), "T": wl.T, "H": wl.H, "E": wl.E, "top_k": wl.top_k, "I": wl.I,
                       "tensor_parallel": tp, "I_per_rank": ip,
                       "launch": "cuda graph replay per step" if use_graph else "eager launches",
                       "l2": f"weights rotate over {n_sets} distinct copies ({n_sets * 3 * wl.E * wl.H * ip * (1 if args.fp8 else 2) / 1e6:.0f} MB per rank) so no step finds them in L2",
                       "all_reduce": "fused k-slot sum + peer-memory all-reduce" if world > 1 else "none (1 GPU)"},
            "us_per_layer": ms_per_step * 1e3, "tokens_per_s": wl.T / (ms_per_step * 1e-3),
            "roofline": roofline, "block": block_stats, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": launches, "clocks": clocks,
        }
        line.update(extras)
        print(json.dumps(line), flush=True)
    if world > 1:
        barrier()
        comm.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
