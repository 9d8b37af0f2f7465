"""Benchmark of the MoE layer forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

One "step" is one forward + backward pass of the layer (router gate, top-k, softmax, routing sort, routed
SwiGLU experts, gate-weighted combine; all gradients) over one batch of synthetic tokens.  At N = 1 the
workload is the Mixtral-shaped configuration (8 experts, top-2, hidden 4096, intermediate 14336, 16384
tokens, bf16).  At N > 1 the experts are sharded over the ranks (expert parallel), every rank keeps its
own 16384 tokens (weak scaling) and rows travel through this package's peer-memory kernels (or NCCL all-to-all with
--ep-exchange nccl).  Before anything is timed at N > 1 the expert-parallel layer is checked against the single-GPU
layer on small seeded cases (`ep_parity`; the run exits non-zero if that fails).  The last key of the line,
`ep_configs`, holds short measurements of the other benchmark configurations on the SAME GLOBAL PROBLEM at this N
(fine-grained 64-expert layer, Zipf-skewed 128-expert layer, 256-expert layer: their token counts divided over the ranks).

Prints ONE JSON line on rank 0.  `value` is TFLOP/s of routed-expert GEMM work (18*T*k*H*I per step) with the
inputs resident in HBM; `e2e` is the same metric with host buffers (pinned) copied in and results copied
out inside the timed region; `roofline` describes the tcgen05 grouped-GEMM kernel (all six launches of a
step) against the measured bf16 peak; `cpu_baseline` times the CPU port of the reference torch path on a
bounded token sample.  `--impl reference` runs only that CPU path and prints its own line.
"""

from __future__ import annotations

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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from kernel_hyperdrive_b200 import synthetic  # noqa: E402

METRIC = "moe_layer_fwd_bwd_tflops"
UNIT = "TFLOP/s"
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}

# dram__bytes_read.sum + dram__bytes_write.sum of the six grouped-GEMM launches of one step, from ncu captures of the
# Mixtral-shaped layer at three token counts (these two counters are a one-pass capture, so the benchmark's own size
# could be captured as well).  Other token counts are interpolated between the neighbouring captures.
NCU_TRAFFIC = {
    "c2": {"captures": {4096: 13.020e9, 8192: 21.187e9, 16384: 45.623e9},
           "per_launch_at_16384_tokens": {"up_forward": 5.525e9, "down_forward": 6.864e9, "down_dgrad": 6.347e9, "down_wgrad": 3.134e9,
                                          "up_wgrad": 7.428e9, "up_dgrad": 16.325e9},
           "algorithmic_bytes_at_16384_tokens": 24.1e9},
}


def ncu_traffic(w):
    rec = NCU_TRAFFIC.get(w.name)
    if not rec:
        return None, None
    pts = sorted(rec["captures"].items())
    if w.tokens in rec["captures"]:
        return rec["captures"][w.tokens], rec
    lo = max([p for p in pts if p[0] <= w.tokens] or [pts[0]])
    hi = min([p for p in pts if p[0] >= w.tokens] or [pts[-1]])
    if lo == hi:  # outside the captured range: extend the nearest segment
        lo, hi = (pts[0], pts[1]) if w.tokens < pts[0][0] else (pts[-2], pts[-1])
    return lo[1] + (hi[1] - lo[1]) * (w.tokens - lo[0]) / (hi[0] - lo[0]), rec


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU while the timed region runs (read-only queries).

    NVML in a thread, one sample every 20 ms, so that even a timed region of a few hundred milliseconds is covered;
    `nvidia-smi -lms` (which needs a few hundred milliseconds to start) only if the NVML module is missing.
    """

    QUERY = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index: int):
        self.index, self.samples, self.proc, self.thread = index, [], None, None
        self.sampler = None
        self.sm, self.mx, self.reasons = [], [], set()
        self.stop = threading.Event()

    def _nvml_loop(self, nvml, handle):
        while not self.stop.is_set():
            try:
                self.sm.append(float(nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM)))
                mask = nvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                for name, bit in self.REASON_BITS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self.stop.wait(0.02)

    def _physical_id(self) -> str:
        """The GPU as the driver tools name it: the entry of CUDA_VISIBLE_DEVICES this process's device index selects
        (an index or a UUID), else the index itself."""
        visible = [v.strip() for v in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if v.strip()]
        return visible[self.index] if self.index < len(visible) else str(self.index)

    def __enter__(self):
        try:
            import pynvml as nvml

            nvml.nvmlInit()
            ident = self._physical_id()
            handle = nvml.nvmlDeviceGetHandleByIndex(int(ident)) if ident.isdigit() else nvml.nvmlDeviceGetHandleByUUID(ident.encode())
            self.mx.append(float(nvml.nvmlDeviceGetMaxClockInfo(handle, nvml.NVML_CLOCK_SM)))
            self.thread = threading.Thread(target=self._nvml_loop, args=(nvml, handle), daemon=True)
            self.thread.start()
            self.sampler = "nvml"
            return self
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self._physical_id()}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            self.sampler = "nvidia-smi"
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def __exit__(self, *exc):
        self.stop.set()
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = list(self.sm), list(self.mx), set(self.reasons)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.samples:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "sampler": self.sampler}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm), "sampler": self.sampler}


# --------------------------------------------------------------------------------------------------
# CPU arm: the port of the reference torch path (oracle) on the host cores, bounded token sample
# --------------------------------------------------------------------------------------------------


def cpu_reference_run(w: synthetic.MoEWorkload, steps: int, warmup: int, sample_tokens: int, weights=None):
    """Times forward + backward of the reference torch formulation on CPU in the workload's dtype.

    Returns (TFLOP/s of the sample, seconds per step, description of the sample, threads used).
    """
    from oracle import moe_oracle as orc  # the one place the benchmark executes the oracle

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    dtype = synthetic.TORCH_DTYPES[w.dtype]
    ws = synthetic.scaled(w, tokens=sample_tokens)
    if weights is None:
        # N(0, std) blocks drawn once per projection; expert e uses the block rolled by 17*e rows (distinct
        # matrices with the same distribution) so that start-up stays short on the host
        g = torch.Generator().manual_seed(0)
        E, H, I = w.num_experts, w.hidden, w.intermediate
        fc = (torch.randn(2 * I, H, generator=g) * w.weight_std).to(dtype)
        pj = (torch.randn(H, I, generator=g) * w.weight_std).to(dtype)
        weights = dict(
            gate=(torch.randn(E, H, generator=g) * w.weight_std).to(dtype),
            w_fc=torch.stack([fc.roll(17 * e, 0) for e in range(E)]),
            w_proj=torch.stack([pj.roll(17 * e, 0) for e in range(E)]),
        )
    x, gy = synthetic.make_tokens(ws, 0)
    x, gy = x.to(dtype), gy.to(dtype)
    rw, sel = synthetic.make_routing(ws, x.float(), weights["gate"].float(), 0)
    rw = rw.to(dtype)
    # warm-up on a small slice (thread pools, first-touch of the weight tensors), then the timed passes on the sample
    n_small = max(8, min(64, sample_tokens))
    for _ in range(max(0, warmup)):
        orc.experts_with_grads(x[:n_small], weights["w_fc"], weights["w_proj"], rw[:n_small], sel[:n_small], gy[:n_small])
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        orc.experts_with_grads(x, weights["w_fc"], weights["w_proj"], rw, sel, gy)
        times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    flops = 18.0 * sample_tokens * w.top_k * w.hidden * w.intermediate
    sample = f"{sample_tokens} of {w.tokens} tokens, all {w.num_experts} experts, full H={w.hidden} I={w.intermediate}, {w.dtype}, {steps} timed passes"
    return flops / sec / 1e12, sec, sample, threads


def run_reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 2)), min(args.warmup, 1)  # bounded: a pass over 1024 tokens takes tens of seconds
    val, sec, sample, threads = cpu_reference_run(w, steps, warmup, args.cpu_sample_tokens)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
        "config": workload_config(w, args.gpus),
        "tokens_per_s": args.cpu_sample_tokens / sec,
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(w, n_gpus, exchange="peer-memory kernels over NVLink"):
    return {
        "workload": f"{w.name}: {w.num_experts} experts top-{w.top_k}, hidden {w.hidden}, SwiGLU intermediate {w.intermediate}, {w.tokens} tokens per GPU, {w.dtype}, routing={w.routing}",
        "tokens_per_gpu": w.tokens, "num_experts": w.num_experts, "top_k": w.top_k, "hidden": w.hidden, "intermediate": w.intermediate,
        "parallelism": "single GPU" if n_gpus == 1 else f"expert parallel ep{n_gpus} (experts sharded, dispatch/combine: {exchange})",
        "l2": "inputs_exceed_l2 (expert weights and activations are GBs, L2 is 126 MB)",
    }


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------


def bind_to_gpu_numa_node(index: int) -> None:
    """Binds this process to the CPU cores next to its GPU (NVML's ideal affinity) before any pinned host buffer is
    allocated, so that with several ranks the host<->device copies of each rank stay on its own NUMA node."""
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cpus = [64 * i + b for i, word in enumerate(words) for b in range(64) if (word >> b) & 1]
        if cpus:
            os.sched_setaffinity(0, cpus)
    except Exception:  # noqa: BLE001 - affinity is an optimisation, never a requirement
        pass


SHARE = {"up_forward": 4, "down_forward": 2, "down_dgrad": 2, "down_wgrad": 2, "up_wgrad": 4, "up_dgrad": 4}  # eighteenths of the step's FLOP


class Job:
    """One workload on this rank: the layer, its resident inputs and the forward closure."""

    def __init__(self, w, world, rank, dev, exchange, placement=None, micro_batches=1, sync_free=False):
        import torch.distributed as dist

        import kernel_hyperdrive_b200 as kh

        self.w, self.world, self.rank, self.dev = w, world, rank, dev
        dtype = self.dtype = synthetic.TORCH_DTYPES[w.dtype]
        E, k, H, I, T = w.num_experts, w.top_k, w.hidden, w.intermediate, w.tokens
        extra = dict(num_shared_experts=w.shared_experts, router_scoring="sigmoid" if w.routing == "sigmoid" else "softmax")
        self.placement_note = None
        if world > 1:
            from kernel_hyperdrive_b200.expert_parallel import MoE_B200_EP

            expected = [1.0] * E
            if w.routing == "zipf":
                # The skew is a property of the routing distribution: experts are placed by their expected load, as a
                # deployment would from running token counts.  The counts come from a separate sample of the same
                # distribution (other seed, 16384 tokens; the same on every rank): the k distinct experts of a token are
                # drawn without replacement, so the popular experts saturate and the loads are flatter than p ~ rank^-1.2.
                _, sample = synthetic.make_routing(synthetic.scaled(w, tokens=16384), torch.zeros(16384, 1), None, 987)
                expected = torch.bincount(sample.flatten(), minlength=E).double().add_(1.0).tolist()
            if placement is None and w.routing == "zipf":
                placement = "balanced"
            self.placement_note = placement or "contiguous"
            rows = (2 if (w.routing != "zipf" or placement == "balanced") else world) * T * k
            if w.routing in ("sigmoid", "normal_logits"):
                rows = int(1.25 * T * k)  # iid logits: the per-rank receive counts stay within a few percent of T * k
            self.layer = MoE_B200_EP(E, k, H, I, kh.swiglu_unchunked_torch, True, False, w.weight_std, group=dist.group.WORLD, device=dev, dtype=dtype, seed=0,
                                     exchange=exchange, exchange_rows=(rows + 127) // 128 * 128, placement=placement, expected_load=expected,
                                     micro_batches=micro_batches, sync_free=sync_free, **extra)
        else:
            torch.manual_seed(0)
            torch.set_default_dtype(dtype)  # build the (large) expert tensors directly in the workload's type
            try:
                with torch.device(dev):
                    self.layer = kh.MoE_B200(E, k, H, I, kh.swiglu_unchunked_torch, True, False, w.weight_std, **extra)
            finally:
                torch.set_default_dtype(torch.float32)
        self.params = list(self.layer.parameters())
        gen = torch.Generator().manual_seed(1000 + rank)
        self.x_host = torch.randn(T, H, generator=gen).to(dtype).pin_memory()
        self.g_host = torch.randn(T, H, generator=gen).to(dtype).pin_memory()
        self.x_dev = self.x_host.to(dev).requires_grad_(True)
        self.g_dev = self.g_host.to(dev)
        self.routing_note = None
        layer = self.layer
        if w.routing == "gate":
            self.forward = lambda x: layer(x)[0]
        else:
            # routing supplied from outside (logits drawn per token and expert, or Zipf-distributed expert choice):
            # enters through the layer's `_compute_experts(hidden_states, router_weights, selected_experts)` seam
            rw_cpu, sel_cpu = synthetic.make_routing(w, self.x_host.float(), torch.zeros(E, 1), seed=1000 + rank)
            rw_dev, sel_dev = rw_cpu.to(dev, dtype), sel_cpu.to(dev)
            counts = torch.bincount(sel_cpu.flatten(), minlength=E)
            self.routing_note = {"rows_min": int(counts.min()), "rows_max": int(counts.max()), "rows_mean": float(counts.float().mean()), "empty_experts": int((counts == 0).sum())}

            def forward(x):
                out = layer._compute_experts(x, rw_dev, sel_dev)
                if w.shared_experts:
                    out = out + layer._compute_shared_experts(x)
                return out

            self.forward = forward

    def step_resident(self):
        for p in self.params:
            p.grad = None
        self.x_dev.grad = None
        y = self.forward(self.x_dev)
        y.backward(self.g_dev)
        return y

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    def timed(self, fn, steps):
        """CUDA-event time of `steps` calls of fn between two rank barriers: the maximum over the ranks, in ms."""
        self.barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        end.record()
        self.barrier()
        ms = torch.tensor([start.elapsed_time(end)], device=self.dev)
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    def measure_resident(self, steps, warm, sample_clocks=False):
        """Warm-up, then `steps` timed steps with every kernel group bracketed by events.  Returns a dict with the step
        time, the per-phase device times per step and (N > 1) the per-rank load report."""
        from kernel_hyperdrive_b200 import _lib, scattermoe

        for _ in range(warm):
            self.step_resident()
        _lib.check_status(self.dev)
        sink = []
        scattermoe.set_timing_sink(sink)
        launches0 = _lib.launch_count()
        if sample_clocks:
            with ClockSampler(self.dev.index or 0) as clocks:
                total_ms = self.timed(self.step_resident, steps)
            clock_summary = clocks.summary()
        else:
            total_ms, clock_summary = self.timed(self.step_resident, steps), None
        launches = _lib.launch_count() - launches0
        scattermoe.set_timing_sink(None)
        torch.cuda.synchronize()
        _lib.check_status(self.dev)
        phases = {}
        for name, s_, e_ in sink:
            phases[name] = phases.get(name, 0.0) + s_.elapsed_time(e_)
        phases = {n: v / steps for n, v in phases.items()}
        w = self.w
        gemm_ms = {n: ms for n, ms in phases.items() if n in SHARE}
        gemm_total = sum(gemm_ms.values())
        local_flops = w.flops_fwd_bwd()
        out = {
            "ms_per_step": total_ms / steps, "tflops": local_flops * self.world / (total_ms / steps * 1e-3) / 1e12, "launches": launches, "clocks": clock_summary,
            "gemm_ms": gemm_total, "gemm_tflops_this_rank": None, "phase_ms": {n: round(v, 4) for n, v in sorted(phases.items())},
            "per_launch": {n: {"ms": ms, "tflops": None} for n, ms in gemm_ms.items()},
        }
        if self.world > 1:
            import torch.distributed as dist

            rows = float(self.layer.received_rows())
            exch = sum(v for n, v in phases.items() if n.startswith("ep_push") or n.startswith("ep_pull"))
            barr = phases.get("ep_barrier", 0.0)
            mine = torch.tensor([rows, gemm_total, exch, barr], device=self.dev, dtype=torch.float64)
            everyone = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(everyone, mine)
            table = torch.stack(everyone).cpu()
            out["per_rank"] = {"received_rows": [int(v) for v in table[:, 0]], "gemm_ms": [round(float(v), 3) for v in table[:, 1]],
                               "exchange_ms": [round(float(v), 3) for v in table[:, 2]], "barrier_ms": [round(float(v), 3) for v in table[:, 3]]}
            # FLOP this rank's experts really did: its received rows (routed experts) plus its own tokens through the shared experts
            local_flops = 18.0 * rows * w.hidden * w.intermediate + 18.0 * w.tokens * w.shared_experts * w.hidden * w.intermediate
        if gemm_total > 0:
            out["gemm_tflops_this_rank"] = local_flops / (gemm_total * 1e-3) / 1e12
            for n, ms in gemm_ms.items():
                out["per_launch"][n]["tflops"] = (SHARE[n] / 18.0) * local_flops / (ms * 1e-3) / 1e12
        return out

    def release(self):
        self.layer = self.params = self.forward = self.x_dev = self.g_dev = None
        import gc

        gc.collect()
        torch.cuda.empty_cache()


def run_ep_configs(args, world, rank, dev, peaks):
    """Short measurements of the other benchmark configurations on the same global problem at this N: tokens divided
    over the ranks, experts sharded.  One entry per configuration; device-resident step time (max over ranks)."""
    out = {}
    names = ["c3", "c4"] + (["c5"] if world > 1 else [])
    for name in names:
        base = synthetic.WORKLOADS[name]
        if base.num_experts % world or base.tokens % world:
            continue
        w = synthetic.scaled(base, tokens=base.tokens // world)
        try:
            job = Job(w, world, rank, dev, args.ep_exchange, micro_batches=args.ep_micro_batches, sync_free=args.ep_sync_free)
            m = job.measure_resident(args.ep_config_steps, 3)
            entry = {
                "tokens_global": base.tokens, "tokens_per_gpu": w.tokens, "experts_per_gpu": base.num_experts // world, "ms_per_step": round(m["ms_per_step"], 4),
                "tflops": round(m["tflops"], 2), "tflops_per_gpu": round(m["tflops"] / world, 2), "frac_of_bf16_peak_burst_per_gpu": round(m["tflops"] / world / peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]), 4),
                "tokens_per_s": round(base.tokens / (m["ms_per_step"] * 1e-3), 1), "gemm_ms_rank0": round(m["gemm_ms"], 4),
                "gemm_tflops_rank0": None if m["gemm_tflops_this_rank"] is None else round(m["gemm_tflops_this_rank"], 1),
                "per_launch_tflops_rank0": {n: round(v["tflops"], 1) for n, v in m["per_launch"].items() if v["tflops"]},
                "phase_ms_rank0": m["phase_ms"], "routing": job.routing_note,
            }
            if world > 1:
                entry["placement"], entry["per_rank"] = job.placement_note, m["per_rank"]
            out[name] = entry
            job.release()
            del job
        except Exception as exc:  # noqa: BLE001 - a configuration that cannot run here is reported, not fatal
            out[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
            import gc

            gc.collect()
            torch.cuda.empty_cache()
    return out


def triton_reference_probe(w, dev, steps):
    """Times the reference package's own Triton MoE layer on this GPU when that package is importable on the box
    (it is not part of this repository); otherwise says so."""
    try:
        import cute_kernels  # noqa: F401
        from cute_kernels import MoE_Triton as RefMoE
    except Exception as exc:  # noqa: BLE001
        return f"unavailable: reference package not installed on this box ({type(exc).__name__})"
    try:
        import kernel_hyperdrive_b200 as kh

        dtype = synthetic.TORCH_DTYPES[w.dtype]
        layer = RefMoE(w.num_experts, w.top_k, w.hidden, w.intermediate, kh.swiglu_unchunked_torch, True, False, w.weight_std).to(dev, dtype)
        x = torch.randn(w.tokens, w.hidden, device=dev, dtype=dtype, requires_grad=True)
        g = torch.randn_like(x)
        for _ in range(3):
            layer(x)[0].backward(g)
        torch.cuda.synchronize()
        s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s_.record()
        for _ in range(steps):
            layer(x)[0].backward(g)
        e_.record()
        torch.cuda.synchronize()
        ms = s_.elapsed_time(e_) / steps
        return {"ms_per_step": ms, "tflops": w.flops_fwd_bwd() / (ms * 1e-3) / 1e12}
    except Exception as exc:  # noqa: BLE001
        return f"unavailable: reference Triton layer failed here ({type(exc).__name__}: {str(exc)[:120]})"


def run_gpu_arm(args, w):
    import torch.distributed as dist

    from kernel_hyperdrive_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world} (launch with torch.distributed.run)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        bind_to_gpu_numa_node(local_rank)
        dist.init_process_group("nccl", device_id=dev)
    _lib.set_option(_lib.OPT_TILE_VARIANT, {"table": -1, "pair": _lib.TILE_PAIR_256x256, "cta": _lib.TILE_CTA_128x256}[args.tile_variant])
    if args.tile_scheduler is not None:
        _lib.set_option(_lib.OPT_DYNAMIC_TILES, args.tile_scheduler)
    if args.tile_order is not None:
        _lib.set_option(_lib.OPT_TILE_ORDER, args.tile_order)
    peaks, peak_kind = measured_peaks()

    # ---- N > 1: correctness of the exchange first ----
    ep_parity = None
    if world > 1 and not args.skip_ep_parity:
        from kernel_hyperdrive_b200.expert_parallel import parity_selfcheck

        ep_parity = parity_selfcheck(dist.group.WORLD, dev)
        if not ep_parity["ok"]:
            if rank == 0:
                print(json.dumps({"metric": METRIC, "n_gpus": world, "error": "expert-parallel parity check failed", "ep_parity": ep_parity}), flush=True)
            dist.destroy_process_group()
            sys.exit(3)

    job = Job(w, world, rank, dev, args.ep_exchange, placement=args.ep_placement, micro_batches=args.ep_micro_batches, sync_free=args.ep_sync_free)
    dtype, T, H = job.dtype, w.tokens, w.hidden
    x_host, g_host, params, forward = job.x_host, job.g_host, job.params, job.forward
    y_host = torch.empty(T, H, dtype=dtype).pin_memory()
    dx_host = torch.empty(T, H, dtype=dtype).pin_memory()

    # End-to-end loop as a host program would run it: inputs start in pinned host memory every step and the
    # results (layer output and input gradient) are read back to the host every step.  Copies run on their own
    # streams, double-buffered, so the upload of step i+1 and the read-back of step i-1 overlap the kernels of
    # step i; every copy of every timed step lies inside the timed region.  The tokens are uploaded before the output
    # gradient (the forward pass needs only the former) and the layer output is read back as soon as the forward pass
    # has produced it, so that only half of a step's traffic is exposed when the pipeline fills and drains.
    copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    x_slots = [torch.empty(T, H, device=dev, dtype=dtype) for _ in range(2)]
    g_slots = [torch.empty(T, H, device=dev, dtype=dtype) for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_in_g = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    ev_fwd = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    keep = [None, None]

    def upload(slot):
        with torch.cuda.stream(copy_in):
            copy_in.wait_event(ev_free[slot])  # the step that last read this slot has finished
            x_slots[slot].copy_(x_host, non_blocking=True)
            ev_in[slot].record(copy_in)
            g_slots[slot].copy_(g_host, non_blocking=True)
            ev_in_g[slot].record(copy_in)

    def run_e2e(steps):
        main = torch.cuda.current_stream(dev)
        for s_ in range(2):
            ev_free[s_].record(main)
        upload(0)
        for i in range(steps):
            slot = i % 2
            if i + 1 < steps:
                upload(1 - slot)
            main.wait_event(ev_in[slot])
            for p in params:
                p.grad = None
            x = x_slots[slot].detach().requires_grad_(True)
            y = forward(x)
            ev_fwd[slot].record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(ev_fwd[slot])
                y_host.copy_(y.detach(), non_blocking=True)
                y.record_stream(copy_out)
            main.wait_event(ev_in_g[slot])
            y.backward(g_slots[slot])
            ev_free[slot].record(main)
            ev_done[slot].record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(ev_done[slot])
                dx_host.copy_(x.grad, non_blocking=True)
                x.grad.record_stream(copy_out)
            keep[slot] = (y, x)  # keep the device results alive until their read-back has been issued and ordered
        main.wait_stream(copy_out)

    n_warm = args.warmup if args.profile else max(args.warmup, 3)
    m = job.measure_resident(args.steps, n_warm, sample_clocks=True)

    if args.profile:
        e2e_ms = float("nan")
    else:
        run_e2e(2)
        torch.cuda.synchronize()
        e2e_ms = job.timed(lambda: run_e2e(args.steps), 1)
    _lib.check_status(dev)

    flops_step = w.flops_fwd_bwd() * world  # every rank brings T tokens
    ms_step = m["ms_per_step"]
    value = flops_step / (ms_step * 1e-3) / 1e12
    e2e_value = flops_step / (e2e_ms / args.steps * 1e-3) / 1e12
    peak = peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"])
    achieved = m["gemm_tflops_this_rank"]
    exchange_ms = {n: v for n, v in m["phase_ms"].items() if n.startswith("ep_")}
    extra_info = {} if job.routing_note is None else {"routing": job.routing_note}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": n_warm,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
        "config": workload_config(w, world, "peer-memory kernels over NVLink" if args.ep_exchange == "p2p" else "NCCL all-to-all"),
        "tokens_per_s": T * world / (ms_step * 1e-3),
        "frac_of_bf16_peak_burst": value / world / peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]),
        "frac_of_bf16_peak_sustained": value / world / peak,
        "clocks": m["clocks"],
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms / args.steps, "h2d_bytes_per_step": 2 * x_host.numel() * x_host.element_size(), "d2h_bytes_per_step": 2 * y_host.numel() * y_host.element_size()},
        "gpu_launches": m["launches"], "ep_micro_batches": args.ep_micro_batches if world > 1 else None, "tile_variant": args.tile_variant, "tile_scheduler": _lib.get_option(_lib.OPT_DYNAMIC_TILES), **extra_info,
        **({"exchange_ms_per_step": exchange_ms} if exchange_ms else {}),
        "roofline": {
            "bound": "tensor", "kernel": "umma2_grouped_kernel (6 launches per step)", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": (achieved / peak) if achieved else None, "peak_kind": f"bf16_tflops_sustained of {peak_kind}",
            "traffic": ncu_traffic(w)[0], "traffic_captures": ncu_traffic(w)[1], "per_launch": m["per_launch"], "gemm_ms_per_step": m["gemm_ms"],
            "phase_ms_per_step": m["phase_ms"],
        },
    }
    if world > 1:
        line["per_rank"] = m["per_rank"]
        line["ep_parity"] = ep_parity if ep_parity is not None else "skipped"
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not args.profile and w.name in ("c1", "c2"):
        layer = job.layer
        cpu_w = dict(gate=layer.gate.weight.detach().cpu(), w_fc=layer.c_fc.weight.detach().cpu(), w_proj=layer.c_proj.weight.detach().cpu())
        val, sec, sample, threads = cpu_reference_run(w, 1, 1, args.cpu_sample_tokens, weights=cpu_w)
        line["cpu_baseline"] = {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}
        del cpu_w
    if world == 1 and not args.profile and not args.no_triton_reference and w.name == "c2":
        line["triton_reference"] = triton_reference_probe(w, dev, min(args.steps, 5))
    # the other configurations on the same global problem: last key of the line
    if not args.profile and not args.no_ep_configs and args.workload == "c2" and args.tokens is None:
        job.release()
        del job, x_slots, g_slots, keep, forward, params
        torch.cuda.empty_cache()
        line["ep_configs"] = run_ep_configs(args, world, rank, dev, peaks)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_micro():
    """Row-kernel timings at the reference's own benchmark sizes (CUDA events): the SwiGLU operator on x = (81920, 8192),
    the histogram and the routing sort on 1M ids.  Prints one JSON line; not the benchmark metric."""
    import kernel_hyperdrive_b200 as kh
    from kernel_hyperdrive_b200.ops import _swiglu_backward, _swiglu_forward

    def timed(fn, iters=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s_.record()
        for _ in range(iters):
            fn()
        e_.record()
        torch.cuda.synchronize()
        return s_.elapsed_time(e_) / iters

    out = {"impl": "micro"}
    n = 81920 * 4096
    for name, dt in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
        x = torch.randn(81920, 8192, device="cuda", dtype=dt)
        y = torch.empty(81920, 4096, device="cuda", dtype=dt)
        dy, dx = torch.randn_like(y), torch.empty_like(x)
        f, b = timed(lambda: _swiglu_forward(x, y)), timed(lambda: _swiglu_backward(x, dy, dx))
        out[f"swiglu_unchunked_forward_{name}"] = {"ms": f, "GB/s": 3 * n * x.element_size() / f / 1e6}
        out[f"swiglu_unchunked_backward_{name}"] = {"ms": b, "GB/s": 5 * n * x.element_size() / b / 1e6}
        del x, y, dy, dx
    # RMSNorm of the layer's input: forward 2 passes over (T, H), backward 3
    from kernel_hyperdrive_b200.ops import _rmsnorm_backward, _rmsnorm_forward

    for name, (T, H) in (("16384x4096", (16384, 4096)), ("131072x2048", (131072, 2048)), ("65536x7168", (65536, 7168))):
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        wn = torch.ones(H, device="cuda", dtype=torch.bfloat16)
        y, dy, dx, dwn = torch.empty_like(x), torch.randn_like(x), torch.empty_like(x), torch.empty_like(wn)
        rstd = torch.empty(T, device="cuda", dtype=torch.float32)
        f = timed(lambda: _rmsnorm_forward(x, wn, y, rstd, 1e-5))
        b = timed(lambda: _rmsnorm_backward(x, wn, dy, rstd, dx, dwn, 1e-5))
        e_ = timed(lambda: torch.nn.functional.rms_norm(x, (H,), wn, 1e-5))
        out[f"rmsnorm_bf16_{name}"] = {"forward_ms": f, "forward_GB/s": 2 * T * H * 2 / f / 1e6, "backward_ms": b, "backward_GB/s": 3 * T * H * 2 / b / 1e6, "torch_forward_ms": e_}
        del x, y, dy, dx
    # router: one fused launch against the eager gate GEMM + top-k + softmax + casts (+ histogram)
    for name, (T, H, E, k) in (("c2_T16384_H4096_E8_k2", (16384, 4096, 8, 2)), ("c5_per_gpu_T16384_H7168_E256_k8", (16384, 7168, 256, 8))):
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        wg = (torch.randn(E, H, device="cuda") * 0.02).to(torch.bfloat16)

        def eager():
            logits = torch.nn.functional.linear(x, wg)
            vals, idx = logits.topk(k, dim=-1)
            return torch.softmax(vals.float(), dim=-1).type_as(x), idx, idx.flatten().bincount(minlength=E)

        f, e_ = timed(lambda: kh.router_forward(x, wg, k, 0)), timed(eager)
        nbytes = (T * H + E * H + T * E + T * k) * 2 + T * k * 8
        out[f"router_{name}"] = {"fused_us": f * 1e3, "eager_us": e_ * 1e3, "fused_GB/s": nbytes / f / 1e6, "fused_TFLOP/s": 2 * T * H * E / f / 1e9}
        del x, wg
    # gate gradient of the expert-parallel return path: row dots against the batched product of the reference
    from kernel_hyperdrive_b200.ops import gate_grad as _gate_grad

    T, k, H = 16384, 2, 4096
    expanded = torch.randn(T * k, H, device="cuda", dtype=torch.bfloat16)
    gy = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    f = timed(lambda: _gate_grad(expanded, gy, k))
    e_ = timed(lambda: torch.bmm(expanded.view(T, k, -1), gy.unsqueeze(2)))
    out["ep_gate_grad_16384x2x4096_bf16"] = {"us": f * 1e3, "GB/s": (T * k + T) * H * 2 / f / 1e6, "torch_bmm_us": e_ * 1e3}
    del expanded, gy
    ids = torch.randint(0, 256, (1 << 20,), device="cuda")
    out["contiguous_count_1M_ids_256_bins"] = {"us": timed(lambda: kh.contiguous_count_cute(ids, 256)) * 1e3}
    out["route_1M_ids_256_experts"] = {"us": timed(lambda: kh.route(ids, 256, 8, True, True)) * 1e3}
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(synthetic.WORKLOADS))
    ap.add_argument("--tokens", type=int, default=None, help="override tokens per GPU (profiling on a small case)")
    ap.add_argument("--experts", type=int, default=None, help="override the number of experts (e.g. the per-GPU expert count of a larger job on fewer GPUs)")
    ap.add_argument("--cpu-sample-tokens", type=int, default=1024, help="tokens of the workload the CPU arm times (1/16 of the Mixtral-shaped batch by default)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ep-exchange", default="p2p", choices=["p2p", "nccl"], help="N > 1: row exchange by this package's kernels over peer memory, or NCCL all-to-all")
    ap.add_argument("--tile-variant", default="table", choices=["table", "pair", "cta"], help="tensor-core tile: per-shape table (default), or force the two-CTA 256x256 / one-CTA 128x256 tile (A/B measurements)")
    ap.add_argument("--tile-scheduler", type=int, default=None, choices=[0, 1, 2, 3], help="two-CTA kernels: 0 = fixed stride, 1 = weight-gradient launches draw tiles from a counter, 2 = those and long-reduction row launches (library default), 3 = every launch")
    ap.add_argument("--ep-placement", default=None, choices=["contiguous", "strided", "balanced"], help="N > 1: expert -> rank placement (default: contiguous; the Zipf workload defaults to balanced by expected load)")
    ap.add_argument("--ep-micro-batches", type=int, default=1, help="N > 1, peer-memory exchange: slices of a rank's tokens whose transfers overlap the expert GEMMs of the other slices")
    ap.add_argument("--ep-sync-free", action="store_true", help="N > 1, peer-memory exchange: no host read per pass (local tensors sized by the buffer capacity)")
    ap.add_argument("--skip-ep-parity", action="store_true", help="N > 1: skip the parity check of the expert-parallel exchange that precedes the timing")
    ap.add_argument("--no-ep-configs", action="store_true", help="skip the short runs of the other benchmark configurations appended as `ep_configs`")
    ap.add_argument("--ep-config-steps", type=int, default=5)
    ap.add_argument("--no-triton-reference", action="store_true")
    ap.add_argument("--tile-order", type=int, default=None, choices=[-1, 0, 1, 2], help="row GEMMs: 1 = column blocks of a row tile first, 0 = row tiles of a column block first, 2 = blocks of 8 x 8 tiles, -1 = by weight-matrix size (library default)")
    ap.add_argument("--micro", action="store_true", help="time the row kernels (SwiGLU operator, histogram, routing sort) instead of the layer")
    ap.add_argument("--profile", action="store_true", help="profiling run under ncu: exactly --warmup warm-up steps, no end-to-end and CPU legs; its numbers are not benchmark values")
    args = ap.parse_args()
    w = synthetic.WORKLOADS[args.workload]
    if args.experts:
        w = synthetic.scaled(w, num_experts=args.experts)
    if args.tokens:
        w = synthetic.scaled(w, tokens=args.tokens)
    elif w.name == "c5":
        w = synthetic.scaled(w, tokens=w.tokens // 8)  # the configuration is stated for 8 GPUs: 131072 tokens over 8 ranks
    if args.micro:
        run_micro()
    elif args.impl == "reference":
        run_reference_arm(args, w)
    else:
        run_gpu_arm(args, w)


if __name__ == "__main__":
    main()
