"""Benchmark of the MegaMoE layer hot path on B200: tokens/s of forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N = 1 runs the per-rank problem of the expert-parallel BF16 configuration on one GPU (EP = 1):
4096 tokens, hidden 4096, 32 experts, softmax top-4, SwiGLU experts with intermediate 1536.
Under torchrun (N > 1) every rank brings its own 4096 tokens and owns 32 / N experts (EP = N,
weak scaling); rows travel through the peer-mapped buffers, NCCL carries only set-up traffic.

One JSON line is printed by rank 0. `value` times the layer with inputs resident in HBM; `e2e`
times the same call through the module API with host buffers (pinned host -> device copies of the
step's inputs and device -> host copies of its results inside the timed region). `parity` is one
forward + backward of the bench shape checked against the CPU oracle (outside the timed region; the
run exits non-zero when it fails). `extra` carries the other configurations of the metric: the MXFP8
layer on both shapes, the router and the residual mix (one GPU), and NVLink figures (N > 1).
`--impl reference` times the CPU restatement of the reference's golden path on the host cores.
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
from dataclasses import dataclass
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "moe_layer_fwd_bwd_tokens_per_s"
UNIT = "tokens/s"


@dataclass(frozen=True)
class Shape:
    """One MoE workload. `experts_per_rank` set: the expert count grows with the number of ranks."""

    name: str
    tokens: int
    hidden: int
    top_k: int
    inter: int
    experts: int | None = None
    experts_per_rank: int | None = None
    zipf: float | None = None

    def num_experts(self, world: int) -> int:
        return self.experts if self.experts is not None else self.experts_per_rank * world

    @property
    def flops_per_token(self) -> int:
        # forward 6*K*H*I flops per token (two GEMMs), backward 12*K*H*I (four GEMMs)
        return 18 * self.top_k * self.hidden * self.inter


# "c2": the per-rank problem of the EP=2 BF16 configuration (the headline). "c3": the per-rank problem of the
# EP=8 MXFP8 configuration (32 experts per rank, Zipf(1.1) expert load, 4 of 8 expert groups per token).
SHAPES = {
    "c2": Shape("c2", tokens=4096, hidden=4096, top_k=4, inter=1536, experts=32),
    "c3": Shape("c3", tokens=8192, hidden=7168, top_k=8, inter=2048, experts_per_rank=32, zipf=1.1),
}


def make_inputs(shape: Shape, rank: int, ep: int, device=None):
    """Seeded synthetic inputs of the configuration's shapes and distributions (CPU, then copied)."""
    tokens, hidden, top_k, inter = shape.tokens, shape.hidden, shape.top_k, shape.inter
    experts = shape.num_experts(ep)
    g = torch.Generator().manual_seed(1234 + rank)
    x = torch.randn(tokens, hidden, generator=g).bfloat16()
    # "uniform-ish" router logits: U(-1, 1) plus small noise, softmax, top-k
    logits = torch.rand(tokens, experts, generator=g) * 2 - 1 + 0.01 * torch.randn(tokens, experts, generator=g)
    if shape.zipf is not None:
        # skewed router logits: expert popularity follows Zipf(s) over a fixed random ranking (Gumbel top-k)
        ranking = torch.randperm(experts, generator=torch.Generator().manual_seed(99))
        popularity = torch.empty(experts)
        popularity[ranking] = torch.arange(1, experts + 1, dtype=torch.float32).pow(-shape.zipf)
        gumbel = -torch.log(-torch.log(torch.rand(tokens, experts, generator=g).clamp_min(1e-9)))
        logits = popularity.log() + gumbel
        # group-limited selection of that configuration: 8 expert groups, the 4 best per token (group score =
        # sum of the two largest scores of the group), then top-k inside them
        scores = logits.sigmoid()
        grouped = scores.view(tokens, 8, experts // 8)
        best_groups = grouped.topk(2, dim=-1).values.sum(dim=-1).topk(4, dim=-1).indices
        keep = torch.zeros(tokens, 8, dtype=torch.bool).scatter_(1, best_groups, True)
        limited = scores.masked_fill(~keep.unsqueeze(-1).expand_as(grouped).reshape(tokens, experts), float("-inf"))
        ids = torch.topk(limited, top_k, dim=-1).indices
        weights = scores.gather(1, ids)
        weights = weights / weights.sum(dim=-1, keepdim=True)
    else:
        weights, ids = torch.topk(logits.softmax(dim=-1), top_k, dim=-1)
    grad_out = torch.randn(tokens, hidden, generator=g).bfloat16()
    local = experts // ep
    if device is not None:
        # large shapes: draw the weights on the GPU (seeded), there is nothing to compare them with on the CPU
        gw = torch.Generator(device=device).manual_seed(4321 + rank)
        w1 = (torch.randn(local, hidden, 2 * inter, generator=gw, device=device) * 0.02).bfloat16()
        w2 = (torch.randn(local, inter, hidden, generator=gw, device=device) * 0.02).bfloat16()
    else:
        gw = torch.Generator().manual_seed(4321 + rank)
        w1 = (torch.randn(local, hidden, 2 * inter, generator=gw) * 0.02).bfloat16()
        w2 = (torch.randn(local, inter, hidden, generator=gw) * 0.02).bfloat16()
    return x, ids, weights.contiguous(), grad_out, w1, w2


def config(shape: Shape, ep: int, precision: str) -> dict:
    experts = shape.num_experts(ep)
    routing = (f"sigmoid top-{shape.top_k} in 4 of 8 expert groups, Zipf({shape.zipf}) load" if shape.zipf
               else f"softmax top-{shape.top_k}")
    return {
        "workload": (f"MegaMoE {precision.upper()} forward+backward, EP={ep}, {shape.tokens} tokens/rank, hidden "
                     f"{shape.hidden}, {experts} experts ({experts // ep}/rank), {routing}, SwiGLU intermediate {shape.inter}"),
        "tokens_per_rank": shape.tokens, "hidden": shape.hidden, "experts": experts, "top_k": shape.top_k,
        "intermediate": shape.inter, "ep": ep, "layout": "EIO",
        "l2": "no flush: each step streams >1.4 GB of weights and activations through the 126 MB L2",
    }


def load_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        peaks = json.loads(path.read_text())
        return {"bf16_sustained": float(peaks["bf16_tflops_sustained"]), "bf16_burst": float(peaks["bf16_tflops"]),
                "hbm_gbs": float(peaks["hbm_gbs"]), "source": "of measured"}
    return {"bf16_sustained": 1400.0, "bf16_burst": 1590.0, "hbm_gbs": 6650.0, "source": "of fallback"}


# ----------------------------------------------------------------------------------- CPU baseline
def cpu_full_problem(shape: Shape, iterations: int, warm: bool) -> dict:
    """Time the oracle (port of the reference's TorchExperts CPU branch) on the FULL per-rank problem:
    every token of rank 0 through every expert, forward + backward, all host threads. The cost of this path
    is nearly flat in the token count (per-expert autograd over all the weights), so a token subsample
    cannot be extrapolated."""
    from oracle import moe as omoe

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    x, ids, weights, grad_out, w1, w2 = make_inputs(shape, 0, 1)
    if warm:
        omoe.experts_forward_backward(x, ids, weights, w1, w2, grad_out)
    times = []
    for _ in range(iterations):
        t0 = time.perf_counter()
        omoe.experts_forward_backward(x, ids, weights, w1, w2, grad_out)
        times.append(time.perf_counter() - t0)
    seconds = statistics.median(times)
    return {
        "value": shape.tokens / seconds, "unit": UNIT, "cores": threads, "kind": "port",
        "sample": (f"full: all {shape.tokens} tokens of rank 0 through all {shape.num_experts(1)} experts, forward+backward, "
                   f"{'1 warm-up + ' if warm else ''}median of {iterations} ({seconds:.2f} s each), torch CPU threads={threads}"),
        "seconds_per_step": seconds,
    }


def run_reference(args) -> None:
    """Reference arm: the CPU restatement of the reference's golden path on the host cores. Every step
    (warm-up and timed alike) is one forward + backward over the full per-rank problem."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import moe as omoe

    shape = SHAPES[args.shape]
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    x, ids, weights, grad_out, w1, w2 = make_inputs(shape, 0, 1)
    per_step = []
    for step in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        omoe.experts_forward_backward(x, ids, weights, w1, w2, grad_out)
        if step >= args.warmup:
            per_step.append(time.perf_counter() - t0)
    seconds = sum(per_step) / len(per_step)
    value = shape.tokens / seconds
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config(shape, 1, "bf16"),
        "cpu_baseline": {
            "value": value, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": (f"full: each step = all {shape.tokens} tokens through all {shape.num_experts(1)} experts, "
                       "forward+backward, on the CPU restatement of the reference's golden path (the reference's "
                       "native path needs Ascend hardware)"),
        },
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------ clock sampler
class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, maxima, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                maxima.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(names, parts[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": max(maxima) if maxima else None,
            "reasons": sorted(reasons), "samples": len(clocks),
        }


# ------------------------------------------------------------------------------------------- GPU arm
class Context:
    """Process-wide state of one bench run: ranks, device, barrier, device-timed loops."""

    def __init__(self, args) -> None:
        import torch.distributed as dist

        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run); "
                             f"got WORLD_SIZE={self.world}")
        self.device = torch.device("cuda", self.local_rank)
        torch.cuda.set_device(self.device)
        self.group = None
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.device)
            self.group = dist.group.WORLD

    def barrier(self) -> None:
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, value: float) -> float:
        if self.world == 1:
            return value
        t = torch.tensor([value], device=self.device, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, step, steps: int, warmup: int, join=()):
        """W untimed steps, then exactly K steps between two events, a barrier + synchronize on both
        sides, the MAX over ranks. Returns (total ms, kernels launched in the timed region)."""
        from hyper_multicore_b200 import _lib

        for _ in range(warmup):
            step()
        self.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches_before = _lib.launch_count()
        start.record()
        for _ in range(steps):
            step()
        for stream in join:  # the last results must be on the host before the clock stops
            torch.cuda.current_stream(self.device).wait_stream(stream)
        stop.record()
        self.barrier()
        return self.max_over_ranks(start.elapsed_time(stop)), _lib.launch_count() - launches_before

    def close(self) -> None:
        if self.world > 1:
            self.dist.destroy_process_group()


class MoeLayerRun:
    """One MoE workload on this rank: module, weights, device-resident inputs, step functions."""

    def __init__(self, ctx: Context, shape: Shape, precision: str, dispatch: str, weights_on_device: bool) -> None:
        from hyper_multicore_b200 import MegaMoeExperts, MegaMoeTuningOptions

        self.ctx, self.shape, self.precision = ctx, shape, precision
        device = ctx.device
        self.host = make_inputs(shape, ctx.rank, ctx.world, device if weights_on_device else None)
        x_h, ids_h, p_h, g_h, w1_h, w2_h = self.host
        self.w1 = w1_h.to(device).requires_grad_(True)
        self.w2 = w2_h.to(device).requires_grad_(True)
        if precision == "mxfp8":
            from hyper_multicore_b200.mxfp8 import attach_mx_fields

            attach_mx_fields(self.w1)
            attach_mx_fields(self.w2)
        self.module = MegaMoeExperts(hidden_size=shape.hidden, intermediate_size=shape.inter,
                                     num_experts=shape.num_experts(ctx.world), top_k=shape.top_k, ep_group=ctx.group,
                                     precision=precision, tuning_options=MegaMoeTuningOptions(dispatch_mode=dispatch))
        self.x = x_h.to(device).requires_grad_(True)
        self.ids = ids_h.to(device)
        self.p = p_h.to(device).requires_grad_(True)
        self.g = g_h.to(device)
        # rows every rank's experts receive (skewed routing loads the ranks unevenly: the step lasts as long as
        # the most loaded rank, so that rank's rows set the work the roofline is computed from)
        local = shape.num_experts(ctx.world) // ctx.world
        received = torch.bincount(ids_h.reshape(-1) // local, minlength=ctx.world).to(device)
        if ctx.world > 1:
            ctx.dist.all_reduce(received)
        self.received_rows = [int(v) for v in received.tolist()]

    def step(self) -> None:
        self.w1.grad = self.w2.grad = self.x.grad = self.p.grad = None
        out = self.module(self.x, self.ids, self.p, expert_weights=(self.w1, self.w2))
        out.backward(self.g)

    def results(self) -> dict:
        """One more forward + backward on the resident inputs; returns this rank's tensors."""
        self.w1.grad = self.w2.grad = self.x.grad = self.p.grad = None
        out = self.module(self.x, self.ids, self.p, expert_weights=(self.w1, self.w2))
        out.backward(self.g)
        self.module.check_status()
        return {"output": out.detach(), "grad_hidden": self.x.grad, "grad_probs": self.p.grad,
                "grad_w1": self.w1.grad, "grad_w2": self.w2.grad}

    def measure(self, steps: int, warmup: int, peaks: dict) -> dict:
        """Device-timed steps plus a profiled pass that separates the GEMM launches from the rest."""
        from hyper_multicore_b200 import _lib

        ctx, shape = self.ctx, self.shape
        # The dominant kernels carry their own CUDA events inside the timed region (recorded by the library on its
        # stream around the GEMM - and for MXFP8 the quantiser - launches only: a few microseconds per step).
        lib = _lib.load()
        kind = "mx_gemm" if self.precision == "mxfp8" else "grouped_gemm"
        watched = [kind, "mx_quant"] if self.precision == "mxfp8" else [kind]
        lib.hmc_profile_enable_kinds(sum(1 << _lib.HMC_PROFILE_KINDS.index(k) for k in watched))
        total_ms, launches = ctx.timed(self.step, steps, warmup)
        lib.hmc_profile_enable(0)
        self.module.check_status()
        per_step = dumped_steps(lib, warmup + steps)[warmup:]
        gemm_ms = ctx.max_over_ranks(statistics.fmean(s["ms"].get(kind, 0.0) for s in per_step))
        quant_ms = ctx.max_over_ranks(statistics.fmean(s["ms"].get("mx_quant", 0.0) for s in per_step))
        gemm_calls = per_step[-1]["calls"].get(kind, 0)
        ms_per_step = total_ms / steps
        rows_max = max(self.received_rows)
        flops = shape.flops_per_token // shape.top_k * rows_max  # 18*H*I per routed row, on the most loaded rank
        return {
            "ms_per_step": ms_per_step, "tokens_per_s": ctx.world * shape.tokens / (ms_per_step * 1e-3),
            "launches": launches, "gemm_ms_per_step": gemm_ms, "gemm_launches_per_step": gemm_calls,
            "quant_ms_per_step": quant_ms, "non_gemm_ms_per_step": ms_per_step - gemm_ms,
            "gemm_tflops": flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None,
            "layer_tflops": flops / (ms_per_step * 1e-3) / 1e12, "flops_per_step": flops,
            "received_rows_max_rank": rows_max, "received_rows_mean": sum(self.received_rows) / len(self.received_rows),
        }

    def close(self) -> None:
        self.module.close()  # collective for EP > 1: every rank unmaps its peers before anyone frees


_ORACLE_CACHE: dict = {}  # (shape, precision, world) -> oracle tensors of rank 0 (the inputs are seeded: computed once)


def parity_check(ctx: Context, run: MoeLayerRun) -> dict:
    """One forward + backward of the bench shape against the CPU oracle, outside any timed region. Rank 0
    checks its own output, dX and dProbs (its tokens through every rank's experts) and its weight-gradient
    shard (every rank's tokens through its experts) on the concatenated global batch."""
    from oracle import compare

    shape, world = run.shape, ctx.world
    got = run.results()
    ctx.barrier()
    verdict = {"checked": True, "shape": f"{shape.name}: {shape.tokens} tokens/rank x {world} ranks, hidden {shape.hidden}, "
                                         f"{shape.num_experts(world)} experts, top-{shape.top_k}, intermediate {shape.inter}",
               "precision": run.precision, "oracle": "oracle.moe (CPU restatement of the reference's TorchExperts golden)"}
    failed = torch.zeros(1, device=ctx.device)
    if ctx.rank == 0:
        t0 = time.perf_counter()
        torch.set_num_threads(os.cpu_count() or 1)
        everyone = [make_inputs(shape, r, world) for r in range(world)]
        w1_all = torch.cat([e[4] for e in everyone])
        w2_all = torch.cat([e[5] for e in everyone])
        x, ids, probs, grad = everyone[0][:4]
        key = (shape.name, run.precision, world)
        if run.precision == "mxfp8":
            from oracle import mxfp8 as omx

            ref = _ORACLE_CACHE.get(key) or omx.experts_forward_backward(x, ids, probs, w1_all, w2_all, grad)
            _ORACLE_CACHE[key] = ref
            names = ["output", "grad_hidden", "grad_probs"] + (["grad_w1", "grad_w2"] if world == 1 else [])
            limits = {"output": 1e-2, "grad_hidden": 3e-2, "grad_probs": 3e-2, "grad_w1": 3e-2, "grad_w2": 3e-2}
            verdict["oracle"] = "oracle.mxfp8 (OCP-MX restatement; the reference pins no MXFP8 numerics: parity unpinned)"
            verdict["rule"] = "relative L2 <= 1e-2 (output), 3e-2 (gradients)"
            report = {}
            for name in names:
                error = float((got[name].detach().float().cpu() - ref[name].float()).norm() / ref[name].float().norm().clamp_min(1e-12))
                report[name] = {"rel_l2": error, "limit": limits[name], "ok": error <= limits[name]}
        else:
            from oracle import moe as omoe

            ref = _ORACLE_CACHE.get(key)
            if ref is None:
                ref = omoe.experts_forward_backward(x, ids, probs, w1_all, w2_all, grad)
                local = w1_all.shape[0] // world
                if world > 1:
                    shard = omoe.experts_forward_backward(
                        torch.cat([e[0] for e in everyone]), torch.cat([e[1] for e in everyone]),
                        torch.cat([e[2] for e in everyone]), w1_all[:local], w2_all[:local],
                        torch.cat([e[3] for e in everyone]))
                    ref["grad_w1"], ref["grad_w2"] = shard["grad_w1"], shard["grad_w2"]
                _ORACLE_CACHE[key] = ref
            verdict["rule"] = (f"rtol {compare.RTOL}, atol {compare.ATOL} x max(1, |ref|max); at most {compare.STRAY_FRACTION:g} "
                               f"of a tensor's elements outside, none beyond {compare.STRAY_FACTOR:g} x, rel L2 < {compare.REL_L2_LIMIT:g}")
            report = {}
            for name in ("output", "grad_hidden", "grad_probs", "grad_w1", "grad_w2"):
                result = compare.report(got[name], ref[name])
                result["ok"] = compare.passes(result)
                report[name] = result
        verdict["tensors"] = report
        verdict["rel_l2"] = {name: r["rel_l2"] for name, r in report.items()}
        verdict["outside_tolerance"] = sum(r.get("outside", 0) for r in report.values())
        verdict["ok"] = all(r["ok"] for r in report.values())
        verdict["oracle_seconds"] = time.perf_counter() - t0
        failed.fill_(0.0 if verdict["ok"] else 1.0)
    if world > 1:
        ctx.dist.broadcast(failed, src=0)
    verdict["ok"] = bool(failed.item() == 0)
    return verdict


def e2e_measure(ctx: Context, run: MoeLayerRun, steps: int, warmup: int) -> dict:
    """The same call through the module API with HOST buffers. The three legs of a step (inputs host ->
    device, forward + backward, results device -> host) run on three streams, so the copies of neighbouring
    steps overlap the compute of this one; every step still copies its own inputs in and its own results
    out. `copy_floor_ms`: the same copies alone, all ranks at once, no compute."""
    shape, device = run.shape, ctx.device
    x_h, ids_h, p_h, g_h = run.host[:4]
    pinned = [t.pin_memory() for t in (x_h, ids_h, p_h, g_h)]
    h2d_bytes = sum(t.numel() * t.element_size() for t in pinned)
    slots = []
    for _ in range(2):
        slots.append({
            "in": [torch.empty_like(t, device=device) for t in pinned],
            "out": [torch.empty(shape.tokens, shape.hidden, dtype=torch.bfloat16).pin_memory(),
                    torch.empty(shape.tokens, shape.hidden, dtype=torch.bfloat16).pin_memory(),
                    torch.empty(shape.tokens, shape.top_k, dtype=torch.float32).pin_memory()],
            "loaded": torch.cuda.Event(), "computed": torch.cuda.Event(), "stored": torch.cuda.Event(), "keep": None,
        })
    d2h_bytes = sum(t.numel() * t.element_size() for t in slots[0]["out"])
    copy_in, copy_out = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    state = {"step": 0, "compute": True}

    def load(slot) -> None:
        with torch.cuda.stream(copy_in):
            copy_in.wait_event(slot["computed"])  # the previous user of this slot has finished with it
            for dst, src in zip(slot["in"], pinned):
                dst.copy_(src, non_blocking=True)
            slot["loaded"].record(copy_in)

    def step_host() -> None:
        main = torch.cuda.current_stream(device)
        index = state["step"]
        slot, other = slots[index % 2], slots[(index + 1) % 2]
        if index == 0:
            load(slot)
        main.wait_event(slot["loaded"])
        main.wait_event(slot["stored"])  # the results of the step that used this slot before are out
        # queued before this step's kernels: the next step's inputs travel while this step computes
        load(other)
        if state["compute"]:
            run.w1.grad = run.w2.grad = None
            x = slot["in"][0].detach().requires_grad_(True)
            p = slot["in"][2].detach().requires_grad_(True)
            out = run.module(x, slot["in"][1], p, expert_weights=(run.w1, run.w2))
            out.backward(slot["in"][3])
            results = (out.detach(), x.grad, p.grad)
        else:
            results = (slot["in"][0], slot["in"][3], slot["in"][2])  # same sizes as the real results
        slot["computed"].record(main)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(slot["computed"])
            for host, dev in zip(slot["out"], results):
                dev.record_stream(copy_out)
                host.copy_(dev, non_blocking=True)
            slot["stored"].record(copy_out)
        slot["keep"] = results
        state["step"] = index + 1

    e2e_ms, _ = ctx.timed(step_host, steps, max(3, warmup), join=(copy_in, copy_out))
    run.module.check_status()
    state["compute"] = False
    floor_ms, _ = ctx.timed(step_host, steps, 3, join=(copy_in, copy_out))
    per_step = e2e_ms / steps
    return {"value": ctx.world * shape.tokens / (per_step * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d_bytes,
            "d2h_bytes_per_step": d2h_bytes, "ms_per_step": per_step, "copy_floor_ms": floor_ms / steps,
            "copy_floor_note": "the same pinned host<->device copies alone, every rank at once, no compute",
            "pipeline": "copies of neighbouring steps overlap this step's compute (3 streams, 2 buffer sets)"}


def nvlink_measure(ctx: Context, run: MoeLayerRun, iterations: int = 10) -> dict:
    """Transport alone, on the bench shape's own routes (N > 1): the stand-alone push dispatch (peer stores +
    arrival counters, then a bounded wait until every expert's rows have landed) and an NCCL
    all_to_all_single of the same expert-major rows with the same split sizes."""
    from hyper_multicore_b200 import _lib, kernels
    from hyper_multicore_b200.modules.mega_moe.route import prepare_route

    shape, device, world, rank = run.shape, ctx.device, ctx.world, ctx.rank
    module = run.module
    experts = shape.num_experts(world)
    local = experts // world
    route = prepare_route(run.x.detach(), run.ids, num_experts=experts, top_k=shape.top_k, ep_size=world, rank=rank,
                          group=ctx.group, status=module._status, control=module._group.control,
                          budget_ns=module._wait_budget_ns)
    module._ensure_workspace(device, route)
    ws = module._workspace
    off = route.offsets
    table = torch.tensor(route.counts_by_source)  # [ep, experts]
    send_rows = [int(table[rank, d * local:(d + 1) * local].sum()) for d in range(world)]
    recv_rows = [int(table[s, rank * local:(rank + 1) * local].sum()) for s in range(world)]
    remote_rows = sum(send_rows) - send_rows[rank]
    row_bytes = shape.hidden * 2
    arrival = ws.ctrl[_lib.HMC_CTRL_ARRIVAL:_lib.HMC_CTRL_ARRIVAL + local]
    times = []
    for it in range(iterations + 3):
        ctx.barrier()
        generation = ws.begin_call()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        kernels.ep_dispatch(run.x.detach(), route.source_of_row, route.expert_of_row, off["dispatch_src_off"],
                            off["dispatch_target_off"], rows=route.routed_rows, top_k=shape.top_k, ep=world,
                            local_experts=local, capacity_rows=ws.capacity_rows, peer_buffers=ws.peer_expert,
                            peer_ctrl=ws.peer_ctrl, local_ctrl=ws.ctrl, generation=generation, status=module._status,
                            budget_ns=module._wait_budget_ns)
        kernels.ep_wait_groups(arrival, off["group_list"], status=module._status, budget_ns=module._wait_budget_ns)
        e1.record()
        torch.cuda.synchronize()
        if it >= 3:
            times.append(e0.elapsed_time(e1))
    push_ms = ctx.max_over_ranks(statistics.median(times))
    module.check_status()
    # NCCL baseline: the same rows, already expert-major (= destination-major) on the source
    permuted = torch.empty(max(route.routed_rows, 1), shape.hidden, dtype=torch.bfloat16, device=device)
    kernels.moe_gather_rows(run.x.detach(), route.source_of_row, shape.top_k, permuted[:route.routed_rows])
    received = torch.empty(max(sum(recv_rows), 1), shape.hidden, dtype=torch.bfloat16, device=device)
    times = []
    for it in range(iterations + 3):
        ctx.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ctx.dist.all_to_all_single(received[:sum(recv_rows)], permuted[:route.routed_rows], recv_rows, send_rows)
        e1.record()
        torch.cuda.synchronize()
        if it >= 3:
            times.append(e0.elapsed_time(e1))
    nccl_ms = ctx.max_over_ranks(statistics.median(times))
    sent = ctx.max_over_ranks(float(remote_rows * row_bytes))
    return {
        "remote_bytes_per_dispatch_max_rank": sent,
        "remote_bytes_per_step_max_rank": 4 * sent,  # dispatch X, combine Y, dispatch dY, combine dX
        "push_dispatch_ms": push_ms, "push_dispatch_gbs_per_direction": sent / (push_ms * 1e-3) / 1e9,
        "push_frac_of_900": sent / (push_ms * 1e-3) / 1e9 / 900.0,
        "nccl_all_to_all_ms": nccl_ms, "nccl_all_to_all_gbs_per_direction": sent / (nccl_ms * 1e-3) / 1e9,
        "note": ("stand-alone transfers of one dispatch (CUDA events, median of %d, max over ranks); the push time includes the "
                 "local copy of the rows a rank keeps and the arrival wait. In the layer the push dispatch rides inside the "
                 "first GEMM of each direction, so most of this time is hidden there" % iterations),
    }


def nccl_layer_measure(ctx: Context, run: MoeLayerRun, steps: int, warmup: int) -> dict:
    """The reference's example baseline for the same layer (examples/_native.py:139-152, 298-397,
    AllToAllTokenDispatcher): rows exchanged with NCCL all_to_all_single and re-ordered on the owner, the same
    grouped GEMMs in between. Forward + backward, explicit (no autograd), timed like the product path."""
    from hyper_multicore_b200 import kernels

    shape, device, world, rank = run.shape, ctx.device, ctx.world, ctx.rank
    experts = shape.num_experts(world)
    local, hid, inter, top_k, tokens = experts // world, shape.hidden, shape.inter, shape.top_k, shape.tokens
    dist = ctx.dist
    bf16 = dict(dtype=torch.bfloat16, device=device)
    w1, w2 = run.w1.detach(), run.w2.detach()
    x, g, probs, ids = run.x.detach(), run.g, run.p.detach(), run.ids

    def exchange(rows_in, send, recv):
        out = torch.empty(max(sum(recv), 1), rows_in.shape[1], **bf16)
        dist.all_to_all_single(out[:sum(recv)], rows_in[:sum(send)], recv, send)
        return out

    def step():
        mapping, sources, _, counts, _ = kernels.moe_sort_routes(ids, experts)
        gathered = torch.empty(world * experts, dtype=torch.int32, device=device)
        dist.all_gather_into_tensor(gathered, counts)
        table = gathered.view(world, experts).cpu()  # the one host synchronisation of the call
        send = [int(table[rank, d * local:(d + 1) * local].sum()) for d in range(world)]
        recv = [int(table[s, rank * local:(rank + 1) * local].sum()) for s in range(world)]
        mine = table[:, rank * local:(rank + 1) * local]  # [source, local expert]
        # received rows are source-major; the GEMMs want them local-expert-major
        start_of = torch.zeros(world, local, dtype=torch.int64)
        flat = mine.reshape(-1).to(torch.int64)
        start_of.view(-1)[1:] = flat.cumsum(0)[:-1]
        order = torch.cat([torch.arange(int(start_of[s, e]), int(start_of[s, e]) + int(mine[s, e]))
                           for e in range(local) for s in range(world)] or [torch.zeros(0, dtype=torch.int64)]).to(device)
        inverse = torch.empty_like(order)
        inverse[order] = torch.arange(order.numel(), device=device)
        group_list = mine.sum(0).to(torch.int64).cumsum(0).to(device)
        rows = max(int(order.numel()), 1)
        routed = tokens * top_k
        permuted = torch.empty(max(routed, 1), hid, **bf16)
        kernels.moe_gather_rows(x, sources, top_k, permuted[:routed])
        x_e = exchange(permuted, send, recv).index_select(0, order) if order.numel() else torch.empty(1, hid, **bf16)
        up, act, down = torch.empty(rows, 2 * inter, **bf16), torch.empty(rows, inter, **bf16), torch.empty(rows, hid, **bf16)
        kernels.grouped_gemm(x_e, w1, up, group_list, mode=kernels.HMC_GEMM_RAGGED_M, epilogue=kernels.HMC_EPI_SWIGLU, aux=act)
        kernels.grouped_gemm(act, w2, down, group_list, mode=kernels.HMC_GEMM_RAGGED_M)
        routed_out = exchange(down.index_select(0, inverse) if order.numel() else down, recv, send)
        out = torch.empty(tokens, hid, **bf16)
        kernels.moe_unpermute(routed_out, mapping, probs, tokens, top_k, out)
        # backward
        grad_routed = torch.empty(max(routed, 1), hid, **bf16)
        grad_probs = torch.empty(tokens, top_k, dtype=torch.float32, device=device)
        kernels.moe_unpermute_grad(routed_out, g, mapping, probs, top_k, grad_routed, grad_probs)
        dy = exchange(grad_routed, send, recv).index_select(0, order) if order.numel() else torch.empty(1, hid, **bf16)
        grad_up, grad_x = torch.empty(rows, 2 * inter, **bf16), torch.empty(rows, hid, **bf16)
        kernels.grouped_gemm(dy, w2, grad_up, group_list, mode=kernels.HMC_GEMM_RAGGED_M, b_major=kernels.HMC_MAJOR_K,
                             epilogue=kernels.HMC_EPI_SWIGLU_GRAD, aux=up)
        kernels.grouped_gemm(grad_up, w1, grad_x, group_list, mode=kernels.HMC_GEMM_RAGGED_M, b_major=kernels.HMC_MAJOR_K)
        grad_w2, grad_w1 = torch.empty_like(w2), torch.empty_like(w1)
        kernels.grouped_gemm(act, dy, grad_w2, group_list, mode=kernels.HMC_GEMM_RAGGED_K)
        kernels.grouped_gemm(x_e, grad_up, grad_w1, group_list, mode=kernels.HMC_GEMM_RAGGED_K)
        returned = exchange(grad_x.index_select(0, inverse) if order.numel() else grad_x, recv, send)
        grad_hidden = torch.empty(tokens, hid, **bf16)
        kernels.moe_token_permute_grad(returned, mapping, tokens, top_k, grad_hidden)
        return out, grad_hidden

    total_ms, _ = ctx.timed(step, steps, warmup)
    return {"ms_per_step": total_ms / steps, "tokens_per_s": world * tokens / (total_ms / steps * 1e-3),
            "what": "NCCL all_to_all_single dispatch/combine + owner-side re-order (torch index_select) around the same "
                    "grouped GEMMs; the baseline of the reference's examples (AllToAllTokenDispatcher)"}


def profiled_steps(ctx: Context, step, steps: int, before=None, after=None) -> list:
    """Device time per kind of native entry point for each of `steps` steps (CUDA events around every entry point,
    recorded by the library on its stream). Two more steps are queued first and dropped from the result, with no
    idle gap after them: the host is then ahead of the device for the steps that count (a start event that runs
    on an idle device would add the host's launch latency to the call). `before` / `after` are called right around
    the counted steps. Returns one {"ms": {kind: ms}, "calls": {kind: n}, "records": [(kind, start_ms, ms), ...]}
    per step."""
    from hyper_multicore_b200 import _lib

    lead = 2
    lib = _lib.load()
    ctx.barrier()
    lib.hmc_profile_enable(1)
    for _ in range(lead):
        step()
    if before is not None:
        before()
    for _ in range(steps):
        step()
    if after is not None:
        after()
    ctx.barrier()
    lib.hmc_profile_enable(0)
    return dumped_steps(lib, lead + steps)[lead:]


def dumped_steps(lib, steps: int) -> list:
    """The library's recorded calls, split evenly into `steps` consecutive steps."""
    import ctypes

    from hyper_multicore_b200 import _lib

    capacity = 1 << 14
    kinds, begins, lengths = (ctypes.c_int32 * capacity)(), (ctypes.c_double * capacity)(), (ctypes.c_double * capacity)()
    count = lib.hmc_profile_dump(kinds, begins, lengths, capacity)
    per_step = count // steps
    out = []
    for s in range(steps):
        records = [(_lib.HMC_PROFILE_KINDS[kinds[i]], begins[i], lengths[i]) for i in range(s * per_step, (s + 1) * per_step)]
        ms, calls = {}, {}
        for name, _, length in records:
            ms[name] = ms.get(name, 0.0) + length
            calls[name] = calls.get(name, 0) + 1
        out.append({"ms": ms, "calls": calls, "records": records})
    return out


def write_timeline(ctx: Context, run: MoeLayerRun, path: str) -> None:
    """Call-by-call device timeline of one forward + backward step (CUDA events around every entry point of
    the native library, on its stream): kind, start, duration and the gap to the previous call. Rank 0 writes it."""
    steps = 3
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    per_step = profiled_steps(ctx, run.step, steps, before=start.record, after=stop.record)
    if ctx.rank != 0:
        return
    records = per_step[-1]["records"]
    lines = [f"# one step of {steps} (the last), rank 0 of {ctx.world}; {config(run.shape, ctx.world, run.precision)['workload']}",
             f"# step time over the {steps} profiled steps: {start.elapsed_time(stop) / steps * 1e3:.1f} us",
             "#   start us    gap us  call kind        duration us"]
    origin = previous_end = records[0][1]
    for name, begin, length in records:
        lines.append(f"{1e3 * (begin - origin):12.1f} {1e3 * (begin - previous_end):9.1f}  {name:14s} {1e3 * length:12.1f}")
        previous_end = begin + length
    lines.append("# per kind (us): " + ", ".join(f"{k} {1e3 * v:.1f}" for k, v in per_step[-1]["ms"].items()))
    Path(path).write_text("\n".join(lines) + "\n")


def side_workload(ctx: Context, workload: str, steps: int, warmup: int, peaks: dict) -> dict:
    import bench_side

    result = bench_side.measure(workload, ctx.rank, ctx.world, ctx.device, steps, warmup, barrier=ctx.barrier,
                                with_e2e=False)
    gbs = result["algorithmic_bytes"] / (result["ms_per_step"] * 1e-3) / 1e9
    return {"workload": bench_side.workload_config(workload)["workload"], "ms_per_step": result["ms_per_step"],
            "tokens_per_s": result["tokens"] / (result["ms_per_step"] * 1e-3),
            "algorithmic_bytes_per_step": result["algorithmic_bytes"], "gbs": gbs, "frac_of_hbm": gbs / peaks["hbm_gbs"],
            "hbm_peak_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"] + " (copy bandwidth)",
            "stage_ms": result["stage_ms"], "launch_mode": result["launch_mode"],
            "eager_ms_per_step": result["eager_ms_per_step"]}


def run_gpu(args) -> None:
    from hyper_multicore_b200 import _lib

    _lib.load()  # fail loudly here if the native library is missing: there is no fallback path
    ctx = Context(args)
    peaks = load_peaks()
    shape = SHAPES[args.shape]
    precision = args.precision
    run = MoeLayerRun(ctx, shape, precision, args.dispatch, weights_on_device=args.shape != "c2")

    sampler = ClockSampler(ctx.local_rank)
    if ctx.rank == 0:
        sampler.start()
    main = run.measure(args.steps, args.warmup, peaks)
    clocks = sampler.stop() if ctx.rank == 0 else None
    if args.timeline:
        write_timeline(ctx, run, args.timeline)
    e2e = e2e_measure(ctx, run, args.steps, args.warmup)
    parity = {"checked": False, "why": "--no-parity"} if args.no_parity or args.shape != "c2" else parity_check(ctx, run)

    extra: dict = {}

    def attempt(name: str, fn) -> None:
        try:
            extra[name] = fn()
        except Exception as error:  # pylint: disable=broad-except
            extra[name] = {"error": f"{type(error).__name__}: {error}"}
            if ctx.world > 1:
                raise  # a rank that skips a collective leg would leave the others waiting

    if not args.no_extra and args.shape == "c2" and precision == "bf16":
        if ctx.world > 1:
            attempt("nvlink", lambda: nvlink_measure(ctx, run))
            attempt("nccl_all_to_all_layer", lambda: nccl_layer_measure(ctx, run, min(args.steps, 10), 3))
        run.close()
        if ctx.world > 1:
            def other_transport(dispatch: str, grow_first: bool):
                """The same layer through another module instance: pull dispatch, or a workspace that must
                grow (a first call with a quarter of the tokens sizes it too small for the full batch: the route
                guard turns the full call into a no-op, all ranks regrow together and run it again)."""
                leg = MoeLayerRun(ctx, shape, "bf16", dispatch, weights_on_device=False)
                out = {"dispatch": dispatch}
                if grow_first:
                    quarter = shape.tokens // 4
                    leg.module(leg.x.detach()[:quarter], leg.ids[:quarter], leg.p.detach()[:quarter],
                               expert_weights=(leg.w1.detach(), leg.w2.detach()))
                    before = leg.module._workspace.capacity_rows
                    leg.step()
                    out["capacity_rows_before"], out["capacity_rows_after"] = before, leg.module._workspace.capacity_rows
                    out["grew"] = out["capacity_rows_after"] > before
                else:
                    result = leg.measure(min(args.steps, 10), 3, peaks)
                    out["ms_per_step"], out["tokens_per_s"] = result["ms_per_step"], result["tokens_per_s"]
                if not args.no_parity:
                    out["parity"] = parity_check(ctx, leg)
                leg.close()
                return out

            attempt("pull_dispatch", lambda: other_transport("pull", grow_first=False))
            attempt("capacity_growth", lambda: other_transport("push", grow_first=True))
        fp8_peak = 2 * peaks["bf16_burst"]

        def mx_leg(name: str, with_parity: bool):
            leg_shape = SHAPES[name]
            leg = MoeLayerRun(ctx, leg_shape, "mxfp8", args.dispatch, weights_on_device=name != "c2")
            result = leg.measure(min(args.steps, 10), max(3, min(args.warmup, 5)), peaks)
            out = {
                "workload": config(leg_shape, ctx.world, "mxfp8")["workload"], "ms_per_step": result["ms_per_step"],
                "tokens_per_s": result["tokens_per_s"], "gemm_ms_per_step": result["gemm_ms_per_step"],
                "quant_ms_per_step": result["quant_ms_per_step"], "gemm_tflops": result["gemm_tflops"],
                "received_rows_max_rank": result["received_rows_max_rank"],
                "received_rows_mean": result["received_rows_mean"],
                "flops_note": "18*H*I flop per routed row x the rows of the most loaded rank (the step lasts as long as that rank)",
                "frac_fp8": result["gemm_tflops"] / fp8_peak if result["gemm_tflops"] else None,
                "layer_frac_fp8": result["layer_tflops"] / fp8_peak,
                "fp8_peak_tflops": fp8_peak,
                "fp8_peak_source": f"2 x the measured cuBLAS BF16 burst rate ({peaks['bf16_burst']} TFLOP/s, {peaks['source']}); "
                                   "no FP8 peak was measured on this pool",
            }
            if with_parity:
                out["parity"] = parity_check(ctx, leg)
            leg.close()
            del leg
            torch.cuda.empty_cache()
            return out

        attempt("mxfp8_c2", lambda: mx_leg("c2", with_parity=not args.no_parity))
        attempt("mxfp8_c3", lambda: mx_leg("c3", with_parity=False))
        if ctx.world == 1:
            attempt("gate_c4", lambda: side_workload(ctx, "gate", args.steps, max(3, args.warmup), peaks))
            attempt("mhc_c5", lambda: side_workload(ctx, "mhc", min(args.steps, 10), 3, peaks))
    else:
        run.close()

    def all_parity_ok() -> bool:
        checks = [parity] + [leg["parity"] for leg in extra.values() if isinstance(leg, dict) and "parity" in leg]
        return all(c["ok"] for c in checks if c.get("checked"))

    if ctx.rank != 0:
        ctx.close()
        if not all_parity_ok():
            sys.exit(1)
        return

    mx = precision == "mxfp8"
    # BF16: the timed region is tens of milliseconds at full clock, so the burst figure is the like-for-like
    # denominator; the sustained one (a seconds-long loop under the power cap) is quoted beside it.
    sustained = (2 if mx else 1) * peaks["bf16_sustained"]
    burst = (2 if mx else 1) * peaks["bf16_burst"]
    gemm_tflops = main["gemm_tflops"]
    tokens, hidden, inter, top_k = shape.tokens, shape.hidden, shape.inter, shape.top_k
    local = shape.num_experts(ctx.world) // ctx.world
    # algorithmic DRAM bytes of the six GEMM launches of one step: every operand read once, every result written once
    rows = tokens * top_k
    gemm_bytes = 2 * (3 * local * hidden * 2 * inter + 3 * local * inter * hidden       # weights read 3x, dW written
                      + rows * (hidden + 2 * inter + inter + inter + hidden)             # forward: X, U, A in/out, Y
                      + rows * (hidden + 2 * inter + 2 * inter + 2 * inter + hidden)     # dY, U, dU out, dU in, dX
                      + rows * (inter + hidden + hidden + 2 * inter))                    # dW operands: A, dY, X, dU
    line = {
        "metric": METRIC, "value": main["tokens_per_s"], "unit": UNIT, "n_gpus": ctx.world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16" if not mx else "mxfp8 (e4m3 + ue8m0/32) operands, bf16 activations",
        "data": "synthetic", "config": config(shape, ctx.world, precision),
        "clocks": clocks, "e2e": e2e, "gpu_launches": main["launches"], "parity": parity,
        "roofline": {
            "bound": "tensor",
            "kernel": ("mx_gemm_pair_kernel (tcgen05 block-scaled FP8 on CTA pairs" if mx else "grouped_gemm_kernel (tcgen05") +
                      f", {main['gemm_launches_per_step']} launches per step)",
            "achieved": gemm_tflops, "peak": burst, "unit": "TFLOP/s", "frac": gemm_tflops / burst,
            "peak_source": (("2 x " if mx else "") + f"cuBLAS bf16 burst rate {peaks['source']}: the timed region is tens of "
                            "milliseconds at full clock, the condition the burst figure was measured under"),
            "frac_burst": gemm_tflops / burst, "frac_sustained": gemm_tflops / sustained,
            "peak_burst": burst, "peak_sustained": sustained,
            "traffic": gemm_bytes / max(main["gemm_launches_per_step"], 1),
            "traffic_note": "algorithmic DRAM bytes per launch (operands read once, results written once)",
            "gemm_ms_per_step": main["gemm_ms_per_step"], "launches_per_step": main["gemm_launches_per_step"],
            "non_gemm_ms_per_step": main["non_gemm_ms_per_step"],
            "algorithmic_flops_per_step": main["flops_per_step"],
            "received_rows_max_rank": main["received_rows_max_rank"], "received_rows_mean": main["received_rows_mean"],
            "layer_frac": main["layer_tflops"] / burst, "layer_frac_sustained": main["layer_tflops"] / sustained,
        },
        "extra": extra,
    }
    if ctx.world == 1 and not args.no_cpu_baseline and args.shape == "c2":
        line["cpu_baseline"] = cpu_full_problem(shape, iterations=3, warm=not parity.get("checked", False))
    print(json.dumps(line), flush=True)
    ctx.close()
    if not all_parity_ok():
        sys.exit(1)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("b200", "reference"), default="b200")
    parser.add_argument("--no-cpu-baseline", action="store_true",
                        help="skip the CPU baseline leg (used when the run is captured by a profiler)")
    parser.add_argument("--no-parity", action="store_true", help="skip the oracle check of the bench shape")
    parser.add_argument("--no-extra", action="store_true", help="skip the MXFP8 / gate / mHC / NVLink legs")
    parser.add_argument("--shape", choices=tuple(SHAPES), default="c2",
                        help="c2 = EP=2 BF16 configuration's per-rank problem (default); c3 = EP=8 MXFP8 configuration's")
    parser.add_argument("--precision", choices=("bf16", "mxfp8"), default="bf16")
    parser.add_argument("--dispatch", choices=("push", "pull"), default="push",
                        help="EP > 1: sources store rows into the owners' buffers (push, default) or owners fetch them (pull)")
    parser.add_argument("--workload", choices=("moe", "gate", "mhc"), default="moe",
                        help="moe = the MoE layer (default, the headline metric); gate / mhc = the router and the "
                             "four-stream residual mix, timed against the HBM roofline")
    parser.add_argument("--timeline", default=None, metavar="FILE",
                        help="also write a call-by-call device timeline of one step (CUDA events) to FILE")
    parser.add_argument("--tokens", type=int, default=None,
                        help="gate / mhc workloads only: run a smaller case of the same kernels (profiler captures)")
    args = parser.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.workload != "moe":
        import bench_side

        if args.impl == "reference":
            bench_side.run_reference(args, args.workload)
        else:
            bench_side.run_gpu(args, args.workload, ClockSampler)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
