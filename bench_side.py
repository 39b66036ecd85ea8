"""Gate and mHC workloads of `bench.py` (`--workload gate` / `--workload mhc`).

Both paths are token-parallel (no exchange step): with N > 1 ranks every rank runs an independent
replica on its own tokens and `value` is the sum over ranks.

gate: the multimodal router problem — 6144 text + 2048 vision tokens, hidden 4096, 64 experts,
      softmax top-6, two correction biases selected by the image mask — followed by the route
      preparation that consumes its indices (per-expert counts and the expert-major permutation).
mhc : MegaMhc forward + backward on 16384 tokens x 4 streams x hidden 7168.
"""

from __future__ import annotations

import json
import os
import statistics
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent

GATE = dict(text=6144, vision=2048, hidden=4096, experts=64, top_k=6, scoring="softmax", scale=1.0)
MHC = dict(tokens=16384, hidden=7168)


# ------------------------------------------------------------------------------------------ inputs
def gate_inputs(rank: int):
    g = torch.Generator().manual_seed(1234 + rank)
    tokens = GATE["text"] + GATE["vision"]
    x = torch.randn(tokens, GATE["hidden"], generator=g)
    channel_scale = torch.rand(GATE["hidden"], generator=g) * 1.5 + 0.5
    x[GATE["text"]:] *= channel_scale
    weight = torch.randn(GATE["experts"], GATE["hidden"], generator=g) * 0.02
    bias = torch.rand(GATE["experts"], generator=g) * 0.2 - 0.1
    bias_vl = torch.rand(GATE["experts"], generator=g) * 0.2 - 0.1
    mask = torch.zeros(1, tokens, dtype=torch.bool)
    mask[:, GATE["text"]:] = True
    return x.bfloat16().unsqueeze(0), weight, bias, bias_vl, mask


def mhc_inputs(rank: int, tokens: int, hidden: int, device=None):
    g = torch.Generator(device=device).manual_seed(1234 + rank) if device is not None else torch.Generator().manual_seed(1234 + rank)
    kw = dict(generator=g, device=device)
    previous_output = torch.randn(tokens, hidden, **kw).bfloat16()
    residual = torch.randn(tokens, 4, hidden, **kw).bfloat16()
    pre = torch.sigmoid(torch.randn(tokens, 4, **kw))
    post = 2 * torch.sigmoid(torch.randn(tokens, 4, **kw))
    mix = torch.softmax(torch.randn(tokens, 4, 4, **kw), dim=-1)
    phi = torch.randn(24, 4 * hidden, **kw) * 0.02
    alpha = torch.ones(3, device=device)
    bias = torch.zeros(24, device=device)
    bias[8:] = (4.0 * torch.eye(4, device=device)).flatten()
    norm_weight = (1 + 0.02 * torch.randn(hidden, **kw)).bfloat16()
    grads = (torch.randn(tokens, 4, hidden, **kw).bfloat16() * 0.1, torch.randn(tokens, 4, **kw) * 0.1,
             torch.randn(tokens, 4, **kw) * 0.1, torch.randn(tokens, 4, 4, **kw) * 0.1,
             torch.randn(tokens, hidden, **kw).bfloat16() * 0.1)
    return (previous_output, residual, pre, post, mix, phi, alpha, bias, norm_weight), grads


# -------------------------------------------------------------------------------------- CPU timing
def gate_cpu(sample: int, iterations: int) -> float:
    """Seconds per pass of the oracle's gate + route preparation on `sample` tokens."""
    from oracle import gate as ogate, route as oroute

    x, weight, bias, bias_vl, mask = gate_inputs(0)
    x, mask = x[0, -sample:], mask[0, -sample:]

    def once() -> None:
        ids = ogate.gate_forward(x, weight, bias, bias_vl, mask, GATE["top_k"], GATE["scoring"], GATE["scale"])["indices"]
        oroute.counts(ids.numpy(), GATE["experts"])
        oroute.permutation(ids.numpy(), GATE["experts"])

    once()
    times = []
    for _ in range(iterations):
        t0 = time.perf_counter()
        once()
        times.append(time.perf_counter() - t0)
    return statistics.median(times)


def mhc_cpu(sample: int, iterations: int) -> float:
    from oracle import mhc as omhc

    inputs, grads = mhc_inputs(0, sample, MHC["hidden"])

    def once() -> None:
        omhc.mega_mhc_grad(grads, inputs)  # runs the forward under autograd, then the backward

    once()
    times = []
    for _ in range(iterations):
        t0 = time.perf_counter()
        once()
        times.append(time.perf_counter() - t0)
    return statistics.median(times)


def cpu_leg(workload: str, budget_s: float) -> dict:
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    if workload == "gate":
        sample, fn, total = 2048, gate_cpu, GATE["text"] + GATE["vision"]
        what = "gate forward + counts + permutation"
    else:
        sample, fn, total = 256, mhc_cpu, MHC["tokens"]
        what = "mHC forward + backward (autograd of the forward restatement)"
    probe = fn(sample, 1)
    iterations = max(1, min(5, int(budget_s / max(probe, 1e-3))))
    seconds = fn(sample, iterations)
    return {"value": sample / seconds, "unit": "tokens/s", "cores": threads, "kind": "port", "sample_tokens": sample,
            "sample": f"{sample} of the {total} tokens, {what}, median of {iterations} ({seconds:.3f} s each), "
                      f"torch CPU threads={threads}"}


def run_reference(args, workload: str) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    leg = cpu_leg(workload, budget_s=120.0)
    line = {"impl": "reference", "metric": f"{workload}_tokens_per_s", "value": leg["value"], "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": leg["sample_tokens"] / leg["value"] * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(workload), "cpu_baseline": leg,
            "e2e": {"value": leg["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(workload: str) -> dict:
    if workload == "gate":
        return {"workload": (f"MegaGate forward + route preparation: {GATE['text']} text + {GATE['vision']} vision tokens, "
                             f"hidden {GATE['hidden']}, {GATE['experts']} experts, softmax top-{GATE['top_k']}, "
                             "two correction biases by image mask; then counts and expert-major permutation"),
                "l2": "256 MiB buffer rewritten between timed steps", **GATE}
    return {"workload": f"MegaMhc forward + backward, {MHC['tokens']} tokens x 4 streams x hidden {MHC['hidden']}",
            "l2": "no flush: each step streams >7 GB through the 126 MB L2", **MHC}


# ---------------------------------------------------------------------------------------- GPU arms
def _peak_hbm():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "of measured (copy bandwidth)"
    return 6650.0, "of fallback"


def measure(workload: str, rank: int, world: int, device, steps: int, warmup: int, *, barrier, tokens=None,
            with_e2e: bool = True, max_over_ranks=None) -> dict:
    """Time one side workload on this rank's device: device-resident steps, optionally the host-buffer
    steps, and a per-stage breakdown (CUDA events on the launch stream). Returns plain numbers."""
    from hyper_multicore_b200 import MegaGate, MegaMhc, _lib, kernels

    if tokens:
        # a smaller case of the same kernels (used for profiler captures)
        if workload == "gate":
            GATE["text"], GATE["vision"] = tokens * 3 // 4, tokens - tokens * 3 // 4
        else:
            MHC["tokens"] = tokens
    reduce_max = max_over_ranks or (lambda value: value)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device) if workload == "gate" else None
    stages: dict[str, list] = {}

    def stage(name: str, fn):
        """Run fn between two events on the launch stream (only while `stages` collection is on)."""
        if not collecting[0]:
            return fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        stages.setdefault(name, []).append((e0, e1))
        return out

    collecting = [False]

    if workload == "gate":
        x_h, weight, bias, bias_vl, mask_h = gate_inputs(rank)
        tokens = x_h.shape[1]
        gate = MegaGate(hidden_size=GATE["hidden"], num_experts=GATE["experts"], top_k=GATE["top_k"],
                        scoring_func=GATE["scoring"], routed_scaling_factor=GATE["scale"], vision_enabled=True).to(device)
        with torch.no_grad():
            gate.weight.copy_(weight)
            gate.bias.copy_(bias)
            gate.bias_vl.copy_(bias_vl)
        x_d, mask_d = x_h.to(device), mask_h.to(device)
        pinned = [x_h.pin_memory(), mask_h.pin_memory()]
        outs_h = [torch.empty(tokens, GATE["top_k"], dtype=torch.float32).pin_memory(),
                  torch.empty(tokens, GATE["top_k"], dtype=torch.int64).pin_memory(),
                  torch.empty(GATE["experts"], dtype=torch.int32).pin_memory(),
                  torch.empty(tokens * GATE["top_k"], dtype=torch.int32).pin_memory()]

        def run(x, mask):
            with torch.no_grad():
                _, weights, ids = stage("gate (projection + route)", lambda: gate(x, mask))
                mapping, _, _, counts, _ = stage("route preparation (counts + permutation)",
                                                 lambda: kernels.moe_sort_routes(ids, GATE["experts"]))
            return weights, ids, counts, mapping

        def step_eager():
            run(x_d, mask_d)

        def capture_step():
            """The step's launches as one CUDA graph, replayed per step: the eager step is bound by the host's launch
            path (two launches of about 25 and 10 us). None when capture is refused or replays differ from eager."""
            try:
                eager = run(x_d, mask_d)  # also caches the weight parts and the kernels' launch attributes
                torch.cuda.synchronize(device)
                graph = torch.cuda.CUDAGraph()
                before = _lib.launch_count()
                with torch.cuda.graph(graph):
                    captured = run(x_d, mask_d)
                per_replay = _lib.launch_count() - before
                for t in captured:
                    t.zero_()
                graph.replay()
                torch.cuda.synchronize(device)
                if per_replay <= 0 or not all(torch.equal(a, b) for a, b in zip(eager, captured)):
                    return None
                return graph, captured, per_replay
            except Exception as exc:  # pylint: disable=broad-except
                print(f"[bench] gate: CUDA graph capture refused ({exc}); timing the eager step", file=sys.stderr, flush=True)
                try:
                    torch.cuda.synchronize(device)
                except Exception:  # pylint: disable=broad-except
                    pass
                return None

        # one rank only: with a process group alive its watchdog thread may touch the device during a capture
        captured_step = capture_step() if world == 1 and os.environ.get("HMC_BENCH_GATE_GRAPH", "1") == "1" else None
        if captured_step is not None:
            graph_launches = captured_step[2]

            def step_resident():
                captured_step[0].replay()
        else:
            step_resident = step_eager

        def step_host():
            results = run(pinned[0].to(device, non_blocking=True), pinned[1].to(device, non_blocking=True))
            for host, dev in zip(outs_h, results):
                host.copy_(dev, non_blocking=True)

        h2d = sum(t.numel() * t.element_size() for t in pinned)
        d2h = sum(t.numel() * t.element_size() for t in outs_h)
        t, h, e, k = tokens, GATE["hidden"], GATE["experts"], GATE["top_k"]
        algorithmic_bytes = t * h * 2 + e * h * 4 + t * e * 4 + t * k * 4 + t * k * 8 + e * 4 + t * k * 4
        kernel_note = "gate_project_promoted_kernel<route> (tcgen05 projection, Route in its epilogue) + sort_routes_fused_kernel"
        dtype = "f32 (bf16 activations, int32/int64 indices)"
    else:
        tokens, hidden = MHC["tokens"], MHC["hidden"]
        inputs, grads = mhc_inputs(rank, tokens, hidden, device=device)
        module = MegaMhc(hidden, device=device)
        with torch.no_grad():
            module.phi.copy_(inputs[5])
            module.alpha.copy_(inputs[6])
            module.bias.copy_(inputs[7])
            module.norm_weight.copy_(inputs[8])
        acts_d = [t.detach().requires_grad_(True) for t in inputs[:5]]
        if with_e2e:
            acts_h = [t.detach().cpu().pin_memory() for t in inputs[:5]]
            grads_h = [g.cpu().pin_memory() for g in grads]
            outs_h = [torch.empty_like(t) for t in acts_h] + [torch.empty(tokens, hidden, dtype=torch.bfloat16).pin_memory(),
                                                              torch.empty(tokens, 4, hidden, dtype=torch.bfloat16).pin_memory()]
        else:
            acts_h, grads_h, outs_h = [], [], []

        def run(acts, upstream):
            for p in module.parameters():
                p.grad = None
            for a in acts:
                a.grad = None
            outputs = stage("forward", lambda: module(*acts))
            stage("backward", lambda: torch.autograd.backward(outputs, upstream))
            return outputs

        def step_resident():
            run(acts_d, grads)

        step_eager = step_resident

        def step_host():
            acts = [t.to(device, non_blocking=True).requires_grad_(True) for t in acts_h]
            upstream = [g.to(device, non_blocking=True) for g in grads_h]
            outputs = run(acts, upstream)
            for host, a in zip(outs_h[:5], acts):
                host.copy_(a.grad, non_blocking=True)
            outs_h[5].copy_(outputs[4].detach(), non_blocking=True)
            outs_h[6].copy_(outputs[0].detach(), non_blocking=True)

        h2d = sum(t.numel() * t.element_size() for t in acts_h + grads_h)
        d2h = sum(t.numel() * t.element_size() for t in outs_h)
        th = tokens * hidden * 2
        # forward: read residual (4TH) + previous_output; write new_residual (4TH), block_input, mixed_input cache.
        # backward: read grad_new_residual, new_residual, residual (3 x 4TH), grad_block_input, mixed_input,
        # previous_output; write grad_residual (4TH), grad_previous_output.
        algorithmic_bytes = (4 + 1 + 4 + 1 + 1) * th + (12 + 3 + 4 + 1) * th
        kernel_note = "mhc_post_kernel, mhc_mapping_kernel, mhc_mapping_grad_kernel, mhc_stream_grad_kernel + 3 tcgen05 contractions"
        dtype = "f32 math on bf16 activations"

    def timed(step, count, warm):
        for _ in range(warm):
            step()
        barrier()
        if flush is not None:
            # per-step events so that the L2 flush between steps stays outside the measured time
            pairs = []
            launches_before = _lib.launch_count()
            for _ in range(count):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                step()
                e1.record()
                pairs.append((e0, e1))
            barrier()
            total = sum(a.elapsed_time(b) for a, b in pairs)
        else:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            launches_before = _lib.launch_count()
            start.record()
            for _ in range(count):
                step()
            stop.record()
            barrier()
            total = start.elapsed_time(stop)
        return reduce_max(total), _lib.launch_count() - launches_before

    total_ms, launches = timed(step_resident, steps, warmup)
    eager_ms = None
    if step_resident is not step_eager:
        launches = graph_launches * steps  # a replay launches what the capture recorded
        eager_ms = timed(step_eager, steps, warmup)[0]
    e2e_ms = timed(step_host, steps, 3)[0] if with_e2e else None

    collecting[0] = True
    profile_steps = min(steps, 5)
    for _ in range(profile_steps):
        if flush is not None:
            flush.zero_()
        step_eager()
    barrier()
    collecting[0] = False
    stage_ms = {name: sum(a.elapsed_time(b) for a, b in pairs) / profile_steps for name, pairs in stages.items()}
    return {"tokens": tokens, "ms_per_step": total_ms / steps, "launches": launches,
            "e2e_ms_per_step": e2e_ms / steps if e2e_ms is not None else None, "h2d": h2d, "d2h": d2h,
            "algorithmic_bytes": algorithmic_bytes, "kernel_note": kernel_note, "dtype": dtype, "stage_ms": stage_ms,
            "launch_mode": "eager" if eager_ms is None else "CUDA graph of the step's launches, replayed per step",
            "eager_ms_per_step": None if eager_ms is None else eager_ms / steps}


def run_gpu(args, workload: str, clock_sampler_cls) -> None:
    import torch.distributed as dist

    from hyper_multicore_b200 import _lib

    _lib.load()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus}; got {world}")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(value: float) -> float:
        if world == 1:
            return value
        ms = torch.tensor([value], device=device)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    sampler = clock_sampler_cls(local_rank)
    if rank == 0:
        sampler.start()
    result = measure(workload, rank, world, device, args.steps, args.warmup, barrier=barrier,
                     tokens=getattr(args, "tokens", None), max_over_ranks=max_over_ranks)
    clocks = sampler.stop() if rank == 0 else None
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peak, note = _peak_hbm()
    tokens, ms_per_step = result["tokens"], result["ms_per_step"]
    achieved = result["algorithmic_bytes"] / (ms_per_step * 1e-3) / 1e9
    line = {
        "metric": f"{workload}_tokens_per_s", "value": world * tokens / (ms_per_step * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak (independent replicas)", "vs_baseline": None, "dtype": result["dtype"],
        "data": "synthetic", "config": workload_config(workload), "clocks": clocks,
        "e2e": {"value": world * tokens / (result["e2e_ms_per_step"] * 1e-3), "unit": "tokens/s",
                "h2d_bytes_per_step": result["h2d"], "d2h_bytes_per_step": result["d2h"],
                "ms_per_step": result["e2e_ms_per_step"]},
        "gpu_launches": result["launches"], "launch_mode": result["launch_mode"],
        "eager_ms_per_step": result["eager_ms_per_step"],
        "roofline": {"bound": "hbm", "kernel": result["kernel_note"], "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_source": note,
                     "traffic": result["algorithmic_bytes"],
                     "traffic_note": "algorithmic bytes per step",
                     "algorithmic_bytes_per_step": result["algorithmic_bytes"], "stage_ms": result["stage_ms"]},
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_leg(workload, budget_s=20.0)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
