"""Benchmark of the MegaMoE layer hot path on B200: tokens/s of forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N = 1 runs the per-rank problem of the expert-parallel BF16 configuration on one GPU (EP = 1):
4096 tokens, hidden 4096, 32 experts, softmax top-4, SwiGLU experts with intermediate 1536.
Under torchrun (N > 1) every rank brings its own 4096 tokens and owns 32 / N experts (EP = N,
weak scaling); rows travel through the peer-mapped buffers, NCCL carries only the count table.

One JSON line is printed by rank 0. `value` times the layer with inputs resident in HBM; `e2e`
times the same call through the module API with host buffers (pinned host -> device copies of the
step's inputs and device -> host copies of its results inside the timed region).
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
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Default: the per-rank problem of the EP=2 BF16 configuration. "c3" is the per-rank problem of the
# EP=8 MXFP8 configuration (32 experts per rank, Zipf(1.1) expert load); its expert count scales with
# the number of ranks so that every rank keeps 32 local experts.
SHAPES = {
    "c2": dict(tokens=4096, hidden=4096, experts=32, top_k=4, inter=1536, experts_per_rank=None, zipf=None),
    "c3": dict(tokens=8192, hidden=7168, experts=None, top_k=8, inter=2048, experts_per_rank=32, zipf=1.1),
}
TOKENS, HIDDEN, EXPERTS, TOP_K, INTER = 4096, 4096, 32, 4, 1536
ZIPF = None
PRECISION = "bf16"


def select_shape(name: str, world: int, precision: str) -> None:
    """Bind the module-level workload constants."""
    global TOKENS, HIDDEN, EXPERTS, TOP_K, INTER, FLOPS_PER_TOKEN, ZIPF, PRECISION  # pylint: disable=global-statement
    shape = SHAPES[name]
    TOKENS, HIDDEN, TOP_K, INTER = shape["tokens"], shape["hidden"], shape["top_k"], shape["inter"]
    EXPERTS = shape["experts"] if shape["experts"] is not None else shape["experts_per_rank"] * world
    ZIPF = shape["zipf"]
    PRECISION = precision
    FLOPS_PER_TOKEN = 18 * TOP_K * HIDDEN * INTER
METRIC = "moe_layer_fwd_bwd_tokens_per_s"
UNIT = "tokens/s"
# forward 6*K*H*I flops per token (two GEMMs), backward 12*K*H*I (four GEMMs)
FLOPS_PER_TOKEN = 18 * TOP_K * HIDDEN * INTER

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of the six grouped-GEMM launches of one
# step at EP=1, from the ncu capture summarised in profiles/grouped_gemm_kernel_bench_moe_bf16_ep1.md.
GEMM_DRAM_BYTES_PER_STEP = 5.02e9


def make_inputs(rank: int, ep: int, device=None):
    """Seeded synthetic inputs of the configuration's shapes and distributions (CPU, then copied)."""
    g = torch.Generator().manual_seed(1234 + rank)
    x = torch.randn(TOKENS, HIDDEN, generator=g).bfloat16()
    # "uniform-ish" router logits: U(-1, 1) plus small noise, softmax, top-4
    logits = torch.rand(TOKENS, EXPERTS, generator=g) * 2 - 1 + 0.01 * torch.randn(TOKENS, EXPERTS, generator=g)
    if ZIPF is not None:
        # skewed router logits: expert popularity follows Zipf(s) over a fixed random ranking (Gumbel top-k)
        ranking = torch.randperm(EXPERTS, generator=torch.Generator().manual_seed(99))
        popularity = torch.empty(EXPERTS)
        popularity[ranking] = torch.arange(1, EXPERTS + 1, dtype=torch.float32).pow(-ZIPF)
        gumbel = -torch.log(-torch.log(torch.rand(TOKENS, EXPERTS, generator=g).clamp_min(1e-9)))
        logits = popularity.log() + gumbel
        # group-limited selection of that configuration: 8 expert groups, the 4 best per token (group score =
        # sum of the two largest scores of the group), then top-k inside them
        scores = logits.sigmoid()
        grouped = scores.view(TOKENS, 8, EXPERTS // 8)
        best_groups = grouped.topk(2, dim=-1).values.sum(dim=-1).topk(4, dim=-1).indices
        keep = torch.zeros(TOKENS, 8, dtype=torch.bool).scatter_(1, best_groups, True)
        limited = scores.masked_fill(~keep.unsqueeze(-1).expand_as(grouped).reshape(TOKENS, EXPERTS), float("-inf"))
        ids = torch.topk(limited, TOP_K, dim=-1).indices
        weights = scores.gather(1, ids)
        weights = weights / weights.sum(dim=-1, keepdim=True)
    else:
        weights, ids = torch.topk(logits.softmax(dim=-1), TOP_K, dim=-1)
    grad_out = torch.randn(TOKENS, HIDDEN, generator=g).bfloat16()
    local = EXPERTS // ep
    if device is not None:
        # large shapes: draw the weights on the GPU (seeded), there is nothing to compare them with on the CPU
        gw = torch.Generator(device=device).manual_seed(4321 + rank)
        w1 = (torch.randn(local, HIDDEN, 2 * INTER, generator=gw, device=device) * 0.02).bfloat16()
        w2 = (torch.randn(local, INTER, HIDDEN, generator=gw, device=device) * 0.02).bfloat16()
    else:
        gw = torch.Generator().manual_seed(4321 + rank)
        w1 = (torch.randn(local, HIDDEN, 2 * INTER, generator=gw) * 0.02).bfloat16()
        w2 = (torch.randn(local, INTER, HIDDEN, generator=gw) * 0.02).bfloat16()
    return x, ids, weights.contiguous(), grad_out, w1, w2


def config(ep: int) -> dict:
    return {
        "workload": (f"MegaMoE {PRECISION.upper()} forward+backward, EP={ep}, {TOKENS} tokens/rank, hidden {HIDDEN}, "
                     f"{EXPERTS} experts ({EXPERTS // ep}/rank), "
                     f"{'sigmoid top-' + str(TOP_K) + ' in 4 of 8 expert groups, Zipf(' + str(ZIPF) + ') load' if ZIPF else 'softmax top-' + str(TOP_K)}, "
                     f"SwiGLU intermediate {INTER}"),
        "tokens_per_rank": TOKENS, "hidden": HIDDEN, "experts": EXPERTS, "top_k": TOP_K, "intermediate": INTER,
        "ep": ep, "layout": "EIO",
        "l2": "no flush: each step streams >1.4 GB of weights and activations through the 126 MB L2",
    }


# ----------------------------------------------------------------------------------- CPU baseline
def cpu_baseline(sample_tokens: int, iterations: int) -> dict:
    """Time the oracle (port of the reference's TorchExperts CPU branch) on a token subsample."""
    from oracle import moe as omoe

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    x, ids, weights, grad_out, w1, w2 = make_inputs(0, 1)
    x, ids, weights, grad_out = x[:sample_tokens], ids[:sample_tokens], weights[:sample_tokens], grad_out[:sample_tokens]
    omoe.experts_forward_backward(x[:64], ids[:64], weights[:64], w1, w2, grad_out[:64])  # warm-up
    times = []
    for _ in range(iterations):
        t0 = time.perf_counter()
        omoe.experts_forward_backward(x, ids, weights, w1, w2, grad_out)
        times.append(time.perf_counter() - t0)
    seconds = statistics.median(times)
    return {
        "value": sample_tokens / seconds, "unit": UNIT, "cores": threads, "kind": "port",
        "sample": (f"{sample_tokens} of the {TOKENS} tokens of rank 0 through all {EXPERTS} experts, "
                   f"forward+backward, median of {iterations} ({seconds:.2f} s each), torch CPU threads={threads}"),
    }


def run_reference(args) -> None:
    """Reference arm: the CPU restatement of the reference's golden path on the host cores.

    Every step (warm-up and timed alike) is one forward+backward over the same token subsample,
    sized from a probe so that the whole run stays within a few minutes.
    """
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import moe as omoe

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    inputs = make_inputs(0, 1)

    def run(sample: int) -> float:
        x, ids, weights, grad_out = (t[:sample] for t in inputs[:4])
        t0 = time.perf_counter()
        omoe.experts_forward_backward(x, ids, weights, inputs[4], inputs[5], grad_out)
        return time.perf_counter() - t0

    probe = run(64)
    per_step_budget = 150.0 / (args.steps + args.warmup)
    sample = 64 * max(1, min(TOKENS // 64, int(per_step_budget / probe)))
    per_step = []
    for step in range(args.warmup + args.steps):
        seconds = run(sample)
        if step >= args.warmup:
            per_step.append(seconds)
    seconds = sum(per_step) / len(per_step)
    value = sample / seconds
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config(1),
        "cpu_baseline": {
            "value": value, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": (f"each step = {sample} of the {TOKENS} tokens through all {EXPERTS} experts, "
                       f"forward+backward, on the CPU restatement of the reference's golden path"),
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
def run_gpu(args) -> None:
    import torch.distributed as dist

    from hyper_multicore_b200 import MegaMoeExperts, kernels
    from hyper_multicore_b200 import _lib

    _lib.load()  # fail loudly here if the native library is missing: there is no fallback path
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run); "
                         f"got WORLD_SIZE={world}")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    x_h, ids_h, p_h, g_h, w1_h, w2_h = make_inputs(rank, world, device if args.shape != "c2" else None)
    w1 = w1_h.to(device).requires_grad_(True)
    w2 = w2_h.to(device).requires_grad_(True)
    if PRECISION == "mxfp8":
        from hyper_multicore_b200.mxfp8 import attach_mx_fields

        attach_mx_fields(w1)
        attach_mx_fields(w2)
    from hyper_multicore_b200 import MegaMoeTuningOptions

    module = MegaMoeExperts(hidden_size=HIDDEN, intermediate_size=INTER, num_experts=EXPERTS, top_k=TOP_K,
                            ep_group=group, precision=PRECISION,
                            tuning_options=MegaMoeTuningOptions(dispatch_mode=args.dispatch))

    # device-resident inputs
    x_d = x_h.to(device).requires_grad_(True)
    ids_d = ids_h.to(device)
    p_d = p_h.to(device).requires_grad_(True)
    g_d = g_h.to(device)

    def step_resident() -> None:
        w1.grad = w2.grad = x_d.grad = p_d.grad = None
        out = module(x_d, ids_d, p_d, expert_weights=(w1, w2))
        out.backward(g_d)

    # host-resident inputs: pinned staging, copies inside the timed region. The three legs of a step
    # (inputs host -> device, forward + backward, results device -> host) run on three streams, so the
    # copies of neighbouring steps overlap the compute of this one; every step still copies its own
    # inputs in and its own results out.
    pinned = [t.pin_memory() for t in (x_h, ids_h, p_h, g_h)]
    h2d_bytes = sum(t.numel() * t.element_size() for t in pinned)
    slots = []
    for _ in range(2):
        slots.append({
            "in": [torch.empty_like(t, device=device) for t in pinned],
            "out": [torch.empty(TOKENS, HIDDEN, dtype=torch.bfloat16).pin_memory(),
                    torch.empty(TOKENS, HIDDEN, dtype=torch.bfloat16).pin_memory(),
                    torch.empty(TOKENS, TOP_K, dtype=torch.float32).pin_memory()],
            "loaded": torch.cuda.Event(), "computed": torch.cuda.Event(), "stored": torch.cuda.Event(), "keep": None,
        })
    d2h_bytes = sum(t.numel() * t.element_size() for t in slots[0]["out"])
    copy_in, copy_out = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    host_state = {"step": 0}

    def load(slot) -> None:
        with torch.cuda.stream(copy_in):
            copy_in.wait_event(slot["computed"])  # the previous user of this slot has finished with it
            for dst, src in zip(slot["in"], pinned):
                dst.copy_(src, non_blocking=True)
            slot["loaded"].record(copy_in)

    def step_host() -> None:
        main = torch.cuda.current_stream(device)
        index = host_state["step"]
        slot, other = slots[index % 2], slots[(index + 1) % 2]
        if index == 0:
            load(slot)
        main.wait_event(slot["loaded"])
        main.wait_event(slot["stored"])  # the results of the step that used this slot before are out
        # queued before this step's kernels (the host waits for the device inside the module's route
        # preparation): the next step's inputs travel while this step computes
        load(other)
        w1.grad = w2.grad = None
        x = slot["in"][0].detach().requires_grad_(True)
        p = slot["in"][2].detach().requires_grad_(True)
        out = module(x, slot["in"][1], p, expert_weights=(w1, w2))
        out.backward(slot["in"][3])
        slot["computed"].record(main)
        results = (out.detach(), x.grad, p.grad)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(slot["computed"])
            for host, dev in zip(slot["out"], results):
                dev.record_stream(copy_out)
                host.copy_(dev, non_blocking=True)
            slot["stored"].record(copy_out)
        slot["keep"] = results
        host_state["step"] = index + 1

    def timed(step, steps: int, warmup: int, join=()):
        for _ in range(warmup):
            step()
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches_before = kernels.LAUNCH_COUNT
        start.record()
        for _ in range(steps):
            step()
        for stream in join:  # the last results must be on the host before the clock stops
            torch.cuda.current_stream(device).wait_stream(stream)
        stop.record()
        barrier()
        ms = torch.tensor([start.elapsed_time(stop)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), kernels.LAUNCH_COUNT - launches_before

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    total_ms, launches = timed(step_resident, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    e2e_ms, _ = timed(step_host, args.steps, max(3, args.warmup), join=(copy_in, copy_out))
    module.check_status()

    # per-launch duration of the dominant kernel (the grouped GEMM), CUDA events on the launch stream
    gemm_name = "mx_gemm" if PRECISION == "mxfp8" else "grouped_gemm"
    original = getattr(kernels, gemm_name)
    pairs: list = []

    def instrumented(*a, **kw):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        original(*a, **kw)
        e1.record()
        pairs.append((e0, e1))

    setattr(kernels, gemm_name, instrumented)
    profile_steps = min(args.steps, 5)
    for _ in range(profile_steps):
        step_resident()
    barrier()
    setattr(kernels, gemm_name, original)
    gemm_ms_per_step = sum(a.elapsed_time(b) for a, b in pairs) / profile_steps
    gemm_launches_per_step = len(pairs) // profile_steps

    module.close()  # collective for EP > 1: every rank unmaps its peers before anyone frees
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks_path = ROOT / "MEASURED_PEAKS.json"
    if peaks_path.exists():
        peaks = json.loads(peaks_path.read_text())
        peak_tflops, peak_note = float(peaks["bf16_tflops_sustained"]), "of measured (sustained cuBLAS bf16)"
    else:
        peak_tflops, peak_note = 1400.0, "of fallback (sustained)"
    if PRECISION == "mxfp8":
        # no FP8 peak was measured on this pool: the dense FP8 rate is twice the BF16 one
        peak_tflops, peak_note = 2 * peak_tflops, "2 x " + peak_note[3:] + " (no FP8 peak measured)"
    flops_per_step = FLOPS_PER_TOKEN * TOKENS  # per rank: every rank owns an equal share in expectation
    achieved = flops_per_step / (gemm_ms_per_step * 1e-3) / 1e12
    ms_per_step = total_ms / args.steps
    value = world * TOKENS / (ms_per_step * 1e-3)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if PRECISION == "bf16" else "mxfp8 (e4m3 + ue8m0/32) operands, bf16 activations",
        "data": "synthetic", "config": config(world),
        "clocks": clocks,
        "e2e": {"value": world * TOKENS / (e2e_ms / args.steps * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                "ms_per_step": e2e_ms / args.steps,
                "pipeline": "copies of neighbouring steps overlap this step's compute (3 streams, 2 buffer sets)"},
        "gpu_launches": launches,
        "roofline": {
            "bound": "tensor",
            "kernel": ("mx_gemm_kernel (tcgen05 block-scaled FP8" if PRECISION == "mxfp8" else "grouped_gemm_kernel (tcgen05") +
                      f", {gemm_launches_per_step} launches per step)",
            "achieved": achieved, "peak": peak_tflops, "unit": "TFLOP/s", "frac": achieved / peak_tflops,
            "peak_source": peak_note,
            "traffic": (GEMM_DRAM_BYTES_PER_STEP / gemm_launches_per_step
                        if world == 1 and gemm_launches_per_step and args.shape == "c2" and PRECISION == "bf16" else None),
            "gemm_ms_per_step": gemm_ms_per_step, "launches_per_step": gemm_launches_per_step,
            "algorithmic_flops_per_step": flops_per_step,
            "layer_frac": flops_per_step / (ms_per_step * 1e-3) / 1e12 / peak_tflops,
        },
    }
    if world == 1 and not args.no_cpu_baseline and args.shape == "c2":
        line["cpu_baseline"] = cpu_baseline(sample_tokens=256, iterations=2)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("b200", "reference"), default="b200")
    parser.add_argument("--no-cpu-baseline", action="store_true",
                        help="skip the CPU baseline leg (used when the run is captured by a profiler)")
    parser.add_argument("--shape", choices=tuple(SHAPES), default="c2",
                        help="c2 = EP=2 BF16 configuration's per-rank problem (default); c3 = EP=8 MXFP8 configuration's")
    parser.add_argument("--precision", choices=("bf16", "mxfp8"), default="bf16")
    parser.add_argument("--dispatch", choices=("push", "pull"), default="push",
                        help="EP > 1: sources store rows into the owners' buffers (push, default) or owners fetch them (pull)")
    parser.add_argument("--workload", choices=("moe", "gate", "mhc"), default="moe",
                        help="moe = the MoE layer (default, the headline metric); gate / mhc = the router and the "
                             "four-stream residual mix, timed against the HBM roofline")
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
    select_shape(args.shape, args.gpus, args.precision)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
