#!/usr/bin/env python
"""MoE-layer throughput benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" = one forward of the Qwen3-30B-A3B-shaped MoE layer (router -> permute -> grouped
SwiGLU expert GEMM -> combine) over one batch of seeded synthetic tokens.  Default workload:
bf16 prefill, T=4096 tokens, H=2048, E=128, top-8, I=768.  Prints ONE JSON line on rank 0.

--impl reference times the CPU restatement of the reference's per-expert-loop path (oracle/) on
the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "mini-qwen-llm_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

H, E, TOPK, I = 2048, 128, 8, 768
T_PREFILL = 4096
METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
CPU_SAMPLE_T = 2048
WORKLOAD = f"bf16 prefill MoE layer, T={T_PREFILL} tokens per GPU, H={H} E={E} top{TOPK} I={I} (seed 1)"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int, period_s: float = 0.02):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None
        self._period = period_s

    def _run(self):
        nv = self._nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self._period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_min_mhz": min(self.samples), "sm_max_mhz": self.max_mhz,
                "samples": len(self.samples), "reasons": sorted(self.reasons)}


def build_dense_block(lay, device, rank=0, world=1, group=None):
    """The layer's experts [rank*E/world, (rank+1)*E/world) on `device` (all of them when world == 1)."""
    from mini_qwen_b200 import Qwen3MoEConfig
    from mini_qwen_b200.model.layers import Qwen3MoEBlock

    cfg = Qwen3MoEConfig(hidden_size=H, intermediate_size=I, num_experts=E, num_experts_per_tok=TOPK)
    el = E // world
    lo, hi = rank * el, (rank + 1) * el
    w13 = torch.cat([lay.gate[lo:hi], lay.up[lo:hi]], dim=1).to(device)
    blk = Qwen3MoEBlock.from_stacked(cfg, lay.router.to(device), w13, lay.down[lo:hi].to(device), ep_group=group)
    return blk


def w4a16_decode_numbers(dev, peaks, iters=200, copies=8, batches=(1, 8, 16, 64), w4_kernel=None):
    """W4A16 decode of the same layer shape: per batch size, the time of one block call under
    CUDA-graph replay, rotating over `copies` independently drawn layers so that no weight byte is
    served from L2 (a layer's active experts are 20-310 MB; 8 layers exceed the 126 MB L2 several
    times over).  Algorithmic bytes = packed weights, scales and zero points of the experts hit
    (2 451 456 B each) + router weight + activations in and out."""
    from mini_qwen_b200 import Qwen3MoEConfig
    from mini_qwen_b200.model.layers import LinearW4A16, Qwen3MoEBlock

    cfg = Qwen3MoEConfig(hidden_size=H, intermediate_size=I, num_experts=E, num_experts_per_tok=TOPK)
    gen = torch.Generator(device=dev).manual_seed(2)

    def stack(kd, n):
        qw = torch.randint(-2 ** 31, 2 ** 31 - 1, (E, kd // 8, n), generator=gen, device=dev, dtype=torch.int32)
        sc = (torch.rand(E, kd // 128, n, generator=gen, device=dev) * 0.015 + 0.005).to(torch.bfloat16)
        qz = torch.randint(-2 ** 31, 2 ** 31 - 1, (E, kd // 128, n // 8), generator=gen, device=dev, dtype=torch.int32)
        return qw, sc, qz

    blocks = []
    for _ in range(copies):
        with torch.device("meta"):
            blk = Qwen3MoEBlock(cfg)
        blk.gate.weight = torch.nn.Parameter(
            (torch.randn(E, H, generator=gen, device=dev) * 0.02).to(torch.bfloat16), requires_grad=False)
        blk._stacks = {"w4": True, "group_size": 128, "gate_proj": stack(H, I), "up_proj": stack(H, I),
                       "down_proj": stack(I, H)}
        blk._ready = lambda st=blk._stacks: st          # stacks are installed directly (random packed words)
        if w4_kernel:
            blk.w4_kernel = w4_kernel
        blocks.append(blk)

    expert_bytes = 3 * (H * I // 2) + 2 * (H // 128) * I * 2 + (I // 128) * H * 2 \
        + 2 * (H // 128) * (I // 8) * 4 + (I // 128) * (H // 8) * 4
    out = []
    for T in batches:
        xs = [torch.randn(T, H, generator=gen, device=dev).to(torch.bfloat16) for _ in range(copies)]
        active = []
        graphs = []
        with torch.no_grad():
            for blk, x in zip(blocks, xs):
                blk(x)                                                   # warm-up, also sets kernel attributes
                from mini_qwen_b200.kernels import moe_router
                ids, _ = moe_router(x, blk.gate.weight, TOPK)
                active.append(int(torch.unique(ids).numel()))
            torch.cuda.synchronize()
            for blk, x in zip(blocks, xs):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    blk(x)
                graphs.append(g)
            for g in graphs:
                g.replay()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for i in range(iters):
                graphs[i % copies].replay()
            e.record()
            torch.cuda.synchronize()
            us_graph = s.elapsed_time(e) * 1e3 / iters
            s.record()
            for i in range(iters):
                blocks[i % copies](xs[i % copies])
            e.record()
            torch.cuda.synchronize()
            us_eager = s.elapsed_time(e) * 1e3 / iters
        a = sum(active) / len(active)
        nbytes = a * expert_bytes + E * H * 2 + 2 * T * H * 2
        gbs = nbytes / (us_graph * 1e-6) / 1e9
        out.append({"T": T, "active_experts": a, "us_per_step_graph": us_graph, "us_per_step_eager": us_eager,
                    "tokens_per_s": T / (us_graph * 1e-6), "algorithmic_mb": nbytes / 1e6, "hbm_gbs": gbs,
                    "hbm_frac": gbs / peaks["hbm_gbs"]})
        del graphs
    return out


def cpu_reference_tokens_per_s(lay, steps, warmup, sample_t):
    """The reference's per-expert-loop path (CPU restatement) on `sample_t`-token slices of the batch."""
    from oracle import moe_oracle as O

    torch.set_num_threads(os.cpu_count())
    T = lay.x.shape[0]
    times = []
    for i in range(warmup + steps):
        lo = (i * sample_t) % max(T - sample_t + 1, 1)
        x = lay.x[lo:lo + sample_t]
        t0 = time.perf_counter()
        O.block_forward(x, lay.router, lay.gate, lay.up, lay.down, lay.top_k, True)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    total = sum(times)
    return sample_t * len(times) / total, 1e3 * total / len(times)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from mini_qwen_b200 import synthetic

    lay = synthetic.dense_layer(1, T_PREFILL, H, E, TOPK, I, torch.bfloat16)
    tps, ms = cpu_reference_tokens_per_s(lay, args.steps, args.warmup, CPU_SAMPLE_T)
    cores = os.cpu_count()
    sample = f"{CPU_SAMPLE_T}-token slices of the {T_PREFILL}-token batch, one slice per step"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample,
                   "parallelism": "reference per-expert loop (CPU restatement) on the host cores of rank 0"},
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_ours(args):
    import torch.distributed as dist

    from mini_qwen_b200 import _cabi, synthetic

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _cabi.load()

    lay = synthetic.dense_layer(1, T_PREFILL, H, E, TOPK, I, torch.bfloat16)
    blk = build_dense_block(lay, dev, rank, world, dist.group.WORLD if world > 1 else None)
    T = T_PREFILL
    if rank > 0:   # every rank routes its own tokens (same distribution, different draw)
        lay.x = torch.randn(T, H, generator=torch.Generator().manual_seed(1000 + rank)).to(torch.bfloat16)
    x_host = lay.x.pin_memory()
    out_host = torch.empty_like(x_host).pin_memory()
    x_dev = lay.x.to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    from mini_qwen_b200.graph import CapturedForward

    # ---- per-kernel times: an eager pass with CUDA events around every stage (not the timed region)
    with torch.no_grad():
        for _ in range(max(3, args.warmup)):
            blk(x_dev)
        barrier()
        blk.kernel_events = []
        for _ in range(min(args.steps, 20)):
            blk(x_dev)
        barrier()
        events, blk.kernel_events = blk.kernel_events, None
    kern = {}
    for name, a, b in events:
        kern.setdefault(name, []).append(a.elapsed_time(b))
    per_call = {}
    for name, _, _ in events[:len(events) // min(args.steps, 20)]:
        per_call[name] = per_call.get(name, 0) + 1
    # a stage that runs several times per call (the rank barriers) is reported as its sum per call
    kern_ms = {k: sum(v) / len(v) * per_call.get(k, 1) for k, v in kern.items()}

    # ---- device-resident throughput: the whole layer call is one CUDA graph (no host synchronisation
    # anywhere in it), so a step is one launch and the host cannot fall behind the GPU
    cap = [CapturedForward(blk, x_dev, warmup=2)]
    cap.append(CapturedForward(blk, x_dev, warmup=1, pool=cap[0].pool()))
    for _ in range(max(3, args.warmup)):
        cap[0].replay()
    barrier()
    _cabi.launch_count = 0
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        start.record()
        for _ in range(args.steps):
            cap[0].replay()
        end.record()
        barrier()
    launches = _cabi.launch_count
    ms_total = max_over_ranks(start.elapsed_time(end))
    ms_step = ms_total / args.steps
    value = world * T * args.steps / (ms_total * 1e-3)

    # the same loop launched kernel by kernel from Python, for comparison
    with torch.no_grad():
        barrier()
        s1, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s1.record()
        for _ in range(args.steps):
            blk(x_dev)
        e1.record()
        barrier()
    eager_ms_step = max_over_ranks(s1.elapsed_time(e1)) / args.steps

    # ---- end to end: pinned host input -> device -> block -> device -> pinned host output, every step.
    # The three legs run on their own streams with two buffers each (one captured graph per buffer), so
    # step i's upload overlaps step i-1's compute and step i-2's download, as a serving loop would
    # pipeline them.
    h2d, d2h = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    comp = torch.cuda.current_stream(dev)
    x_in = [c.x for c in cap]
    out_pinned = [torch.empty_like(x_host).pin_memory() for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]       # compute has consumed x_in[b]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    ev_down = [torch.cuda.Event() for _ in range(2)]       # download of out_pinned[b] finished

    def e2e_steps(n):
        for i in range(n):
            b = i & 1
            with torch.cuda.stream(h2d):
                if i >= 2:
                    h2d.wait_event(ev_free[b])
                x_in[b].copy_(x_host, non_blocking=True)
                ev_in[b].record(h2d)
            comp.wait_event(ev_in[b])
            if i >= 2:
                comp.wait_event(ev_down[b])                 # the graph's output buffer has been downloaded
            out = cap[b].replay()
            ev_free[b].record(comp)
            ev_out[b].record(comp)
            with torch.cuda.stream(d2h):
                d2h.wait_event(ev_out[b])
                out_pinned[b].copy_(out, non_blocking=True)
                ev_down[b].record(d2h)
        comp.wait_stream(d2h)
        comp.wait_stream(h2d)

    with torch.no_grad():
        e2e_steps(max(4, args.warmup // 2))
        barrier()
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s2.record()
        e2e_steps(args.steps)
        e2.record()
        barrier()
    e2e_ms = max_over_ranks(s2.elapsed_time(e2))
    e2e_value = world * T * args.steps / (e2e_ms * 1e-3)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    S = T * TOPK
    gemm1_flops = 2.0 * S * (2 * I) * H          # gate+up projections of all slots
    gemm1_ms = kern_ms.get("grouped_swiglu")
    roofline = None
    if gemm1_ms:
        achieved = gemm1_flops / (gemm1_ms * 1e-3) / 1e12
        # algorithmic bytes of one launch: this rank's gate/up weights once, every token row once, h once
        alg_bytes = (E // world) * 2 * I * H * 2 + T * H * 2 + S * I * 2
        roofline = {"bound": "tensor", "kernel": "grouped gate/up GEMM + SwiGLU (rows gathered in the kernel)",
                    "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["bf16_tflops"],
                    "peak_source": f"{peaks['source']} burst bf16 GEMM",
                    # dram__bytes_read.sum + dram__bytes_write.sum of this kernel at this workload, one ncu
                    # capture (profiles/grouped_gemm_tc5_c2.md): 892.8 MB read + 45.1 MB written
                    "traffic": 937.9e6 if world == 1 else None,
                    "flops_per_launch": gemm1_flops, "ms_per_launch": gemm1_ms}
        if world == 1:
            # the layer is on the ridge: the same launch seen from the HBM side
            gbs = alg_bytes / (gemm1_ms * 1e-3) / 1e9
            roofline["hbm"] = {"achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                               "frac": gbs / peaks["hbm_gbs"], "algorithmic_bytes": alg_bytes}

    cpu_base = None
    if world == 1 and not args.no_cpu_baseline:
        tps, _ = cpu_reference_tokens_per_s(lay, steps=6, warmup=1, sample_t=T_PREFILL // 2)
        cpu_base = {"value": tps, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                    "sample": f"6 passes over {T_PREFILL // 2}-token halves of the batch after 1 warm-up"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "l2": "per-step working set 1.2 GB of expert weights > 126 MB L2; no flush needed",
                   "parallelism": "single GPU" if world == 1 else
                   f"expert parallel ep{world}: {E // world} experts per GPU, {T} tokens per GPU, "
                   "dispatch by NVLink stores out of the permute kernel, return by NVLink stores out of the down "
                   "projection's epilogue, stream-ordered flag barriers between ranks"},
        "roofline": roofline, "cpu_baseline": cpu_base,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * 2,
                "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": e2e_ms / args.steps,
                "pipeline": "upload, compute and download on three streams, two buffers each"},
        "gpu_launches": launches, "clocks": clocks.summary(),
        "launch": "one CUDA graph per step", "eager_ms_per_step": eager_ms_step,
        "kernels_ms": kern_ms,
    }
    if world == 1 and not args.no_decode:
        del blk
        torch.cuda.empty_cache()
        batches = tuple(int(b) for b in args.decode_batches.split(","))
        line["w4a16_decode"] = w4a16_decode_numbers(dev, peaks, iters=args.decode_iters, batches=batches)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="skip the W4A16 decode numbers")
    ap.add_argument("--decode-only", action="store_true",
                    help="only the W4A16 decode numbers (small profiling runs); prints their JSON list")
    ap.add_argument("--decode-iters", type=int, default=200)
    ap.add_argument("--decode-batches", default="1,8,16,64")
    ap.add_argument("--w4-kernel", default=None, choices=["auto", "tc", "mma"],
                    help="W4A16 kernel of the decode numbers (default: the block's own choice)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.decode_only:
        assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        batches = tuple(int(b) for b in args.decode_batches.split(","))
        print(json.dumps({"w4a16_decode": w4a16_decode_numbers(dev, measured_peaks(), iters=args.decode_iters,
                                                                batches=batches, w4_kernel=args.w4_kernel)}))
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
