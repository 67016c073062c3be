#!/usr/bin/env python
"""MoE-layer throughput benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c4|c5]

One "step" = one pass of the MoE hot path (router -> permute -> grouped SwiGLU expert GEMM -> combine)
over one batch of seeded synthetic tokens.  Workloads (the Qwen3-30B-A3B MoE layer: H=2048, E=128, top-8,
I=768):

  c2 (default)  bf16 prefill layer, 4096 tokens per GPU (weak scaling under expert parallelism)
  c3            W4A16 decode layer, batches 1/8/16/64, one GPU; the line's value is batch 64
  c4            bf16 layer with Zipf(1.2)-skewed routing, 16384 tokens in total split over the GPUs
                (strong scaling), experts sharded
  c5            48 independently drawn W4A16 layers chained (a weight-free RMS norm between them), decode
                batch 16 in total (--c5-batch 8 for the other size), experts sharded over the GPUs;
                tokens/s per full 48-layer pass

Prints ONE JSON line on rank 0.  Every line carries a parity sample (rows of the timed configuration
checked against the CPU restatement of the reference before the timed loop, on every rank) and the device
status words read after it.

--impl reference times the CPU restatement of the reference's per-expert-loop path (oracle/) on the host
cores of rank 0, on a bounded sample of the same workload.
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
GROUP = 128
T_PREFILL = 4096
T_SKEWED = 16384
LAYERS = 48
METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
RTOL, ATOL = 2e-2, 2e-3
# bytes of one expert's W4A16 tensors (three projections: packed weights, bf16 scales, packed zero points)
EXPERT_BYTES_W4 = 3 * (H * I // 2) + 2 * (H // GROUP) * I * 2 + (I // GROUP) * H * 2 \
    + 2 * (H // GROUP) * (I // 8) * 4 + (I // GROUP) * (H // 8) * 4
GATE_UP_BYTES_W4 = 2 * (H * I // 2 + (H // GROUP) * I * 2 + (H // GROUP) * (I // 8) * 4)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def recorded_traffic(key):
    """DRAM bytes per launch of a kernel from its ncu capture, if one is on record (profiles/dram_traffic.json,
    written when a profile summary is made); None otherwise."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as f:
            entry = json.load(f).get(key)
        return None if entry is None else float(entry["dram_bytes_read"]) + float(entry["dram_bytes_write"])
    except (OSError, ValueError, KeyError):
        return None


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


# --------------------------------------------------------------------------------------------- harness
class Harness:
    """One process per GPU: device, process group, barriers and reductions over the ranks."""

    def __init__(self):
        import torch.distributed as dist
        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.group = None
        if self.world > 1:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer loads/stores only
            dist.init_process_group("nccl", device_id=self.dev)
            self.group = dist.group.WORLD
        from mini_qwen_b200 import _cabi
        self.cabi = _cabi
        _cabi.load()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        if self.world > 1:
            t = torch.tensor([v], device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            return float(t.item())
        return v

    def all_ok(self, ok: bool) -> bool:
        if self.world > 1:
            t = torch.tensor([1 if ok else 0], device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
            return bool(t.item())
        return ok

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def stage_times(hn, model, blocks, x_dev, warmup, calls):
    """Per-stage CUDA-event times of an eager pass (not the timed region): {stage: ms per model call}."""
    with torch.no_grad():
        for _ in range(max(3, warmup)):
            model(x_dev)
        hn.barrier()
        for b in blocks:
            b.kernel_events = []
        for _ in range(calls):
            model(x_dev)
        hn.barrier()
    sums = {}
    for b in blocks:
        events, b.kernel_events = b.kernel_events, None
        for name, a, e in events:
            sums[name] = sums.get(name, 0.0) + a.elapsed_time(e)
    return {k: v / calls for k, v in sums.items()}


def timed_replays(hn, cap, steps, warmup):
    for _ in range(max(3, warmup)):
        cap.replay()
    hn.barrier()
    hn.cabi.launch_count = 0
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(hn.local) as clocks:
        start.record()
        for _ in range(steps):
            cap.replay()
        end.record()
        hn.barrier()
    return hn.max_over_ranks(start.elapsed_time(end)), hn.cabi.launch_count, clocks.summary()


def timed_eager(hn, model, x_dev, steps):
    with torch.no_grad():
        hn.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(steps):
            model(x_dev)
        e.record()
        hn.barrier()
    return hn.max_over_ranks(s.elapsed_time(e)) / steps


def timed_e2e(hn, caps, x_host, steps, warmup):
    """Pinned host input -> device -> model -> device -> pinned host output, every step.  The three legs run on
    their own streams with two buffers each (one captured graph per buffer), so step i's upload overlaps step
    i-1's compute and step i-2's download, as a serving loop would pipeline them.  Returns total ms."""
    dev = hn.dev
    h2d, d2h = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    comp = torch.cuda.current_stream(dev)
    x_in = [c.x for c in caps]
    out_pinned = [torch.empty(caps[0].out.shape, dtype=caps[0].out.dtype).pin_memory() for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]       # compute has consumed x_in[b]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    ev_down = [torch.cuda.Event() for _ in range(2)]       # download of out_pinned[b] finished

    def run(n):
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
            out = caps[b].replay()
            ev_free[b].record(comp)
            ev_out[b].record(comp)
            with torch.cuda.stream(d2h):
                d2h.wait_event(ev_out[b])
                out_pinned[b].copy_(out, non_blocking=True)
                ev_down[b].record(d2h)
        comp.wait_stream(d2h)
        comp.wait_stream(h2d)

    with torch.no_grad():
        run(max(4, warmup // 2))
        hn.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        run(steps)
        e.record()
        hn.barrier()
    return hn.max_over_ranks(s.elapsed_time(e)), out_pinned[0].numel() * out_pinned[0].element_size()


def device_status(blocks):
    """OR of the blocks' device status words (bounded wait expired = 1, receive buffer overflow = 2)."""
    bits = 0
    for b in blocks:
        if b._status is not None:
            bits |= int(b._status.item())
        if b._peer is not None:
            bits |= int(b._peer.status.item())
    return bits


def literal_close(out, ref):
    out, ref = out.float(), ref.float()
    return bool(((out - ref).abs() <= ATOL + RTOL * ref.abs()).all())


# --------------------------------------------------------------------------------- dense workloads (c2, c4)
def dense_setup(name):
    from mini_qwen_b200 import synthetic
    if name == "c2":
        lay = synthetic.dense_layer(1, T_PREFILL, H, E, TOPK, I, torch.bfloat16)
        return lay, None, f"bf16 prefill MoE layer, T={T_PREFILL} tokens per GPU, H={H} E={E} top{TOPK} I={I} (seed 1)"
    lay = synthetic.dense_layer(4, T_SKEWED, H, E, TOPK, I, torch.bfloat16)
    bias = synthetic.zipf_router_bias(5, E, s=1.2, strength=1.0)
    return lay, bias, (f"bf16 MoE layer with Zipf(1.2)-skewed routing, T={T_SKEWED} tokens in total split over the GPUs, "
                       f"H={H} E={E} top{TOPK} I={I} (seed 4, router bias seed 5)")


def cpu_dense_tokens_per_s(lay, bias, steps, warmup, sample_t):
    """The reference's per-expert-loop path (CPU restatement) on `sample_t`-token slices of the batch."""
    from oracle import moe_oracle as O
    torch.set_num_threads(os.cpu_count())
    T = lay.x.shape[0]
    times = []
    for i in range(warmup + steps):
        lo = (i * sample_t) % max(T - sample_t + 1, 1)
        x = lay.x[lo:lo + sample_t]
        t0 = time.perf_counter()
        O.block_forward(x, lay.router, lay.gate, lay.up, lay.down, lay.top_k, True, bias)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    total = sum(times)
    return sample_t * len(times) / total, 1e3 * total / len(times)


def run_dense(args, name):
    from mini_qwen_b200 import Qwen3MoEConfig
    from mini_qwen_b200.graph import CapturedForward
    from mini_qwen_b200.model.layers import Qwen3MoEBlock
    from oracle import moe_oracle as O

    hn = Harness()
    world, rank, dev = hn.world, hn.rank, hn.dev
    lay, bias, desc = dense_setup(name)
    cfg = Qwen3MoEConfig(hidden_size=H, intermediate_size=I, num_experts=E, num_experts_per_tok=TOPK)
    el = E // world
    lo, hi = rank * el, (rank + 1) * el
    w13 = torch.cat([lay.gate[lo:hi], lay.up[lo:hi]], dim=1).to(dev)
    if name == "c2":
        T = T_PREFILL                                           # weak scaling: every rank routes its own 4096 tokens
        x_cpu = lay.x if rank == 0 else \
            torch.randn(T, H, generator=torch.Generator().manual_seed(1000 + rank)).to(torch.bfloat16)
        tokens_per_step, scaling = world * T, "weak"
    else:
        T = T_SKEWED // world                                   # strong scaling: the batch is split over the ranks
        x_cpu = lay.x[rank * T:(rank + 1) * T].contiguous()
        tokens_per_step, scaling = T_SKEWED, "strong"
    blk = Qwen3MoEBlock.from_stacked(cfg, lay.router.to(dev), w13, lay.down[lo:hi].to(dev), ep_group=hn.group,
                                     ep_max_tokens=T)
    if bias is not None:
        blk.router_bias = bias.to(dev)
    x_host = x_cpu.pin_memory()
    x_dev = x_cpu.to(dev)

    # ---- parity sample: this rank's first 64 rows against the CPU restatement of the reference (all experts)
    with torch.no_grad():
        out = blk(x_dev)
    torch.cuda.synchronize()
    rows = min(64, T)
    ref, ref_ids, _, _ = O.block_forward(x_cpu[:rows], lay.router, lay.gate, lay.up, lay.down, TOPK, True, bias)
    from mini_qwen_b200.kernels import moe_router
    ids, _ = moe_router(x_dev[:rows], blk.gate.weight, TOPK, bias=blk.router_bias)
    sample_ok = torch.equal(ids.cpu(), ref_ids) and literal_close(out[:rows].cpu(), ref)
    parity_ok = hn.all_ok(sample_ok)
    if not parity_ok:
        if rank == 0 or not sample_ok:
            print(f"rank {rank}: parity sample {'FAILED' if not sample_ok else 'ok'} (a rank failed: no number is reported)",
                  file=sys.stderr)
        hn.barrier()
        hn.close()
        sys.exit(3)

    kern_ms = stage_times(hn, blk, [blk], x_dev, args.warmup, min(args.steps, 20))
    # the whole layer call is one CUDA graph (no host synchronisation anywhere in it): a step is one launch
    caps = [CapturedForward(blk, x_dev, warmup=2)]
    caps.append(CapturedForward(blk, x_dev, warmup=1, pool=caps[0].pool()))
    ms_total, launches, clocks = timed_replays(hn, caps[0], args.steps, args.warmup)
    eager_ms = timed_eager(hn, blk, x_dev, args.steps)
    e2e_ms, out_bytes = timed_e2e(hn, caps, x_host, args.steps, args.warmup)
    status = device_status([blk])
    status = int(hn.max_over_ranks(float(status)))
    if rank != 0:
        hn.close()
        return

    peaks = measured_peaks()
    S = T * TOPK
    roofline = None
    gemm1_ms = kern_ms.get("grouped_swiglu")
    if gemm1_ms:
        # slots this rank's gate/up launch multiplies: its own under weak scaling on one GPU; under expert
        # parallelism the rows it received, about S for uniform routing (exact counts are routing dependent)
        gemm1_flops = 2.0 * S * (2 * I) * H
        achieved = gemm1_flops / (gemm1_ms * 1e-3) / 1e12
        alg_bytes = (E // world) * 2 * I * H * 2 + T * H * 2 + S * I * 2
        roofline = {"bound": "tensor", "kernel": "grouped gate/up GEMM + SwiGLU (rows gathered in the kernel)",
                    "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["bf16_tflops"], "peak_source": f"{peaks['source']} burst bf16 GEMM",
                    "traffic": recorded_traffic(f"grouped_gemm_tc5_gate_up_{name}") if world == 1 else None,
                    "flops_per_launch": gemm1_flops, "ms_per_launch": gemm1_ms}
        if world == 1:
            gbs = alg_bytes / (gemm1_ms * 1e-3) / 1e9            # the same launch seen from the HBM side
            roofline["hbm"] = {"achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                               "frac": gbs / peaks["hbm_gbs"], "algorithmic_bytes": alg_bytes}
    cpu_base = None
    if world == 1 and not args.no_cpu_baseline:
        tps, _ = cpu_dense_tokens_per_s(lay, bias, steps=4, warmup=1, sample_t=T_PREFILL)
        cpu_base = {"value": tps, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                    "sample": f"4 passes over {T_PREFILL}-token slices of the batch after 1 warm-up"}
    line = {
        "metric": METRIC, "value": tokens_per_step * args.steps / (ms_total * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": desc,
                   "l2": "per-step working set 1.2 GB of expert weights > 126 MB L2; no flush needed",
                   "parallelism": "single GPU" if world == 1 else
                   f"expert parallel ep{world}: {E // world} experts per GPU, {T} tokens per GPU, dispatch by NVLink "
                   "stores out of the permute kernel, return by NVLink stores out of the down projection's epilogue, "
                   "stream-ordered flag barriers between ranks"},
        "roofline": roofline, "cpu_baseline": cpu_base,
        "e2e": {"value": tokens_per_step * args.steps / (e2e_ms * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": out_bytes,
                "ms_per_step": e2e_ms / args.steps,
                "pipeline": "upload, compute and download on three streams, two buffers each"},
        "gpu_launches": launches, "clocks": clocks,
        "parity_sample": "ok", "status": status,
        "parity_note": f"every rank: expert ids bit-exact and outputs within rtol {RTOL} / atol {ATOL} of the CPU "
                       f"restatement of the reference on its first {rows} rows, before the timed loop; status = OR of "
                       "the device status words after it (0 = no bounded wait expired, no receive buffer overflowed)",
        "launch": "one CUDA graph per step", "eager_ms_per_step": eager_ms, "kernels_ms": kern_ms,
    }
    if status != 0:
        line["invalid"] = "a device status bit is set: the timed steps are not valid"
    if name == "c2" and world == 1 and not args.no_decode:
        del blk, caps
        torch.cuda.empty_cache()
        batches = tuple(int(b) for b in args.decode_batches.split(","))
        line["w4a16_decode"] = w4_decode_numbers(dev, peaks, iters=args.decode_iters, batches=batches,
                                                 w4_kernel=args.w4_kernel)
    print(json.dumps(line))
    hn.close()


# ----------------------------------------------------------------------------------- W4A16 workloads (c3, c5)
def w4_stacks(dev, seed, experts):
    from mini_qwen_b200 import synthetic
    return synthetic.w4a16_stacks_on_device(dev, seed, experts, H, I, GROUP)


def w4_router(dev, seed):
    from mini_qwen_b200 import synthetic
    return synthetic.router_weight_on_device(dev, seed, E, H)


def w4_block(dev, layer_seed, rank=0, world=1, group=None, max_tokens=None, w4_kernel=None):
    """One W4A16 layer (this rank's experts) as a block.  The experts of rank r of layer L are drawn from the seed
    (L, r), so any rank can redraw any other rank's experts for a parity check."""
    from mini_qwen_b200 import Qwen3MoEConfig
    from mini_qwen_b200.model.layers import Qwen3MoEBlock
    cfg = Qwen3MoEConfig(hidden_size=H, intermediate_size=I, num_experts=E, num_experts_per_tok=TOPK)
    gate, up, down = w4_stacks(dev, 1_000_003 * layer_seed + 17 * rank + 1, E // world)
    blk = Qwen3MoEBlock.from_stacked_w4(cfg, w4_router(dev, 7919 * layer_seed + 5), gate, up, down, GROUP,
                                        ep_group=group, ep_max_tokens=max_tokens)
    if w4_kernel:
        blk.w4_kernel = w4_kernel
    return blk


def w4_parity_sample(dev, layer_seed, world, x_rows, out_rows, router_w):
    """Rows of one W4A16 layer against the CPU restatement of the reference: the experts the rows hit are redrawn
    (seeds as in w4_block), dequantised on the CPU and multiplied the way the reference's loop does."""
    from oracle import moe_oracle as O
    el = E // world
    shards = {}

    def expert_fn(e, x_e):
        r, j = divmod(e, el)
        if r not in shards:
            shards[r] = [[t.cpu() for t in p] for p in w4_stacks(dev, 1_000_003 * layer_seed + 17 * r + 1, el)]
        trios = [tuple(t[j] for t in p) for p in shards[r]]
        return O.w4a16_expert(x_e, *trios, GROUP)
    ref, ref_ids, _, _ = O.block_forward(x_rows.cpu(), router_w.cpu(), None, None, None, TOPK, True, expert_fn=expert_fn)
    from mini_qwen_b200.kernels import moe_router
    ids, _ = moe_router(x_rows, router_w, TOPK)
    # the quantised layer's outputs reach magnitude 10-100 from bf16 intermediates; the sample is held to rtol 2e-2
    # with the absolute term scaled by the output magnitude (the full bar, against exact sums, is a test)
    out, ref = out_rows.cpu().float(), ref.float()
    close = bool(((out - ref).abs() <= ATOL * max(1.0, ref.abs().max().item()) + RTOL * ref.abs()).all())
    return torch.equal(ids.cpu(), ref_ids) and close


def cpu_w4_layer_ms(dev, layer_seed, x_cpu, steps=3, warmup=1):
    """The reference's per-expert loop on the CPU with each W4A16 projection's weight dequantised to fp32 once
    (its Triton W4A16 kernel cannot run on a CPU): ms per layer call, all experts the batch hits."""
    from oracle import moe_oracle as O
    import torch.nn.functional as F
    torch.set_num_threads(os.cpu_count())
    stacks = [[t.cpu() for t in p] for p in w4_stacks(dev, 1_000_003 * layer_seed + 1, E)]
    router_w = w4_router(dev, 7919 * layer_seed + 5).cpu()
    ids, _ = O.router(x_cpu, router_w, TOPK)
    weights = {}
    for e in sorted(set(ids.reshape(-1).tolist())):
        weights[e] = [O.dequantise(p[0][e], p[1][e], p[2][e], GROUP) for p in stacks]

    def expert_fn(e, x_e):
        g, u, d = weights[e]
        gg = (x_e.float() @ g).to(torch.bfloat16)
        uu = (x_e.float() @ u).to(torch.bfloat16)
        return ((F.silu(gg) * uu).float() @ d).to(torch.bfloat16)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        O.block_forward(x_cpu, router_w, None, None, None, TOPK, True, expert_fn=expert_fn)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    return 1e3 * sum(times) / len(times), len(weights)


def w4_decode_numbers(dev, peaks, iters=200, copies=8, batches=(1, 8, 16, 64), w4_kernel=None):
    """W4A16 decode of the layer: per batch size, the time of one block call under CUDA-graph replay, rotating
    over `copies` independently drawn layers so that no weight byte is served from L2 (a layer's active experts
    are 20-310 MB; 8 layers exceed the 126 MB L2 several times over).  A replay holds one call of each layer
    (`us_per_step_graph` = replay time / layers); `us_per_step_one_call_graph` replays a one-call graph per step.  Algorithmic bytes = packed weights, scales
    and zero points of the experts hit (2 451 456 B each) + router weight + activations in and out."""
    from mini_qwen_b200.kernels import moe_router
    blocks = [w4_block(dev, 100 + i, w4_kernel=w4_kernel) for i in range(copies)]
    gen = torch.Generator(device=dev).manual_seed(2)
    out = []
    for T in batches:
        xs = [torch.randn(T, H, generator=gen, device=dev).to(torch.bfloat16) for _ in range(copies)]
        active, graphs = [], []
        with torch.no_grad():
            for blk, x in zip(blocks, xs):
                blk(x)                                                   # warm-up, also sets kernel attributes
                ids, _ = moe_router(x, blk.gate.weight, TOPK)
                active.append(int(torch.unique(ids).numel()))
            torch.cuda.synchronize()
            # one graph holds a call of each of the rotating layers, the way a decoder's graph holds its layers: a
            # replay is `copies` layer calls (= steps), and the one-replay-per-call figure rides along
            g_all = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_all):
                for blk, x in zip(blocks, xs):
                    blk(x)
            for blk, x in zip(blocks, xs):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    blk(x)
                graphs.append(g)
            for g in graphs + [g_all]:
                g.replay()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            replays = max(1, iters // copies)
            s.record()
            for i in range(replays):
                g_all.replay()
            e.record()
            torch.cuda.synchronize()
            us_graph = s.elapsed_time(e) * 1e3 / (replays * copies)
            s.record()
            for i in range(iters):
                graphs[i % copies].replay()
            e.record()
            torch.cuda.synchronize()
            us_single = s.elapsed_time(e) * 1e3 / iters
            s.record()
            for i in range(iters):
                blocks[i % copies](xs[i % copies])
            e.record()
            torch.cuda.synchronize()
            us_eager = s.elapsed_time(e) * 1e3 / iters
            blocks[0].kernel_events = []
            for _ in range(10):
                for blk, x in zip(blocks, xs):                            # rotate: the timed block finds its weights in HBM
                    blk(x)
            torch.cuda.synchronize()
            ev, blocks[0].kernel_events = blocks[0].kernel_events, None
        stages = {}
        for name, a, b in ev:
            stages[name] = stages.get(name, 0.0) + a.elapsed_time(b) * 1e3 / 10
        a = sum(active) / len(active)
        nbytes = a * EXPERT_BYTES_W4 + E * H * 2 + 2 * T * H * 2
        gbs = nbytes / (us_graph * 1e-6) / 1e9
        out.append({"T": T, "active_experts": a, "us_per_step_graph": us_graph, "us_per_step_one_call_graph": us_single,
                    "us_per_step_eager": us_eager,
                    "tokens_per_s": T / (us_graph * 1e-6), "algorithmic_mb": nbytes / 1e6, "hbm_gbs": gbs,
                    "hbm_frac": gbs / peaks["hbm_gbs"], "stage_us_eager": stages})
        del graphs, g_all
    for blk in blocks:
        bits = device_status([blk])
        if bits:
            out.append({"invalid": f"device status {bits}"})
    return out


def run_c3(args):
    """W4A16 decode layer on one GPU: the line's value is batch 64; the other batch sizes ride along."""
    from mini_qwen_b200.graph import CapturedForward
    hn = Harness()
    assert hn.world == 1, "workload c3 is a single-GPU workload (c5 is the expert-parallel W4A16 one)"
    dev = hn.dev
    peaks = measured_peaks()
    batches = tuple(int(b) for b in args.decode_batches.split(","))
    table = w4_decode_numbers(dev, peaks, iters=max(args.steps, 50), batches=batches, w4_kernel=args.w4_kernel)
    top = [r for r in table if r.get("T") == max(batches)][0]
    T = top["T"]
    # parity sample and the end-to-end loop on one layer at the largest batch
    blk = w4_block(dev, 100, w4_kernel=args.w4_kernel)
    x = torch.randn(T, H, generator=torch.Generator(device=dev).manual_seed(2), device=dev).to(torch.bfloat16)
    with torch.no_grad():
        out = blk(x)
    rows = min(4, T)
    ok = w4_parity_sample(dev, 100, 1, x[:rows], out[:rows], blk.gate.weight)
    if not ok:
        print("parity sample FAILED: no number is reported", file=sys.stderr)
        sys.exit(3)
    caps = [CapturedForward(blk, x, warmup=2)]
    caps.append(CapturedForward(blk, x, warmup=1, pool=caps[0].pool()))
    x_host = x.cpu().pin_memory()
    e2e_ms, out_bytes = timed_e2e(hn, caps, x_host, max(args.steps, 50), args.warmup)
    e2e_steps = max(args.steps, 50)
    gu_us = top["stage_us_eager"].get("grouped_swiglu")
    roofline = None
    if gu_us:
        gu_bytes = top["active_experts"] * GATE_UP_BYTES_W4 + T * TOPK * (H + I) * 2
        gbs = gu_bytes / (gu_us * 1e-6) / 1e9
        roofline = {"bound": "hbm", "kernel": "W4A16 gate/up + SwiGLU stream kernel", "achieved": gbs,
                    "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                    "peak_source": f"{peaks['source']} copy bandwidth",
                    "traffic": recorded_traffic("w4a16_stream_gate_up_c3_t64") if T == 64 else None,
                    "algorithmic_bytes": gu_bytes, "us_per_launch": gu_us,
                    "layer": {"achieved": top["hbm_gbs"], "frac": top["hbm_frac"], "unit": "GB/s",
                              "algorithmic_bytes": top["algorithmic_mb"] * 1e6, "us_per_step": top["us_per_step_graph"]}}
    cpu_base = None
    if not args.no_cpu_baseline:
        ms, hit = cpu_w4_layer_ms(dev, 100, x.cpu())
        cpu_base = {"value": T / (ms * 1e-3), "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                    "sample": f"3 calls of the per-expert loop on the {T}-token batch ({hit} experts hit, each projection's "
                              "weight dequantised to fp32 once beforehand) after 1 warm-up"}
    line = {
        "metric": METRIC, "value": top["tokens_per_s"], "unit": UNIT, "n_gpus": 1, "steps": max(args.steps, 50),
        "warmup": args.warmup, "ms_per_step": top["us_per_step_graph"] * 1e-3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "w4a16 (int4 weights, bf16 activations, fp32 sums)",
        "data": "synthetic",
        "config": {"workload": f"W4A16 decode MoE layer, batch {T}, H={H} E={E} top{TOPK} I={I}, group {GROUP}",
                   "l2": "steps rotate over 8 independently drawn layers (2.5 GB of weights), so no weight byte is served "
                         "from the 126 MB L2",
                   "parallelism": "single GPU"},
        "roofline": roofline, "cpu_baseline": cpu_base,
        "e2e": {"value": T * e2e_steps / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * 2,
                "d2h_bytes_per_step": out_bytes, "ms_per_step": e2e_ms / e2e_steps,
                "note": "one layer replayed (its weights stay in L2 between steps at small batches); the device-resident "
                        "value rotates layers"},
        "gpu_launches": caps[0].launches * max(args.steps, 50), "clocks": None,
        "parity_sample": "ok", "status": device_status([blk]),
        "launch": "one CUDA graph replay per 8 steps (a call of each of the 8 rotating layers, as a decoder's graph holds "
                  "its layers); w4a16_decode[].us_per_step_one_call_graph is one replay per step",
        "w4a16_decode": table,
    }
    with ClockSampler(hn.local) as clocks:
        for _ in range(200):
            caps[0].replay()
        torch.cuda.synchronize()
    line["clocks"] = clocks.summary()
    print(json.dumps(line))
    hn.close()


def run_c5(args):
    """48 W4A16 layers chained, decode batch, experts sharded over the GPUs."""
    from mini_qwen_b200.graph import CapturedForward
    hn = Harness()
    world, rank, dev = hn.world, hn.rank, hn.dev
    B = args.c5_batch
    assert B % world == 0, f"a batch of {B} tokens does not split over {world} GPUs"
    T = B // world
    blocks = [w4_block(dev, 200 + L, rank, world, hn.group, max_tokens=T, w4_kernel=args.w4_kernel) for L in range(LAYERS)]

    # between the layers: an RMS norm with a weight of ones (the stack has no attention and no learnt norms; without
    # it SwiGLU's quadratic growth overflows within a few layers), on the library's own norm kernel
    from mini_qwen_b200.model.layers import rms_norm
    ones = torch.ones(H, dtype=torch.bfloat16, device=dev)

    def model(x):
        for i, blk in enumerate(blocks):
            x = blk(rms_norm(x, ones, 1e-6) if i else x)
        return x
    x_all = torch.randn(B, H, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    x_cpu = x_all[rank * T:(rank + 1) * T].contiguous()
    x_host, x_dev = x_cpu.pin_memory(), x_cpu.to(dev)

    # parity sample: the first layer's output for this rank's first token(s) against the CPU restatement
    with torch.no_grad():
        first = blocks[0](x_dev)
        final = model(x_dev)
    torch.cuda.synchronize()
    rows = min(2, T)
    sample_ok = w4_parity_sample(dev, 200, world, x_dev[:rows], first[:rows], blocks[0].gate.weight) \
        and bool(torch.isfinite(final.float()).all())
    if not hn.all_ok(sample_ok):
        print(f"rank {rank}: parity sample {'FAILED' if not sample_ok else 'ok'} (a rank failed: no number is reported)",
              file=sys.stderr)
        hn.barrier()
        hn.close()
        sys.exit(3)

    kern_ms = stage_times(hn, model, blocks, x_dev, 2, 3)
    caps = [CapturedForward(model, x_dev, warmup=2)]
    caps.append(CapturedForward(model, x_dev, warmup=1, pool=caps[0].pool()))
    ms_total, launches, clocks = timed_replays(hn, caps[0], args.steps, args.warmup)
    eager_ms = timed_eager(hn, model, x_dev, max(2, args.steps // 4))
    e2e_ms, out_bytes = timed_e2e(hn, caps, x_host, args.steps, args.warmup)
    status = int(hn.max_over_ranks(float(device_status(blocks))))
    # experts hit per layer (this rank's tokens over all experts), for the algorithmic bytes
    from mini_qwen_b200.kernels import moe_router
    if rank != 0:
        hn.close()
        return
    peaks = measured_peaks()
    ms_step = ms_total / args.steps
    # algorithmic bytes of a pass, per GPU: the experts the WHOLE batch hits among this GPU's (expected value for
    # uniform routing: E/world * (1 - (1 - 1/E)^(B*top_k))), their W4A16 tensors, plus router weight and activations
    exp_hit = (E / world) * (1.0 - (1.0 - 1.0 / E) ** (B * TOPK))
    bytes_gpu = LAYERS * (exp_hit * EXPERT_BYTES_W4 + E * H * 2 + 2 * T * H * 2)
    gbs = bytes_gpu / (ms_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "whole 48-layer pass, per GPU (W4A16 stream kernels dominate)",
                "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                "peak_source": f"{peaks['source']} copy bandwidth", "traffic": None,
                "algorithmic_bytes": bytes_gpu, "ms_per_pass": ms_step,
                "note": "expected experts hit per GPU and layer: %.1f of %d" % (exp_hit, E // world)}
    cpu_base = None
    if world == 1 and not args.no_cpu_baseline:
        ms, hit = cpu_w4_layer_ms(dev, 200, x_all)
        cpu_base = {"value": B / (LAYERS * ms * 1e-3), "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                    "sample": f"one of the {LAYERS} layers ({hit} experts hit, weights dequantised to fp32 once beforehand), "
                              f"3 calls after 1 warm-up; a pass is taken as {LAYERS} times that"}
    line = {
        "metric": "moe_stack_tokens_per_s", "value": B * args.steps / (ms_total * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "w4a16 (int4 weights, bf16 activations, fp32 sums)",
        "data": "synthetic",
        "config": {"workload": f"{LAYERS} W4A16 MoE layers chained (weight-free RMS norm between layers), decode batch {B} in "
                               f"total, H={H} E={E} top{TOPK} I={I}, group {GROUP}; tokens/s per full {LAYERS}-layer pass",
                   "l2": f"a pass streams {LAYERS} different layers ({bytes_gpu / 1e9:.2f} GB per GPU): no weight byte is reused "
                         "from L2 between passes",
                   "parallelism": "single GPU" if world == 1 else
                   f"expert parallel ep{world}: {E // world} experts per GPU and layer, {T} token(s) per GPU; every rank "
                   "gathers all tokens over NVLink, routes them, runs its own experts and sends fp32 partial sums to the "
                   "tokens' owners; two flag barriers between the ranks per layer"},
        "roofline": roofline, "cpu_baseline": cpu_base,
        "e2e": {"value": B * args.steps / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * 2,
                "d2h_bytes_per_step": out_bytes, "ms_per_step": e2e_ms / args.steps,
                "pipeline": "upload, compute and download on three streams, two buffers each"},
        "gpu_launches": launches, "clocks": clocks, "parity_sample": "ok", "status": status,
        "launch": f"one CUDA graph per {LAYERS}-layer pass", "eager_ms_per_step": eager_ms, "kernels_ms": kern_ms,
    }
    if status != 0:
        line["invalid"] = "a device status bit is set: the timed steps are not valid"
    print(json.dumps(line))
    hn.close()


# ------------------------------------------------------------------------------------------ reference arm
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count()
    name = args.workload
    if name in ("c2", "c4"):
        lay, bias, desc = dense_setup(name)
        tps, ms = cpu_dense_tokens_per_s(lay, bias, args.steps, args.warmup, T_PREFILL)
        sample = (f"{T_PREFILL}-token slices of the batch, one slice per step" if name == "c4" else
                  f"the {T_PREFILL}-token batch, once per step")
        dtype, scaling, metric = "bf16", ("weak" if name == "c2" else "strong"), METRIC
    else:
        # the W4A16 layers are drawn on a device in the GPU arm; the CPU arm draws the same distributions on the CPU
        dev = torch.device("cpu")
        B = max(int(b) for b in args.decode_batches.split(",")) if name == "c3" else args.c5_batch
        x = torch.randn(B, H, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
        ms, hit = cpu_w4_layer_ms(dev, 200, x, steps=max(1, min(args.steps, 5)), warmup=min(args.warmup, 1))
        layers = 1 if name == "c3" else LAYERS
        tps = B / (layers * ms * 1e-3)
        ms = layers * ms
        desc = (f"W4A16 decode MoE layer, batch {B}, H={H} E={E} top{TOPK} I={I}, group {GROUP}" if name == "c3" else
                f"{LAYERS} W4A16 MoE layers chained, decode batch {B} in total; tokens/s per full {LAYERS}-layer pass")
        sample = (f"per-expert loop over the {hit} experts the batch hits, weights dequantised to fp32 once beforehand "
                  "(the reference's W4A16 kernel needs a GPU)" +
                  ("" if name == "c3" else f"; one layer timed, a pass taken as {LAYERS} times that"))
        dtype, scaling = "w4a16 (fp32 dequantised weights on the CPU)", ("weak" if name == "c3" else "strong")
        metric = METRIC if name == "c3" else "moe_stack_tokens_per_s"
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": tps, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": {"workload": desc, "sample": sample,
                   "parallelism": "reference per-expert loop (CPU restatement) on the host cores of rank 0"},
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c4", "c5"])
    ap.add_argument("--c5-batch", type=int, default=16, help="decode batch of workload c5 (8 or 16)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="c2: skip the W4A16 decode numbers")
    ap.add_argument("--decode-only", action="store_true",
                    help="only the W4A16 decode table (small profiling runs); prints its JSON list")
    ap.add_argument("--decode-iters", type=int, default=200)
    ap.add_argument("--decode-batches", default="1,8,16,64")
    ap.add_argument("--w4-kernel", default=None, choices=["stream", "auto", "tc", "mma"],
                    help="W4A16 kernels of the decode numbers (default: the block's own choice)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.decode_only:
        assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        batches = tuple(int(b) for b in args.decode_batches.split(","))
        print(json.dumps({"w4a16_decode": w4_decode_numbers(dev, measured_peaks(), iters=args.decode_iters,
                                                            batches=batches, w4_kernel=args.w4_kernel)}))
    elif args.workload in ("c2", "c4"):
        run_dense(args, args.workload)
    elif args.workload == "c3":
        run_c3(args)
    else:
        run_c5(args)


if __name__ == "__main__":
    main()
