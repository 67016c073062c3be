"""Generates the golden vectors under tests/golden/ by running the REFERENCE implementation
(mini-qwen-llm's own PyTorch per-expert-loop path, imported unmodified) on seeded inputs.

Run where the reference checkout is available:
    python tests/golden/make_golden.py --reference /path/to/mini-qwen-llm
The inputs are not stored: tests regenerate them from the same seeds (mini_qwen_b200.synthetic
and the helpers in tests/cases.py), so only the reference's outputs are committed.
bf16 tensors are stored as their raw 16-bit patterns (int16).
"""
from __future__ import annotations

import argparse
import os
import sys
import time
from types import SimpleNamespace

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "mini-qwen-llm_b200"))
sys.path.insert(0, os.path.join(ROOT, "tests"))

import cases  # noqa: E402  (tests/cases.py)


def bits(t: torch.Tensor) -> np.ndarray:
    """Storable numpy form of a tensor (bf16 as raw int16 bit patterns)."""
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy()
    return t.contiguous().numpy()


def ref_block(ref, cfg, router, gate, up, down, dtype):
    """The reference's Qwen3MoEBlock holding the given dense weights."""
    blk = ref.moe.Qwen3MoEBlock(cfg).to(dtype)
    blk.gate.weight.data = router.clone()
    for e, ex in enumerate(blk.experts):
        ex.gate_proj.weight.data = gate[e]
        ex.up_proj.weight.data = up[e]
        ex.down_proj.weight.data = down[e]
    return blk


class DequantisedLinear(nn.Module):
    """Stands in for the reference's LinearW4A16 on CPU (its Triton kernel needs CUDA): the same
    buffers, multiplied out in fp32 by the formula of the reference's tests/test_w4a16_gemm.py:19-44,
    result rounded to bf16 as LinearW4A16.forward returns bf16."""

    def __init__(self, ref, layer):
        super().__init__()
        unpack = ref.packing.unpack_int4
        g = layer.group_size
        q = unpack(layer.qweight.T.contiguous()).T.float()
        z = unpack(layer.qzeros).float().repeat_interleave(g, 0)
        s = layer.scales.float().repeat_interleave(g, 0)
        self.w = (q - z) * s

    def forward(self, x):
        return (x.float() @ self.w).to(torch.bfloat16)


def run_dense(ref, name, lay, norm=True, bias=None, sample_rows=None):
    T, H = lay.x.shape
    E, I = lay.gate.shape[0], lay.gate.shape[1]
    cfg = SimpleNamespace(hidden_size=H, intermediate_size=I, num_experts=E,
                          num_experts_per_tok=lay.top_k, norm_topk_prob=norm)
    blk = ref_block(ref, cfg, lay.router, lay.gate, lay.up, lay.down, lay.x.dtype)
    if bias is not None:
        # the reference router has no bias: its three lines (moe_router.py:19-21) plus the bias add
        def biased_router(hs, rw, top_k=8):
            scores = F.softmax(F.linear(hs.float(), rw.float()) + bias, dim=-1)
            w, i = torch.topk(scores, top_k, dim=-1)
            return i, w
        ref.moe.moe_router = biased_router
        route = biased_router
    else:
        route = ref.router.moe_router
    with torch.no_grad():
        ids, wts = route(lay.x, lay.router, lay.top_k)
        _, off = ref.permute.moe_permute(lay.x, ids, E)
        out = blk(lay.x)
    if bias is not None:
        ref.moe.moe_router = ref.router.moe_router
    rec = {"ids": ids.numpy().astype(np.uint8 if E <= 256 else np.int32), "weights": wts.numpy(),
           "offsets": off.numpy()}
    rows = slice(None) if sample_rows is None else slice(0, sample_rows)
    rec["out"] = bits(out[rows])
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
    return ids, off


def run_w4(ref, name, lay, Ts):
    T, H = lay.x.shape
    E = lay.router.shape[0]
    I = lay.gate.qweight.shape[2]
    cfg = SimpleNamespace(hidden_size=8, intermediate_size=8, num_experts=E,
                          num_experts_per_tok=lay.top_k, norm_topk_prob=True)
    blk = ref.moe.Qwen3MoEBlock(cfg).to(torch.bfloat16)   # tiny dense skeleton, projections replaced below
    # the reference loader casts the dense router to bf16 (model/loader.py:253-259)
    blk.gate.weight.data = lay.router.to(torch.bfloat16)
    from_gptq = ref.linear_w4a16.LinearW4A16.from_gptq
    for e, ex in enumerate(blk.experts):
        for pname, p in (("gate_proj", lay.gate), ("up_proj", lay.up), ("down_proj", lay.down)):
            layer = from_gptq(p.qweight[e], p.qzeros[e], p.scales[e], lay.group_size, zero_plus_one=True)
            setattr(ex, pname, DequantisedLinear(ref, layer))
    rec = {}
    with torch.no_grad():
        for t in Ts:
            x = lay.x[:t]
            ids, wts = ref.router.moe_router(x, blk.gate.weight, lay.top_k)
            _, off = ref.permute.moe_permute(x, ids, E)
            out = blk(x)
            rec[f"ids_T{t}"] = ids.numpy().astype(np.uint8)
            rec[f"weights_T{t}"] = wts.numpy()
            rec[f"offsets_T{t}"] = off.numpy()
            rec[f"out_T{t}"] = bits(out)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a mini-qwen-llm checkout (the reference)")
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import mini_qwen.kernels.moe_permute as r_permute
    import mini_qwen.kernels.moe_router as r_router
    import mini_qwen.kernels.moe_unpermute as r_unpermute
    import mini_qwen.kernels.moe_grouped_gemm as r_gg
    import mini_qwen.model.layers.linear_w4a16 as r_lin
    import mini_qwen.model.layers.moe as r_moe
    import mini_qwen.quantization.awq as r_awq
    import mini_qwen.quantization.packing as r_packing
    ref = SimpleNamespace(router=r_router, permute=r_permute, unpermute=r_unpermute, gg=r_gg, moe=r_moe,
                          linear_w4a16=r_lin, packing=r_packing, awq=r_awq)
    torch.set_num_threads(os.cpu_count())
    want = lambda n: (not args.only) or n in args.only.split(",")

    if want("script"):
        # the five cases of the reference's scripts/test_moe_synthetic.py:106-133, its own generator
        rec = {}
        for i, c in enumerate(cases.SCRIPT_CASES):
            x, gate_w, gw, uw, dw = cases.script_case_inputs(c)
            ids, w = r_router.moe_router(x, gate_w, c["K"])
            if c["norm"]:
                w = w / w.sum(dim=-1, keepdim=True)
            permuted, off = r_permute.moe_permute(x, ids, c["E"])
            out_perm = torch.zeros_like(permuted)
            for e in range(c["E"]):
                s, t = off[e].item(), off[e + 1].item()
                if s == t:
                    continue
                xe = permuted[s:t]
                out_perm[s:t] = F.linear(F.silu(F.linear(xe, gw[e])) * F.linear(xe, uw[e]), dw[e])
            out = r_unpermute.moe_unpermute(out_perm, w, ids, c["T"])
            rec[f"ids_{i}"], rec[f"weights_{i}"] = ids.numpy(), w.numpy()
            rec[f"offsets_{i}"], rec[f"permuted_{i}"] = off.numpy(), bits(permuted)
            rec[f"out_{i}"] = bits(out)
        np.savez_compressed(os.path.join(HERE, "script_cases.npz"), **rec)
        print("script_cases done")

    if want("kernels"):
        # shapes and seeds of the reference's tests/test_moe_kernels.py (run there on CUDA only)
        rec = {}
        for i, (T, E, K, H, D) in enumerate(cases.KERNEL_SHAPES):
            hidden, router_w = cases.kernel_router_inputs(T, E, K, H)
            ids, w = r_router.moe_router(hidden, router_w, top_k=K)
            rec[f"router_ids_{i}"], rec[f"router_w_{i}"] = ids.numpy(), w.numpy()
            permuted, off = r_permute.moe_permute(hidden, ids, E)
            rec[f"permute_off_{i}"] = off.numpy()
            xg, wg = cases.kernel_gemm_inputs(T, E, K, H, D)
            rec[f"gemm_out_{i}"] = bits(r_gg._moe_grouped_gemm_oracle(permuted, wg, off))
        np.savez_compressed(os.path.join(HERE, "kernel_cases.npz"), **rec)
        print("kernel_cases done")

    if want("quant"):
        rec = {}
        for i, (M, K, N, g) in enumerate(cases.W4_GEMM_SHAPES):
            x, w = cases.w4_gemm_inputs(M, K, N)
            qw, sc, qz = r_awq._per_group_minmax_quantize(w, g)
            lin = DequantisedLinear(ref, SimpleNamespace(qweight=qw, scales=sc, qzeros=qz, group_size=g))
            rec[f"qweight_sum_{i}"] = np.array([int(qw.to(torch.int64).sum())])
            rec[f"out_{i}"] = bits((x.double() @ lin.w.double()).to(torch.bfloat16))
        # from_gptq zero fix-up on every stored nibble value
        stored = r_packing.pack_int4(torch.arange(16, dtype=torch.int32).reshape(1, 16))
        layer = r_lin.LinearW4A16.from_gptq(torch.zeros(16, 16, dtype=torch.int32), stored,
                                            torch.ones(1, 16) * 0.0123, group_size=128)
        rec["gptq_zeros"] = layer.qzeros.numpy()
        rec["gptq_scales"] = bits(layer.scales)
        np.savez_compressed(os.path.join(HERE, "quant_cases.npz"), **rec)
        print("quant_cases done")

    if want("glue"):
        # post-attention RMSNorm -> MoE block -> residual add, as the reference's decoder layer does it
        import mini_qwen.model.layers.rms_norm as r_norm
        rec = {}
        for i, c in enumerate(cases.GLUE_CASES):
            lay, h, norm_w = cases.glue_case_inputs(c)
            cfg = SimpleNamespace(hidden_size=c["H"], intermediate_size=c["I"], num_experts=c["E"],
                                  num_experts_per_tok=c["K"], norm_topk_prob=True)
            blk = ref_block(ref, cfg, lay.router, lay.gate, lay.up, lay.down, c["dtype"])
            norm = r_norm.RMSNorm(c["H"], eps=c["eps"]).to(c["dtype"])
            norm.weight.data = norm_w.clone()
            with torch.no_grad():
                xn = norm(h)
                ids, _ = r_router.moe_router(xn, lay.router, c["K"])
                out = h + blk(xn)
            rec[f"normed_{i}"], rec[f"ids_{i}"], rec[f"out_{i}"] = bits(xn), ids.numpy(), bits(out)
        np.savez_compressed(os.path.join(HERE, "glue_cases.npz"), **rec)
        print("glue_cases done")

    if want("c1"):
        run_dense(ref, "c1", cases.config1())
        print("c1 done")
    if want("c3"):
        t0 = time.time()
        run_w4(ref, "c3", cases.config3(), cases.C3_TS)
        print("c3 done", time.time() - t0)
    if want("c2"):
        t0 = time.time()
        run_dense(ref, "c2", cases.config2(), sample_rows=cases.C2_SAMPLE_ROWS)
        print("c2 done", time.time() - t0)
    if want("c4"):
        t0 = time.time()
        lay = cases.config4()
        ids, off = run_dense(ref, "c4", lay, bias=cases.config4_bias(), sample_rows=cases.C4_SAMPLE_ROWS)
        counts = (off[1:] - off[:-1])
        print("c4 done", time.time() - t0, "empty experts:", int((counts == 0).sum()), "max:", int(counts.max()))


if __name__ == "__main__":
    main()
