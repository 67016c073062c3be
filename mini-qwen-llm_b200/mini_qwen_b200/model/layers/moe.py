"""Qwen3 MoE FFN block with the module tree and interface of the reference's
``mini_qwen/model/layers/moe.py:28-78`` (``gate``, ``experts[e].{gate,up,down}_proj``,
``forward``, ``quantize_to_w4a16``), executed as a fixed chain of grouped kernels instead of a
Python loop over experts.

The per-expert modules stay the owners of the weights as far as ``state_dict`` /
``load_state_dict`` / ``set_submodule`` are concerned.  Before the first forward (or when
:meth:`finalize` is called) their tensors are gathered once into expert-major stacks and the
module tensors are re-pointed at views of those stacks, so nothing is stored twice and in-place
loads keep working.  Replacing an expert projection module, or moving the block to another
device or dtype, invalidates the stacks; the next forward rebuilds them.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ...kernels.moe_grouped_gemm import (gather_swiglu_supported, moe_grouped_gemm, moe_grouped_gemm_scatter,
                                          moe_grouped_swiglu, moe_grouped_swiglu_gather, scatter_gemm_supported)
from ...kernels.moe_permute import gather_rows, moe_permute_plan
from ...kernels.moe_router import moe_route_small, moe_router, route_small_supported, route_small_workspace
from ...kernels.moe_unpermute import unpermute_combine
from .rms_norm import RMSNorm
from ...kernels.w4a16_gemm import (w4a16_grouped_gemm, w4a16_grouped_swiglu, w4a16_stream_supported,
                                     w4a16_stream_swiglu, w4a16_tc_gemm, w4a16_tc_prep, w4a16_tc_supported,
                                     w4a16_tc_swiglu)
from ... import parallel
from .linear_w4a16 import LinearW4A16

_PROJ = ("gate_proj", "up_proj", "down_proj")


class _ExpertMLP(nn.Module):
    """SwiGLU MLP of one expert; names match HF ``experts[e].gate_proj / up_proj / down_proj``."""

    def __init__(self, config, epoch: list):
        super().__init__()
        object.__setattr__(self, "_epoch", epoch)      # shared counter, not a submodule/buffer
        self.gate_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.up_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.down_proj = nn.Linear(config.intermediate_size, config.hidden_size, bias=False)

    def __setattr__(self, name, value):
        if name in _PROJ:
            self._epoch[0] += 1                        # a projection was swapped: stacks are stale
        super().__setattr__(name, value)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Single-expert path (kept for callers that address one expert; the block does not use it)."""
        return self.down_proj(nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


class Qwen3MoEBlock(nn.Module):
    """router -> permute -> grouped gate/up + SwiGLU -> grouped down -> weighted combine.

    With ``ep_group`` (a ``torch.distributed`` process group of G ranks) the block is expert
    parallel: it holds only the ``num_experts / G`` experts of its rank (``experts[j]`` is global
    expert ``expert_offset + j``), routes its own tokens over all experts, and exchanges rows with
    the other ranks in one all-to-all each way (see ``mini_qwen_b200.parallel``).
    """

    def __init__(self, config, ep_group=None, ep_mode: str = "p2p", ep_max_tokens: int | None = None):
        super().__init__()
        self.num_experts = config.num_experts
        self.num_experts_per_tok = config.num_experts_per_tok
        self.norm_topk_prob = getattr(config, "norm_topk_prob", True)
        self._epoch = [0]
        self._stacked_epoch = -1
        self._stacks = None
        self.ep_group = ep_group
        # "p2p": dispatch/combine fused into the permute/unpermute kernels over peer memory (CUDA only);
        # "nccl": materialise, then torch.distributed all-to-all (any backend; one host sync per call)
        self.ep_mode = ep_mode
        self.ep_max_tokens = ep_max_tokens     # most tokens per rank and call (sizes the peer buffers)
        # "fused": the down projection writes its rows into the source ranks' buffers itself;
        # "pull": the combine kernel reads them from the owners (the only way for W4A16 experts)
        self.ep_return = "fused"
        # "unique": a token row crosses NVLink once per destination rank and the owner's gate/up kernel
        # gathers through a slot table; "slots": one copy per slot (W4A16 experts, more than 8 ranks)
        self.ep_dispatch = "unique"
        # W4A16 experts: "stream" = activations prepared once (rows gathered in the k order the MMA wants, group
        # sums), gate/up on the TMA-staged stream kernel, down on the cp.async kernel (the default);
        # "mma" = both projections on the cp.async kernel from materialised rows; "tc" = the tcgen05 kernel
        # with the weights dequantised into tensor memory; "auto" = "tc" by the number of slots per expert
        self.w4_kernel = "stream"
        # the stream kernel's activations as row-scaled fp16 (exact up to elements 2^28 times smaller than their
        # row's largest): its weights then unpack with five instead of seven integer instructions per word.
        # Measured: the same output bits and 1 % less time in the gate/up kernel, nothing on the layer call; off.
        self.w4_rows_f16 = False
        # small batches (up to 64 tokens): router, top-k, permute plan (and, on one GPU, the W4A16 activation
        # preparation) as ONE launch instead of three or four; same ids and plan, weights equal up to the order of
        # the fp32 logit sums
        self.fuse_small_batches = True
        self.fuse_max_tokens = 64
        # expert-parallel W4A16 decode batches (at most 64 tokens over all ranks): "replicate" = every rank holds
        # all tokens and runs its own experts (two rank barriers per call), "dispatch" = the prefill path
        self.ep_decode = "replicate"
        self._route_ws = None
        self._peer = None
        self.ep_size = 1 if ep_group is None else torch.distributed.get_world_size(ep_group)
        self.ep_rank = 0 if ep_group is None else torch.distributed.get_rank(ep_group)
        if self.num_experts % self.ep_size != 0:
            raise ValueError(f"{self.num_experts} experts do not shard evenly over {self.ep_size} ranks")
        self.num_local_experts = self.num_experts // self.ep_size
        self.expert_offset = self.ep_rank * self.num_local_experts
        self.gate = nn.Linear(config.hidden_size, config.num_experts, bias=False)
        self.experts = nn.ModuleList([_ExpertMLP(config, self._epoch) for _ in range(self.num_local_experts)])
        self.router_bias = None       # optional fp32 [E] logit bias (not in the reference)
        self._status = None
        self.kernel_events = None     # set to a list to collect (stage, start, end) CUDA events per forward

    # ------------------------------------------------------------------ weight stacks
    def _apply(self, fn, *args, **kwargs):
        self._epoch[0] += 1           # .to()/.cuda()/.half() re-create the parameter storage
        return super()._apply(fn, *args, **kwargs)

    def _sentinel(self):
        first, last = self.experts[0].gate_proj, self.experts[-1].down_proj
        a = first.qweight if isinstance(first, LinearW4A16) else first.weight
        b = last.qweight if isinstance(last, LinearW4A16) else last.weight
        return (a.data_ptr(), b.data_ptr())

    def finalize(self) -> None:
        """Gather the per-expert tensors into expert-major stacks (idempotent)."""
        kinds = {isinstance(getattr(ex, p), LinearW4A16) for ex in self.experts for p in _PROJ}
        if len(kinds) != 1:
            raise ValueError("experts mix nn.Linear and LinearW4A16 projections; quantise all or none")
        quantised = kinds.pop()
        with torch.no_grad():
            if quantised:
                stacks = {"w4": True}
                groups = {getattr(ex, p).group_size for ex in self.experts for p in _PROJ}
                if len(groups) != 1:
                    raise ValueError("all expert projections must share one group_size")
                stacks["group_size"] = groups.pop()
                for p in _PROJ:
                    mods = [getattr(ex, p) for ex in self.experts]
                    trio = []
                    for buf in ("qweight", "scales", "qzeros"):
                        st = torch.stack([getattr(m, buf) for m in mods]).contiguous()
                        for e, m in enumerate(mods):
                            m._buffers[buf] = st[e]
                        trio.append(st)
                    stacks[p] = tuple(trio)
            else:
                stacks = {"w4": False}
                g = [ex.gate_proj.weight for ex in self.experts]
                u = [ex.up_proj.weight for ex in self.experts]
                d = [ex.down_proj.weight for ex in self.experts]
                inter = g[0].shape[0]
                w13 = torch.cat([torch.stack([w.data for w in g]), torch.stack([w.data for w in u])], dim=1).contiguous()
                w2 = torch.stack([w.data for w in d]).contiguous()
                for e, ex in enumerate(self.experts):
                    ex.gate_proj.weight.data = w13[e, :inter]
                    ex.up_proj.weight.data = w13[e, inter:]
                    ex.down_proj.weight.data = w2[e]
                stacks["w13"], stacks["w2"] = w13, w2
        self._stacks = stacks
        self._stacked_epoch = self._epoch[0]
        self._stacked_sentinel = self._sentinel()

    @classmethod
    def from_stacked(cls, config, router_weight: torch.Tensor, gate_up_proj: torch.Tensor,
                     down_proj: torch.Tensor, ep_group=None, ep_mode: str = "p2p",
                     ep_max_tokens: int | None = None) -> "Qwen3MoEBlock":
        """Builds a dense block from expert-major tensors without copying them:
        ``router_weight`` [E, H], ``gate_up_proj`` [E, 2I, H] (gate rows, then up rows: the fused
        layout of HF Qwen3-MoE checkpoints), ``down_proj`` [E, H, I].  The per-expert modules become
        views of the given tensors.  With ``ep_group`` the expert tensors hold this rank's experts
        only (``num_experts / G`` of them); the router weight always covers all experts."""
        E, I2, H = gate_up_proj.shape
        with torch.device("meta"):
            blk = cls(config, ep_group=ep_group, ep_mode=ep_mode, ep_max_tokens=ep_max_tokens)
        assert E == blk.num_local_experts and I2 == 2 * config.intermediate_size and H == config.hidden_size
        assert tuple(down_proj.shape) == (E, H, I2 // 2)
        assert tuple(router_weight.shape) == (config.num_experts, H)
        w13, w2 = gate_up_proj.contiguous(), down_proj.contiguous()
        blk.gate.weight = nn.Parameter(router_weight, requires_grad=False)
        inter = I2 // 2
        for e, ex in enumerate(blk.experts):
            ex.gate_proj.weight = nn.Parameter(w13[e, :inter], requires_grad=False)
            ex.up_proj.weight = nn.Parameter(w13[e, inter:], requires_grad=False)
            ex.down_proj.weight = nn.Parameter(w2[e], requires_grad=False)
        blk._stacks = {"w4": False, "w13": w13, "w2": w2}
        blk._stacked_epoch = blk._epoch[0]
        blk._stacked_sentinel = blk._sentinel()
        return blk

    @classmethod
    def from_stacked_w4(cls, config, router_weight: torch.Tensor, gate, up, down, group_size: int = 128,
                        ep_group=None, ep_mode: str = "p2p", ep_max_tokens: int | None = None) -> "Qwen3MoEBlock":
        """Builds a W4A16 block from expert-major stacks without copying them.  ``gate``, ``up`` and ``down``
        are ``(qweight [E, K/8, N] int32, scales [E, K/g, N] bf16, qzeros [E, K/g, N/8] int32)`` in the
        convention of the module buffers, i.e. what ``LinearW4A16.from_gptq`` stores (bf16 scales, zero
        points already incremented and clamped).  The per-expert ``LinearW4A16`` modules become views of the
        stacks.  With ``ep_group`` the stacks hold this rank's experts only; the router weight covers all."""
        with torch.device("meta"):
            blk = cls(config, ep_group=ep_group, ep_mode=ep_mode, ep_max_tokens=ep_max_tokens)
        E = blk.num_local_experts
        H, I = config.hidden_size, config.intermediate_size
        shapes = {"gate_proj": (H, I), "up_proj": (H, I), "down_proj": (I, H)}
        stacks = {"w4": True, "group_size": group_size}
        for name, trio in (("gate_proj", gate), ("up_proj", up), ("down_proj", down)):
            kd, n = shapes[name]
            qw, sc, qz = (t.contiguous() for t in trio)
            assert tuple(qw.shape) == (E, kd // 8, n) and qw.dtype == torch.int32, f"{name}: qweight {tuple(qw.shape)}"
            assert tuple(sc.shape) == (E, kd // group_size, n) and sc.dtype == torch.bfloat16, f"{name}: scales"
            assert tuple(qz.shape) == (E, kd // group_size, n // 8) and qz.dtype == torch.int32, f"{name}: qzeros"
            stacks[name] = (qw, sc, qz)
        assert tuple(router_weight.shape) == (config.num_experts, H)
        blk.gate.weight = nn.Parameter(router_weight, requires_grad=False)
        for e, ex in enumerate(blk.experts):
            for name, (kd, n) in shapes.items():
                with torch.device("meta"):
                    lin = LinearW4A16(kd, n, group_size)
                for buf, st in zip(("qweight", "scales", "qzeros"), stacks[name]):
                    lin._buffers[buf] = st[e]
                setattr(ex, name, lin)
        blk._stacks = stacks
        blk._stacked_epoch = blk._epoch[0]
        blk._stacked_sentinel = blk._sentinel()
        return blk

    def _ready(self):
        if (self._stacks is None or self._stacked_epoch != self._epoch[0]
                or self._stacked_sentinel != self._sentinel()):
            self.finalize()
        return self._stacks

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """The block on ``x`` [..., H].  With ``residual`` (same shape and dtype) the result is
        ``residual + block(x)``, the add done by the combine kernel as an add of two model-dtype tensors."""
        shape = x.shape
        x2d = x.reshape(-1, shape[-1])
        if not x2d.is_contiguous():
            x2d = x2d.contiguous()
        T = x2d.shape[0]
        res = None
        if residual is not None:
            if residual.shape != x.shape or residual.dtype != x.dtype:
                raise ValueError("residual must have the shape and dtype of the block's input")
            res = residual.reshape(-1, shape[-1]).contiguous()
        K, E = self.num_experts_per_tok, self.num_experts
        st = self._ready()

        run = self._stage
        xp_tok = xs_tok = None
        if self._replicated_decode(st, x2d, T, E, K):
            return self._forward_replicated(x2d, st, T, K, E, res).reshape(shape)
        if self.fuse_small_batches and 0 < T <= self.fuse_max_tokens and route_small_supported(T, E, K):
            # decode batches: logits, top-k, plan and (one GPU) the W4A16 activation preparation in one launch
            prepare = (self.ep_size == 1 and st["w4"] and x2d.dtype == torch.bfloat16 and self._w4_stream(st)
                       and T <= E)
            if self._route_ws is None or self._route_ws.device != x2d.device:
                self._route_ws = route_small_workspace(E, x2d.device)     # zero-filled once, reused by every call
            if prepare and self.w4_rows_f16 and x2d.shape[1] <= 3968:
                prepare = "f16"
            ids32, weights, perm, inv, off32, xp_tok, xs_tok = run(
                "route_small", moe_route_small, x2d, self.gate.weight, K, bias=self.router_bias,
                renormalize=self.norm_topk_prob, prepare=prepare, workspace=self._route_ws)
        else:
            _, weights, ids32 = run("router", moe_router, x2d, self.gate.weight, K, bias=self.router_bias,
                                    renormalize=self.norm_topk_prob, return_int32_ids=True)
            perm, inv, off32, _ = run("permute_plan", moe_permute_plan, ids32, E, want_int64_offsets=False)
        if self.ep_size > 1 and self.ep_mode == "p2p":
            return self._forward_peer(x2d, st, weights, ids32, perm, inv, off32, T, K, E, res).reshape(shape)
        if self.ep_size == 1 and not st["w4"] and gather_swiglu_supported(x2d, st["w13"]):
            # the gate/up kernel fetches the rows through the permutation itself: no permuted copy
            status = self._status_word(x2d.device)
            h = run("grouped_swiglu", moe_grouped_swiglu_gather, x2d, perm, K, st["w13"], off32, status=status)
            out_perm = run("grouped_down", moe_grouped_gemm, h, st["w2"], off32, zero_init=False, status=status)
            return run("unpermute_combine", unpermute_combine, out_perm, weights, inv, T, K, residual=res).reshape(shape)
        if self.ep_size == 1 and st["w4"] and self._w4_stream(st):
            # decode path: one preparation launch replaces the row gather, the gate/up kernel then needs no byte
            # permutes and no extra MMAs for the group sums
            status = self._status_word(x2d.device)
            if xp_tok is not None:
                # prepared per token by the routing launch: the gate/up kernel gathers through the permutation
                h = run("grouped_swiglu", w4a16_stream_swiglu, xp_tok, xs_tok, st["gate_proj"], st["up_proj"], off32,
                        st["group_size"], shuffle_out=False, status=status, perm=perm, top_k=K)
            else:
                xp, xs = run("w4_prep", w4a16_tc_prep, x2d, perm, K,
                             f16=self.w4_rows_f16 and x2d.shape[1] <= 3968)
                h = run("grouped_swiglu", w4a16_stream_swiglu, xp, xs, st["gate_proj"], st["up_proj"], off32,
                        st["group_size"], shuffle_out=False, status=status)
            out_perm = run("grouped_down", w4a16_grouped_gemm, h, *st["down_proj"], off32, st["group_size"],
                           zero_init=False)
            return run("unpermute_combine", unpermute_combine, out_perm, weights, inv, T, K, residual=res).reshape(shape)
        if self.ep_size == 1 and st["w4"] and self._w4_tc(st, T * K):
            # decode-size groups: weights dequantised into tensor memory, activations prepared once
            status = self._status_word(x2d.device)
            xp, xs = run("w4_prep", w4a16_tc_prep, x2d, perm, K)
            out_perm = self._experts_w4_tc(st, xp, xs, off32, status)
            return run("unpermute_combine", unpermute_combine, out_perm, weights, inv, T, K, residual=res).reshape(shape)
        plan = None
        if self.ep_size > 1:
            all_counts = parallel.gather_counts(off32[1:] - off32[:-1], self.ep_group)
        permuted = run("gather_rows", gather_rows, x2d, perm, K)
        if self.ep_size > 1:
            plan = parallel.make_plan(all_counts, self.ep_rank)
            permuted = run("dispatch", parallel.dispatch, permuted, plan, self.ep_group)
            off32 = plan.seg_offsets
        out_perm = self._experts(st, permuted, off32)
        if plan is not None:
            out_perm = run("combine", parallel.combine, out_perm, plan, self.ep_group)
        out = run("unpermute_combine", unpermute_combine, out_perm, weights, inv, T, K, residual=res)
        return out.reshape(shape)

    def half_layer(self, h: torch.Tensor, norm: "RMSNorm") -> torch.Tensor:
        """Second half of the reference's MoE decoder layer (``mini_qwen/model/qwen3_moe.py:63-66``):
        ``h + self(norm(h))`` with ``norm`` the layer's post-attention RMSNorm; the add runs in the combine kernel."""
        return self.forward(norm(h), residual=h)

    def _experts(self, st, rows, off32, out=None):
        """Grouped gate/up + SwiGLU and down projection over rows grouped by `off32`."""
        run = self._stage
        # the groups of a routing cover every row that is read later, so no output needs a zero fill
        if st["w4"]:
            h = run("grouped_swiglu", w4a16_grouped_swiglu, rows, st["gate_proj"], st["up_proj"], off32,
                    st["group_size"], zero_init=False)
            return run("grouped_down", w4a16_grouped_gemm, h, *st["down_proj"], off32, st["group_size"],
                       zero_init=False, out=out)
        status = self._status_word(rows.device)
        h = run("grouped_swiglu", moe_grouped_swiglu, rows, st["w13"], off32, zero_init=False, status=status)
        return run("grouped_down", moe_grouped_gemm, h, st["w2"], off32, zero_init=False, out=out, status=status)

    def _w4_stream(self, st) -> bool:
        """Whether the prepared-activation path applies (``w4_kernel == "stream"`` and the shapes are covered)."""
        if self.w4_kernel != "stream":
            return False
        H = st["gate_proj"][0].shape[1] * 8
        I = st["gate_proj"][0].shape[2]
        return w4a16_stream_supported(H, I, st["group_size"], self.num_local_experts)

    def _w4_tc(self, st, slots: int) -> bool:
        """Whether the W4A16 projections run on the tensor-memory kernel (``w4_kernel``: "auto", "tc", "mma")."""
        if self.w4_kernel in ("mma", "stream"):
            return False
        H = st["gate_proj"][0].shape[1] * 8
        I = st["gate_proj"][0].shape[2]
        ok = w4a16_tc_supported(H, I, st["group_size"]) and w4a16_tc_supported(I, H, st["group_size"])
        if self.w4_kernel == "tc":
            return ok
        # tuned for groups of at most 32 rows: decode batches
        return ok and slots <= 32 * st["gate_proj"][0].shape[0]

    def _experts_w4_tc(self, st, xp, xs, off32, status, out=None):
        run = self._stage
        h = run("grouped_swiglu", w4a16_tc_swiglu, xp, xs, st["gate_proj"], st["up_proj"], off32, st["group_size"],
                status=status)
        _, xs2 = run("w4_sums", w4a16_tc_prep, h, shuffle=False, want_rows=False)
        return run("grouped_down", w4a16_tc_gemm, h, xs2, *st["down_proj"], off32, st["group_size"], status=status,
                   out=out)

    def _status_word(self, device) -> torch.Tensor:
        """Device status word of this block's kernels (bit 0: a bounded wait expired); allocated once."""
        if self._status is None or self._status.device != device:
            self._status = torch.zeros(1, dtype=torch.int32, device=device)
        return self._status

    def check_status(self) -> None:
        """Raises if a kernel of this block reported a device-side error (synchronises)."""
        if self._status is not None and int(self._status.item()) & 1:
            raise RuntimeError("a bounded wait expired inside a grouped GEMM kernel; the last output is invalid")
        if self._peer is not None:
            self._peer.check_status()

    def _ensure_peer(self, x2d, T, K):
        if self._peer is None:
            max_t = self.ep_max_tokens or T
            self._peer = parallel.PeerExchange(self.ep_group, x2d.device, self.ep_size * max_t * K, x2d.shape[1],
                                               x2d.dtype)
            self.ep_max_tokens = max_t
        peer = self._peer
        if T > self.ep_max_tokens or x2d.dtype != peer.dtype:
            raise ValueError(f"expert-parallel buffers were sized for {self.ep_max_tokens} tokens of {peer.dtype} per "
                             f"rank; got {T} of {x2d.dtype} (pass ep_max_tokens at construction)")
        return peer

    def _replicated_decode(self, st, x2d, T, E, K) -> bool:
        """Decode batches of an expert-parallel W4A16 block go by replication (``ep_decode = "replicate"``): every
        rank holds all G*T tokens, runs its own experts and sends partial sums; see ``_forward_replicated``."""
        B = self.ep_size * T
        return (self.ep_size > 1 and self.ep_mode == "p2p" and self.ep_decode == "replicate" and st["w4"]
                and x2d.dtype == torch.bfloat16 and self._w4_stream(st) and 0 < B <= self.fuse_max_tokens
                and B <= E and route_small_supported(B, E, K) and K >= 2)

    def _forward_replicated(self, x2d, st, T, K, E, res=None):
        """Expert parallelism for decode batches: all-gather the step's tokens (a few rows), route them on every
        rank (same kernel, same bytes: same plan everywhere), run this rank's experts on the slots they own, send
        every token's partial weighted sum to the rank that owns the token, add the partial sums up in rank order.
        Two rank barriers per call instead of four, and each rank streams only its own experts' weights.  Every
        rank must call with the same number of tokens.  Outputs equal the dispatch path's up to the order of the
        fp32 sums of the combine."""
        run = self._stage
        peer = self._ensure_peer(x2d, T, K)
        G, el = self.ep_size, E // self.ep_size
        x_all = run("gather_tokens", peer.gather_tokens, x2d)                        # [G*T, H], barrier inside
        if self._route_ws is None or self._route_ws.device != x2d.device:
            self._route_ws = route_small_workspace(E, x2d.device)
        prepare = "f16" if (self.w4_rows_f16 and x2d.shape[1] <= 3968) else True
        ids32, weights, perm, inv, off32, xp_tok, xs_tok = run(
            "route_small", moe_route_small, x_all, self.gate.weight, K, bias=self.router_bias,
            renormalize=self.norm_topk_prob, prepare=prepare, workspace=self._route_ws)
        # this rank's experts: the offsets from its first expert on; rows keep their positions in the sorted order
        off_local = off32[self.ep_rank * el: self.ep_rank * el + el + 1]
        status = self._status_word(x2d.device)
        h = run("grouped_swiglu", w4a16_stream_swiglu, xp_tok, xs_tok, st["gate_proj"], st["up_proj"], off_local,
                st["group_size"], shuffle_out=False, status=status, perm=perm, top_k=K)
        out_perm = run("grouped_down", w4a16_grouped_gemm, h, *st["down_proj"], off_local, st["group_size"],
                       zero_init=False)
        run("send_partials", peer.send_partials, out_perm, weights, ids32, inv, T, K, el)   # barrier inside
        return run("sum_partials", peer.sum_partials, T, res)

    def _forward_peer(self, x2d, st, weights, ids32, perm, inv, off32, T, K, E, res=None):
        """Expert-parallel path over peer memory: rows go straight from x into the owners' receive
        buffers and expert outputs are read straight from the owners while combining."""
        run = self._stage
        peer = self._ensure_peer(x2d, T, K)
        tc5 = (not st["w4"]) and scatter_gemm_supported(peer.recv_rows(), st["w2"]) \
            and gather_swiglu_supported(peer.recv_rows(), st["w13"])
        fused_return = tc5 and self.ep_return == "fused"
        unique = tc5 and self.ep_dispatch == "unique" and self.ep_size <= 8
        # counts to every peer, rank barrier, plan: one launch
        send_base, seg = run("exchange_plan", peer.exchange_plan, off32)
        if unique:
            # one copy of a token row per destination rank; the owners gather through their slot tables
            slot_dst = run("dispatch", peer.dispatch_unique, x2d, ids32, perm, off32, send_base, K, E,
                           self.ep_max_tokens)
        else:
            slot_dst = run("dispatch", peer.dispatch, x2d, perm, off32, send_base, K, E)
        run("rank_barrier", peer.rank_barrier)
        if tc5:
            status = self._status_word(x2d.device)
            if unique:
                h = run("grouped_swiglu", moe_grouped_swiglu_gather, peer.recv_rows(), peer.slot_table(), 1,
                        st["w13"], seg, status=status)
            else:
                h = run("grouped_swiglu", moe_grouped_swiglu, peer.recv_rows(), st["w13"], seg, zero_init=False,
                        status=status)
            if fused_return:
                run("grouped_down", moe_grouped_gemm_scatter, h, st["w2"], seg, peer.home_table(), peer.y_ptrs,
                    status=status)
                run("rank_barrier", peer.rank_barrier)
                # every row of this rank's sorted order is back in its own buffer
                return run("unpermute_combine", unpermute_combine, peer.y_rows()[:T * K], weights, inv, T, K,
                           residual=res)
            run("grouped_down", moe_grouped_gemm, h, st["w2"], seg, zero_init=False, out=peer.y_rows(), status=status)
            run("rank_barrier", peer.rank_barrier)
            return run("combine", peer.combine, weights, inv, slot_dst, T, K, residual=res)
        self._experts(st, peer.recv_rows(), seg, out=peer.y_rows())
        run("rank_barrier", peer.rank_barrier)
        return run("combine", peer.combine, weights, inv, slot_dst, T, K, residual=res)

    def _stage(self, name, fn, *args, **kwargs):
        """Runs one stage; with ``kernel_events`` set, brackets it with CUDA events on the current stream."""
        events = self.kernel_events
        if events is None:
            return fn(*args, **kwargs)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        result = fn(*args, **kwargs)
        end.record()
        events.append((name, start, end))
        return result

    def quantize_to_w4a16(self, group_size: int = 128) -> None:
        """Replace every expert Linear by a min-max quantised ``LinearW4A16`` on the same device."""
        device = next(self.parameters()).device
        for expert in self.experts:
            for p in _PROJ:
                setattr(expert, p, LinearW4A16.from_float(getattr(expert, p), group_size).to(device))
