"""A routed feed-forward (mixture of experts), with an optional expert that every token uses.

Router: ``z = W_router h`` in float32 (h as the activation dtype holds it), ``s = softmax(z)`` over
all experts.  Experts are chosen by ``s + correction`` (a stored vector): they form
``n_groups`` equal groups of neighbours, a group counts by its best choice score, only experts of
the ``keep_groups`` best groups can be chosen, and of those the ``top`` best are.  The chosen
experts' weights are their ``s`` (not renormalised) times ``weight_scale``.  An expert is
``W_down (silu(W_gate h) * (W_up h))``; the output is the weighted sum of the chosen experts'.
The shared expert has the same form (its own inner size) and is added multiplied by
``sigmoid(W_sg h)``, one number per token.

The router's matrix and the shared expert's gate row are kept as one float32 matrix, so one product
on the CUDA cores gives the logits and the gate's input in float32.  The experts' products read
only the chosen experts' weights (``kernels/ops.moe_gate_up``, ``moe_down``); the shared expert runs
through the dense products.  Nothing here reads a choice back to the host, so a step through this
part can be captured in a graph.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..kernels.linear import EPI_STORE, EPI_SWIGLU, linear
from .base import FEED_FORWARDS, FeedForward, ParamSpec


@FEED_FORWARDS.register("routed_mlp")
class RoutedMLP(FeedForward):
    graph_safe = True

    def __init__(self, width: int, n_experts: int, top: int, inner: int, n_groups: int = 1, keep_groups: int = 1,
                 shared_inner: Optional[int] = None, correction: bool = True, weight_scale: float = 1.0):
        if n_experts < 1 or not 1 <= top <= n_experts or inner < 1:
            raise ValueError(f"routed feed-forward: bad sizes experts={n_experts} top={top} inner={inner}")
        if n_groups < 1 or n_experts % n_groups != 0 or not 1 <= keep_groups <= n_groups:
            raise ValueError(f"routed feed-forward: {n_experts} experts in {n_groups} groups, {keep_groups} kept")
        if keep_groups * (n_experts // n_groups) < top:
            raise ValueError(f"routed feed-forward: {keep_groups} groups of {n_experts // n_groups} experts cannot give {top}")
        self.width, self.n_experts, self.top, self.inner = int(width), int(n_experts), int(top), int(inner)
        self.n_groups, self.keep_groups = int(n_groups), int(keep_groups)
        self.shared_inner = None if shared_inner is None else int(shared_inner)
        self.has_correction, self.weight_scale = bool(correction), float(weight_scale)

    def param_specs(self) -> Dict[str, ParamSpec]:
        w = self.width
        specs = {"router": ParamSpec((self.n_experts, w))}
        if self.has_correction:
            specs["correction"] = ParamSpec((self.n_experts,))
        for e in range(self.n_experts):
            specs[f"experts.{e}.gate_proj"] = ParamSpec((self.inner, w))
            specs[f"experts.{e}.up_proj"] = ParamSpec((self.inner, w))
            specs[f"experts.{e}.down_proj"] = ParamSpec((w, self.inner))
        if self.shared_inner is not None:
            specs["shared.gate_proj"] = ParamSpec((self.shared_inner, w))
            specs["shared.up_proj"] = ParamSpec((self.shared_inner, w))
            specs["shared.down_proj"] = ParamSpec((w, self.shared_inner))
            specs["shared.gate"] = ParamSpec((1, w))
        return specs

    def load(self, tensors, runtime) -> None:
        def stack(kind):
            mats = [tensors[f"experts.{e}.{kind}"] for e in range(self.n_experts)]
            if len({m.dtype for m in mats}) > 1 or mats[0].dtype != runtime.dtype:
                mats = [m.to(runtime.dtype) if runtime.dtype == torch.float32 else m for m in mats]
            return torch.stack(mats, dim=0).contiguous()

        self.w_gate, self.w_up, self.w_down = stack("gate_proj"), stack("up_proj"), stack("down_proj")
        rows = [tensors["router"].float()]
        if self.shared_inner is not None:
            rows.append(tensors["shared.gate"].float())
            g, u = tensors["shared.gate_proj"], tensors["shared.up_proj"]
            if g.dtype != u.dtype:
                g, u = g.float(), u.float()
            self.ws_gate_up = torch.stack([g, u], dim=1).reshape(2 * self.shared_inner, self.width).contiguous()
            self.ws_down = tensors["shared.down_proj"]
        self.w_router = torch.cat(rows, dim=0).contiguous()          # float32: the product runs on the CUDA cores
        self.correction = tensors["correction"].float().contiguous() if self.has_correction else None

    def forward_store(self, ctx, h, out) -> None:
        self._run(ctx, h, out, accumulate=False)

    def forward(self, ctx, h, residual) -> None:
        self._run(ctx, h, residual, accumulate=True)

    def _run(self, ctx, h, target, accumulate: bool) -> None:
        n = h.shape[0]
        shared = self.shared_inner is not None
        z = ctx.rows("moe.logits", self.w_router.shape[0], torch.float32)
        linear(h, self.w_router, z, EPI_STORE)
        idx = ctx.rows("moe.idx", self.top, torch.int32)
        wts = ctx.rows("moe.weight", self.top, torch.float32)
        gate = ctx.rows("moe.gate", 1, torch.float32).view(-1) if shared else None
        ops.moe_route(z, self.n_experts, self.correction, idx, wts, self.top, self.n_groups, self.keep_groups,
                      self.weight_scale, gate)
        ys = None
        if shared:
            act_s = ctx.rows("moe.shared.act", self.shared_inner)
            linear(h, self.ws_gate_up, act_s, EPI_SWIGLU)
            ys = ctx.rows("moe.shared.out", self.width, torch.float32)
            linear(act_s, self.ws_down, ys, EPI_STORE)
        act = ctx.rows("moe.act", self.top * self.inner).view(n * self.top, self.inner)
        ops.moe_gate_up(h, self.w_gate, self.w_up, idx, ctx.token_slot, act)
        ops.moe_down(act, self.w_down, idx, wts, ctx.token_slot, target, ys, gate, accumulate)
