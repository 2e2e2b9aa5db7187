"""A routed feed-forward (mixture of experts), with an optional expert that every token uses.

Router: ``z = W_router h`` in float32 (h as the activation dtype holds it), ``s = softmax(z)`` over
all experts.  Experts are chosen by ``s + correction`` (a stored vector): they form
``n_groups`` equal groups of neighbours, a group counts by its best choice score, only experts of
the ``keep_groups`` best groups can be chosen, and of those the ``top`` best are.  The chosen
experts' weights are their ``s`` (not renormalised) times ``weight_scale``.  An expert is
``W_down (silu(W_gate h) * (W_up h))``; the output is the weighted sum of the chosen experts'.
The shared expert has the same form (its own inner size) and is added multiplied by
``sigmoid(W_sg h)``, one number per token.

The router's matrix and the shared expert's gate row are kept as one float32 matrix; one kernel
makes the logits and the gate's input from it in float32 and decides (``kernels/ops.moe_router``).  The experts' weights are kept
as two matrices for all experts (gate and up rows interleaved, expert after expert; the down
matrices side by side), which serve two ways of computing: a step with few (token, expert) pairs
reads only the chosen experts' weights (``kernels/ops.moe_gate_up``, ``moe_down``); a bfloat16 step
with at least ``DENSE_PAIRS_PER_EXPERT`` pairs per expert, which touches nearly every expert anyway,
runs the two dense products over all experts on the tensor cores and multiplies the activations by
the chosen experts' weights, 0 for the others, in between (``moe_weigh_dense``); the shared expert
stands behind the routed ones in both matrices and is weighed by its gate there, so the dense way is
two products and one kernel between them.  In the other way the shared expert runs through dense
products of its own.  Nothing here reads a choice back to the host, so a step through
this part can be captured in a graph.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..kernels.linear import EPI_ACCUMULATE, EPI_STORE, EPI_SWIGLU, linear
from .base import FEED_FORWARDS, FeedForward, ParamSpec


DENSE_PAIRS_PER_EXPERT = 2      # from this many (token, expert) pairs per expert on, every expert is computed for every token


@FEED_FORWARDS.register("mixture_of_experts")
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
        mats = [tensors[f"experts.{e}.{kind}"] for e in range(self.n_experts) for kind in ("gate_proj", "up_proj", "down_proj")]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        gu = [torch.stack([mats[3 * e], mats[3 * e + 1]], dim=1).reshape(2 * self.inner, self.width) for e in range(self.n_experts)]
        downs = [mats[3 * e + 2] for e in range(self.n_experts)]
        rows = [tensors["router"].float()]
        if self.shared_inner is not None:
            # the shared expert stands behind the routed ones in both matrices, so the dense way is two
            # products for all of them; the other way reads it through views (and its own down matrix)
            rows.append(tensors["shared.gate"].float())
            g, u, dn = tensors["shared.gate_proj"], tensors["shared.up_proj"], tensors["shared.down_proj"]
            if len({g.dtype, u.dtype, dn.dtype, gu[0].dtype}) > 1:
                g, u, dn, gu, downs = g.float(), u.float(), dn.float(), [m.float() for m in gu], [m.float() for m in downs]
            gu.append(torch.stack([g, u], dim=1).reshape(2 * self.shared_inner, self.width))
            downs.append(dn)
            self.ws_down = dn.contiguous()
        self.w_gu_all = torch.cat(gu, dim=0).contiguous()                  # [(E * ff + shared) * 2, width]
        self.w_down_all = torch.cat(downs, dim=1).contiguous()             # [width, E * ff + shared]
        routed = self.n_experts * self.inner
        self.w_gu = self.w_gu_all[:2 * routed]                             # [E * 2 * ff, width]
        self.w_down = self.w_down_all[:, :routed]                          # [width, E * ff], rows of the wider matrix
        self.routed_rows = 2 * routed                                      # the shared expert's gate/up rows follow
        self.w_router = torch.cat(rows, dim=0).contiguous()                # float32: the logits are float32 sums
        self.correction = tensors["correction"].float().contiguous() if self.has_correction else None

    def forward_store(self, ctx, h, out) -> None:
        self._run(ctx, h, out, accumulate=False)

    def forward(self, ctx, h, residual) -> None:
        self._run(ctx, h, residual, accumulate=True)

    def _run(self, ctx, h, target, accumulate: bool) -> None:
        n = h.shape[0]
        shared = self.shared_inner is not None
        idx = ctx.rows("moe.idx", self.top, torch.int32)
        wts = ctx.rows("moe.weight", self.top, torch.float32)
        gate = ctx.rows("moe.gate", 1, torch.float32).view(-1) if shared else None
        ops.moe_router(h, self.w_router, self.n_experts, self.correction, ctx.token_slot, idx, wts, self.top, self.n_groups,
                       self.keep_groups, self.weight_scale, gate)
        if h.dtype == torch.bfloat16 and self.w_gu_all.dtype == torch.bfloat16 \
                and n * self.top >= DENSE_PAIRS_PER_EXPERT * self.n_experts:
            tail = self.shared_inner or 0
            act = ctx.rows("moe.act.dense", self.n_experts * self.inner + tail)
            linear(h, self.w_gu_all, act, EPI_SWIGLU)
            ops.moe_weigh_dense(act, self.n_experts, idx, wts, ctx.token_slot, tail, gate)
            linear(act, self.w_down_all, target, EPI_ACCUMULATE if accumulate else EPI_STORE)
            return
        ys = None
        if shared:
            act_s = ctx.rows("moe.shared.act", self.shared_inner)
            linear(h, self.w_gu_all[self.routed_rows:], act_s, EPI_SWIGLU)
            ys = ctx.rows("moe.shared.out", self.width, torch.float32)
            linear(act_s, self.ws_down, ys, EPI_STORE)
        act = ctx.rows("moe.act", self.top * self.inner).view(n * self.top, self.inner)
        ops.moe_gate_up(h, self.w_gu, self.n_experts, idx, ctx.token_slot, act)
        ops.moe_down(act, self.w_down, self.n_experts, idx, wts, ctx.token_slot, target, ys, gate, accumulate)
