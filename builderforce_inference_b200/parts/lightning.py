"""Linear attention with a decay per head ("lightning attention"), as a mixer.

With ``q = silu(W_q h)``, ``k = silu(W_k h)`` (``heads x dim``) and ``v = silu(W_v h)``
(``heads x vdim``), every head keeps a ``dim x vdim`` state per sequence:

    S_t = decay_h * S_(t-1) + k_t v_t^T        o_t = S_t^T q_t

The heads of a token are RMS-normed together (one weight over ``heads * vdim``), multiplied by
``sigmoid(W_g h)`` and projected by ``W_o`` into the residual stream.  The state is float32, zero
when a slot is taken (the cache clears it), and the only thing a sequence keeps: a step may bring
whole prompts, further pieces of one, or single tokens.

The four input projections are one matrix product over the concatenated weights; the activations
are applied where the values are read (the recurrence kernels, the gated norm), in float32.
"""
from __future__ import annotations

from typing import Dict, Sequence

import torch

from ..kernels import ops
from ..kernels.linear import EPI_ACCUMULATE, EPI_STORE, linear
from .base import MIXERS, Mixer, ParamSpec, StateNeed


@MIXERS.register("lightning")
class LightningAttention(Mixer):
    graph_safe = True

    def __init__(self, width: int, n_heads: int, dim: int, vdim: int, decay: Sequence[float], eps: float = 1e-6):
        if n_heads < 1 or dim < 1 or vdim < 1:
            raise ValueError(f"lightning attention: bad sizes heads={n_heads} dim={dim} vdim={vdim}")
        if len(decay) != n_heads:
            raise ValueError(f"lightning attention: {len(decay)} decays for {n_heads} heads")
        self.width, self.n_heads, self.dim, self.vdim = int(width), int(n_heads), int(dim), int(vdim)
        self.decay_values = tuple(float(x) for x in decay)
        self.eps = float(eps)
        self.w_in = self.w_o = self.norm = self.decay = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        qk, vv, w = self.n_heads * self.dim, self.n_heads * self.vdim, self.width
        return {"q_proj": ParamSpec((qk, w)), "k_proj": ParamSpec((qk, w)), "v_proj": ParamSpec((vv, w)),
                "g_proj": ParamSpec((vv, w)), "o_proj": ParamSpec((w, vv)), "norm": ParamSpec((vv,), "norm")}

    def cache_need(self):
        return StateNeed((self.n_heads, self.dim, self.vdim), "float32")

    def load(self, tensors, runtime) -> None:
        mats = [tensors[n] for n in ("q_proj", "k_proj", "v_proj", "g_proj")]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_o = tensors["o_proj"]
        self.norm = tensors["norm"]
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=runtime.device)

    def forward(self, ctx, h, residual, run) -> None:
        state = run.state
        if state is None or not run.writes_cache:
            raise RuntimeError("lightning attention needs a state of its own for its run")
        qk, vv = self.n_heads * self.dim, self.n_heads * self.vdim
        proj = ctx.rows("light.proj", 2 * qk + 2 * vv)
        linear(h, self.w_in, proj, EPI_STORE)
        o = ctx.rows("light.o", vv, torch.float32)
        self.recur(ctx, proj, o, state)
        y = ctx.rows("light.y", vv)
        ops.gated_rmsnorm(o, proj[:, 2 * qk + vv:], self.norm, self.eps, y)
        linear(y, self.w_o, residual, EPI_ACCUMULATE)

    def recur(self, ctx, proj, o, state) -> None:
        qk = self.n_heads * self.dim
        if proj.dtype == torch.bfloat16:
            from ..kernels import fast_ops
            if ctx.max_seq_tokens >= fast_ops.LIGHTNING_CHUNK_MIN_TOKENS and fast_ops.lightning_chunks_bf16(
                    proj, 0, qk, 2 * qk, o, state, self.decay, ctx.cu_seqlens, ctx.seq_slot, ctx.n_seqs,
                    self.n_heads, self.dim, self.vdim):
                return
        ops.lightning_scan(proj, 0, qk, 2 * qk, o, state, self.decay, ctx.cu_seqlens, ctx.seq_slot, ctx.n_seqs,
                           self.n_heads, self.dim, self.vdim, ops.LIGHT_ACT_SILU, few_tokens=ctx.max_seq_tokens == 1,
                           single_tokens=ctx.max_seq_tokens == 1 and ctx.n_tokens == ctx.n_seqs)
