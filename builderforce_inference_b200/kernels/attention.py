"""Choice of the attention kernel for a step.  Returns False when no specialised kernel takes
the step; the caller then runs the general paged kernel."""
from __future__ import annotations

import torch


def attend(ctx, qkv, out, kv, n_heads: int, scale: float, sink=None, exact_weights: bool = False) -> bool:
    """``exact_weights``: the design wants its attention weights in float32; only kernels that keep
    them so (in effect) are chosen."""
    if qkv.dtype != torch.bfloat16:
        return False
    if not kv.plain or isinstance(sink, torch.Tensor) or exact_weights:
        # a chunked mask or a learned sink per head: steps with more than one token per sequence have
        # the tensor-core kernel with 64-token tiles (keys and values of one size, 64 or 128); single
        # tokens and values of another size than the keys run the general kernel
        if kv.value_dim != kv.head_dim or (ctx.max_seq_tokens == 1 and ctx.n_tokens == ctx.n_seqs):
            return False
        if isinstance(sink, torch.Tensor) and (sink.dtype != torch.float32 or not sink.is_contiguous()):
            return False
        from . import fast_ops
        return fast_ops.attention_prefill_bf16(ctx, qkv, out, kv, n_heads, scale, sink, exact_weights)
    from . import fast_ops
    if ctx.max_seq_tokens == 1 and ctx.n_tokens == ctx.n_seqs:
        return fast_ops.attention_decode_bf16(ctx, qkv, out, kv, n_heads, scale, sink=sink)
    if ctx.max_seq_tokens >= fast_ops.TCGEN05_ATTENTION_MIN_TOKENS and \
            fast_ops.attention_prefill_tcgen05_bf16(ctx, qkv, out, kv, n_heads, scale, sink):
        return True
    return fast_ops.attention_prefill_bf16(ctx, qkv, out, kv, n_heads, scale, sink)
