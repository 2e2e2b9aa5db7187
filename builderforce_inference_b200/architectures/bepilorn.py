"""Bepilorn as data: its configuration turned into a ``ModelSpec``.

Every layer is a sandwich block (a norm before and after each sublayer, all with weights stored
around zero that enter as ``1 + w``).  Its mixer is the state-space part (``mamba2`` layers), or the
weighted sum of two members side by side (``parallel`` layers): the attention part in the variant
"biases on q, k, v, rotate-half rotation of the first ``rot.dims`` values, value heads of their own
size, a chunked mask and a learned sink per head", and the gated linear attention part.  The
feed-forward, where a layer has one, is the routed part with a shared expert.  The head is a
tensor of its own; the logits are multiplied by ``logit_scale``.

Tensor names: ``embed``, ``final.norm``, ``head``, and per layer ``l<i>.norm1``, ``norm1b``, ``norm2``,
``norm2b``; ``l<i>.mix.*`` (state space: in, conv, conv.b, dt_bias, A_log, D, norm, o; parallel:
``left.{q,k,v}`` with biases ``.b``, ``left.sink``, ``left.o``, ``right.{q,k,v,g,o,norm,a1,a2,a2.b}``);
``l<i>.mlp.router``, ``correction``, ``e<j>.{gate,up,down}``, ``shared.{gate,up,down,sg}``; matrices are
``[out, in]``.
"""
from __future__ import annotations

from typing import Any, Dict

from ..config.bepilorn import BepilornConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunSpec

NORM_OFFSET = 1.0       # the block norms' weights are stored around zero


def bepilorn_spec(cfg: BepilornConfig) -> ModelSpec:
    norm = PartSpec("rms", {"width": cfg.width, "eps": cfg.eps, "offset": NORM_OFFSET})
    layers, unused = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        names = {"norm1.weight": p + "norm1", "norm1b.weight": p + "norm1b"}
        m = layer.mixer
        if layer.type == "mamba2":
            mixer = PartSpec("state_space", {"width": cfg.width, "n_heads": m.heads, "vdim": m.vdim, "state": m.state,
                                             "groups": m.groups, "conv_taps": m.conv, "norm_groups": m.norm_groups,
                                             "eps": cfg.eps})
            names.update({"mixer.in_proj": p + "mix.in", "mixer.conv": p + "mix.conv", "mixer.conv.bias": p + "mix.conv.b",
                          "mixer.dt_bias": p + "mix.dt_bias", "mixer.A_log": p + "mix.A_log", "mixer.D": p + "mix.D",
                          "mixer.norm": p + "mix.norm", "mixer.o_proj": p + "mix.o"})
        else:
            a, g = m.left, m.right
            position = None
            if a.rot_base is not None:
                position = PartSpec("rotary", {"theta": a.rot_base, "rot_dim": a.rot_dims, "pairing": "half"})
            left = PartSpec("attention", {
                "width": cfg.width, "n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim, "v_dim": a.vdim,
                "position": position, "eps": cfg.eps, "scale": a.scale, "chunk": a.chunk, "bias": True,
                "out_bias": False, "sink": "learned", "exact_weights": True})
            right = PartSpec("gated_linear", {"width": cfg.width, "n_heads": g.heads, "dim": g.dim, "vdim": g.vdim,
                                              "tau": g.tau, "decay_rank": g.rank, "eps": cfg.eps})
            mixer = PartSpec("weighted_sum", {"members": {"left": left, "right": right},
                                              "scales": {"left": m.left_scale, "right": m.right_scale}})
            lp, rp = p + "mix.left.", p + "mix.right."
            names.update({"mixer.left.q_proj": lp + "q", "mixer.left.q_proj.bias": lp + "q.b",
                          "mixer.left.k_proj": lp + "k", "mixer.left.k_proj.bias": lp + "k.b",
                          "mixer.left.v_proj": lp + "v", "mixer.left.v_proj.bias": lp + "v.b",
                          "mixer.left.sink": lp + "sink", "mixer.left.o_proj": lp + "o",
                          "mixer.right.q_proj": rp + "q", "mixer.right.k_proj": rp + "k", "mixer.right.v_proj": rp + "v",
                          "mixer.right.g_proj": rp + "g", "mixer.right.o_proj": rp + "o", "mixer.right.norm": rp + "norm",
                          "mixer.right.a1_proj": rp + "a1", "mixer.right.a2_proj": rp + "a2",
                          "mixer.right.a2_proj.bias": rp + "a2.b"})
        params = {"norm1": norm, "mixer": mixer, "norm1b": norm}
        if layer.mlp is not None:
            f = layer.mlp
            params.update({"norm2": norm, "norm2b": norm, "ffn": PartSpec("mixture_of_experts", {
                "width": cfg.width, "n_experts": f.experts, "top": f.top, "inner": f.ff, "n_groups": f.groups,
                "keep_groups": f.keep, "shared_inner": f.shared_ff})})
            q = p + "mlp."
            names.update({"norm2.weight": p + "norm2", "norm2b.weight": p + "norm2b", "ffn.router": q + "router",
                          "ffn.correction": q + "correction"})
            for e in range(f.experts):
                for kind in ("gate", "up", "down"):
                    names[f"ffn.experts.{e}.{kind}_proj"] = f"{q}e{e}.{kind}"
            if f.shared_ff is not None:
                names.update({"ffn.shared.gate_proj": q + "shared.gate", "ffn.shared.up_proj": q + "shared.up",
                              "ffn.shared.down_proj": q + "shared.down", "ffn.shared.gate": q + "shared.sg"})
        else:       # a checkpoint may still carry the norms of the feed-forward the layer does not have
            unused += [p + "norm2", p + "norm2b"]
        layers.append(LayerSpec(block=PartSpec("sandwich", params), names=names))
    return ModelSpec(
        vocab_size=cfg.vocab, width=cfg.width, embedding_name="embed", layers=tuple(layers),
        schedule=tuple(RunSpec(layer=i) for i in range(len(layers))),
        final_norm=norm, final_norm_names={"weight": "final.norm"}, head_name="head", ignored_names=tuple(unused),
        max_positions=cfg.max_positions, stop_ids=tuple(cfg.eos_token_ids), logit_scale=cfg.logit_scale)


def describe(config: Dict[str, Any]) -> ModelSpec:
    return bepilorn_spec(BepilornConfig.from_dict(config))
