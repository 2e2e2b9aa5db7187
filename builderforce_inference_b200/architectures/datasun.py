"""Datasun as data: its configuration turned into a ``ModelSpec``.

Every layer is a parallel block; its mixer is the attention part in the variant "biases, a norm
over the whole q and k projections, values that are the keys, adjacent-pair rotation of the first
``rot.dims`` values with yarn-scaled frequencies, a window and a sink of score 0", or the lightning
part.  The feed-forward is the gated one with gate slope 1.702, the configured clamp and an up
shift of 1.  The head is the embedding table (without the embedding's scale).

Tensor names: ``embed``, ``final.norm``, and per layer ``l<i>.norm1``, ``l<i>.mix.<name>`` (q, k, v,
g, o, norm, q.norm, k.norm; biases with ``.b`` appended) and ``l<i>.mlp.{gate,up,down}``, all
``[out, in]``.
"""
from __future__ import annotations

from typing import Any, Dict

from ..config.datasun import DatasunConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunSpec

GATE_SLOPE = 1.702      # sigmoid(1.702 g) in the feed-forward's gate
UP_SHIFT = 1.0          # the up branch enters as (u + 1)
SINK_SCORE = 0.0        # the softmax's denominator carries exp(0)


def datasun_spec(cfg: DatasunConfig) -> ModelSpec:
    norm = PartSpec("rms", {"width": cfg.width, "eps": cfg.eps})
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        names = {"norm1.weight": p + "norm1"}
        m = layer.mixer
        if layer.type == "attention":
            position = None
            if m.rotary is not None:
                position = PartSpec("rotary", {"theta": m.rotary.base, "rot_dim": m.rotary.dims, "pairing": "adjacent",
                                               "scaling": dict(m.rotary.scaling) if m.rotary.scaling else None})
            mixer = PartSpec("attention", {
                "width": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim,
                "position": position, "qk_norm": "row", "eps": cfg.eps, "window": m.window, "scale": m.scale,
                "bias": True, "values": "keys", "sink": SINK_SCORE})
            names.update({"mixer.q_proj": p + "mix.q", "mixer.q_proj.bias": p + "mix.q.b",
                          "mixer.k_proj": p + "mix.k", "mixer.k_proj.bias": p + "mix.k.b",
                          "mixer.q_norm": p + "mix.q.norm", "mixer.k_norm": p + "mix.k.norm",
                          "mixer.o_proj": p + "mix.o", "mixer.o_proj.bias": p + "mix.o.b"})
        else:
            mixer = PartSpec("lightning", {"width": cfg.width, "n_heads": m.heads, "dim": m.dim, "vdim": m.vdim,
                                           "decay": m.decay, "eps": cfg.eps})
            names.update({"mixer.q_proj": p + "mix.q", "mixer.k_proj": p + "mix.k", "mixer.v_proj": p + "mix.v",
                          "mixer.g_proj": p + "mix.g", "mixer.o_proj": p + "mix.o", "mixer.norm": p + "mix.norm"})
        ffn = None
        if layer.mlp is not None:
            ffn = PartSpec("gated_mlp", {"width": cfg.width, "inner": layer.mlp.ff, "gate_alpha": GATE_SLOPE,
                                         "limit": layer.mlp.limit, "up_shift": UP_SHIFT})
            names.update({"ffn.gate_proj": p + "mlp.gate", "ffn.up_proj": p + "mlp.up", "ffn.down_proj": p + "mlp.down"})
        layers.append(LayerSpec(block=PartSpec("parallel", {"norm1": norm, "mixer": mixer, "ffn": ffn}), names=names))
    return ModelSpec(
        vocab_size=cfg.vocab, width=cfg.width, embedding_name="embed", layers=tuple(layers),
        schedule=tuple(RunSpec(layer=i) for i in range(len(layers))),
        final_norm=norm, final_norm_names={"weight": "final.norm"}, head_name=None,
        max_positions=cfg.max_positions, stop_ids=tuple(cfg.eos_token_ids), embedding_scale=cfg.embedding_scale)


def describe(config: Dict[str, Any]) -> ModelSpec:
    return datasun_spec(DatasunConfig.from_dict(config))
