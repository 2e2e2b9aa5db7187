"""``BepilornConfig``: the sizes and constants of a Bepilorn decoder, read from its config.json.

A Bepilorn model is a stack of blocks with a norm before and after each sublayer, whose mixer is,
layer by layer, a Mamba-2 state-space mixer or a pair of mixers side by side (chunked softmax
attention with a learned sink per head, and gated linear attention with a decay per key channel),
and whose feed-forward, where a layer has one, is a mixture of experts with a shared expert.
config.json carries:

    architecture        "Bepilorn"
    vocab, width        vocabulary size, residual width
    norm.eps            epsilon of every RMS norm
    logit_scale         factor on the logits (default 1)
    layers[i].type      "mamba2" | "parallel"
    layers[i].mixer     mamba2:   heads, vdim, state, groups, conv (taps), norm_groups
                        parallel: left_scale, right_scale,
                                  left:  heads, kv_heads, dim, vdim, scale, mask.size (chunk),
                                         rot.{base, dims}
                                  right: heads, dim, vdim, tau, rank (optional: width between the decay's
                                         two projections; absent, the tensor's shape gives it)
    layers[i].mlp       null, or {kind: "moe", expert.ff, router.{experts, top, groups.{count, keep}},
                                  shared.ff}

Every value is checked here, so a bad folder fails by key before any weight is read.  Sizes that
only a tensor's shape gives (the rank of the decay's two-step projection) are read from the
safetensors header by the architecture's ``describe``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ConfigReader
from .datasun import _sub


@dataclass(frozen=True)
class BepilornStateSpace:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class BepilornSoftmax:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: Optional[int]
    rot_base: Optional[float]
    rot_dims: int


@dataclass(frozen=True)
class BepilornGatedLinear:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: Optional[int]       # width between the decay's two projections; None: the tensor's shape gives it


@dataclass(frozen=True)
class BepilornParallel:
    left: BepilornSoftmax
    right: BepilornGatedLinear
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class BepilornMoE:
    experts: int
    top: int
    ff: int
    groups: int
    keep: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class BepilornLayer:
    type: str
    mixer: Any
    mlp: Optional[BepilornMoE]


def _state_space(r: ConfigReader) -> BepilornStateSpace:
    heads = r.integer("heads", minimum=1)
    groups = r.integer("groups", default=1, minimum=1)
    if heads % groups != 0:
        raise ConfigError(f"{r.what}: {heads} heads do not divide into {groups} groups")
    vdim = r.integer("vdim", minimum=1)
    parts = r.integer("norm_groups", default=1, minimum=1)
    if (heads * vdim) % parts != 0:
        raise ConfigError(f"{r.what}: heads * vdim = {heads * vdim} does not cut into {parts} norm_groups")
    conv = r.integer("conv", minimum=1)
    if conv > 16:
        raise ConfigError(f"{r.what}: key 'conv' must be at most 16 taps, got {conv}")
    return BepilornStateSpace(heads=heads, vdim=vdim, state=r.integer("state", minimum=1), groups=groups, conv=conv,
                              norm_groups=parts)


def _softmax(r: ConfigReader) -> BepilornSoftmax:
    heads = r.integer("heads", minimum=1)
    kv = r.integer("kv_heads", default=heads, minimum=1)
    if heads % kv != 0:
        raise ConfigError(f"{r.what}: {heads} query heads do not divide into {kv} key/value heads")
    dim = r.integer("dim", minimum=2)
    if dim % 2 != 0 or dim > 512:
        raise ConfigError(f"{r.what}: key 'dim' must be even and at most 512, got {dim}")
    vdim = r.integer("vdim", default=dim, minimum=1)
    if vdim > 512:
        raise ConfigError(f"{r.what}: key 'vdim' must be at most 512, got {vdim}")
    scale = r.number("scale", default=dim ** -0.5, positive=True)
    chunk = None
    mask = _sub(r, "mask", required=False)
    if mask is not None:
        chunk = mask.integer("size", minimum=1)
    base, dims = None, 0
    rot = _sub(r, "rot", required=False)
    if rot is not None:
        dims = rot.integer("dims", minimum=2)
        if dims % 2 != 0 or dims > dim:
            raise ConfigError(f"{rot.what}: key 'dims' must be even and at most dim {dim}, got {dims}")
        base = rot.number("base", positive=True)
    return BepilornSoftmax(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, chunk=chunk, rot_base=base,
                           rot_dims=dims)


def _gated_linear(r: ConfigReader) -> BepilornGatedLinear:
    return BepilornGatedLinear(heads=r.integer("heads", minimum=1), dim=r.integer("dim", minimum=1),
                               vdim=r.integer("vdim", minimum=1), tau=r.number("tau", positive=True),
                               rank=r.integer("rank", default=None, minimum=1))


def _moe(r: ConfigReader) -> BepilornMoE:
    kind = r.string("kind", default="moe")
    if kind != "moe":
        raise ConfigError(f"{r.what}: key 'kind' must be \"moe\", got {kind!r}")
    router = _sub(r, "router")
    experts = router.integer("experts", minimum=1)
    top = router.integer("top", minimum=1)
    if top > experts:
        raise ConfigError(f"{router.what}: key 'top' {top} exceeds the {experts} experts")
    count = keep = 1
    groups = _sub(router, "groups", required=False)
    if groups is not None:
        count = groups.integer("count", default=1, minimum=1)
        keep = groups.integer("keep", default=count, minimum=1)
        if experts % count != 0 or keep > count:
            raise ConfigError(f"{groups.what}: {experts} experts in {count} groups, {keep} kept")
        if keep * (experts // count) < top:
            raise ConfigError(f"{groups.what}: {keep} groups of {experts // count} experts cannot give top {top}")
    shared = _sub(r, "shared", required=False)
    return BepilornMoE(experts=experts, top=top, ff=_sub(r, "expert").integer("ff", minimum=1), groups=count, keep=keep,
                       shared_ff=None if shared is None else shared.integer("ff", minimum=1))


@dataclass(frozen=True)
class BepilornConfig:
    vocab: int
    width: int
    eps: float
    logit_scale: float
    layers: Tuple[BepilornLayer, ...]
    max_positions: int
    eos_token_ids: Tuple[int, ...]

    @classmethod
    def from_dict(cls, data: Dict[str, Any], what: str = "config.json") -> "BepilornConfig":
        r = ConfigReader(data, what)
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        eps = _sub(r, "norm").number("eps", positive=True)
        raw_layers = r.raw("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(f"{what}: key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            lr = ConfigReader(entry, f"{what}: layers[{i}]")
            kind = lr.string("type")
            mixer = _sub(lr, "mixer")
            if kind == "mamba2":
                m = _state_space(mixer)
            elif kind == "parallel":
                m = BepilornParallel(left=_softmax(_sub(mixer, "left")), right=_gated_linear(_sub(mixer, "right")),
                                     left_scale=mixer.number("left_scale", default=1.0),
                                     right_scale=mixer.number("right_scale", default=1.0))
            else:
                raise ConfigError(f"{lr.what}: key 'type' must be \"mamba2\" or \"parallel\", got {kind!r}")
            mr = _sub(lr, "mlp", required=False)
            layers.append(BepilornLayer(type=kind, mixer=m, mlp=None if mr is None else _moe(mr)))
        return cls(vocab=vocab, width=width, eps=eps, logit_scale=r.number("logit_scale", default=1.0),
                   layers=tuple(layers), max_positions=r.integer("max_positions", default=0, minimum=0),
                   eos_token_ids=tuple(r.int_or_list("eos_token_id")))
