"""``DatasunConfig``: the sizes and constants of a Datasun decoder, read from its config.json.

A Datasun model is a stack of parallel blocks (one norm; mixer and feed-forward both read it), each
with one of two mixers: windowed softmax attention whose values are its keys, with a sink in the
softmax's denominator, or linear attention with a decay per head.  config.json carries:

    architecture        "Datasun"
    vocab, width        vocabulary size, residual width
    norm.eps            epsilon of every RMS norm
    embedding.scale     factor on the embedding rows (the tied head does not carry it)
    layers[i].type      "attention" | "lightning"
    layers[i].mixer     attention: heads, kv_heads, dim, vdim (= dim), scale, mask.size (window),
                                   rot.{base, dims, scaling.{factor, original, fast, slow}}
                        lightning: heads, dim, vdim, decay[heads]
    layers[i].mlp       null, or {kind: "dense", ff, limit}

Every value is checked here, so a bad folder fails by key before any weight is read.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ConfigReader


@dataclass(frozen=True)
class DatasunRotary:
    base: float
    dims: int
    scaling: Optional[Tuple[Tuple[str, float], ...]]      # (factor, original, fast, slow) by name, or None


@dataclass(frozen=True)
class DatasunAttention:
    heads: int
    kv_heads: int
    dim: int
    scale: float
    window: Optional[int]
    rotary: Optional[DatasunRotary]


@dataclass(frozen=True)
class DatasunLightning:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class DatasunMLP:
    ff: int
    limit: Optional[float]


@dataclass(frozen=True)
class DatasunLayer:
    type: str
    mixer: Any
    mlp: Optional[DatasunMLP]


def _sub(r: ConfigReader, key: str, required: bool = True) -> Optional[ConfigReader]:
    v = r.raw(key)
    if v is None:
        if required:
            raise ConfigError(f"{r.what}: missing required key '{key}'")
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"{r.what}: key '{key}' must be an object, got {v!r}")
    return ConfigReader(v, f"{r.what}: {key}")


def _attention(r: ConfigReader) -> DatasunAttention:
    heads = r.integer("heads", minimum=1)
    kv = r.integer("kv_heads", default=heads, minimum=1)
    if heads % kv != 0:
        raise ConfigError(f"{r.what}: {heads} query heads do not divide into {kv} key/value heads")
    dim = r.integer("dim", minimum=2)
    if dim % 2 != 0:
        raise ConfigError(f"{r.what}: key 'dim' must be even, got {dim}")
    vdim = r.integer("vdim", default=dim, minimum=1)
    if vdim != dim:
        raise ConfigError(f"{r.what}: the values are the keys, so 'vdim' {vdim} must equal 'dim' {dim}")
    scale = r.number("scale", default=dim ** -0.5, positive=True)
    window = None
    mask = _sub(r, "mask", required=False)
    if mask is not None:
        window = mask.integer("size", minimum=1)
    rotary = None
    rot = _sub(r, "rot", required=False)
    if rot is not None:
        dims = rot.integer("dims", minimum=2)
        if dims % 2 != 0 or dims > dim:
            raise ConfigError(f"{rot.what}: key 'dims' must be even and at most dim {dim}, got {dims}")
        base = rot.number("base", positive=True)
        scaling = None
        sc = _sub(rot, "scaling", required=False)
        if sc is not None:
            if not base > 1.0:
                raise ConfigError(f"{rot.what}: frequency scaling needs a base above 1, got {base}")
            scaling = tuple((k, sc.number(k, positive=True)) for k in ("factor", "original", "fast", "slow"))
        rotary = DatasunRotary(base=base, dims=dims, scaling=scaling)
    return DatasunAttention(heads=heads, kv_heads=kv, dim=dim, scale=scale, window=window, rotary=rotary)


def _lightning(r: ConfigReader) -> DatasunLightning:
    heads = r.integer("heads", minimum=1)
    dim = r.integer("dim", minimum=1)
    vdim = r.integer("vdim", default=dim, minimum=1)
    decay = r.raw("decay")
    if isinstance(decay, (int, float)) and not isinstance(decay, bool):
        decay = [decay] * heads
    if not isinstance(decay, (list, tuple)) or len(decay) != heads or \
            not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
        raise ConfigError(f"{r.what}: key 'decay' must list one number per head ({heads})")
    return DatasunLightning(heads=heads, dim=dim, vdim=vdim, decay=tuple(float(x) for x in decay))


@dataclass(frozen=True)
class DatasunConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: Tuple[DatasunLayer, ...]
    max_positions: int
    eos_token_ids: Tuple[int, ...]

    @classmethod
    def from_dict(cls, data: Dict[str, Any], what: str = "config.json") -> "DatasunConfig":
        r = ConfigReader(data, what)
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        eps = _sub(r, "norm").number("eps", positive=True)
        emb = _sub(r, "embedding", required=False)
        scale = emb.number("scale", default=1.0) if emb is not None else 1.0
        raw_layers = r.raw("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(f"{what}: key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            lr = ConfigReader(entry, f"{what}: layers[{i}]")
            kind = lr.string("type")
            mixer = _sub(lr, "mixer")
            if kind == "attention":
                m = _attention(mixer)
            elif kind == "lightning":
                m = _lightning(mixer)
            else:
                raise ConfigError(f"{lr.what}: key 'type' must be \"attention\" or \"lightning\", got {kind!r}")
            mlp = None
            mr = _sub(lr, "mlp", required=False)
            if mr is not None:
                mk = mr.string("kind", default="dense")
                if mk != "dense":
                    raise ConfigError(f"{mr.what}: key 'kind' must be \"dense\", got {mk!r}")
                mlp = DatasunMLP(ff=mr.integer("ff", minimum=1), limit=mr.number("limit", default=None, positive=True))
            layers.append(DatasunLayer(type=kind, mixer=m, mlp=mlp))
        return cls(vocab=vocab, width=width, eps=eps, embedding_scale=scale, layers=tuple(layers),
                   max_positions=r.integer("max_positions", default=0, minimum=0),
                   eos_token_ids=tuple(r.int_or_list("eos_token_id")))
