"""Shared by the Bepilorn tests: small configurations with sizes of their own, weights made here
(larger than the package's random fill, so that softmaxes are sharp, decays spread out and routers
decide), and model folders written from them."""
import json
import math
import os
import struct
import tempfile

import torch

F32, BF16 = torch.float32, torch.bfloat16


def ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def par(left, right, ls, rs):
    return {"left": left, "right": right, "left_scale": ls, "right_scale": rs}


def soft(heads, kv, dim, vdim, scale, chunk=None, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


def gla(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def moe(experts, top, ff, count=None, keep=None, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if count:
        m["router"]["groups"] = {"count": count, "keep": keep}
    if shared:
        m["shared"] = {"ff": shared}
    return m


# odd sizes everywhere: a chunk shorter than a page and one that crosses page borders, rotation over
# part of a head, value heads wider and narrower than the keys, 1 and 3 key/value heads, convolutions
# of 2 and 5 taps, one and several norm parts, a layer without feed-forward, a router without groups
# and one that keeps 2 of 3, a feed-forward without shared expert, top 1 and top 3
BP_ODD = {"architecture": "Bepilorn", "vocab": 131, "width": 40, "norm": {"eps": 2e-5}, "logit_scale": 0.7,
          "layers": [
              {"type": "mamba2", "mixer": ssm(3, 8, 12, 1, 2, 1), "mlp": moe(6, 3, 24, 3, 2, 40)},
              {"type": "parallel", "mixer": par(soft(4, 2, 24, 10, 0.21, 9, (5000.0, 12)), gla(3, 8, 20, 4.0, 5), 0.7, 1.3),
               "mlp": None},
              {"type": "mamba2", "mixer": ssm(4, 6, 5, 2, 5, 3), "mlp": moe(5, 1, 16)},
              {"type": "parallel", "mixer": par(soft(3, 3, 16, 28, 0.3, 70, (100.0, 16)), gla(2, 24, 8, 32.0, 3), -0.8, 0.5),
               "mlp": moe(4, 2, 20, 2, 1, 12)},
              {"type": "parallel", "mixer": par(soft(2, 1, 32, 32, 0.15), gla(1, 16, 16, 1.0, 8), 1.0, 1.0),
               "mlp": moe(8, 2, 8, 4, 2)}]}
# sizes nearer to a served model's: heads of 64, a state of 64, chunks of 128
BP_WIDE = {"architecture": "Bepilorn", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
           "layers": [
               {"type": "mamba2", "mixer": ssm(6, 64, 64, 3, 4, 2), "mlp": moe(8, 2, 64, 4, 2, 128)},
               {"type": "parallel", "mixer": par(soft(8, 2, 64, 64, 0.11, 128, (1e4, 32)), gla(2, 64, 64, 12.0, 8), 0.5, 1.5),
                "mlp": moe(12, 3, 48, 3, 2, 64)},
               {"type": "mamba2", "mixer": ssm(2, 32, 128, 1, 4, 1), "mlp": None}]}
CONFIGS = {"odd": BP_ODD, "wide": BP_WIDE}


def tensor_shapes(cfg):
    """name -> (shape, kind) of every tensor of a Bepilorn model, from its config alone."""
    w = cfg["width"]
    out = {"embed": ((cfg["vocab"], w), "table"), "final.norm": ((w,), "norm0"), "head": ((cfg["vocab"], w), "matrix")}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = ((w,), "norm0")
        out[p + "norm1b"] = ((w,), "norm0")
        if layer["type"] == "mamba2":
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            c = inner + 2 * gn
            out.update({p + "mix.in": ((2 * inner + 2 * gn + m["heads"], w), "matrix"), p + "mix.conv": ((c, m["conv"]), "conv"),
                        p + "mix.conv.b": ((c,), "bias"), p + "mix.dt_bias": ((m["heads"],), "step"),
                        p + "mix.A_log": ((m["heads"],), "step"), p + "mix.D": ((m["heads"],), "norm"),
                        p + "mix.norm": ((inner,), "norm"), p + "mix.o": ((w, inner), "matrix")})
        else:
            a, g = m["left"], m["right"]
            lp, rp = p + "mix.left.", p + "mix.right."
            nq, nk, nv = a["heads"] * a["dim"], a["kv_heads"] * a["dim"], a["kv_heads"] * a["vdim"]
            out.update({lp + "q": ((nq, w), "matrix"), lp + "q.b": ((nq,), "bias"), lp + "k": ((nk, w), "matrix"),
                        lp + "k.b": ((nk,), "bias"), lp + "v": ((nv, w), "matrix"), lp + "v.b": ((nv,), "bias"),
                        lp + "sink": ((a["heads"],), "sink"), lp + "o": ((w, a["heads"] * a["vdim"]), "matrix")})
            gq, gv = g["heads"] * g["dim"], g["heads"] * g["vdim"]
            out.update({rp + "q": ((gq, w), "matrix"), rp + "k": ((gq, w), "matrix"), rp + "v": ((gv, w), "matrix"),
                        rp + "g": ((gv, w), "matrix"), rp + "o": ((w, gv), "matrix"), rp + "norm": ((g["vdim"],), "norm"),
                        rp + "a1": ((g["rank"], w), "matrix"), rp + "a2": ((gq, g["rank"]), "matrix"),
                        rp + "a2.b": ((gq,), "decay")})
        f = layer.get("mlp")
        if f:
            q = p + "mlp."
            out[p + "norm2"] = ((w,), "norm0")
            out[p + "norm2b"] = ((w,), "norm0")
            out[q + "router"] = ((f["router"]["experts"], w), "router")
            out[q + "correction"] = ((f["router"]["experts"],), "correction")
            for e in range(f["router"]["experts"]):
                ff = f["expert"]["ff"]
                out.update({f"{q}e{e}.gate": ((ff, w), "matrix"), f"{q}e{e}.up": ((ff, w), "matrix"),
                            f"{q}e{e}.down": ((w, ff), "matrix")})
            if f.get("shared"):
                ff = f["shared"]["ff"]
                out.update({q + "shared.gate": ((ff, w), "matrix"), q + "shared.up": ((ff, w), "matrix"),
                            q + "shared.down": ((w, ff), "matrix"), q + "shared.sg": ((1, w), "matrix")})
    return out


def make_weights(cfg, seed, dt, steady=False):
    """``steady``: routers that decide by wide gaps (corrections a quarter apart, logits that move
    the scores by less), so that the rounding of a bfloat16 run cannot turn a choice and with it the
    whole output; the float32 models' routers decide by the scores."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        t = torch.randn(shape, generator=g)
        if kind == "norm":
            t = 1.0 + 0.2 * t
        elif kind == "norm0":
            t = 0.25 * t
        elif kind == "bias":
            t = 0.3 * t
        elif kind == "table":
            t = 0.7 * t
        elif kind == "conv":
            t = 0.6 * t
        elif kind == "step":
            t = 0.8 * t
        elif kind == "sink":
            t = 1.5 * t
        elif kind == "decay":
            t = 2.0 + 1.5 * t
        elif kind == "correction":
            # mostly negative: a masked expert must count as minus infinity, not 0
            t = 0.25 * torch.randperm(shape[0], generator=g).float() - 1.0 if steady else 0.15 * t - 0.2
        elif kind == "router":
            t = t * ((0.1 if steady else 3.0) / math.sqrt(shape[1]))
        else:
            # milder matrices in the steady models: a design that norms every sublayer's output doubles a
            # rounding error from layer to layer when its softmaxes and gates are sharp
            t = t * ((1.0 if steady else 1.6) / math.sqrt(shape[1]))
        out[name] = t.to(dt)
    return out


def write_folder(cfg, weights):
    folder = tempfile.mkdtemp(prefix="bfi_bepilorn_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    for name, t in weights.items():
        raw = t.contiguous().view(torch.uint8).numpy().tobytes() if t.dtype != BF16 else \
            t.contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": {F32: "F32", BF16: "BF16"}[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    return folder


_MODELS = {}


def model(name, dtype, seed=3):
    """(folder, config, float64 weights as stored) of a test model; the store is the run dtype's."""
    key = (name, dtype, seed)
    if key not in _MODELS:
        cfg = CONFIGS[name]
        w = make_weights(cfg, seed, F32 if dtype == "float32" else BF16, steady=dtype != "float32")
        _MODELS[key] = (write_folder(cfg, w), cfg, {k: v.to(torch.float64) for k, v in w.items()})
    return _MODELS[key]


def prompts(vocab, lengths, seed=5):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def _divisors(n):
    return [d for d in range(1, n + 1) if n % d == 0]


def random_config(seed):
    """A configuration drawn from a seed: two to five layers in any order, sizes from lists that hold
    odd ones and ones past what the register kernels take, chunks that are and are not whole pages,
    routers with and without groups, layers with and without a feed-forward or a shared expert."""
    import random
    rng = random.Random(seed)
    width = rng.choice([48, 64, 96, 160, 256])
    layers = []
    for _ in range(rng.randint(2, 5)):
        if rng.random() < 0.55:
            heads, vdim = rng.choice([1, 2, 3, 4, 6, 8]), rng.choice([8, 16, 24, 32, 48, 64])
            mixer = ssm(heads, vdim, rng.choice([4, 16, 48, 64, 96, 136]), rng.choice(_divisors(heads)), rng.choice([1, 2, 3, 4, 6]),
                        rng.choice([g for g in _divisors(heads * vdim) if g <= 8]))
            kind = "mamba2"
        else:
            heads = rng.choice([1, 2, 4, 6, 8])
            kv, dim = rng.choice(_divisors(heads)), rng.choice([16, 32, 48, 64, 80, 128])
            vdim, chunk = rng.choice([8, 16, 32, 64, 128, dim]), rng.choice([None, 7, 33, 64, 100, 128, 200])
            rot = (rng.choice([100.0, 1e4, 5e5]), rng.choice(list(range(2, dim + 1, 2)))) if rng.random() < 0.8 else None
            left = soft(heads, kv, dim, vdim, rng.choice([0.05, 0.125, dim ** -0.5, 0.3]), chunk, rot)
            right = gla(rng.choice([1, 2, 3, 4]), rng.choice([8, 16, 48, 64, 144]), rng.choice([8, 16, 40, 64, 128]),
                        rng.choice([1.0, 4.0, 16.0, 64.0]), rng.choice([4, 16, 24]))
            mixer = par(left, right, rng.choice([0.3, 0.7, 1.0, -0.5]), rng.choice([0.4, 1.0, 1.7]))
            kind = "parallel"
        mlp = None
        if rng.random() < 0.85:
            experts = rng.choice([2, 4, 6, 8, 12, 16, 32])
            count = rng.choice(_divisors(experts))
            keep = rng.randint(1, count)
            top = rng.randint(1, min(keep * (experts // count), 6))
            mlp = moe(experts, top, rng.choice([8, 20, 32, 64, 72]), count if rng.random() < 0.8 else None, keep, rng.choice([None, 16, 40, 96]))
            if "groups" not in mlp["router"]:
                mlp["router"]["top"] = min(top, experts)
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Bepilorn", "vocab": rng.choice([97, 256, 333, 1000]), "width": width, "norm": {"eps": rng.choice([1e-6, 1e-5])},
            "logit_scale": rng.choice([0.5, 1.0, 0.7]), "layers": layers}
