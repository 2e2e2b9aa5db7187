"""A plain, slow implementation of the Datasun design: whole sequences, no cache, float64, one
function per mechanism, written from the design's equations and sharing nothing with the
package.  The tests compare the package's kernels, parts and engine with it.

Notation: ``x`` is the residual stream ``[T, width]``; ``h`` a normed copy of it; linear weights
are ``[out, in]`` and act as ``W x``.
"""
import json
import math
import os
import struct

import torch

F = torch.float64


# ------------------------------------------------------------------------------- files
def read_tensors(path):
    """name -> tensor of a safetensors file (8-byte length, JSON header, raw data)."""
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(blob[a:b]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        out[name] = t.to(F) if t.is_floating_point() else t
    return out


def load_folder(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_tensors(os.path.join(folder, "model.safetensors"))


# ------------------------------------------------------------------------------- mechanisms
def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last dimension; eps sits inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def rotary_frequencies(base, dims, scaling=None):
    """The dims/2 angular frequencies and the factor on cos and sin.  Without scaling:
    f_i = base^(-2i/dims), factor 1.  With yarn scaling (factor s, original L, fast b, slow a):
    frequencies below the ramp keep f_i, those above it become f_i / s, linear in between."""
    i = torch.arange(dims // 2, dtype=F)
    f = torch.tensor(float(base), dtype=F) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    s, L, b, a = (float(scaling[k]) for k in ("factor", "original", "fast", "slow"))

    def turns_to_dim(t):
        return dims * math.log(L / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turns_to_dim(b)), 0)
    hi = min(math.ceil(turns_to_dim(a)), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / s * ramp + f * (1.0 - ramp), 0.1 * math.log(s) + 1.0


def rotate_adjacent(x, positions, base, dims, scaling=None):
    """x [T, heads, d]: values (2i, 2i+1), i < dims/2, of every head turn by positions * f_i;
    values from dims on pass unchanged."""
    f, mag = rotary_frequencies(base, dims, scaling)
    ang = torch.as_tensor(list(positions), dtype=F)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def sink_attention(q, k, v, scale, window=None, sink=None, first_position=0):
    """q [T, H, d] at positions first_position .. ; k, v [first_position + T, G, d] from position 0.
    Query at position i sees keys j with 0 <= i - j < window (all j <= i without a window).
    p_j = exp(s_j) / (exp(sink) + sum exp(s)) when there is a sink, the usual softmax otherwise."""
    T, H, d = q.shape
    G = k.shape[1]
    n = k.shape[0]
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    for t in range(T):
        i = first_position + t
        lo = 0 if window is None else max(0, i - window + 1)
        for hh in range(H):
            g = hh // (H // G)
            s = (k[lo:i + 1, g] @ q[t, hh]) * scale
            m = s.max() if sink is None else torch.maximum(s.max(), torch.tensor(float(sink), dtype=F))
            e = torch.exp(s - m)
            den = e.sum() + (0.0 if sink is None else math.exp(float(sink) - float(m)))
            out[t, hh] = (e / den) @ v[lo:i + 1, g]
    assert n >= first_position + T
    return out


def lightning_recurrence(q, k, v, decay, state=None):
    """q, k [T, H, D], v [T, H, V]; per head S <- decay_h S + k_t v_t^T, o_t = S^T q_t.
    Returns (o [T, H, V], the state after the last token [H, D, V])."""
    T, H, D = q.shape
    V = v.shape[-1]
    S = torch.zeros(H, D, V, dtype=F) if state is None else state.clone().to(F)
    w = torch.as_tensor(list(decay), dtype=F)
    o = torch.zeros(T, H, V, dtype=F)
    for t in range(T):
        for hh in range(H):
            S[hh] = w[hh] * S[hh] + torch.outer(k[t, hh], v[t, hh])
            o[t, hh] = S[hh].t() @ q[t, hh]
    return o, S


def silu(x):
    return x * torch.sigmoid(x)


def clamped_gate(g, u, limit=None, slope=1.702, shift=1.0):
    """min(g, limit) * sigmoid(slope * min(g, limit)) * (clamp(u, -limit, limit) + shift)."""
    if limit is not None:
        g = torch.clamp(g, max=limit)
        u = torch.clamp(u, -limit, limit)
    return g * torch.sigmoid(slope * g) * (u + shift)


# ------------------------------------------------------------------------------- sublayers
def attention_mixer(h, w, p, m, eps, first_position=0, h_before=None):
    """The attention mixer on h [T, width]; ``h_before`` are the normed inputs of the earlier tokens
    of the sequence (their keys are recomputed here: there is no cache)."""
    hh = h if h_before is None else torch.cat([h_before, h])
    n, T = hh.shape[0], h.shape[0]
    H, G, d = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    q = h @ w[p + "q"].t() + w[p + "q.b"]
    k = hh @ w[p + "k"].t() + w[p + "k.b"]
    v = k.reshape(n, G, d)                                   # the values are the keys as projected
    q = rms_norm(q, w[p + "q.norm"], eps).reshape(T, H, d)
    k = rms_norm(k, w[p + "k.norm"], eps).reshape(n, G, d)
    rot = m.get("rot")
    if rot:
        q = rotate_adjacent(q, range(first_position, first_position + T), rot["base"], rot["dims"], rot.get("scaling"))
        k = rotate_adjacent(k, range(n), rot["base"], rot["dims"], rot.get("scaling"))
    window = m["mask"]["size"] if m.get("mask") else None
    o = sink_attention(q, k, v, m.get("scale", d ** -0.5), window, 0.0, first_position)
    return o.reshape(T, H * d) @ w[p + "o"].t() + w[p + "o.b"]


def lightning_mixer(h, w, p, m, eps, state=None):
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m.get("vdim", m["dim"])
    q = silu(h @ w[p + "q"].t()).reshape(T, H, D)
    k = silu(h @ w[p + "k"].t()).reshape(T, H, D)
    v = silu(h @ w[p + "v"].t()).reshape(T, H, V)
    o, S = lightning_recurrence(q, k, v, m["decay"], state)
    y = rms_norm(o.reshape(T, H * V), w[p + "norm"], eps) * torch.sigmoid(h @ w[p + "g"].t())
    return y @ w[p + "o"].t(), S


def feed_forward(h, w, p, m):
    return clamped_gate(h @ w[p + "gate"].t(), h @ w[p + "up"].t(), m.get("limit")) @ w[p + "down"].t()


# ------------------------------------------------------------------------------- the model
def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of the whole sequence."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(list(tokens))] * cfg.get("embedding", {}).get("scale", 1.0)
    for i, layer in enumerate(cfg["layers"]):
        h = rms_norm(x, w[f"l{i}.norm1"], eps)
        if layer["type"] == "attention":
            y = attention_mixer(h, w, f"l{i}.mix.", layer["mixer"], eps)
        else:
            y, _ = lightning_mixer(h, w, f"l{i}.mix.", layer["mixer"], eps)
        if layer.get("mlp"):
            y = y + feed_forward(h, w, f"l{i}.mlp.", layer["mlp"])
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["embed"].t()


def greedy(cfg, w, prompt, n_new):
    """Greedy continuation (lowest index wins a tie), recomputing the sequence every step."""
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(torch.argmax(forward(cfg, w, ids)[-1])))
    return ids[len(prompt):]
