"""A plain, slow implementation of the Bepilorn design: whole sequences, no cache, float64, one
function per mechanism, written from the design's equations and sharing nothing with the
package.  The tests compare the package's kernels, parts and engine with it.

Notation: ``x`` is the residual stream ``[T, width]``; ``h`` a normed copy of it; linear weights
are ``[out, in]`` and act as ``W x``; ``w[name]`` is a tensor of the checkpoint.

A layer is ``x += norm1b(mixer(norm1(x)))`` and, when it has a feed-forward,
``x += norm2b(ff(norm2(x)))``; every one of these norms multiplies by ``1 + weight``.
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


# ------------------------------------------------------------------------------- small functions
def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    """log(1 + e^z), evaluated so that large |z| neither overflows nor loses the small term."""
    return torch.clamp(z, min=0.0) + torch.log1p(torch.exp(-z.abs()))


def rms(x, eps):
    """x divided by its root mean square over the last dimension; eps sits inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x, weight, eps):
    """The block's norm: the weight is stored around zero and enters as 1 + weight."""
    return rms(x, eps) * (1.0 + weight)


# ------------------------------------------------------------------------------- rotary
def rotate_half(x, positions, base, dims):
    """x [T, heads, d].  Of each head's first ``dims`` values, value i (i < dims/2) and value
    i + dims/2 form a pair that turns by the angle position * base^(-2i/dims); the rest pass."""
    half = dims // 2
    i = torch.arange(half, dtype=F)
    freq = torch.tensor(float(base), dtype=F) ** (-2.0 * i / dims)
    ang = torch.as_tensor(list(positions), dtype=F)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ------------------------------------------------------------------------------- softmax attention
def chunk_sink_attention(q, k, v, scale, chunk=None, sink=None, first_position=0):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key/value head h // (H/G).
    Token i (position first_position + i) sees token j <= i, and with ``chunk`` only if both
    positions fall into the same block of ``chunk`` consecutive positions counted from 0.
    ``sink`` [H]: one more term exp(sink_h) in the denominator, with no value."""
    T, H, d = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    pos = torch.arange(T) + first_position
    seen = pos[None, :] <= pos[:, None]
    if chunk is not None:
        seen &= (pos[None, :] // chunk) == (pos[:, None] // chunk)
    for h in range(H):
        g = h // rep
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = s.masked_fill(~seen, -math.inf)
        m = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            m = torch.clamp(m, min=float(sink[h]))
        e = torch.exp(s - m)
        den = e.sum(dim=-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - m)
        out[:, h, :] = (e / den) @ v[:, g, :]
    return out


def softmax_mixer(h, w, p, m, positions):
    """The softmax half of a parallel mixer: biased q/k/v projections, rotation of q and k,
    chunked causal attention with a learned sink per head, output projection."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        q = rotate_half(q, positions, rot["base"], rot["dims"])
        k = rotate_half(k, positions, rot["base"], rot["dims"])
    chunk = m["mask"]["size"] if m.get("mask") else None
    o = chunk_sink_attention(q, k, v, m["scale"], chunk, w[p + "sink"], first_position=positions[0])
    return o.reshape(T, H * dv) @ w[p + "o"].T


# ------------------------------------------------------------------------------- recurrences
def channel_decay_recurrence(q, k, v, alpha, state=None):
    """q, k, alpha [T, H, D]; v [T, H, V].  Per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T
    (S is D x V, the decay acts on rows) and o_t = S_t^T q_t.  Returns o [T, H, V] and S."""
    T, H, D = q.shape
    V = v.shape[-1]
    S = torch.zeros(H, D, V, dtype=F) if state is None else state.clone()
    o = torch.zeros(T, H, V, dtype=F)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o, S


def gated_linear_mixer(h, w, p, m, eps, state=None):
    """The recurrent half of a parallel mixer: q scaled by dim^(-1/2), a decay per key channel
    alpha = sigmoid(z)^(1/tau) with z from a two-step projection, the recurrence, an RMS norm of
    every head's output over vdim (plain weight, shared by the heads), a silu gate, W_o."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, V)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / m["tau"]).view(T, H, D)
    o, S = channel_decay_recurrence(q, k, v, alpha, state)
    o = rms(o, eps) * w[p + "norm"]
    y = o.reshape(T, H * V) * silu(h @ w[p + "g"].T)
    return y @ w[p + "o"].T, S


def causal_conv(u, weight, bias, history=None):
    """u [T, C]; weight [C, taps], the last column multiplies the current token; zeros (or
    ``history`` [taps-1, C], the inputs just before) come before the first token."""
    T, C = u.shape
    taps = weight.shape[1]
    past = torch.zeros(taps - 1, C, dtype=F) if history is None else history
    full = torch.cat([past, u], dim=0)
    out = torch.zeros(T, C, dtype=F)
    for j in range(taps):
        out += full[j:j + T] * weight[:, j]
    return out + bias, full[T:]


def state_space_mixer(h, w, p, m, eps, state=None, history=None):
    """Mamba-2: one projection gives z, x, B, C and dt; x, B, C pass a short causal convolution
    and silu; per head S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T and
    y_t = S_t^T C_t + D x_t; y is gated by silu(z), normed in equal parts, projected."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc, history = causal_conv(xbc, w[p + "conv"], w[p + "conv.b"], history)
    xbc = silu(xbc)
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])                       # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)         # [T, H]
    S = torch.zeros(H, N, P, dtype=F) if state is None else state.clone()
    y = torch.zeros(T, H, P, dtype=F)
    per = H // G
    for t in range(T):
        for hh in range(H):
            g = hh // per
            S[hh] = decay[t, hh] * S[hh] + dt[t, hh] * torch.outer(B[t, g], x[t, hh])
            y[t, hh] = S[hh].T @ C[t, g] + w[p + "D"][hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T, S, history


# ------------------------------------------------------------------------------- feed-forward
def gated_expert(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, router, correction, top, n_groups=1, keep=1, report=None):
    """Which experts each token uses and with which weights.  s = softmax(router h); the choice is
    made on s + correction: experts form ``n_groups`` equal groups of neighbours, a group counts by
    its best choice score, only experts of the ``keep`` best groups can be chosen, and of those
    the ``top`` best are; the weights are the chosen experts' s, not renormalised.  ``report`` (a
    list) receives the smallest gap by which any decision here was made."""
    s = torch.softmax(h @ router.T, dim=-1)
    choice = s + correction
    T, E = s.shape
    per = E // n_groups
    best = choice.view(T, n_groups, per).max(dim=-1).values
    kept = torch.zeros(T, n_groups, dtype=torch.bool)
    kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
    choice = choice.masked_fill(~kept.repeat_interleave(per, dim=1), -math.inf)
    idx = choice.topk(top, dim=-1).indices
    if report is not None:
        gaps = []
        if keep < n_groups:
            order = best.sort(dim=-1, descending=True).values
            gaps.append(float((order[:, keep - 1] - order[:, keep]).min()))
        if top < keep * per:
            order = choice.sort(dim=-1, descending=True).values
            gaps.append(float((order[:, top - 1] - order[:, top]).min()))
        report.append(min(gaps) if gaps else math.inf)
    return idx, s.gather(1, idx)


def mixture(h, w, p, mlp, report=None):
    r = mlp["router"]
    groups = r.get("groups") or {}
    count = groups.get("count", 1)
    idx, weight = route(h, w[p + "router"], w[p + "correction"], r["top"], count, groups.get("keep", count), report)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), weight[t]):
            out[t] += a * gated_expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + gated_expert(h, w, p + "shared.") * torch.sigmoid(h @ w[p + "shared.sg"].T)
    return out


# ------------------------------------------------------------------------------- the model
def forward(cfg, w, tokens, layer_outputs=None, report=None):
    """Logits [T, vocab] of a whole sequence that starts at position 0.  ``layer_outputs`` (a list)
    receives the residual stream after every layer, ``report`` every router's smallest gap."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(list(tokens))]
    T = x.shape[0]
    positions = list(range(T))
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = offset_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "mamba2":
            y, _, _ = state_space_mixer(h, w, p + "mix.", m, eps)
        elif layer["type"] == "parallel":
            left = softmax_mixer(h, w, p + "mix.left.", m["left"], positions)
            right, _ = gated_linear_mixer(h, w, p + "mix.right.", m["right"], eps)
            y = m["left_scale"] * left + m["right_scale"] * right
        else:
            raise ValueError(layer["type"])
        x = x + offset_norm(y, w[p + "norm1b"], eps)
        if layer.get("mlp"):
            h = offset_norm(x, w[p + "norm2"], eps)
            x = x + offset_norm(mixture(h, w, p + "mlp.", layer["mlp"], report), w[p + "norm2b"], eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return (offset_norm(x, w["final.norm"], eps) @ w["head"].T if "head" in w
            else offset_norm(x, w["final.norm"], eps) @ w["embed"].T) * cfg.get("logit_scale", 1.0)


def greedy(cfg, w, prompt, n_new):
    """The ids a greedy decoder appends to ``prompt`` (lowest id wins a tie)."""
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(torch.argmax(forward(cfg, w, ids)[-1])))
    return ids[len(prompt):]
