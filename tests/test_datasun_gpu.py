"""Datasun through the package against the plain implementation (tests/plain/datasun_plain.py):
every mechanism's kernel alone, then whole models with sizes of their own, stepped whole, token by
token, in portions, in unequal batches, over reused slots and pages, and generated from greedily.

The weights are made here (larger than the package's random fill, so that softmaxes are sharp and
clamps bite), and some tests shape them or their inputs so that one key, one edge or the sink
decides the result."""
import json
import math
import os
import struct
import tempfile

import pytest
import torch

from helpers import rel_err
from plain import datasun_plain as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
F32, BF16 = torch.float32, torch.bfloat16


def tol(dt):
    return 2e-5 if dt in (F32, "float32") else 2.5e-2


def ops():
    from builderforce_inference_b200.kernels import ops as o
    return o


def i32(xs):
    return torch.tensor(xs, dtype=torch.int32, device=DEV)


def q64(t, dt):
    """The values a tensor of storage type ``dt`` holds, as float64."""
    return t.to(dt).to(torch.float64)


# ------------------------------------------------------------------------------------------------
# model folders with weights of this file's making
# ------------------------------------------------------------------------------------------------
def yarn(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def att(heads, kv, dim, scale, window=None, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = rot
    return m


def mlp(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


# odd sizes everywhere: head sizes 24 and 16, 2 of 4 and 3 of 3 kv heads, a window shorter than a page and
# one that crosses a page border, rotation over part of a head and over all of it, scaled and unscaled
# frequencies, a layer without window and rotation, a layer without feed-forward, vdim above and below dim
DS_ODD = {"architecture": "Datasun", "vocab": 131, "width": 40, "norm": {"eps": 2e-5}, "embedding": {"scale": 1.7},
          "layers": [
              {"type": "attention", "mixer": att(4, 2, 24, 0.21, 9, {"base": 5000.0, "dims": 12, "scaling": yarn(4.0, 64, 16.0, 2.0)}),
               "mlp": mlp(56, 0.8)},
              {"type": "lightning", "mixer": {"heads": 3, "dim": 8, "vdim": 20, "decay": [0.5, 0.93, 0.999]}, "mlp": None},
              {"type": "attention", "mixer": att(3, 3, 16, 0.3, 70, {"base": 100.0, "dims": 16}), "mlp": mlp(72, 2.5)},
              {"type": "lightning", "mixer": {"heads": 2, "dim": 24, "vdim": 8, "decay": [0.97, 0.8]}, "mlp": mlp(56, 0.8)},
              {"type": "attention", "mixer": att(2, 1, 32, 0.15), "mlp": mlp(24, 1.1)}]}
# the sizes the bfloat16 tensor-core kernels take: attention heads of 64 and 128, recurrent heads of 64 and 128
DS_WIDE = {"architecture": "Datasun", "vocab": 300, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.6},
           "layers": [
               {"type": "lightning", "mixer": {"heads": 2, "dim": 64, "vdim": 64, "decay": [0.9, 0.995]}, "mlp": mlp(192, 1.5)},
               {"type": "attention", "mixer": att(8, 2, 64, 0.11, 100, {"base": 1e4, "dims": 32, "scaling": yarn(2.0, 128, 8.0, 1.0)}),
                "mlp": mlp(192, 1.5)},
               {"type": "lightning", "mixer": {"heads": 2, "dim": 32, "vdim": 128, "decay": [0.7, 0.98]}, "mlp": mlp(160, 3.0)},
               {"type": "attention", "mixer": att(2, 2, 128, 0.08, 40, {"base": 1e6, "dims": 128}), "mlp": None}]}
CONFIGS = {"odd": DS_ODD, "wide": DS_WIDE}


def tensor_shapes(cfg):
    """name -> (shape, kind) of every tensor of a Datasun model, from its config alone."""
    w = cfg["width"]
    out = {"embed": ((cfg["vocab"], w), "table"), "final.norm": ((w,), "norm")}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = ((w,), "norm")
        if layer["type"] == "attention":
            nq, nk = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
            out.update({p + "mix.q": ((nq, w), "matrix"), p + "mix.q.b": ((nq,), "bias"), p + "mix.k": ((nk, w), "matrix"),
                        p + "mix.k.b": ((nk,), "bias"), p + "mix.q.norm": ((nq,), "norm"), p + "mix.k.norm": ((nk,), "norm"),
                        p + "mix.o": ((w, nq), "matrix"), p + "mix.o.b": ((w,), "bias")})
        else:
            nq, nv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            out.update({p + "mix.q": ((nq, w), "matrix"), p + "mix.k": ((nq, w), "matrix"), p + "mix.v": ((nv, w), "matrix"),
                        p + "mix.g": ((nv, w), "matrix"), p + "mix.o": ((w, nv), "matrix"), p + "mix.norm": ((nv,), "norm")})
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            out.update({p + "mlp.gate": ((ff, w), "matrix"), p + "mlp.up": ((ff, w), "matrix"), p + "mlp.down": ((w, ff), "matrix")})
    return out


def make_weights(cfg, seed, dt):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        t = torch.randn(shape, generator=g)
        if kind == "norm":
            t = 1.0 + 0.2 * t
        elif kind == "bias":
            t = 0.3 * t
        elif kind == "table":
            t = 0.7 * t
        else:
            t = t * (1.6 / math.sqrt(shape[1]))
        out[name] = t.to(dt)
    return out


def write_folder(cfg, weights):
    folder = tempfile.mkdtemp(prefix="bfi_datasun_")
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
        w = make_weights(cfg, seed, F32 if dtype == "float32" else BF16)
        _MODELS[key] = (write_folder(cfg, w), cfg, {k: v.to(torch.float64) for k, v in w.items()})
    return _MODELS[key]


def engine(name, dtype, **kw):
    from builderforce_inference_b200.engine.engine import Engine
    folder, cfg, w = model(name, dtype)
    return Engine.load(folder, dtype=dtype, max_tokens=kw.pop("max_tokens", 2048), **kw), cfg, w


def prompts(vocab, lengths, seed=5):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def S(slot, tokens, want=None):
    from builderforce_inference_b200.engine.engine import SequenceStep
    return SequenceStep(slot, tokens, list(range(len(tokens))) if want is None else want)


# ------------------------------------------------------------------------------------------------
# the kernels, one mechanism each
# ------------------------------------------------------------------------------------------------
class Pages:
    """A hand-made paged cache whose pages are handed out in a scrambled order and start as NaN."""

    def __init__(self, n_slots, max_len, n_kv, d, dt, window=None, seed=0):
        from builderforce_inference_b200.cache import KVView
        blocks = (max_len + 63) // 64
        n_pages = n_slots * blocks + 3
        perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
        self.table = torch.tensor(perm[:n_slots * blocks], dtype=torch.int32).reshape(n_slots, blocks)
        self.k = torch.full((n_pages, n_kv, 64, d), float("nan"), dtype=dt, device=DEV)
        self.v = torch.full((n_pages, n_kv, 64, d), float("nan"), dtype=dt, device=DEV)
        self.view = KVView(self.k, self.v, self.table.to(DEV), n_kv, d, window)

    def write(self, slot, pos0, k, v):
        for t in range(k.shape[0]):
            p = pos0 + t
            page = int(self.table[slot, p // 64])
            self.k[page, :, p % 64, :] = k[t].to(self.k.dtype).to(DEV)
            self.v[page, :, p % 64, :] = v[t].to(self.v.dtype).to(DEV)

    def read(self, slot, n):
        k = torch.stack([self.k[int(self.table[slot, p // 64]), :, p % 64, :] for p in range(n)])
        v = torch.stack([self.v[int(self.table[slot, p // 64]), :, p % 64, :] for p in range(n)])
        return k.double().cpu(), v.double().cpu()


def run_paged(q, pages, seqs, n_q, scale, dt, sink):
    cu = [0]
    for _, _, t in seqs:
        cu.append(cu[-1] + t)
    out = torch.full((cu[-1], q.shape[1]), float("nan"), dtype=dt, device=DEV)
    ops().attention_paged(q.to(dt).to(DEV), q.shape[1], out, pages.view, i32(cu), i32([s for s, _, _ in seqs]),
                          i32([st for _, st, _ in seqs]), len(seqs), max(t for _, _, t in seqs), n_q, scale, sink)
    return out.double().cpu()


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("n_q,n_kv,d,window,sink", [(4, 2, 24, 9, 0.0), (6, 1, 64, 70, 0.0), (3, 3, 40, None, 1.5),
                                                    (2, 2, 128, 64, -2.0)])
def test_sink_attention_kernel_in_a_mixed_batch(dt, n_q, n_kv, d, window, sink):
    g = torch.Generator().manual_seed(n_q * 100 + d)
    seqs = [(2, 0, 75), (0, 130, 1), (1, 61, 7)]          # a prompt, a single token far in, a continuation over a page border
    pages = Pages(3, 256, n_kv, d, dt, window)
    qs, refs = [], []
    for slot, start, t in seqs:
        k = torch.randn(start + t, n_kv, d, generator=g)
        v = torch.randn(start + t, n_kv, d, generator=g)
        q = torch.randn(t, n_q, d, generator=g)
        pages.write(slot, 0, k, v)
        kk, vv = pages.read(slot, start + t)
        refs.append(P.sink_attention(q64(q, dt), kk, vv, 0.2, window, sink, start).reshape(t, n_q * d))
        qs.append(q.reshape(t, n_q * d))
    got = run_paged(torch.cat(qs), pages, seqs, n_q, 0.2, dt, sink)
    assert rel_err(got, torch.cat(refs)) < (3e-6 if dt == F32 else 1e-2)


@pytest.mark.parametrize("dt", [F32, BF16])
def test_the_sink_takes_the_weight_when_every_score_is_low_and_none_when_one_is_high(dt):
    n_q = n_kv = 1
    d, n = 16, 50
    pages = Pages(1, 64, n_kv, d, dt)
    k = torch.zeros(n, 1, d)
    k[:, 0, 0] = 1.0
    v = torch.ones(n, 1, d)
    pages.write(0, 0, k, v)
    for q0, want in ((-30.0, 0.0), (30.0, 1.0), (0.0, 50.0 / 51.0)):
        q = torch.zeros(1, d)
        q[0, 0] = q0
        got = run_paged(q, pages, [(0, n - 1, 1)], n_q, 1.0, dt, 0.0)
        assert abs(float(got[0, 0]) - want) < 1e-2, (q0, got[0, 0])
    # without a sink the same rows average the values whatever the scores
    got = run_paged(torch.zeros(1, d), pages, [(0, n - 1, 1)], n_q, 1.0, dt, None)
    assert abs(float(got[0, 0]) - 1.0) < 1e-2


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("window", [5, 64, 65, 100])
def test_one_loud_key_just_inside_and_just_outside_the_window(dt, window):
    """Key ``far`` carries a score that beats everything and a value of its own: a query sees it
    exactly while its distance is below the window, in a prompt and as a single token."""
    d, n, far = 32, 230, 17
    pages = Pages(1, 256, 1, d, dt, window)
    g = torch.Generator().manual_seed(window)
    k = 0.1 * torch.randn(n, 1, d, generator=g)
    v = 0.1 * torch.randn(n, 1, d, generator=g)
    k[far, 0] = 0.0
    k[far, 0, 3] = 40.0
    v[far, 0] = 5.0
    pages.write(0, 0, k, v)
    q = 0.1 * torch.randn(n, d, generator=g)
    q[:, 3] = 1.0
    whole = run_paged(q, pages, [(0, 0, n)], 1, 1.0, dt, 0.0)
    for i in (far, far + window - 1, far + window, far + window + 1):
        if i >= n:
            continue
        alone = run_paged(q[i:i + 1], pages, [(0, i, 1)], 1, 1.0, dt, 0.0)
        seen = i - far < window
        for row in (whole[i], alone[0]):
            assert (float(row.mean()) > 4.5) == seen, (i, window, float(row.mean()))


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("n_q,n_kv,d,rot,norm", [(4, 2, 24, 12, "row"), (6, 1, 64, 16, "row"), (3, 3, 16, 16, "head"),
                                                 (2, 1, 32, 0, None)])
def test_prepare_kernel_bias_row_norm_adjacent_rotation_values_from_keys(dt, n_q, n_kv, d, rot, norm):
    from builderforce_inference_b200.parts.rotary import rotary_table
    o = ops()
    g = torch.Generator().manual_seed(d + rot)
    T, width, eps = 9, 20, 3e-5
    scaling = yarn(3.0, 40, 6.0, 1.5) if rot == 12 else None
    pos = [0, 1, 2, 63, 64, 65, 100, 7, 8]
    slots = [0, 0, 0, 0, 0, 0, 0, 1, 1]
    pages = Pages(2, 128, n_kv, d, dt)
    qk = torch.randn(T, (n_q + n_kv) * d, generator=g).to(dt)
    bq, bk, bo = (0.5 * torch.randn(n, generator=g).to(dt) for n in (n_q * d, n_kv * d, width))
    nq_w = (1 + 0.3 * torch.randn(n_q * d if norm == "row" else d, generator=g)).to(dt)
    nk_w = (1 + 0.3 * torch.randn(n_kv * d if norm == "row" else d, generator=g)).to(dt)
    res = torch.randn(T, width, generator=g)
    table = rotary_table(777.0, rot, 128, DEV, scaling) if rot else None
    buf, res_dev = qk.clone().to(DEV), res.clone().to(DEV)
    o.qk_prepare(buf, n_q, n_kv, d, i32(pos), i32(slots), pages.view, o.FLAG_WRITE_CACHE | o.FLAG_VALUES_ARE_KEYS,
                 q_bias=bq.to(DEV), k_bias=bk.to(DEV), q_norm_w=nq_w.to(DEV) if norm else None,
                 k_norm_w=nk_w.to(DEV) if norm else None,
                 norm_mode={None: o.NORM_NONE, "head": o.NORM_HEAD, "row": o.NORM_ROW}[norm], eps=eps, rope_table=table,
                 rot_dim=rot, pairing=o.PAIR_ADJACENT, residual=res_dev, out_bias=bo.to(DEV))
    q = qk[:, :n_q * d].double() + bq.double()
    k = qk[:, n_q * d:].double() + bk.double()
    v_ref = k.reshape(T, n_kv, d)
    if norm == "row":
        q, k = P.rms_norm(q, nq_w.double(), eps), P.rms_norm(k, nk_w.double(), eps)
    q, k = q.reshape(T, n_q, d), k.reshape(T, n_kv, d)
    if norm == "head":
        q, k = P.rms_norm(q, nq_w.double(), eps), P.rms_norm(k, nk_w.double(), eps)
    if rot:
        q, k = (P.rotate_adjacent(x, pos, 777.0, rot, scaling) for x in (q, k))
    t = 3e-6 if dt == F32 else 1e-2
    assert rel_err(buf[:, :n_q * d].double().cpu(), q.reshape(T, -1)) < t
    for i, (p, s) in enumerate(zip(pos, slots)):
        page = int(pages.table[s, p // 64])
        assert rel_err(pages.k[page, :, p % 64].double().cpu(), k[i]) < t, i
        assert rel_err(pages.v[page, :, p % 64].double().cpu(), v_ref[i]) < t, i
    assert rel_err(res_dev.cpu(), res.double() + bo.double()) < 1e-6


def test_rotation_table_with_scaled_frequencies():
    from builderforce_inference_b200.parts.rotary import rotary_table
    for base, dims, sc in ((3e5, 24, yarn(3.0, 256, 24.0, 1.5)), (5000.0, 12, yarn(4.0, 64, 16.0, 2.0)), (100.0, 8, None),
                           (1e4, 64, yarn(8.0, 4096, 32.0, 1.0))):
        f, mag = P.rotary_frequencies(base, dims, sc)
        ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None]
        table = rotary_table(base, dims, 300, "cpu", sc).double()
        assert torch.allclose(table[..., 0], torch.cos(ang) * mag, atol=1e-6)
        assert torch.allclose(table[..., 1], torch.sin(ang) * mag, atol=1e-6)
        if sc:      # the ramp really splits the frequencies: the fastest is untouched, the slowest divided
            plain, _ = P.rotary_frequencies(base, dims)
            assert abs(float(f[0] / plain[0]) - 1.0) < 1e-12 and abs(float(f[-1] / plain[-1]) - 1.0 / sc["factor"]) < 1e-12


def scan(proj, state, decay, seqs, H, D, V, few=False):
    """seqs: [(slot, rows)] over consecutive rows of proj; returns o [rows, H*V] (float64, cpu)."""
    cu = [0]
    for _, n in seqs:
        cu.append(cu[-1] + n)
    o = torch.full((cu[-1], H * V), float("nan"), dtype=F32, device=DEV)
    ops().lightning_scan(proj, 0, H * D, 2 * H * D, o, state, decay, i32(cu), i32([s for s, _ in seqs]), len(seqs), H, D, V,
                         ops().LIGHT_ACT_SILU, few, few and all(n == 1 for _, n in seqs))
    return o.double().cpu()


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("H,D,V", [(3, 8, 20), (2, 64, 64), (1, 24, 130), (4, 128, 32)])
def test_lightning_kernel_whole_in_portions_and_token_by_token(dt, H, D, V):
    g = torch.Generator().manual_seed(H * D + V)
    lens = [150, 1, 67]
    slots = [3, 0, 2]
    decay = [0.999, 0.6, 0.93, 0.97][:H]
    dec = torch.tensor(decay, dtype=F32, device=DEV)
    cols = 2 * H * D + 2 * H * V
    projs = [torch.randn(n, cols, generator=g).to(dt) for n in lens]
    projs[0][5] *= 6.0                                   # one loud early token: it lasts under decay 0.999 and not under 0.6
    refs = []
    for p in projs:
        x = P.silu(p.double())
        n = p.shape[0]
        o, S = P.lightning_recurrence(x[:, :H * D].reshape(n, H, D), x[:, H * D:2 * H * D].reshape(n, H, D),
                                      x[:, 2 * H * D:2 * H * D + H * V].reshape(n, H, V), decay)
        refs.append((o.reshape(n, H * V), S))
    t = 2e-5 if dt == F32 else 2e-5
    # whole, as one mixed batch
    state = torch.zeros(4, H, D, V, dtype=F32, device=DEV)
    state[1] = float("nan")                              # a slot nobody uses
    got = scan(torch.cat(projs).to(DEV), state, dec, list(zip(slots, lens)), H, D, V)
    at = 0
    for (o, S), n, s in zip(refs, lens, slots):
        assert rel_err(got[at:at + n], o) < t
        assert rel_err(state[s].double().cpu(), S) < t
        at += n
    # sequence 0 in portions of many sizes down to two tokens and one, the state carried between the calls
    state.zero_()
    cuts, at, outs = [64, 2, 1, 3, 65, 1, 1, 13], 0, []
    for c in cuts:
        outs.append(scan(projs[0][at:at + c].to(DEV), state, dec, [(3, c)], H, D, V, few=c == 1))
        at += c
    assert at == lens[0]
    assert rel_err(torch.cat(outs), refs[0][0]) < t
    assert rel_err(state[3].double().cpu(), refs[0][1]) < t


def test_lightning_chunked_kernel_against_the_plain_recurrence_on_the_same_bfloat16_values():
    """The tensor-core kernel rounds the activated q, k, v to bfloat16 and nothing else: against
    the plain recurrence on those rounded values it is exact to float32-like accuracy, whatever the
    decay; whole, in portions that end inside a chunk, and mixed with short sequences."""
    from builderforce_inference_b200.kernels import fast_ops
    for H, D, V, decay in ((2, 64, 64, [0.999, 0.6]), (3, 32, 128, [1.0, 0.93, 0.05]), (1, 128, 48, [0.97]), (2, 16, 16, [0.9, 0.5])):
        g = torch.Generator().manual_seed(H + D + V)
        lens, slots = [200, 9, 70], [3, 0, 2]
        dec = torch.tensor(decay, dtype=F32, device=DEV)
        cols = 2 * H * D + 2 * H * V
        projs = [torch.randn(n, cols, generator=g).to(BF16) for n in lens]
        projs[0][5] *= 6.0
        refs = []
        for p in projs:
            x = P.silu(p.double()).to(BF16).double()
            n = p.shape[0]
            o, S = P.lightning_recurrence(x[:, :H * D].reshape(n, H, D), x[:, H * D:2 * H * D].reshape(n, H, D),
                                          x[:, 2 * H * D:2 * H * D + H * V].reshape(n, H, V), decay)
            refs.append((o.reshape(n, H * V), S))

        def run(proj, state, seqs):
            cu = [0]
            for _, n in seqs:
                cu.append(cu[-1] + n)
            o = torch.full((cu[-1], H * V), float("nan"), dtype=F32, device=DEV)
            assert fast_ops.lightning_chunks_bf16(proj.to(DEV), 0, H * D, 2 * H * D, o, state, dec, i32(cu),
                                                  i32([s for s, _ in seqs]), len(seqs), H, D, V)
            return o.double().cpu()

        state = torch.zeros(4, H, D, V, dtype=F32, device=DEV)
        got = run(torch.cat(projs), state, list(zip(slots, lens)))
        at = 0
        for (o, S), n, sl in zip(refs, lens, slots):
            assert rel_err(got[at:at + n], o) < 3e-3, (H, D, V)
            assert rel_err(state[sl].double().cpu(), S) < 3e-3
            at += n
        state.zero_()
        outs, at = [], 0
        for c in (64, 2, 70, 63, 1):
            outs.append(run(projs[0][at:at + c], state, [(3, c)]))
            at += c
        assert at == lens[0] and rel_err(torch.cat(outs), refs[0][0]) < 3e-3
        # and the two kernels agree on a state they hand to one another
        mid = scan(projs[0][:100].to(DEV), state.zero_(), dec, [(3, 100)], H, D, V)
        rest = run(projs[0][100:], state, [(3, 100)])
        assert rel_err(torch.cat([mid, rest]), refs[0][0]) < 3e-3
    assert not fast_ops.lightning_chunks_bf16(torch.zeros(4, 2 * 24 + 2 * 20, dtype=BF16, device=DEV), 0, 24, 48,
                                              torch.zeros(4, 20, device=DEV), torch.zeros(1, 1, 24, 20, device=DEV),
                                              torch.ones(1, device=DEV), i32([0, 4]), i32([0]), 1, 1, 24, 20)


class StepShape:
    """The fields of a step context the bfloat16 attention kernels read."""

    def __init__(self, seqs):
        from builderforce_inference_b200.engine.context import Workspace
        cu = [0]
        for _, _, t in seqs:
            cu.append(cu[-1] + t)
        self.n_seqs, self.n_tokens = len(seqs), cu[-1]
        self.max_seq_tokens = max(t for _, _, t in seqs)
        self.cu_seqlens, self.seq_slot, self.seq_start = i32(cu), i32([s for s, _, _ in seqs]), i32([st for _, st, _ in seqs])
        self.workspace = Workspace(DEV)


@pytest.mark.parametrize("kernel", ["decode", "mma", "tcgen05"])
@pytest.mark.parametrize("n_q,n_kv,d,window,sink", [(8, 2, 64, 100, 0.0), (6, 1, 64, 40, 0.0), (4, 4, 128, None, 2.0), (2, 1, 128, 70, -1.0)])
def test_sink_in_the_bfloat16_attention_kernels(kernel, n_q, n_kv, d, window, sink, monkeypatch):
    from builderforce_inference_b200.kernels import fast_ops
    g = torch.Generator().manual_seed(n_q + d)
    if kernel == "decode":
        seqs = [(0, 0, 1), (1, 63, 1), (2, 64, 1), (3, 300, 1), (4, 39, 1), (5, 40, 1)]
    else:
        seqs = [(2, 0, 33), (0, 0, 1), (1, 31, 34), (4, 64, 64), (5, 0, 200), (3, 63, 130)]
    pages = Pages(6, 400, n_kv, d, BF16, window, seed=d)
    qs, refs = [], []
    for slot, start, t in seqs:
        k = torch.randn(start + t, n_kv, d, generator=g)
        v = torch.randn(start + t, n_kv, d, generator=g)
        q = torch.randn(t, n_q, d, generator=g)
        pages.write(slot, 0, k, v)
        kk, vv = pages.read(slot, start + t)
        refs.append(P.sink_attention(q64(q, BF16), kk, vv, 0.17, window, sink, start).reshape(t, n_q * d))
        qs.append(q.reshape(t, n_q * d))
    q_all = torch.cat(qs).to(BF16).to(DEV)
    ref = torch.cat(refs)
    fn = {"decode": fast_ops.attention_decode_bf16, "mma": fast_ops.attention_prefill_bf16,
          "tcgen05": fast_ops.attention_prefill_tcgen05_bf16}[kernel]
    for forced in ((None, 1, 3) if kernel == "decode" else (None,)):      # one page range per sequence, and several merged
        if forced is not None:
            monkeypatch.setattr(fast_ops, "decode_splits", lambda *a, f=forced: f)
        out = torch.full(q_all.shape, float("nan"), dtype=BF16, device=DEV)
        assert fn(StepShape(seqs), q_all, out, pages.view, n_q, 0.17, sink=sink)
        assert rel_err(out.double().cpu(), ref) < 1e-2, forced
        # the same launch without the sink differs: the test would see a sink that is left out
        out2 = torch.full(q_all.shape, float("nan"), dtype=BF16, device=DEV)
        assert fn(StepShape(seqs), q_all, out2, pages.view, n_q, 0.17)
        assert rel_err(out2.double().cpu(), ref) > 3e-2
    st = fast_ops.tc_status(DEV)
    assert int(st[0]) == 0
    st.zero_()


@pytest.mark.parametrize("dt", [F32, BF16])
def test_gate_mul_clamps_and_shifts(dt):
    g = torch.Generator().manual_seed(0)
    x = (3.0 * torch.randn(7, 2 * 50, generator=g)).to(dt)
    for alpha, limit, shift in ((1.702, 0.8, 1.0), (1.0, None, 0.0), (0.5, 2.5, -0.25)):
        out = torch.empty(7, 50, dtype=dt, device=DEV)
        ops().gate_mul(x.to(DEV), out, True, alpha, limit or 0.0, shift)
        ref = P.clamped_gate(x[:, 0::2].double(), x[:, 1::2].double(), limit, alpha, shift)
        assert rel_err(out.double().cpu(), ref) < (1e-6 if dt == F32 else 6e-3)
    assert float(x.abs().max()) > 2.5                    # the clamps had something to do


@pytest.mark.parametrize("dt", [F32, BF16])
def test_feed_forward_part_applies_the_clamped_gate_in_every_product_kernel(dt):
    """Few rows, many rows and 128+ rows take different matrix-product kernels; each applies the gate
    in its epilogue.  The plain SiLU form beside it must stay what it was."""
    from builderforce_inference_b200.engine.context import Workspace, build_context
    from builderforce_inference_b200.engine.decoder import Runtime
    from builderforce_inference_b200.parts import FEED_FORWARDS, PartSpec
    rt, ws = Runtime(DEV, dt), Workspace(DEV)
    width, inner = 96, 160
    g = torch.Generator().manual_seed(2)
    w = {"gate_proj": torch.randn(inner, width, generator=g) * 0.3, "up_proj": torch.randn(inner, width, generator=g) * 0.3,
         "down_proj": torch.randn(width, inner, generator=g) * 0.1}
    w = {k: v.to(dt) for k, v in w.items()}
    for params, (limit, slope, shift) in (({"gate_alpha": 1.702, "limit": 0.8, "up_shift": 1.0}, (0.8, 1.702, 1.0)),
                                          ({}, (None, 1.0, 0.0)), ({"gate_alpha": 0.5, "up_shift": -0.5}, (None, 0.5, -0.5))):
        ffn = FEED_FORWARDS.build(PartSpec("gated_mlp", dict(width=width, inner=inner, **params)))
        ffn.load_all({k: v.to(DEV) for k, v in w.items()}, rt)
        for rows in (1, 5, 40, 130, 300):
            h = torch.randn(rows, width, generator=g).to(dt)
            res = torch.randn(rows, width, generator=g)
            out = res.clone().to(DEV)
            ffn.forward(build_context([(0, 0, [1] * rows)], dt, ws, DEV), h.to(DEV), out)
            f = {k: v.double() for k, v in w.items()}
            act = P.clamped_gate(h.double() @ f["gate_proj"].t(), h.double() @ f["up_proj"].t(), limit, slope, shift)
            ref = res.double() + act @ f["down_proj"].t()
            assert rel_err(out, ref) < (5e-6 if dt == F32 else 1.5e-2), (params, rows)


@pytest.mark.parametrize("dt", [F32, BF16])
def test_gated_rmsnorm(dt):
    g = torch.Generator().manual_seed(1)
    x, gate = torch.randn(5, 70, generator=g) * 4, torch.randn(5, 100, generator=g).to(dt)
    w = (1 + 0.2 * torch.randn(70, generator=g)).to(dt)
    out = torch.empty(5, 70, dtype=dt, device=DEV)
    ops().gated_rmsnorm(x.to(DEV), gate.to(DEV)[:, 30:], w.to(DEV), 1e-3, out)
    ref = P.rms_norm(x.double(), w.double(), 1e-3) * torch.sigmoid(gate[:, 30:].double())
    assert rel_err(out.double().cpu(), ref) < (1e-6 if dt == F32 else 6e-3)


def test_embedding_scale():
    table = torch.randn(11, 24)
    out = torch.empty(3, 24, device=DEV)
    ops().embed_rows(table.to(DEV), i32([4, 0, 10]), out, None, 2.5)
    assert torch.equal(out.cpu(), table[[4, 0, 10]] * 2.5)


# ------------------------------------------------------------------------------------------------
# whole models through the engine
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_whole_prompts_and_every_layer(name, dtype):
    eng, cfg, w = engine(name, dtype)
    for p in prompts(cfg["vocab"], [1, 2, 9, 70, 150]):
        ref = P.forward(cfg, w, p)
        s = eng.acquire()
        assert rel_err(eng.step([S(s, p)]).cpu(), ref) < tol(dtype), len(p)
        eng.release(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,graphs", [("odd", True), ("odd", False), ("wide", True)])
def test_prompt_then_token_by_token_far_past_every_window(name, dtype, graphs):
    eng, cfg, w = engine(name, dtype, use_graphs=graphs)
    (p,) = prompts(cfg["vocab"], [260], seed=8)
    ref = P.forward(cfg, w, p)
    s = eng.acquire()
    got = [eng.step([S(s, p[:3])]).cpu().clone()]            # the first tokens, then one by one through two page borders
    for t in range(3, len(p)):
        got.append(eng.step([S(s, [p[t]])]).cpu().clone())
    assert rel_err(torch.cat(got), ref) < tol(dtype)
    eng.release(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_portions_of_a_prompt_down_to_two_tokens(name, dtype):
    eng, cfg, w = engine(name, dtype, prefill_chunk_tokens=64)    # the engine cuts long portions itself as well
    (p,) = prompts(cfg["vocab"], [200], seed=9)
    ref = P.forward(cfg, w, p)
    for cuts in ([2, 2, 60, 1, 64, 71], [130, 2, 68], [63, 1, 1, 135]):
        s = eng.acquire()
        got, at = [], 0
        for c in cuts:
            got.append(eng.step([S(s, p[at:at + c])]).cpu().clone())
            at += c
        assert at == len(p) and rel_err(torch.cat(got), ref) < tol(dtype), cuts
        eng.release(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_unequal_batches_reused_slots_and_poisoned_pages(name, dtype):
    eng, cfg, w = engine(name, dtype, max_tokens=1024)
    ps = prompts(cfg["vocab"], [90, 3, 41, 140], seed=10)
    refs = [P.forward(cfg, w, p) for p in ps]
    for round_ in range(2):                                   # the second round reuses slots, pages and states
        eng.cache.poison()
        slots = [eng.acquire() for _ in ps]
        pre = [70, 2, 40, 129]
        lg = eng.step([S(s, p[:k]) for s, p, k in zip(slots, ps, pre)]).cpu().clone()
        got, o = [[] for _ in ps], 0
        for i, k in enumerate(pre):
            got[i].append(lg[o:o + k])
            o += k
        pos, live = list(pre), list(range(len(ps)))
        while live:
            lg = eng.step([S(slots[i], [ps[i][pos[i]]]) for i in live]).cpu().clone()
            for j, i in enumerate(live):
                got[i].append(lg[j:j + 1])
                pos[i] += 1
            for i in list(live):
                if pos[i] == len(ps[i]):
                    eng.release(slots[i])
                    live.remove(i)
        for i, r in enumerate(refs):
            assert rel_err(torch.cat(got[i]), r) < tol(dtype), (round_, i)
        eng.cache.check()
    shapes = {(m["heads"], m["dim"], m["vdim"]) for m in (x["mixer"] for x in cfg["layers"] if x["type"] == "lightning")}
    assert len(eng.cache.state_groups) == len(shapes)


def test_batch_against_each_alone_to_the_bit_in_float32():
    eng, cfg, w = engine("odd", "float32")
    ps = prompts(cfg["vocab"], [30, 77, 5], seed=11)
    alone = []
    for p in ps:
        s = eng.acquire()
        alone.append(eng.step([S(s, p)]).cpu().clone())
        eng.release(s)
    slots = [eng.acquire() for _ in ps]
    together = eng.step([S(s, p) for s, p in zip(slots, ps)]).cpu()
    assert rel_err(together, torch.cat(alone)) < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_public_entry_point(dtype):
    from builderforce_inference_b200 import Model, SampleParams
    folder, cfg, w = model("odd", dtype)
    m = Model.load(folder, dtype=dtype, max_tokens=2048)
    ps = prompts(cfg["vocab"], [12, 3, 70], seed=12)
    outs = m.generate_batch(ps, SampleParams(max_tokens=20), ignore_eos=True)
    for p, out in zip(ps, outs):
        if dtype == "float32":
            assert list(out) == P.greedy(cfg, w, p, 20)
        else:   # bfloat16: every chosen id is the plain model's choice for the same history, or within rounding of it
            ids = list(p)
            for t in out:
                lg = P.forward(cfg, w, ids)[-1]
                assert float(lg.max() - lg[t]) < 0.05 * float(lg.abs().max()), (len(ids), t)
                ids.append(int(t))


def test_trace_replay_and_command_line_take_the_model():
    folder, cfg, w = model("odd", "float32")
    (p,) = prompts(cfg["vocab"], [40], seed=13)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": p[:33], "want": [0, 32]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": p[33:34], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": p[34:], "want": [5]}], "end": ["a"]}]
    import numpy as np
    import subprocess
    import sys
    out_dir = tempfile.mkdtemp(prefix="bfi_trace_")
    from helpers import ROOT
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", out_dir, "--max-tokens", "128"], input="".join(json.dumps(s) + "\n" for s in steps),
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    ref = P.forward(cfg, w, p)
    got = [np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"]) for i in range(3)]
    assert rel_err(torch.from_numpy(np.concatenate(got)), ref[[0, 32, 33, 39]]) < 2e-5
