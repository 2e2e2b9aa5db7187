"""Bepilorn through the package against the plain implementation (tests/plain/bepilorn_plain.py):
every mechanism's kernel alone, then whole models with sizes of their own, stepped whole, token by
token, in portions, in unequal batches, over reused slots and pages, and generated from greedily.

Some tests shape their inputs so that one key, one edge, the sink or one expert decides the result."""
import json
import math
import os

import pytest
import torch

from bepilorn_models import BF16, CONFIGS, F32, make_weights, model, prompts, random_config, write_folder
from helpers import rel_err
from plain import bepilorn_plain as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def tol(dt):
    # bfloat16: the rounding of five layers whose outputs are all normed again; a lost state, a wrong key
    # or a turned choice shows as 0.3 and more
    return 3e-5 if dt in (F32, "float32") else 6e-2


def close(got, ref, dtype):
    """Whether a model's output is the plain implementation's.  float32: every value, to 3e-5 of the
    largest.  bfloat16: rounding is amplified where a token happens to be badly conditioned (a normed
    output that is nearly zero, a softmax on the edge), so 95 % of the rows (all but one, of few) must
    lie within the tolerance and every row must be finite and within 1; the float32 run is the sharp test."""
    if dtype in (F32, "float32"):
        return rel_err(got, ref) < tol(dtype)
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    if got.shape != ref.shape or not torch.isfinite(got).all():
        return False
    rows = (got - ref).abs().reshape(got.shape[0], -1).max(dim=1).values / max(1e-6, float(ref.abs().max()))
    return int((rows > tol(dtype)).sum()) <= max(1, rows.numel() // 20) and float(rows.max()) < 1.0


def ops():
    from builderforce_inference_b200.kernels import ops as o
    return o


def i32(xs):
    return torch.tensor(xs, dtype=torch.int32, device=DEV)


def q64(t, dt):
    """The values a tensor of storage type ``dt`` holds, as float64."""
    return t.to(dt).to(torch.float64)


def engine(name, dtype, **kw):
    from builderforce_inference_b200.engine.engine import Engine
    folder, cfg, w = model(name, dtype)
    return Engine.load(folder, dtype=dtype, max_tokens=kw.pop("max_tokens", 2048), **kw), cfg, w


def S(slot, tokens, want=None):
    from builderforce_inference_b200.engine.engine import SequenceStep
    return SequenceStep(slot, tokens, list(range(len(tokens))) if want is None else want)


def steady_prompt(cfg, w, length, dtype, seed0=5):
    """A prompt for a model test.  The bfloat16 models' routers decide by wide gaps (see
    ``bepilorn_models.make_weights``), which is checked here: rounding must not turn a choice."""
    ids = prompts(cfg["vocab"], [length], seed0)[0]
    if dtype != "float32":
        rep = []
        P.forward(cfg, w, ids, None, rep)
        assert min(rep) > 0.03, rep
    return ids


# ------------------------------------------------------------------------------------------------
# the attention kernel: values of their own size, chunks, a sink per head
# ------------------------------------------------------------------------------------------------
class Pages:
    """A hand-made paged cache whose pages are handed out in a scrambled order and start as NaN."""

    def __init__(self, n_slots, max_len, n_kv, d, dv, dt, chunk=None, seed=0):
        from builderforce_inference_b200.cache import KVView
        blocks = (max_len + 63) // 64
        n_pages = n_slots * blocks + 3
        perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
        self.table = torch.tensor(perm[:n_slots * blocks], dtype=torch.int32).reshape(n_slots, blocks)
        self.k = torch.full((n_pages, n_kv, 64, d), float("nan"), dtype=dt, device=DEV)
        self.v = torch.full((n_pages, n_kv, 64, dv), float("nan"), dtype=dt, device=DEV)
        self.view = KVView(self.k, self.v, self.table.to(DEV), n_kv, d, None, v_dim=dv, chunk=chunk)

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


def run_paged(q, pages, seqs, n_q, dv, scale, dt, sink):
    cu = [0]
    for _, _, t in seqs:
        cu.append(cu[-1] + t)
    out = torch.full((cu[-1], n_q * dv), float("nan"), dtype=dt, device=DEV)
    ops().attention_paged(q.to(dt).to(DEV), q.shape[1], out, pages.view, i32(cu), i32([s for s, _, _ in seqs]),
                          i32([st for _, st, _ in seqs]), len(seqs), max(t for _, _, t in seqs), n_q, scale,
                          None if sink is None else sink.float().to(DEV))
    return out.double().cpu()


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("n_q,n_kv,d,dv,chunk", [(4, 2, 24, 10, 9), (6, 3, 64, 24, 70), (3, 3, 16, 40, None), (2, 2, 32, 128, 64),
                                                 (8, 2, 64, 64, 128)])
def test_chunked_sink_attention_kernel_in_a_mixed_batch(dt, n_q, n_kv, d, dv, chunk):
    g = torch.Generator().manual_seed(n_q * 100 + d)
    seqs = [(2, 0, 150), (0, 130, 1), (1, 61, 7)]       # a prompt over chunk borders, a single token far in, a continuation
    pages = Pages(3, 256, n_kv, d, dv, dt, chunk)
    sink = torch.randn(n_q, generator=g)
    qs, refs = [], []
    for slot, start, t in seqs:
        k = torch.randn(start + t, n_kv, d, generator=g)
        v = torch.randn(start + t, n_kv, dv, generator=g)
        q = torch.randn(start + t, n_q, d, generator=g)
        pages.write(slot, 0, k, v)
        kk, vv = pages.read(slot, start + t)
        ref = P.chunk_sink_attention(q64(q, dt), kk, vv, 0.2, chunk, sink.double())
        refs.append(ref[start:].reshape(t, n_q * dv))
        qs.append(q[start:].reshape(t, n_q * d))
    got = run_paged(torch.cat(qs), pages, seqs, n_q, dv, 0.2, dt, sink)
    assert rel_err(got, torch.cat(refs)) < (3e-6 if dt == F32 else 1e-2)


@pytest.mark.parametrize("n_q,n_kv,d,chunk", [(8, 2, 64, 128), (4, 4, 128, 70), (2, 1, 64, 9), (4, 2, 128, None)])
def test_tensor_core_prompt_attention_with_chunks_and_a_sink_per_head(n_q, n_kv, d, chunk):
    """The bfloat16 kernel that steps with more than one token per sequence run when keys and values
    have one size of 64 or 128: the same mixed batch as above, through the choice the attention part makes."""
    from builderforce_inference_b200.engine.context import Workspace, build_context
    from builderforce_inference_b200.kernels import attention as choose
    from builderforce_inference_b200.kernels.library import library
    g = torch.Generator().manual_seed(n_q + d)
    seqs = [(2, 0, 150), (0, 130, 2), (1, 61, 7)]
    pages = Pages(3, 256, n_kv, d, d, BF16, chunk)
    sink = torch.randn(n_q, generator=g)
    qs, refs = [], []
    for slot, start, t in seqs:
        k, v, q = (torch.randn(start + t, h, d, generator=g) for h in (n_kv, n_kv, n_q))
        pages.write(slot, 0, k, v)
        kk, vv = pages.read(slot, start + t)
        ref = P.chunk_sink_attention(q64(q, BF16), kk, vv, 0.2, chunk, sink.double())
        refs.append(ref[start:].reshape(t, n_q * d))
        qs.append(q[start:].reshape(t, n_q * d))
    ctx = build_context([(slot, start, [0] * t) for slot, start, t in seqs], BF16, Workspace(DEV), DEV)
    qd = torch.cat(qs).to(BF16).to(DEV)
    out = torch.full((qd.shape[0], n_q * d), float("nan"), dtype=BF16, device=DEV)
    before = library("fast").calls
    assert choose.attend(ctx, qd, out, pages.view, n_q, 0.2, sink.float().to(DEV))
    assert library("fast").calls == before + 1
    assert rel_err(out, torch.cat(refs)) < 1.5e-2
    # with the weights kept float32 in effect (two bfloat16 terms each) only the output's own rounding is left
    exact = torch.full((qd.shape[0], n_q * d), float("nan"), dtype=BF16, device=DEV)
    assert choose.attend(ctx, qd, exact, pages.view, n_q, 0.2, sink.float().to(DEV), exact_weights=True)
    ref = torch.cat(refs)
    err_exact = float((exact.double().cpu() - ref).abs().max())
    assert err_exact <= float((out.double().cpu() - ref).abs().max()) + 1e-6
    assert float((exact.double().cpu() - ref.to(BF16).double()).abs().max()) <= 2.0 * float(ref.abs().max()) * 2.0 ** -9


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("chunk", [5, 64, 65, 100])
def test_one_loud_key_just_inside_and_just_outside_the_chunk(dt, chunk):
    """Among a few hundred quiet keys one key is loud (a large score with every query) and carries
    a value of its own.  A query reads it exactly when both lie in one chunk: the first position of
    the query's chunk is read, the last position of the chunk before is not, in a prompt and as a
    single decoded token."""
    n_q, n_kv, d, dv = 2, 1, 16, 8
    n = 3 * chunk + 3
    g = torch.Generator().manual_seed(chunk)
    sink = torch.zeros(n_q)
    for loud in (2 * chunk, 2 * chunk - 1, 3 * chunk - 1):
        k = 0.05 * torch.randn(n, n_kv, d, generator=g)
        v = 0.05 * torch.randn(n, n_kv, dv, generator=g)
        q = 0.05 * torch.randn(n, n_q, d, generator=g)
        k[loud, 0, 0], q[:, :, 0], v[loud, 0, :] = 40.0, 40.0, 7.0
        pages = Pages(2, n + 64, n_kv, d, dv, dt, chunk, seed=loud)
        pages.write(0, 0, k, v)
        pages.write(1, 0, k, v)
        kk, vv = pages.read(0, n)
        ref = P.chunk_sink_attention(q64(q, dt), kk, vv, 0.25, chunk, sink.double()).reshape(n, n_q * dv)
        whole = run_paged(q.reshape(n, -1), pages, [(0, 0, n)], n_q, dv, 0.25, dt, sink)
        assert rel_err(whole, ref) < (1e-5 if dt == F32 else 2e-2)
        for p in (loud, loud + 1, (loud // chunk + 1) * chunk - 1, (loud // chunk + 1) * chunk):
            if p >= n:
                continue
            one = run_paged(q[p:p + 1].reshape(1, -1), pages, [(1, p, 1)], n_q, dv, 0.25, dt, sink)
            assert rel_err(one, ref[p:p + 1]) < (1e-5 if dt == F32 else 2e-2)
            heard = abs(float(one[0, 0])) > 3.0
            assert heard == (p >= loud and p // chunk == loud // chunk), (loud, p)


@pytest.mark.parametrize("dt", [F32, BF16])
def test_one_loud_key_far_back_among_hundreds_and_the_first_tokens(dt):
    """Without a chunk every earlier key is read: a loud key at position 3 decides the output of a query
    400 positions on (in a prompt, as a continuation over a page border and as a single token), and the
    first three tokens, which come before it, do not hear it."""
    n_q, n_kv, d, dv, n, loud = 3, 1, 24, 12, 404, 3
    g = torch.Generator().manual_seed(17)
    k = 0.05 * torch.randn(n, n_kv, d, generator=g)
    v = 0.05 * torch.randn(n, n_kv, dv, generator=g)
    q = 0.05 * torch.randn(n, n_q, d, generator=g)
    k[loud, 0, 0], q[:, :, 0], v[loud, 0, :] = 40.0, 40.0, 7.0
    sink = torch.tensor([0.0, -1.0, 2.0])
    pages = Pages(3, n + 60, n_kv, d, dv, dt)
    for slot in range(3):
        pages.write(slot, 0, k, v)
    kk, vv = pages.read(0, n)
    ref = P.chunk_sink_attention(q64(q, dt), kk, vv, 0.25, None, sink.double()).reshape(n, n_q * dv)
    t = 1e-5 if dt == F32 else 2e-2
    whole = run_paged(q.reshape(n, -1), pages, [(0, 0, n)], n_q, dv, 0.25, dt, sink)
    assert rel_err(whole, ref) < t
    assert float(whole[:loud].abs().max()) < 1.0 and float(whole[loud:, 0].min()) > 3.0
    rest = run_paged(q[380:].reshape(n - 380, -1), pages, [(1, 380, n - 380)], n_q, dv, 0.25, dt, sink)
    assert rel_err(rest, ref[380:]) < t
    one = run_paged(q[n - 1:].reshape(1, -1), pages, [(2, n - 1, 1)], n_q, dv, 0.25, dt, sink)
    assert rel_err(one, ref[n - 1:]) < t and float(one[0, 0]) > 3.0
    first = run_paged(q[:1].reshape(1, -1), pages, [(2, 0, 1)], n_q, dv, 0.25, dt, sink)
    assert rel_err(first, ref[:1]) < t


@pytest.mark.parametrize("dt", [F32, BF16])
def test_a_sink_per_head_takes_the_weight_of_its_head_only(dt):
    n_q, n_kv, d, dv, n = 4, 2, 8, 4, 70
    g = torch.Generator().manual_seed(3)
    k, v, q = (0.1 * torch.randn(n, h, e, generator=g) for h, e in ((n_kv, d), (n_kv, dv), (n_q, d)))
    v += 1.0
    sink = torch.tensor([-30.0, 30.0, 0.0, 30.0])
    pages = Pages(1, n, n_kv, d, dv, dt)
    pages.write(0, 0, k, v)
    kk, vv = pages.read(0, n)
    ref = P.chunk_sink_attention(q64(q, dt), kk, vv, 1.0, None, sink.double())
    got = run_paged(q.reshape(n, -1), pages, [(0, 0, n)], n_q, dv, 1.0, dt, sink).reshape(n, n_q, dv)
    assert rel_err(got, ref) < (1e-5 if dt == F32 else 2e-2)
    assert float(got[:, 0].min()) > 0.5 and float(got[:, 1].abs().max()) < 1e-6 and float(got[:, 3].abs().max()) < 1e-6
    # the sink of score 0 is one more key: the first token's only key has weight exp(s) / (exp(s) + 1)
    s = float((q64(q, dt)[0, 2] * kk[0, 1]).sum())
    assert math.isclose(float(got[0, 2, 0]), float(vv[0, 1, 0]) * math.exp(s) / (math.exp(s) + 1.0), rel_tol=2e-2 if dt == BF16 else 1e-5)


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("n_q,n_kv,d,dv,rot", [(4, 2, 24, 10, 12), (2, 1, 16, 40, 16), (3, 3, 32, 32, 0)])
def test_prepare_kernel_with_values_of_their_own_size(dt, n_q, n_kv, d, dv, rot):
    from builderforce_inference_b200.parts.rotary import rotary_table
    g = torch.Generator().manual_seed(d + dv)
    n, start = 9, 60                                    # positions 60..68 cross a page border
    row = (n_q + n_kv) * d + n_kv * dv
    x = torch.randn(n, row, generator=g)
    bq, bk, bv = (0.5 * torch.randn(m, generator=g) for m in (n_q * d, n_kv * d, n_kv * dv))
    pages = Pages(1, 128, n_kv, d, dv, dt)
    qkv = x.to(dt).to(DEV)
    table = rotary_table(300.0, rot, 128, DEV) if rot else None
    o = ops()
    o.qk_prepare(qkv, n_q, n_kv, d, i32(list(range(start, start + n))), i32([0] * n), pages.view, o.FLAG_WRITE_CACHE,
                 q_bias=bq.to(dt).to(DEV), k_bias=bk.to(dt).to(DEV), v_bias=bv.to(dt).to(DEV), rope_table=table,
                 rot_dim=rot, v_dim=dv)
    xs = q64(x, dt)
    q = (xs[:, :n_q * d] + q64(bq, dt)).view(n, n_q, d)
    k = (xs[:, n_q * d:(n_q + n_kv) * d] + q64(bk, dt)).view(n, n_kv, d)
    v = (xs[:, (n_q + n_kv) * d:] + q64(bv, dt)).view(n, n_kv, dv)
    if rot:
        q = P.rotate_half(q, range(start, start + n), 300.0, rot)
        k = P.rotate_half(k, range(start, start + n), 300.0, rot)
    t = 1e-6 if dt == F32 else 8e-3
    assert rel_err(qkv[:, :n_q * d].double().cpu().view(n, n_q, d), q) < t
    for j in range(n):
        page, r = int(pages.table[0, (start + j) // 64]), (start + j) % 64
        assert rel_err(pages.k[page, :, r, :], k[j]) < t
        assert rel_err(pages.v[page, :, r, :], v[j]) < t


# ------------------------------------------------------------------------------------------------
# the recurrence, the convolution, the gated norm
# ------------------------------------------------------------------------------------------------
def scan(o, mode, dt, qk, v, raw, bias, rate, skip, seqs, state, H, D, V, hpg, q_scale=1.0, inv_tau=1.0, offs=(0, 0, 0, 0),
         chunk_len=0):
    cu = [0]
    for _, t in seqs:
        cu.append(cu[-1] + t)
    out = torch.full((cu[-1], H * V), float("nan"), dtype=F32, device=DEV)
    f = lambda t: None if t is None else t.float().to(DEV)
    chunked = {}
    if chunk_len:
        n_chunks = cu[-1] // chunk_len + len(seqs)
        chunked = {"chunk_len": chunk_len, "max_chunks": (max(t for _, t in seqs) + chunk_len - 1) // chunk_len,
                   "chunk_state": torch.full((n_chunks, H * D * V), float("nan"), dtype=F32, device=DEV),
                   "chunk_decay": torch.full((n_chunks, H * D), float("nan"), dtype=F32, device=DEV)}
    o.decay_scan(qk.to(dt).to(DEV), offs[0], offs[1], v.to(dt).to(DEV), offs[2], raw.to(dt).to(DEV), offs[3], out, state,
                 i32(cu), i32([s for s, _ in seqs]), len(seqs), H, D, V, hpg, mode, f(bias), rate=f(rate), skip=f(skip),
                 q_scale=q_scale, inv_tau=inv_tau, few_tokens=max(t for _, t in seqs) == 1,
                 single_tokens=all(t == 1 for _, t in seqs), **chunked)
    return out.double().cpu()


@pytest.fixture(params=["registers", "shared memory"])
def scan_kernels(request):
    """Both families of recurrence kernels: the state in registers (the default up to 128 rows) and
    the general ones with the state in shared memory."""
    from builderforce_inference_b200.kernels.library import library
    lib = library("core").lib
    lib.bfi_decay_scan_general(1 if request.param == "shared memory" else 0)
    yield request.param
    lib.bfi_decay_scan_general(0)


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("mode", ["sigmoid", "step"])
@pytest.mark.parametrize("chunk_len,H,G,D,V", [(64, 4, 2, 24, 40), (16, 2, 1, 64, 64), (50, 2, 2, 128, 33), (64, 1, 1, 130, 20)])
def test_chunked_recurrence_is_the_recurrence_in_order(dt, mode, chunk_len, H, G, D, V, scan_kernels):
    """The chunked form (chunks side by side, a carry over the chunks, then the earlier tokens' part)
    against the walk in order, in a batch of unequal sequences that all continue a state: lengths
    that are whole chunks, one token more, one less, a single token."""
    o = ops()
    g = torch.Generator().manual_seed(chunk_len)
    lens = [3 * chunk_len, chunk_len + 1, 1, 2 * chunk_len - 1, 7]
    seqs = list(zip([4, 0, 2, 1, 3], lens))
    n = sum(lens)
    x = torch.randn(n, H * V, generator=g)
    if mode == "sigmoid":
        qk, raw, hpg = torch.randn(n, 2 * H * D, generator=g), 2.0 * torch.randn(n, H * D, generator=g), 1
        kw = dict(bias=1.0 + torch.randn(H * D, generator=g), rate=None, skip=None, q_scale=D ** -0.5, inv_tau=0.25, offs=(0, H * D, 0, 0))
        m = o.DECAY_SIGMOID
    else:
        qk, raw, hpg = torch.randn(n, 2 * G * D, generator=g), torch.randn(n, H, generator=g), H // G
        kw = dict(bias=torch.randn(H, generator=g), rate=torch.exp(torch.randn(H, generator=g)), skip=torch.randn(H, generator=g),
                  offs=(G * D, 0, 0, 0))
        m = o.DECAY_STEP
    start = 0.3 * torch.randn(5, H, D, V, generator=g)
    s_seq, s_chk = start.clone().to(DEV), start.clone().to(DEV)
    ref = scan(o, m, dt, qk, x, raw, seqs=seqs, state=s_seq, H=H, D=D, V=V, hpg=hpg, **kw)
    got = scan(o, m, dt, qk, x, raw, seqs=seqs, state=s_chk, H=H, D=D, V=V, hpg=hpg, chunk_len=chunk_len, **kw)
    assert rel_err(got, ref) < 2e-5
    assert rel_err(s_chk, s_seq) < 2e-5


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("H,D,V", [(3, 8, 20), (2, 24, 8), (2, 64, 64), (1, 48, 130)])
def test_channel_decay_recurrence_whole_in_portions_and_token_by_token(dt, H, D, V, scan_kernels):
    o = ops()
    g = torch.Generator().manual_seed(H * D + V)
    n, tau = 75, 4.0
    qk = torch.randn(n, 2 * H * D, generator=g)
    v = torch.randn(n, H * V, generator=g)
    raw = 2.0 * torch.randn(n, H * D, generator=g)
    bias = 1.0 + torch.randn(H * D, generator=g)
    alpha = torch.exp(torch.nn.functional.logsigmoid(q64(raw, dt) + bias.float().double()) / tau).view(n, H, D)
    ref, S_ref = P.channel_decay_recurrence(q64(qk, dt)[:, :H * D].view(n, H, D) * D ** -0.5, q64(qk, dt)[:, H * D:].view(n, H, D),
                                            q64(v, dt).view(n, H, V), alpha)
    ref = ref.reshape(n, H * V)
    t = 2e-5 if dt == F32 else 2e-5      # the inputs are the same rounded values; the arithmetic is float32 either way
    for cuts in ([n], [1, 2, 40, 32], [1] * n):
        state = torch.zeros(3, H, D, V, dtype=F32, device=DEV)
        state[0].fill_(float("nan"))      # another slot's state must not matter
        outs, at = [], 0
        for c in cuts:
            outs.append(scan(o, o.DECAY_SIGMOID, dt, qk[at:at + c], v[at:at + c], raw[at:at + c], bias, None, None, [(1, c)], state,
                             H, D, V, 1, q_scale=D ** -0.5, inv_tau=1.0 / tau, offs=(0, H * D, 0, 0)))
            at += c
        assert rel_err(torch.cat(outs), ref) < t, cuts
        assert rel_err(state[1], S_ref) < t
        assert float(state[2].abs().max()) == 0.0


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("H,G,N,Pd", [(3, 1, 12, 8), (4, 2, 5, 6), (4, 4, 64, 64), (2, 1, 128, 32)])
def test_state_space_recurrence_with_groups_steps_and_skip(dt, H, G, N, Pd, scan_kernels):
    o = ops()
    g = torch.Generator().manual_seed(H * N + Pd)
    seqs = [(2, 40), (0, 1), (1, 7)]                     # three sequences of one step, slots out of order
    n = sum(t for _, t in seqs)
    bc = torch.randn(n, 2 * G * N, generator=g)           # B then C
    x = torch.randn(n, H * Pd, generator=g)
    raw = torch.randn(n, H, generator=g)
    dt_bias, a_log, skip = (torch.randn(H, generator=g) for _ in range(3))
    rate = torch.exp(a_log.float())
    state = torch.zeros(3, H, N, Pd, dtype=F32, device=DEV)
    got = scan(o, o.DECAY_STEP, dt, bc, x, raw, dt_bias, rate, skip, seqs, state, H, N, Pd, H // G, offs=(G * N, 0, 0, 0))
    at = 0
    for slot, t in seqs:
        B = q64(bc, dt)[at:at + t, :G * N].view(t, G, N)
        C = q64(bc, dt)[at:at + t, G * N:].view(t, G, N)
        xs = q64(x, dt)[at:at + t].view(t, H, Pd)
        step = P.softplus(q64(raw, dt)[at:at + t] + dt_bias.float().double())
        decay = torch.exp(-rate.double() * step)
        Sr = torch.zeros(H, N, Pd, dtype=P.F)
        ref = torch.zeros(t, H, Pd, dtype=P.F)
        for i in range(t):
            for h in range(H):
                gg = h // (H // G)
                Sr[h] = decay[i, h] * Sr[h] + step[i, h] * torch.outer(B[i, gg], xs[i, h])
                ref[i, h] = Sr[h].T @ C[i, gg] + skip.float().double()[h] * xs[i, h]
        assert rel_err(got[at:at + t], ref.reshape(t, H * Pd)) < 2e-5
        assert rel_err(state[slot], Sr) < 2e-5
        at += t


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("taps,C", [(1, 7), (2, 5), (3, 130), (4, 64), (5, 33)])
def test_causal_convolution_over_portions_single_tokens_and_reused_slots(dt, taps, C):
    o = ops()
    g = torch.Generator().manual_seed(taps * 7 + C)
    w, b = 0.6 * torch.randn(C, taps, generator=g), 0.3 * torch.randn(C, generator=g)
    off = 3                                               # the channels start at column 3 of the input's rows
    state = torch.zeros(4, taps - 1, C, dtype=F32, device=DEV)

    def run(pieces, single=False):
        """pieces: [(slot, tokens [t, C])] of one step."""
        rows = torch.cat([u for _, u in pieces])
        full = torch.cat([torch.randn(rows.shape[0], off, generator=g), rows, torch.randn(rows.shape[0], 2, generator=g)], dim=1)
        cu, slots, tok_slot = [0], [], []
        for s, u in pieces:
            cu.append(cu[-1] + u.shape[0])
            slots.append(s)
            tok_slot += [s] * u.shape[0]
        y = torch.full((rows.shape[0], C), float("nan"), dtype=dt, device=DEV)
        o.causal_conv(full.to(dt).to(DEV), off, C, w.to(dt).to(DEV), b.to(dt).to(DEV), state, y, i32(tok_slot), i32(cu), i32(slots),
                      len(pieces), single_tokens=single)
        return y.double().cpu()

    def plain(u, hist=None):
        y, hist = P.causal_conv(q64(u, dt), q64(w, dt), q64(b, dt), hist)
        return P.silu(y), hist

    t = 1e-6 if dt == F32 else 8e-3
    a, c = torch.randn(23, C, generator=g), torch.randn(9, C, generator=g)
    ref_a, _ = plain(a)
    ref_c, _ = plain(c)
    # a step with two sequences: the second one's first tokens must not read the first one's last
    got = run([(2, a), (0, c)])
    assert rel_err(got[:23], ref_a) < t and rel_err(got[23:], ref_c) < t
    # sequence a again in another slot, in portions of 1, 2, 1 (shorter than the taps), 10, then single tokens
    cuts, at, outs = [1, 2, 1, 10], 0, []
    for n in cuts:
        outs.append(run([(3, a[at:at + n])]))
        at += n
    for i in range(at, 23):
        outs.append(run([(3, a[i:i + 1]), (1, c[i - at:i - at + 1])], single=True)[:1])
    assert rel_err(torch.cat(outs), ref_a) < t
    _, hist = plain(a)
    if taps > 1:
        assert rel_err(state[3], hist) < 1e-6
    # slot 2 is given back and used again: its state is cleared by the cache; here by hand
    state[2].zero_()
    assert rel_err(run([(2, c)]), ref_c) < t


@pytest.mark.parametrize("dt", [F32, BF16])
def test_gated_group_norm_gate_before_and_after(dt):
    o = ops()
    g = torch.Generator().manual_seed(8)
    n, width = 5, 96
    x = torch.randn(n, width, generator=g)
    gate = torch.randn(n, width + 7, generator=g).to(dt)
    for parts, w_len, first in ((1, 96, True), (3, 96, True), (4, 24, False), (96, 1, False)):
        w = (1.0 + 0.2 * torch.randn(w_len, generator=g)).to(dt)
        y = torch.empty(n, width, dtype=dt, device=DEV)
        o.gated_group_norm(x.to(DEV), gate.to(DEV)[:, 3:3 + width], w.to(DEV), 1e-5, y, parts, gate_first=first)
        gs = P.silu(gate.double()[:, 3:3 + width])
        xs = x.double() * gs if first else x.double()
        ref = P.rms(xs.view(n, parts, width // parts), 1e-5).reshape(n, width) * w.double().repeat(width // w_len)
        if not first:
            ref = ref * gs
        assert rel_err(y, ref) < (1e-6 if dt == F32 else 8e-3), (parts, first)


def test_sublayer_output_kernels():
    o = ops()
    g = torch.Generator().manual_seed(4)
    x, y, y2 = (torch.randn(6, 40, generator=g) for _ in range(3))
    w = 1.0 + 0.25 * torch.randn(40, generator=g)
    xd = x.to(DEV)
    o.norm_add(xd, y.to(DEV), w.to(DEV), 2e-5)
    assert rel_err(xd, x.double() + P.rms(y.double(), 2e-5) * w.double()) < 1e-6
    # the same with the next norm of the new x in the same kernel
    for dt in (F32, BF16):
        xd2, w2 = x.to(DEV), (1.0 + 0.25 * torch.randn(40, generator=g))
        hn = torch.full((6, 40), float("nan"), dtype=dt, device=DEV)
        o.norm_add(xd2, y.to(DEV), w.to(DEV), 2e-5, next_w=w2.to(DEV), next_eps=3e-5, out=hn)
        assert torch.equal(xd2, xd)
        assert rel_err(hn, P.rms(xd.double().cpu(), 3e-5) * w2.double()) < (1e-6 if dt == F32 else 8e-3)
    out = torch.empty(6, 40, device=DEV)
    o.weighted_sum(out, y.to(DEV), -0.8, y2.to(DEV), 1.3)
    assert rel_err(out, -0.8 * y.double() + 1.3 * y2.double()) < 1e-6
    big = torch.randn(3, 50, generator=g).to(DEV)
    view = big[:, :41]
    ref = view.double().cpu() * 0.3
    o.scale_rows(view, 0.3)
    assert rel_err(view, ref) < 1e-6 and torch.equal(big[:, 41:].cpu(), big[:, 41:].cpu())


# ------------------------------------------------------------------------------------------------
# the routed feed-forward
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("E,top,groups,keep", [(12, 2, 3, 1), (6, 3, 3, 2), (5, 1, 1, 1), (64, 6, 8, 3), (40, 8, 1, 1)])
def test_router_against_the_plain_router(E, top, groups, keep):
    o = ops()
    g = torch.Generator().manual_seed(E + top)
    n = 200
    z = 2.0 * torch.randn(n, E + 1, generator=g)
    corr = 0.1 * torch.randn(E, generator=g) - 0.3        # choice scores are mostly negative
    idx = torch.empty(n, top, dtype=torch.int32, device=DEV)
    wt = torch.empty(n, top, dtype=F32, device=DEV)
    gate = torch.empty(n, dtype=F32, device=DEV)
    o.moe_route(z.to(DEV), E, corr.to(DEV), idx, wt, top, groups, keep, 1.0, gate)
    ridx, rw = P.route(z.double()[:, :E], torch.eye(E, dtype=P.F), corr.double(), top, groups, keep)
    got = idx.cpu().long()
    assert torch.equal(got.sort(dim=1).values, ridx.sort(dim=1).values)
    assert torch.equal(got, ridx)                          # best first, as the plain top-k lists them
    assert rel_err(wt, rw) < 1e-5
    assert rel_err(gate, torch.sigmoid(z.double()[:, E])) < 1e-6
    # the same decision with the logits made in the kernel, from float32 and from bfloat16 inputs
    width = 72
    w_r = torch.randn(E + 1, width, generator=g) * (3.0 / math.sqrt(width))
    h = torch.randn(n, width, generator=g)
    slots = [0] * n
    slots[5] = -1
    for dt in (F32, BF16):
        idx.fill_(-7)
        o.moe_router(h.to(dt).to(DEV), w_r.to(DEV), E, corr.to(DEV), i32(slots), idx, wt, top, groups, keep, 1.0, gate)
        zz = q64(h, dt) @ w_r.double().T
        rep = []
        ridx, rw = P.route(zz[:, :E], torch.eye(E, dtype=P.F), corr.double(), top, groups, keep, rep)
        rows = [t for t in range(n) if t != 5]
        got = idx.cpu().long()
        assert torch.equal(got[rows], ridx[rows]) or rep[0] < 1e-5
        assert rel_err(wt.cpu()[rows], rw[rows]) < 1e-5 and rel_err(gate.cpu()[rows], torch.sigmoid(zz[rows, E])) < 1e-5
        assert int(got[5, 0]) == -7                       # a padding row is left alone


@pytest.mark.parametrize("dt", [F32, BF16])
@pytest.mark.parametrize("width,ff,E,top", [(40, 24, 6, 3), (128, 64, 8, 2), (72, 20, 4, 1)])
def test_expert_products_read_the_chosen_experts(dt, width, ff, E, top):
    o = ops()
    g = torch.Generator().manual_seed(width + ff)
    n = 11
    h = torch.randn(n, width, generator=g)
    wg, wu = (torch.randn(E, ff, width, generator=g) / math.sqrt(width) for _ in range(2))
    wd = torch.randn(E, width, ff, generator=g) / math.sqrt(ff)
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(n)]).to(torch.int32)
    wt = torch.rand(n, top, generator=g)
    shared, gate = torch.randn(n, width, generator=g), torch.rand(n, generator=g)
    slots = [0] * n
    slots[4] = -1                                          # a padding row is left alone
    # the layouts the part keeps: gate and up rows interleaved, expert after expert; the down matrices side by side
    w_gu = torch.cat([torch.stack([wg[e], wu[e]], dim=1).reshape(2 * ff, width) for e in range(E)]).to(dt).to(DEV)
    w_dn = torch.cat([wd[e] for e in range(E)], dim=1).contiguous().to(dt).to(DEV)
    act = torch.full((n * top, ff), float("nan"), dtype=dt, device=DEV)
    o.moe_gate_up(h.to(dt).to(DEV), w_gu, E, idx.to(DEV), i32(slots), act)
    out = torch.full((n, width), 5.0, dtype=F32, device=DEV)
    o.moe_down(act, w_dn, E, idx.to(DEV), wt.to(DEV), i32(slots), out, shared.to(DEV), gate.to(DEV))
    acc = torch.full((n, width), 5.0, dtype=F32, device=DEV)
    o.moe_down(act, w_dn, E, idx.to(DEV), wt.to(DEV), i32(slots), acc, accumulate=True)
    # the dense way's weighing: every expert's activations times the token's weight of it, 0 where it was not chosen
    dense = torch.ones(n, E * ff + 5, dtype=dt, device=DEV)             # five more columns: an expert every token uses
    o.moe_weigh_dense(dense, E, idx.to(DEV), wt.to(DEV), i32(slots), 5, gate.to(DEV))
    comb = torch.zeros(n, E, dtype=P.F)
    comb.scatter_(1, idx.long(), wt.double())
    keep_rows = [t for t in range(n) if t != 4]
    want = torch.cat([comb.repeat_interleave(ff, dim=1), gate.double()[:, None].expand(n, 5)], dim=1)
    assert rel_err(dense.cpu()[keep_rows], q64(want, dt)[keep_rows]) < 1e-6
    # the down matrices as the first columns of a wider matrix
    wide = torch.cat([w_dn, torch.full((width, 9), float("nan"), dtype=dt, device=DEV)], dim=1)
    out2 = torch.full((n, width), 5.0, dtype=F32, device=DEV)
    o.moe_down(act, wide[:, :E * ff], E, idx.to(DEV), wt.to(DEV), i32(slots), out2, shared.to(DEV), gate.to(DEV))
    assert rel_err(out2.cpu()[keep_rows], out.cpu()[keep_rows]) < 1e-5      # rows that are not 16-byte aligned sum in another order
    g_out = torch.full((n, width), 2.0, dtype=F32, device=DEV)
    o.gated_rows(g_out, shared.to(DEV), gate.to(DEV), accumulate=True)
    assert rel_err(g_out, 2.0 + gate.double()[:, None] * shared.double()) < 1e-6
    hs, ref, ref_acc = q64(h, dt), torch.zeros(n, width, dtype=P.F), torch.zeros(n, width, dtype=P.F)
    for t in range(n):
        for k in range(top):
            e = int(idx[t, k])
            a = P.silu(q64(wg, dt)[e] @ hs[t]) * (q64(wu, dt)[e] @ hs[t])
            a = q64(a, dt)                                 # the activations are stored in the run dtype
            ref_acc[t] += float(wt[t, k]) * (q64(wd, dt)[e] @ a)
        ref[t] = ref_acc[t] + float(gate[t]) * shared.double()[t]
    keep = [t for t in range(n) if t != 4]
    assert rel_err(out.cpu()[keep], ref[keep]) < (1e-5 if dt == F32 else 1e-2)
    assert rel_err(acc.cpu()[keep], 5.0 + ref_acc[keep]) < (1e-5 if dt == F32 else 1e-2)
    assert float((out[4] - 5.0).abs().max()) == 0.0


# ------------------------------------------------------------------------------------------------
# whole models
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_whole_prompts_and_every_layer(name, dtype):
    from builderforce_inference_b200.engine.context import build_context
    eng, cfg, w = engine(name, dtype)
    ids = steady_prompt(cfg, w, 260, dtype)       # long enough for the chunked form of the recurrences
    layers = []
    ref = P.forward(cfg, w, ids, layers)
    slot = eng.acquire()
    assert close(eng.step([S(slot, ids)]), ref, dtype)
    eng.release(slot)
    # the residual stream after every layer
    slot = eng.acquire()
    eng.cache.begin_step([slot], [len(ids)])
    ctx = build_context([(slot, 0, ids)], eng.dtype, eng.workspace, eng.device, eng.status)
    x = eng.decoder.embed(ctx)
    for i in range(len(cfg["layers"])):
        eng.decoder.run_layers(ctx, x, eng.cache, i, i + 1)
        assert close(x, layers[i], dtype), i
    eng.cache.end_step([slot], [len(ids)])
    eng.release(slot)
    eng.cache.check()


@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_prompt_then_token_by_token_far_past_every_chunk(name, dtype, graphs):
    eng, cfg, w = engine(name, dtype, use_graphs=graphs)
    ids = steady_prompt(cfg, w, 300, dtype, seed0=40)     # chunks of 9, 70 and 128 are crossed token by token
    ref = P.forward(cfg, w, ids)
    slot = eng.acquire()
    head = 3
    outs = [eng.step([S(slot, ids[:head])]).clone()]
    for t in ids[head:]:
        outs.append(eng.step([S(slot, [t])]).clone())
    assert close(torch.cat(outs), ref, dtype)
    # a chunked layer holds the pages of its current chunk only
    for gkv in eng.cache.kv_groups:
        if gkv.need.chunk:
            held = sum(1 for p in gkv.table.rows[slot] if p >= 0)
            assert held <= (gkv.need.chunk + 62) // 64 + 1
    eng.release(slot)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_portions_of_a_prompt_down_to_two_tokens(name, dtype):
    eng, cfg, w = engine(name, dtype)
    ids = steady_prompt(cfg, w, 201, dtype, seed0=70)
    ref = P.forward(cfg, w, ids)
    for cuts in ([2, 2, 3, 64, 65, 63, 2], [128, 73], [1, 7, 1, 130, 62], [1, 200], [193, 2, 6]):
        slot = eng.acquire()
        outs, at = [], 0
        for c in cuts:
            outs.append(eng.step([S(slot, ids[at:at + c])]).clone())
            at += c
        assert at == len(ids)
        assert close(torch.cat(outs), ref, dtype), cuts
        eng.release(slot)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_unequal_batches_reused_slots_and_poisoned_pages(name, dtype):
    eng, cfg, w = engine(name, dtype, max_tokens=1024)
    eng.cache.poison()
    lengths = [70, 5, 131, 1]
    seqs = [steady_prompt(cfg, w, n + 6, dtype, seed0=100 + 20 * i) for i, n in enumerate(lengths)]
    refs = [P.forward(cfg, w, s) for s in seqs]
    for round_ in range(2):                               # the second round runs in slots and pages that were used
        slots = [eng.acquire() for _ in seqs]
        got = eng.step([S(sl, s[:n]) for sl, s, n in zip(slots, seqs, lengths)])
        want = torch.cat([r[:n] for r, n in zip(refs, lengths)])
        assert close(got, want, dtype), round_
        live = list(range(len(seqs)))
        for step in range(6):                             # decoded together; the shortest leave first
            got = eng.step([S(slots[i], [seqs[i][lengths[i] + step]]) for i in live])
            want = torch.stack([refs[i][lengths[i] + step] for i in live])
            assert close(got, want, dtype), (round_, step)
            if step in (1, 3):
                eng.release(slots[live.pop(1)])
        for i in live:
            eng.release(slots[i])
        eng.cache.check()
        eng.cache.poison()


def test_batch_against_each_alone_in_float32():
    eng, cfg, w = engine("odd", "float32")
    seqs = prompts(cfg["vocab"], [33, 140, 2, 71], seed=9)
    slots = [eng.acquire() for _ in seqs]
    together = eng.step([S(sl, s) for sl, s in zip(slots, seqs)]).clone()
    nxt = eng.step([S(sl, [7]) for sl in slots]).clone()
    for sl in slots:
        eng.release(sl)
    at = 0
    for i, s in enumerate(seqs):
        sl = eng.acquire()
        alone = eng.step([S(sl, s)]).clone()
        # the products' tiles differ with the number of rows, so sums differ in their last bits
        assert rel_err(together[at:at + len(s)], alone) < 1e-5
        assert rel_err(nxt[i:i + 1], eng.step([S(sl, [7])])) < 1e-5
        eng.release(sl)
        at += len(s)


@pytest.mark.parametrize("seed", range(101, 113))
def test_random_configurations_in_float32(seed):
    """Configurations drawn from a seed (layer order, every size, chunks, groups, with and without
    feed-forward, shared expert and rotation): an unequal batch of prompts, five tokens decoded
    together, and the longest prompt again in portions, against the plain implementation.  A prompt
    whose routers decide by less than 1e-4 somewhere is not compared (a float32 sum may turn it)."""
    from builderforce_inference_b200.engine.engine import Engine
    cfg = random_config(seed)
    w = make_weights(cfg, seed, F32)
    eng = Engine.load(write_folder(cfg, w), dtype="float32", max_tokens=2048)
    w64 = {k: v.to(torch.float64) for k, v in w.items()}
    lens = [(1, 5, 70, 130, 260)[seed % 5], (2, 33, 200)[seed % 3], (1, 64, 129)[seed % 2]]
    seqs = prompts(cfg["vocab"], [n + 5 for n in lens], seed)
    refs, steady = [], []
    for s in seqs:
        rep = []
        refs.append(P.forward(cfg, w64, s, None, rep))
        steady.append(not rep or min(rep) > 1e-4)
    slots = [eng.acquire() for _ in seqs]
    got = eng.step([S(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)])
    at = 0
    for i, n in enumerate(lens):
        if steady[i]:
            assert rel_err(got[at:at + n], refs[i][:n]) < 4e-4, (i, cfg)
        at += n
    for step in range(5):
        got = eng.step([S(sl, [s[n + step]]) for sl, s, n in zip(slots, seqs, lens)])
        for i, n in enumerate(lens):
            if steady[i]:
                assert rel_err(got[i:i + 1], refs[i][n + step:n + step + 1]) < 4e-4, (i, step, cfg)
    for sl in slots:
        eng.release(sl)
    i = max(range(3), key=lambda k: lens[k])
    sl, outs, at = eng.acquire(), [], 0
    for c in [max(1, lens[i] // 3), 2, 1, 97, 10 ** 6]:
        c = min(c, lens[i] - at)
        if c > 0:
            outs.append(eng.step([S(sl, seqs[i][at:at + c])]).clone())
            at += c
    if steady[i]:
        assert rel_err(torch.cat(outs), refs[i][:lens[i]]) < 4e-4, cfg
    eng.release(sl)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_public_entry_point(dtype):
    from builderforce_inference_b200.engine.api import Model
    from builderforce_inference_b200.sampling.params import SampleParams
    folder, cfg, w = model("odd", dtype)
    m = Model.load(folder, dtype=dtype, max_tokens=1024)
    ps = prompts(cfg["vocab"], [12, 3, 40], seed=21)
    n_new = 24
    outs = m.generate_batch(ps, SampleParams(temperature=0.0, max_tokens=n_new), ignore_eos=True)
    for p, got in zip(ps, outs):
        got = list(got)
        assert len(got) == n_new
        # every generated id is the plain model's best id given the ids before it, or (bfloat16) a near tie
        full = p + got
        ref = P.forward(cfg, w, full)
        for i, tok in enumerate(got):
            row = ref[len(p) + i - 1]
            if int(torch.argmax(row)) != tok:
                assert dtype == "bfloat16" and float(row.max() - row[tok]) < 0.05 * float(row.max() - row.min())


def test_trace_replay_and_command_line_take_the_model():
    from helpers import run_trace
    folder, cfg, w = model("odd", "float32")
    a, b = prompts(cfg["vocab"], [40, 9], seed=31)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}, {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]}, {"id": "b", "tokens": b[8:9], "want": []}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[31:40], "want": [8]}], "end": ["a"]}]
    import numpy as np
    import subprocess
    import sys
    import tempfile
    from helpers import ROOT
    out_dir = tempfile.mkdtemp(prefix="bfi_trace_")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out_dir,
                        "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    assert [line for line in r.stdout.splitlines() if line.startswith("done ")] == ["done 0", "done 1", "done 2"]
    ra, rb = P.forward(cfg, w, a), P.forward(cfg, w, b)
    got0 = torch.from_numpy(np.fromfile(os.path.join(out_dir, "0.f32"), dtype="<f4").reshape(3, -1).copy())
    assert rel_err(got0, torch.stack([ra[0], ra[29], rb[7]])) < 3e-5
    got1 = torch.from_numpy(np.fromfile(os.path.join(out_dir, "1.f32"), dtype="<f4").reshape(1, -1).copy())
    assert rel_err(got1, ra[30:31]) < 3e-5
    got2 = torch.from_numpy(np.fromfile(os.path.join(out_dir, "2.f32"), dtype="<f4").reshape(1, -1).copy())
    assert rel_err(got2, ra[39:40]) < 3e-5
