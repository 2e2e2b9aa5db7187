"""Bepilorn without a GPU: the configuration reader and its refusals by key, the model as data, the
cache's bookkeeping for chunked layers and for values of their own size, and the plain
implementation (tests/plain/bepilorn_plain.py) against closed forms."""
import copy
import math

import pytest
import torch

from bepilorn_models import BP_ODD, BP_WIDE, make_weights, tensor_shapes
from plain import bepilorn_plain as P

from builderforce_inference_b200.cache.pages import PAGE_TOKENS, PageTable
from builderforce_inference_b200.cache.plan import kv_bytes_per_token
from builderforce_inference_b200.config.base import ConfigError
from builderforce_inference_b200.config.bepilorn import BepilornConfig
from builderforce_inference_b200.engine.decoder import expected_tensors
from builderforce_inference_b200.parts.base import KVNeed, StateNeed
from builderforce_inference_b200.registry import architecture_for, describe_model


# ------------------------------------------------------------------------------------------------ configuration
def test_config_reads_every_size_and_constant():
    c = BepilornConfig.from_dict(BP_ODD)
    assert (c.vocab, c.width, c.eps, c.logit_scale, len(c.layers)) == (131, 40, 2e-5, 0.7, 5)
    s = c.layers[0].mixer
    assert (s.heads, s.vdim, s.state, s.groups, s.conv, s.norm_groups) == (3, 8, 12, 1, 2, 1)
    p = c.layers[1].mixer
    assert (p.left.heads, p.left.kv_heads, p.left.dim, p.left.vdim, p.left.scale, p.left.chunk) == (4, 2, 24, 10, 0.21, 9)
    assert (p.left.rot_base, p.left.rot_dims) == (5000.0, 12)
    assert (p.right.heads, p.right.dim, p.right.vdim, p.right.tau, p.right.rank) == (3, 8, 20, 4.0, 5)
    assert (p.left_scale, p.right_scale) == (0.7, 1.3)
    assert c.layers[1].mlp is None
    f = c.layers[0].mlp
    assert (f.experts, f.top, f.ff, f.groups, f.keep, f.shared_ff) == (6, 3, 24, 3, 2, 40)
    f = c.layers[2].mlp
    assert (f.groups, f.keep, f.shared_ff) == (1, 1, None)
    last = c.layers[4].mixer.left
    assert last.chunk is None and last.rot_base is None
    assert architecture_for(BP_ODD).name == "bepilorn"


def _changed(path, value):
    cfg = copy.deepcopy(BP_ODD)
    node = cfg
    for k in path[:-1]:
        node = node[k]
    if value is KeyError:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return cfg


@pytest.mark.parametrize("path,value,names", [
    (("vocab",), KeyError, "vocab"),
    (("norm",), KeyError, "norm"),
    (("layers", 0, "type"), "mamba3", "type"),
    (("layers", 0, "mixer", "groups"), 2, "groups"),                 # 3 heads in 2 groups
    (("layers", 0, "mixer", "norm_groups"), 5, "norm_groups"),       # 24 values in 5 parts
    (("layers", 0, "mixer", "conv"), 40, "conv"),
    (("layers", 1, "mixer", "left", "kv_heads"), 3, "key/value heads"),
    (("layers", 1, "mixer", "left", "dim"), 23, "dim"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 26, "dims"),
    (("layers", 1, "mixer", "right", "tau"), 0.0, "tau"),
    (("layers", 1, "mixer", "right"), KeyError, "right"),
    (("layers", 0, "mlp", "kind"), "dense", "kind"),
    (("layers", 0, "mlp", "router", "top"), 7, "top"),
    (("layers", 0, "mlp", "router", "groups", "count"), 4, "groups"),   # 6 experts in 4 groups
    (("layers", 0, "mlp", "router", "groups", "keep"), 1, "top"),       # 1 group of 2 cannot give 3
])
def test_config_refuses_by_key(path, value, names):
    with pytest.raises(ConfigError) as e:
        BepilornConfig.from_dict(_changed(path, value))
    assert names in str(e.value)


def test_a_layer_without_feed_forward_ignores_stray_norms_and_one_tap_is_a_convolution():
    spec = describe_model(BP_ODD)
    assert set(spec.ignored_names) == {"l1.norm2", "l1.norm2b"}
    cfg = _changed(("layers", 0, "mixer", "conv"), 1)
    from builderforce_inference_b200.parts.base import BLOCKS
    need = BLOCKS.build(describe_model(cfg).layers[0].block).mixer().cache_need()
    assert need == (StateNeed((3, 12, 8), "float32"),)             # nothing is kept for the convolution


def test_model_as_data_names_every_tensor_with_its_shape():
    for cfg in (BP_ODD, BP_WIDE):
        want = {n: s for n, (s, _) in tensor_shapes(cfg).items()}
        got = {n: tuple(p.shape) for n, p in expected_tensors(describe_model(cfg)).items()}
        assert got == want
    # without the rank in the configuration the decay's two projections leave that size to the checkpoint
    cfg = copy.deepcopy(BP_ODD)
    del cfg["layers"][1]["mixer"]["right"]["rank"]
    got = expected_tensors(describe_model(cfg))
    assert got["l1.mix.right.a1"].shape == (-1, 40) and got["l1.mix.right.a2"].shape == (24, -1)
    spec = describe_model(BP_ODD)
    assert spec.logit_scale == 0.7 and spec.head_name == "head"
    assert [layer.block.kind for layer in spec.layers] == ["sandwich"] * 5


def test_cache_needs_of_the_mixers():
    from builderforce_inference_b200.parts.base import BLOCKS
    spec = describe_model(BP_ODD)
    needs = [BLOCKS.build(layer.block).mixer().cache_need() for layer in spec.layers]
    assert needs[0] == (StateNeed((3, 12, 8), "float32"), StateNeed((1, 8 * 3 + 2 * 12), "float32"))
    assert needs[1] == (KVNeed(2, 24, None, v_dim=10, chunk=9), StateNeed((3, 8, 20), "float32"))
    assert needs[4] == (KVNeed(1, 32, None), StateNeed((1, 16, 16), "float32"))
    # bytes per token: keys of 24 and values of 10 for 2 heads; 16 + 28 for 3; 32 + 32 for 1
    assert kv_bytes_per_token(needs, [None] * 5, 2) == 2 * (2 * 34 + 3 * 44 + 64)


# ------------------------------------------------------------------------------------------------ pages of chunked layers
def test_chunked_page_table_keeps_the_current_chunk_only():
    t = PageTable(16, chunk=100)
    t.open(0)
    assert [t.first_kept_position(n) for n in (0, 99, 100, 199, 200, 250)] == [0, 0, 100, 100, 200, 200]
    t.ensure(0, 0, 130)                    # a prompt of 130 tokens: pages 0, 1, 2
    assert t.held_pages() == 3
    assert t.trim(0, 130)                  # the next token (130) reads 100..130: page 0 (0..63) goes, page 1 holds 100
    assert t.rows[0][0] == -1 and t.rows[0][1] >= 0 and t.held_pages() == 2
    for n in range(130, 200):
        t.ensure(0, n, n + 1)
        t.trim(0, n + 1)
    assert t.first_kept_position(200) == 200 and t.rows[0][:3] == [-1, -1, -1] and t.rows[0][3] >= 0
    t.check()
    t.close(0)
    assert t.pool.n_free == 16
    # a chunk that is a whole number of pages gives every page back at its border
    t = PageTable(4, chunk=PAGE_TOKENS)
    t.open(3)
    for n in range(3 * PAGE_TOKENS):
        t.ensure(3, n, n + 1)
        t.trim(3, n + 1)
        assert t.held_pages() <= 1
    # a window and a chunk together: whichever starts later
    assert PageTable(4, window=10, chunk=64).first_kept_position(70) == 64
    assert PageTable(4, window=3, chunk=64).first_kept_position(70) == 68


# ------------------------------------------------------------------------------------------------ the plain implementation
def test_plain_rotation_turns_pairs_half_a_width_apart_and_leaves_the_rest():
    x = torch.zeros(2, 1, 8, dtype=P.F)
    x[:, 0, 0] = 1.0                      # pair (0, 2) of a rotated width of 4
    x[:, 0, 5] = 3.0
    y = P.rotate_half(x, [0, 2], 100.0, 4)
    assert torch.allclose(y[0], x[0])
    assert math.isclose(float(y[1, 0, 0]), math.cos(2.0)) and math.isclose(float(y[1, 0, 2]), math.sin(2.0))
    assert float(y[1, 0, 5]) == 3.0 and float(y[1, 0, 1]) == 0.0
    x = torch.zeros(1, 1, 8, dtype=P.F)
    x[0, 0, 1] = 1.0                      # pair (1, 3): frequency 100^(-2/4) = 0.1
    y = P.rotate_half(x, [5], 100.0, 4)
    assert math.isclose(float(y[0, 0, 1]), math.cos(0.5)) and math.isclose(float(y[0, 0, 3]), math.sin(0.5))


def test_plain_attention_chunks_and_sink():
    T, C = 7, 3
    q = torch.zeros(T, 1, 2, dtype=P.F)
    k = torch.zeros(T, 1, 2, dtype=P.F)
    v = torch.arange(T, dtype=P.F).reshape(T, 1, 1) + 1.0
    # all scores 0: a token averages the values of its chunk so far; the sink of score 0 counts as one more key
    out = P.chunk_sink_attention(q, k, v, 1.0, C, torch.zeros(1, dtype=P.F))
    for i in range(T):
        seen = [j for j in range(T) if j <= i and j // C == i // C]
        assert math.isclose(float(out[i, 0, 0]), sum(j + 1.0 for j in seen) / (len(seen) + 1))
    # positions count from the sequence's start, not from where the piece starts
    out = P.chunk_sink_attention(q[:3], k[:3], v[:3], 1.0, C, None, first_position=2)
    assert [round(float(x), 9) for x in out[:, 0, 0]] == [1.0, 2.0, 2.5]
    # a sink far above every score takes all the weight
    out = P.chunk_sink_attention(q, k, v, 1.0, None, torch.full((1,), 50.0, dtype=P.F))
    assert float(out.abs().max()) < 1e-18


def test_plain_recurrences_against_sums():
    g = torch.Generator().manual_seed(1)
    T, H, D, V = 6, 2, 3, 4
    q, k, a = (torch.rand(T, H, D, generator=g, dtype=P.F) for _ in range(3))
    v = torch.rand(T, H, V, generator=g, dtype=P.F)
    o, S = P.channel_decay_recurrence(q, k, v, a)
    for t in (0, 3, 5):
        ref = torch.zeros(H, V, dtype=P.F)
        for j in range(t + 1):
            w = torch.ones(H, D, dtype=P.F)
            for i in range(j + 1, t + 1):
                w = w * a[i]
            ref += torch.einsum("hd,hv->hv", q[t] * w * k[j], v[j])
        assert torch.allclose(o[t], ref)
    # carried on from a state, two pieces give what one piece gives
    o1, S1 = P.channel_decay_recurrence(q[:2], k[:2], v[:2], a[:2])
    o2, S2 = P.channel_decay_recurrence(q[2:], k[2:], v[2:], a[2:], S1)
    assert torch.allclose(torch.cat([o1, o2]), o) and torch.allclose(S2, S)


def test_plain_convolution_and_its_history():
    u = torch.arange(1.0, 6.0, dtype=P.F).reshape(5, 1)
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=P.F)          # the last column is the current token's
    y, hist = P.causal_conv(u, w, torch.tensor([0.5], dtype=P.F))
    assert y[:, 0].tolist() == [1.5, 12.5, 123.5, 234.5, 345.5]
    assert hist[:, 0].tolist() == [4.0, 5.0]
    y1, h1 = P.causal_conv(u[:1], w, torch.tensor([0.5], dtype=P.F))
    y2, h2 = P.causal_conv(u[1:], w, torch.tensor([0.5], dtype=P.F), h1)
    assert torch.equal(torch.cat([y1, y2]), y) and torch.equal(h2, hist) and h1[:, 0].tolist() == [0.0, 1.0]


def test_plain_router_groups_negative_scores_and_weights():
    # one token, 6 experts in 3 groups; logits make s known; corrections make every choice score negative
    z = torch.tensor([[0.0, 1.0, 2.0, 0.5, 3.0, -1.0]], dtype=P.F)
    s = torch.softmax(z, dim=-1)
    router = torch.eye(6, dtype=P.F)
    corr = torch.tensor([-2.0, -2.0, -5.0, -2.0, -5.0, -1.2], dtype=P.F)
    # choice = s + corr; group bests: g0 = max(s0, s1) - 2, g1 = s3 - 2 (s2 - 5 is lower), g2 = s5 - 1.2
    idx, w = P.route(z, router, corr, 2, 3, 2)
    # kept groups: g2 and g0 (s1 > s3); the best two of experts {0, 1, 4, 5}: 5 then 1; expert 4 has the largest s but -5
    assert idx.tolist() == [[5, 1]]
    assert torch.allclose(w, s[:, [5, 1]])                      # the weights are s without the correction, not renormalised
    # masked experts count as minus infinity, not 0: with one group kept nothing outside it can be chosen
    idx, _ = P.route(z, router, corr, 2, 3, 1)
    assert sorted(idx.tolist()[0]) == [4, 5]
    rep = []
    P.route(z, router, corr, 2, 3, 2, rep)
    assert rep and rep[0] > 0


def test_plain_model_decodes_and_counts_layers():
    w = {k: v.to(P.F) for k, v in make_weights(BP_ODD, 2, torch.float32).items()}
    outs, rep = [], []
    logits = P.forward(BP_ODD, w, [3, 1, 4, 1, 5, 9, 2, 6], outs, rep)
    assert logits.shape == (8, 131) and len(outs) == 5 and len(rep) == 4
    # causal: a longer sequence leaves earlier logits alone
    more = P.forward(BP_ODD, w, [3, 1, 4, 1, 5, 9, 2, 6, 5, 3])
    assert torch.allclose(more[:8], logits)
    assert len(P.greedy(BP_ODD, w, [3, 1, 4], 3)) == 3
