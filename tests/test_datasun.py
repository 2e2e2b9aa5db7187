"""Datasun without a GPU: its configuration reader, the model it describes, and the plain
implementation checked against closed forms of its own."""
import copy
import math

import pytest
import torch

from plain import datasun_plain as P

CFG = {"architecture": "Datasun", "vocab": 90, "width": 32, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
       "layers": [
           {"type": "lightning", "mixer": {"heads": 2, "dim": 8, "vdim": 12, "decay": [0.9, 0.5]},
            "mlp": {"kind": "dense", "ff": 48, "limit": 2.0}},
           {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.2, "mask": {"size": 7},
                                           "rot": {"base": 1e4, "dims": 8, "scaling": {"factor": 2.0, "original": 64,
                                                                                      "fast": 8.0, "slow": 1.0}}},
            "mlp": None}]}


def test_config_is_read_and_registered():
    from builderforce_inference_b200 import describe_model, registered_architectures
    from builderforce_inference_b200.config.datasun import DatasunConfig
    from builderforce_inference_b200.engine.decoder import expected_tensors
    assert "Datasun" in registered_architectures()
    c = DatasunConfig.from_dict(CFG)
    assert (c.vocab, c.width, c.eps, c.embedding_scale, len(c.layers)) == (90, 32, 1e-5, 2.0, 2)
    assert c.layers[0].mixer.decay == (0.9, 0.5) and c.layers[0].mlp.limit == 2.0 and c.layers[1].mlp is None
    a = c.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.window, a.scale, a.rotary.dims) == (4, 2, 16, 7, 0.2, 8)
    spec = describe_model(CFG)
    assert spec.embedding_scale == 2.0 and spec.head_name is None
    names = expected_tensors(spec)
    assert names["l0.mix.v"].shape == (24, 32) and names["l0.mix.norm"].shape == (24,)
    assert names["l1.mix.q.norm"].shape == (64,) and names["l1.mix.k.b"].shape == (32,) and names["l1.mix.o.b"].shape == (32,)
    assert "l1.mix.v" not in names and "l1.mlp.gate" not in names and names["l0.mlp.down"].shape == (32, 48)
    from builderforce_inference_b200.parts import KVNeed, StateNeed
    from builderforce_inference_b200.parts.base import BLOCKS
    needs = [BLOCKS.build(layer.block).mixer().cache_need() for layer in spec.layers]
    assert needs == [StateNeed((2, 8, 12), "float32"), KVNeed(2, 16, 7)]


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "divide"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "kind"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "dims"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_bad_configurations_are_refused_by_key(edit, word):
    from builderforce_inference_b200.config import ConfigError
    from builderforce_inference_b200.config.datasun import DatasunConfig
    c = copy.deepcopy(CFG)
    edit(c)
    with pytest.raises(ConfigError, match=word):
        DatasunConfig.from_dict(c)


def test_optional_keys_have_plain_meanings():
    from builderforce_inference_b200.config.datasun import DatasunConfig
    c = copy.deepcopy(CFG)
    m = c["layers"][1]["mixer"]
    del m["mask"], m["rot"], m["scale"], m["kv_heads"]
    a = DatasunConfig.from_dict(c).layers[1].mixer
    assert a.window is None and a.rotary is None and a.kv_heads == 4 and a.scale == 16 ** -0.5


def test_a_written_folder_loads_by_name_on_the_cpu_side(tmp_path):
    from builderforce_inference_b200 import write_model_folder
    folder = write_model_folder(CFG, 4, str(tmp_path / "m"), torch.float32)
    cfg, w = P.load_folder(folder)
    assert cfg == CFG and w["l1.mix.q.b"].shape == (64,)
    assert P.forward(cfg, w, [1, 2, 3, 4, 5]).shape == (5, 90)


# ---- the plain implementation against closed forms ---------------------------------------------
def test_plain_recurrence_is_the_decayed_sum():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(9, 2, n, generator=g, dtype=torch.float64) for n in (4, 4, 5))
    o, S = P.lightning_recurrence(q, k, v, [0.8, 1.0])
    for h, w in enumerate((0.8, 1.0)):
        for t in range(9):
            want = sum(w ** (t - j) * float(q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1))
            assert torch.allclose(o[t, h], want, atol=1e-12)
    o2, S2 = P.lightning_recurrence(q[5:], k[5:], v[5:], [0.8, 1.0], P.lightning_recurrence(q[:5], k[:5], v[:5], [0.8, 1.0])[1])
    assert torch.allclose(o2, o[5:], atol=1e-12) and torch.allclose(S2, S, atol=1e-12)


def test_plain_sink_softmax_and_window():
    k = torch.zeros(6, 1, 2, dtype=torch.float64)
    v = torch.arange(6, dtype=torch.float64).reshape(6, 1, 1).expand(6, 1, 2).clone()
    q = torch.zeros(6, 1, 2, dtype=torch.float64)
    out = P.sink_attention(q, k, v, 1.0, window=3, sink=0.0)
    # every score is 0, so every seen key weighs 1 / (1 + seen)
    assert torch.allclose(out[0, 0, 0], torch.tensor(0.0, dtype=torch.float64))
    assert torch.allclose(out[1, 0, 0], torch.tensor((0 + 1) / 3.0, dtype=torch.float64))
    assert torch.allclose(out[5, 0, 0], torch.tensor((3 + 4 + 5) / 4.0, dtype=torch.float64))
    assert torch.allclose(P.sink_attention(q, k, v, 1.0, window=3)[5, 0, 0], torch.tensor(4.0, dtype=torch.float64))


def test_plain_rotation_and_gate():
    f, mag = P.rotary_frequencies(1e4, 8, {"factor": 1.0, "original": 64, "fast": 8.0, "slow": 1.0})
    plain, one = P.rotary_frequencies(1e4, 8)
    assert torch.allclose(f, plain) and mag == 1.0 and one == 1.0
    x = torch.randn(3, 2, 10, dtype=torch.float64)
    y = P.rotate_adjacent(x, [0, 5, 9], 1e4, 6)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 6:], x[..., 6:])
    assert torch.allclose((y[..., 0:6:2] ** 2 + y[..., 1:6:2] ** 2), (x[..., 0:6:2] ** 2 + x[..., 1:6:2] ** 2))
    a = 5 * float(P.rotary_frequencies(1e4, 6)[0][1])
    assert torch.allclose(y[1, 0, 2], x[1, 0, 2] * math.cos(a) - x[1, 0, 3] * math.sin(a))
    g = P.clamped_gate(torch.tensor([5.0, -1.0], dtype=torch.float64), torch.tensor([-9.0, 0.5], dtype=torch.float64), 2.0)
    assert torch.allclose(g, torch.tensor([2.0 / (1 + math.exp(-3.404)) * (-1.0), -1.0 / (1 + math.exp(1.702)) * 1.5],
                                          dtype=torch.float64))
