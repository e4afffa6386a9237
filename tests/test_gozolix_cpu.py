"""The Gozolix design on the CPU: its configuration, tensor names, schedule and cache needs in the library,
and the plain implementation's own sanity."""
import copy
import json

import numpy as np
import pytest
import torch

import gozolix_models as gm
import plain_gozolix as pg
from gopherllm_b200.api import build_model
from gopherllm_b200.cache.sequence_cache import KVView, SequenceCache, StateView
from gopherllm_b200.config.registry import architecture_from_config
from gopherllm_b200.parts.base import KVRequest, StateRequest
from gopherllm_b200.weights.loader import check_folder, tensor_table


def build(cfg):
    arch = architecture_from_config(cfg)
    typed = arch.config_class.from_dict(cfg)
    return arch, typed, build_model(arch, typed)


@pytest.mark.parametrize("cfg", [gm.ALPHA, gm.BETA, gm.GAMMA], ids=["ALPHA", "BETA", "GAMMA"])
def test_declared_tensors_are_the_files_tensors(cfg):
    arch, typed, model = build(cfg)
    assert arch.name == "gozolix"
    table = tensor_table(model.parameters(), arch.tensor_names(typed))
    want = gm.tensor_shapes(cfg)
    assert set(table) == set(want)
    for name, (shape, _) in want.items():
        assert tuple(table[name][1].shape) == tuple(shape), name


def test_every_constant_of_the_file_reaches_the_spec():
    _, typed, model = build(gm.ALPHA)
    spec = model.spec
    assert spec.embedding_scale == 3.0 and spec.final_norm.eps == 1e-5 and not spec.head_bias
    pair = spec.pair_embedding
    assert (pair.buckets, pair.mul_prev, pair.mul_cur) == (101, 13, 5)
    d, a, reader, d2 = (b.mixer for b in spec.layers)
    assert (d.kind, d.num_heads, d.num_kv_heads, d.head_dim, d.value_dim) == ("gated_delta", 4, 2, 16, 24)
    assert d.option("conv") == 3 and d.q_scale == 16 ** -0.5 and d.option("norm_eps") == 1e-5
    assert a.option("score_scale") == 0.2 and a.option("softcap") == 5.0 and a.option("q_temp") == (0.5, 7.0)
    assert a.bias and not a.option("shared_kv") and reader.option("shared_kv") and reader.option("q_temp") == (0.2, 50.0)
    moe = spec.layers[1].ffn
    assert moe.kind == "moe" and moe.intermediate == 40
    assert [moe.option(k) for k in ("experts", "top", "groups", "keep", "router_scale", "shared")] == [8, 3, 4, 2, 2.5, 24]
    plain = spec.layers[3].ffn
    assert [plain.option(k) for k in ("experts", "top", "groups", "keep", "shared")] == [6, 2, 1, 1, 0]
    assert spec.layers[0].ffn.activation == "relu2" and spec.layers[2].ffn is None
    assert typed.to_dict()["layers"] == gm.ALPHA["layers"]
    # no pair table, no soft cap, no temperature
    _, _, other = build(gm.BETA)
    assert other.spec.pair_embedding is None and other.spec.embedding_cache_entry is None
    first = other.spec.layers[0].mixer
    assert first.option("softcap") is None and first.option("q_temp") is None


def test_schedule_and_cache_of_layers_that_share_keys():
    _, _, model = build(gm.BETA)
    runs = model.spec.schedule
    assert [(e.layer, e.cache, e.writes) for e in runs] == [(0, 0, True), (1, 1, True), (2, 2, True), (3, 0, False),
                                                            (4, 0, False)]
    reqs = model.cache_requests()
    assert reqs[0] == KVRequest(3, 16, 0, value_dim=48) and isinstance(reqs[1], StateRequest) and len(reqs) == 3
    _, _, with_pair = build(gm.ALPHA)
    reqs = with_pair.cache_requests()
    assert reqs[-1] == StateRequest((1,)) and with_pair.spec.embedding_cache_entry == len(reqs) - 1
    # the delta layer keeps its memory and the filter's last inputs: 4 heads x 16 x 24, and 2 taps back of 160 channels
    assert reqs[0] == StateRequest((4 * 16 * 24 + (2 * 2 * 16 + 4 * 24) * 2,))
    cache = SequenceCache(reqs, max_tokens=256, max_positions=256, dtype=torch.float32, device="cpu", max_slots=2)
    assert isinstance(cache.view(1), KVView) and isinstance(cache.view(0), StateView)
    assert tuple(cache.view(1).k.shape[1:]) == (2, 64, 32) and tuple(cache.view(1).v.shape[1:]) == (2, 64, 16)
    s = cache.open()
    cache.view(len(reqs) - 1).rows[s].fill_(7.0)
    cache.close(s)
    assert cache.open() == s and float(cache.view(len(reqs) - 1).rows[s].abs().max()) == 0.0


def _with(cfg, path, value):
    out = copy.deepcopy(cfg)
    at = out
    for k in path[:-1]:
        at = at[k]
    if value is KeyError:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    return out


@pytest.mark.parametrize("path,value", [
    (("layers", 2, "mixer", "kv_from"), 3), (("layers", 2, "mixer", "kv_from"), 0), (("layers", 2, "mixer", "kv_from"), 2),
    (("layers", 2, "mixer", "vdim"), 32), (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 1, "mixer", "scale"), KeyError),
    (("layers", 1, "mlp", "router", "groups", "count"), 3), (("layers", 1, "mlp", "router", "top"), 5),
    (("layers", 1, "mlp", "kind"), "sparse"), (("layers", 0, "type"), "mamba"), (("layers", 0, "mixer", "conv"), 0),
    (("embedding", "bigram", "buckets"), 0), (("norm", "eps"), 0.0), (("width",), KeyError)])
def test_configurations_that_are_refused(path, value):
    with pytest.raises((ValueError, KeyError)):
        build(_with(gm.ALPHA, path, value))


def test_plain_layers_do_not_look_ahead():
    for cfg in (gm.ALPHA, gm.GAMMA):
        t = {k: v.double() for k, v in gm.draw(cfg, 2).items()}
        toks = [int(x) for x in np.random.default_rng(0).integers(0, cfg["vocab"], size=12)]
        a = pg.forward(toks, t, cfg)
        b = pg.forward(toks[:7], t, cfg)
        assert torch.allclose(a[:7], b, atol=1e-10)


def test_plain_delta_rule_written_out():
    """With a decay of one and beta of one the memory holds, under a key of unit length, exactly the value last
    written under it: reading with the same key returns that value."""
    torch.manual_seed(0)
    T, W = 6, 8
    w = {"q": torch.randn(4, W), "k": torch.randn(4, W), "v": torch.randn(3, W), "g": torch.randn(3, W), "o": torch.eye(3),
         "norm": torch.ones(3), "b": torch.zeros(1, W), "a": torch.zeros(1, W), "A_log": torch.tensor([0.0]),
         "dt_bias": torch.tensor([-1e4]), "q.conv": torch.ones(4, 1), "k.conv": torch.ones(4, 1), "v.conv": torch.ones(3, 1)}
    w = {k: v.double() for k, v in w.items()}
    w["q"] = w["k"].clone()                        # the query is the key
    w["b"][:] = 0.0
    h = torch.randn(T, W).double()
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 3, "conv": 1}
    # beta = sigmoid(0) = 1/2 here; write the recurrence out by hand for two tokens
    silu = lambda z: z * torch.sigmoid(z)
    k = silu(h @ w["k"].T)
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    v = silu(h @ w["v"].T)
    S = torch.zeros(4, 3, dtype=torch.float64)
    outs = []
    for t in range(T):
        S = S + torch.outer(k[t], 0.5 * (v[t] - S.T @ k[t]))
        outs.append(S.T @ (k[t] * 0.5))
    o = torch.stack(outs)
    gate = h @ w["g"].T
    want = o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-6) * silu(gate)
    got = pg.delta_mixer(h, w, "", m, 1e-6)
    assert torch.allclose(got, want, atol=1e-9)


def test_plain_router_on_an_example_by_hand():
    """Eight experts in four pairs, two pairs stay, three experts chosen."""
    z = torch.tensor([[2.0, -1.0, 0.5, 0.4, 3.0, -3.0, 1.0, 0.9]], dtype=torch.float64)
    w = {"router": torch.eye(8, dtype=torch.float64)}
    r = {"experts": 8, "top": 3, "scale": 2.0, "groups": {"count": 4, "keep": 2}}
    s = torch.sigmoid(z[0])
    # pair scores: (0,1) s0+s1, (2,3), (4,5), (6,7): the best two are (0,1)? and (6,7)?
    pair = [float(s[2 * i] + s[2 * i + 1]) for i in range(4)]
    best = sorted(range(4), key=lambda i: -pair[i])[:2]
    allowed = sorted(e for g in best for e in (2 * g, 2 * g + 1))
    top = sorted(allowed, key=lambda e: -float(s[e]))[:3]
    chosen, weights = pg.route(z, w, "", r)
    assert chosen[0].tolist() == top
    assert torch.allclose(weights[0], s[top] / s[top].sum() * 2.0)
    # without groups the three largest of all
    chosen, _ = pg.route(z, w, "", {"experts": 8, "top": 3, "scale": 1.0})
    assert chosen[0].tolist() == [4, 0, 6]


def test_plain_first_token_takes_the_tables_last_row():
    cfg = gm.GAMMA
    t = {k: v.double() for k, v in gm.draw(cfg, 1).items()}
    x = pg.embedding(torch.tensor([5, 9]), t, cfg)
    n = cfg["embedding"]["bigram"]["buckets"]
    assert torch.allclose(x[0], t["embed"][5] * 0.7 + t["bigram"][n])
    assert torch.allclose(x[1], t["embed"][9] * 0.7 + t["bigram"][(5 * 2000000011 + 9) % n])


def test_command_line_inspects_and_writes_a_random_folder(tmp_path, capsys):
    from gopherllm_b200.cli import main
    cfg_file = tmp_path / "c.json"
    cfg_file.write_text(json.dumps(gm.GAMMA))
    folder = str(tmp_path / "m")
    assert main([folder, "--random-config", str(cfg_file), "--seed", "3"]) == 0
    arch, typed, model = build(gm.GAMMA)
    check_folder(folder, tensor_table(model.parameters(), arch.tensor_names(typed)))
    capsys.readouterr()
    assert main([folder, "--inspect"]) == 0
    out = capsys.readouterr().out
    assert "architecture: Gozolix" in out and "supported: true" in out
    cfg, t = gm.read_folder(folder)
    assert torch.isfinite(pg.forward([1, 2, 3, 4, 5], t, cfg)).all()
