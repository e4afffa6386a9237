"""The Vopedra design's host side: configuration, schedule, tensor names, cache requests; and the
plain implementation's own consistency (no GPU)."""
import copy

import numpy as np
import pytest
import torch

import plain_vopedra as pv
import vopedra_models as vm
from gopherllm_b200.api import build_model
from gopherllm_b200.cache.sequence_cache import KVView, SequenceCache, StateView
from gopherllm_b200.config import architecture_from_config, looped_schedule
from gopherllm_b200.config.vopedra import VopedraConfig
from gopherllm_b200.parts.base import KVRequest, StateRequest
from gopherllm_b200.weights.loader import check_folder, tensor_table


def build(cfg):
    arch = architecture_from_config(cfg)
    typed = arch.config_class.from_dict(cfg)
    return arch, typed, build_model(arch, typed)


def test_architecture_is_found_by_its_plain_key():
    arch = architecture_from_config({"architecture": "Vopedra"})
    assert arch.name == "vopedra" and arch.config_class is VopedraConfig
    with pytest.raises(ValueError):
        architecture_from_config({"architecture": "Nonesuch"})


@pytest.mark.parametrize("cfg", [vm.ALPHA, vm.BETA, vm.GAMMA, vm.DELTA], ids=["alpha", "beta", "gamma", "delta"])
def test_declared_tensors_are_the_files_tensors(cfg):
    """The names and shapes the parts declare are the ones the tests write by the design's naming
    rules; a folder written that way passes the loader's check."""
    arch, typed, model = build(cfg)
    table = tensor_table(model.parameters(), arch.tensor_names(typed))
    want = {n: tuple(s) for n, (s, _) in vm.tensor_shapes(cfg).items()}
    assert {n: tuple(spec.shape) for n, (_, spec) in table.items()} == want
    folder = vm.write_folder(cfg, vm.draw(cfg, 1))
    check_folder(folder, table)


def test_schedule_of_a_loop():
    runs = looped_schedule(6, 1, 5, 2)
    assert [r.layer for r in runs] == [0, 1, 2, 3, 4, 1, 2, 3, 4, 5]
    assert [r.cache for r in runs] == list(range(10))                     # every run its own entry
    marks = [(i, r.enter.index, r.enter.add_embedding) for i, r in enumerate(runs) if r.enter is not None]
    assert marks == [(1, 0, False), (5, 1, True)]
    once = looped_schedule(3, 0, 2, 1)
    assert [r.layer for r in once] == [0, 1, 2] and once[0].enter.index == 0 and not once[0].enter.add_embedding
    assert [i for i, _, _ in pv.layer_order({"layers": [0] * 6, "loop": {"start": 1, "stop": 5, "times": 2}})] == [r.layer for r in runs]
    with pytest.raises(ValueError):
        looped_schedule(3, 2, 1, 2)


def test_spec_carries_every_constant_of_the_file():
    cfg = copy.deepcopy(vm.ALPHA)
    cfg["layers"][2]["mixer"]["left"].update(scale=0.37, rot={"dims": 8, "base": 77.0})
    cfg["layers"][0]["mixer"]["gate_cap"] = 3.5
    cfg["norm"]["eps"] = 2e-3
    _, _, model = build(cfg)
    spec = model.spec
    left = spec.layers[2].mixer.option("left")
    assert left.q_scale == 0.37 and left.position.rotary_dim == 8 and left.position.theta == 77.0
    assert left.value_dim == 16 and left.head_dim == 32 and left.num_kv_heads == 2
    assert spec.layers[0].mixer.option("gate_cap") == 3.5 and spec.layers[0].norm.eps == 2e-3
    assert spec.layers[1].ffn is None and spec.layers[1].norm2 is None
    assert spec.pass_vectors == 3 and spec.embedding_norm is not None and not spec.head_bias


@pytest.mark.parametrize("change", [
    lambda c: c["layers"][0].update(type="gru"),
    lambda c: c["layers"][2]["mixer"]["left"].update(heads=3),                 # not a multiple of kv_heads
    lambda c: c["layers"][2]["mixer"]["left"]["rot"].update(dims=7),
    lambda c: c["layers"][1]["mixer"].pop("state"),
    lambda c: c["loop"].update(stop=9),
    lambda c: c.pop("norm"),
    lambda c: c["layers"][0]["mixer"].update(gate_cap=0),
])
def test_bad_configurations_are_refused(change):
    cfg = copy.deepcopy(vm.ALPHA)
    change(cfg)
    with pytest.raises(ValueError):
        VopedraConfig.from_dict(cfg)


def test_cache_requests_and_views_of_a_pair():
    _, _, model = build(vm.ALPHA)
    reqs = model.cache_requests()
    assert len(reqs) == 1 + 2 * 3                                          # a run, an entry
    pair = reqs[2]
    assert isinstance(pair, tuple) and pair[0] == KVRequest(2, 32, 0, value_dim=16) and isinstance(pair[1], StateRequest)
    cache = SequenceCache(reqs, 256, 256, torch.float32, "cpu")
    view = cache.view(2)
    assert isinstance(view[0], KVView) and isinstance(view[1], StateView)
    assert tuple(view[0].k.shape[1:]) == (2, 64, 32) and tuple(view[0].v.shape[1:]) == (2, 64, 16)
    assert len(cache.groups) == 1 and len(cache.groups[0].entries) == 3     # the three passes' attention entries
    s = cache.open()
    view[1].rows[s].fill_(3.0)
    cache.close(s)
    assert cache.open() == s and float(view[1].rows[s].abs().max()) == 0.0  # state rows start at zero again


def test_plain_mixers_do_not_look_ahead():
    """Causality of the plain implementation itself: a later token changes no earlier logits."""
    cfg = vm.ALPHA
    t = {k: v.double() for k, v in vm.draw(cfg, 2).items()}
    toks = [int(x) for x in np.random.default_rng(0).integers(0, cfg["vocab"], size=12)]
    a = pv.forward(cfg, t, toks)
    b = pv.forward(cfg, t, toks[:7])
    assert torch.allclose(a[:7], b, atol=1e-10)


def test_plain_gated_memory_matches_its_closed_form():
    """The recurrence with a running maximum equals the same sums written out without it."""
    torch.manual_seed(0)
    T, W = 9, 16
    m = {"heads": 1, "dim": 4, "vdim": 5, "gate_cap": 8.0}
    t = {"q": torch.randn(4, W), "k": torch.randn(4, W), "v": torch.randn(5, W), "g": torch.randn(5, W),
         "o": torch.eye(5), "norm": torch.ones(5), "i": torch.randn(1, W), "i.b": torch.randn(1),
         "f": torch.randn(1, W), "f.b": torch.randn(1)}
    t = {k: v.double() for k, v in t.items()}
    h = torch.randn(T, W).double()
    got = pv.mlstm_mixer(h, t, "", m, 1e-6)
    q, k, v = (h @ t["q"].T) * 0.5, h @ t["k"].T, h @ t["v"].T
    gi = 8 * torch.tanh((h @ t["i"].T + t["i.b"]) / 8)[:, 0]
    gf = pv.log_sigmoid(8 * torch.tanh((h @ t["f"].T + t["f.b"]) / 8))[:, 0]
    rows = []
    for s in range(T):
        logw = torch.stack([gi[j] + gf[j + 1:s + 1].sum() for j in range(s + 1)])
        mx = torch.maximum(torch.tensor(0.0, dtype=torch.float64) + gf[:s + 1].sum(), logw.max())   # the maximum started at 0
        w = torch.exp(logw - mx)
        num = (w[:, None] * (k[:s + 1] @ q[s])[:, None] * v[:s + 1]).sum(0)
        den = torch.maximum(torch.abs((w * (k[:s + 1] @ q[s])).sum()), torch.exp(-mx)) + 1e-6
        rows.append(num / den)
    o = torch.stack(rows)
    want = pv.rms_norm(o, None, 1e-6) * torch.sigmoid(h @ t["g"].T)
    assert torch.allclose(got, want, atol=1e-9)


def test_command_line_inspects_and_writes_a_random_folder(tmp_path, capsys):
    """--random-config writes a Vopedra folder the loader's check accepts; --inspect names the design."""
    import json
    from gopherllm_b200.cli import main
    cfg_file = tmp_path / "c.json"
    cfg_file.write_text(json.dumps(vm.GAMMA))
    folder = str(tmp_path / "m")
    assert main([folder, "--random-config", str(cfg_file), "--seed", "3"]) == 0
    arch, typed, model = build(vm.GAMMA)
    check_folder(folder, tensor_table(model.parameters(), arch.tensor_names(typed)))
    capsys.readouterr()
    assert main([folder, "--inspect"]) == 0
    out = capsys.readouterr().out
    assert "architecture: Vopedra" in out and "supported: true" in out
    _, t = pv.read_folder(folder)
    logits = pv.forward(vm.GAMMA, t, [1, 2, 3, 4, 5])
    assert torch.isfinite(logits).all()
