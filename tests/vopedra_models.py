"""Small Vopedra configurations for the tests, with weights made by the tests themselves.

The tensors are drawn here by name (the design's own naming rules, restated), written with the
library's container writer and read back by the library and by the plain implementation, so a wrong
name or shape on either side shows.  Sizes differ between the configurations in every respect:
widths, head counts (also one head, and as many key/value heads as query heads), key sizes above and
below 64, value sizes other than key sizes, memories wider than one block of columns, states of more
than eight entries a channel, a low rank that is no multiple of 8, filters of one to four taps, a
rotation over the whole head, over a part and over nothing, a loop run once, three times, over no layer
and no loop, layers without a feed-forward, sizes that are multiples of nothing, more query heads a
key/value head and more key/value heads than the fast one-token kernel takes.
"""
import json
import os
import tempfile

import torch

ALPHA = dict(
    architecture="Vopedra", vocab=300, width=64, norm={"eps": 1e-5},
    layers=[
        {"type": "mlstm", "mixer": {"heads": 2, "dim": 16, "vdim": 24, "gate_cap": 10.0}, "mlp": {"kind": "dense", "ff": 96}},
        {"type": "mamba1", "mixer": {"inner": 96, "state": 12, "dt_rank": 8, "conv": 4}, "mlp": None},
        {"type": "parallel", "mixer": {
            "left": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "rot": {"dims": 16, "base": 10000.0}, "scale": 0.2},
            "right": {"heads": 2, "dim": 24, "vdim": 40}}, "mlp": {"kind": "dense", "ff": 128}},
    ],
    loop={"start": 1, "stop": 3, "times": 3})

BETA = dict(
    architecture="Vopedra", vocab=257, width=96, norm={"eps": 1e-6},
    layers=[
        {"type": "parallel", "mixer": {
            "left": {"heads": 3, "kv_heads": 3, "dim": 16, "vdim": 48, "rot": {"dims": 16, "base": 500.0}, "scale": 0.3},
            "right": {"heads": 1, "dim": 72, "vdim": 8}}, "mlp": {"kind": "dense", "ff": 64}},
        {"type": "mamba1", "mixer": {"inner": 40, "state": 20, "dt_rank": 5, "conv": 2}, "mlp": {"kind": "dense", "ff": 64}},
        {"type": "mlstm", "mixer": {"heads": 1, "dim": 80, "vdim": 130, "gate_cap": 15.0}, "mlp": None},
    ])

GAMMA = dict(
    architecture="Vopedra", vocab=128, width=48, norm={"eps": 1e-4},
    layers=[
        {"type": "mamba1", "mixer": {"inner": 24, "state": 4, "dt_rank": 16, "conv": 1}, "mlp": {"kind": "dense", "ff": 40}},
        {"type": "parallel", "mixer": {
            "left": {"heads": 2, "kv_heads": 1, "dim": 24, "vdim": 24, "rot": {"dims": 0, "base": 10000.0}, "scale": 0.25},
            "right": {"heads": 3, "dim": 8, "vdim": 8}}, "mlp": None},
        {"type": "mlstm", "mixer": {"heads": 3, "dim": 8, "vdim": 8, "gate_cap": 6.0}, "mlp": {"kind": "dense", "ff": 24}},
    ],
    loop={"start": 0, "stop": 2, "times": 1})


# sizes that are multiples of nothing convenient, nine query heads on one key/value head, an empty loop
DELTA = dict(
    architecture="Vopedra", vocab=91, width=36, norm={"eps": 3e-6},
    layers=[
        {"type": "parallel", "mixer": {
            "left": {"heads": 9, "kv_heads": 1, "dim": 6, "vdim": 10, "rot": {"dims": 4, "base": 100.0}, "scale": 0.4},
            "right": {"heads": 2, "dim": 5, "vdim": 7}}, "mlp": {"kind": "dense", "ff": 20}},
        {"type": "mamba1", "mixer": {"inner": 10, "state": 3, "dt_rank": 2, "conv": 3}, "mlp": {"kind": "dense", "ff": 11}},
        {"type": "mlstm", "mixer": {"heads": 3, "dim": 5, "vdim": 9, "gate_cap": 4.0}, "mlp": None},
        {"type": "parallel", "mixer": {
            "left": {"heads": 20, "kv_heads": 10, "dim": 16, "vdim": 16, "rot": {"dims": 16, "base": 300.0}, "scale": 0.25},
            "right": {"heads": 1, "dim": 3, "vdim": 2}}, "mlp": None},
    ],
    loop={"start": 2, "stop": 2, "times": 2})


def only(cfg, index, mlp=True, loop=None):
    """A model of one layer of ``cfg`` (a mechanism alone), with or without its feed-forward."""
    layer = json.loads(json.dumps(cfg["layers"][index]))
    if not mlp:
        layer["mlp"] = None
    elif layer["mlp"] is None:
        layer["mlp"] = {"kind": "dense", "ff": 32}
    out = {k: v for k, v in cfg.items() if k not in ("layers", "loop")}
    out["layers"] = [layer]
    if loop:
        out["loop"] = loop
    return out


def tensor_shapes(cfg):
    """name -> (shape, how it is drawn)."""
    W, V = cfg["width"], cfg["vocab"]
    s = {"embed": ((V, W), "embed"), "embed.norm": ((W,), "gamma"), "final.norm": ((W,), "gamma"), "head": ((V, W), "matrix")}
    if cfg.get("loop"):
        s["loop.step"] = ((cfg["loop"]["times"], W), "small")
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s[p + "norm1"] = ((W,), "gamma")
        if L["type"] == "mlstm":
            H, D, Vd = m["heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * D), ("k", H * D), ("v", H * Vd), ("g", H * Vd), ("i", H), ("f", H)):
                s[p + "mix." + n] = ((rows, W), "matrix")
            s[p + "mix.o"] = ((W, H * Vd), "matrix")
            s[p + "mix.norm"] = ((H * Vd,), "gamma")
            s[p + "mix.i.b"] = ((H,), "wide")
            s[p + "mix.f.b"] = ((H,), "forget")
        elif L["type"] == "mamba1":
            C, N, R, K = m["inner"], m["state"], m["dt_rank"], m["conv"]
            s.update({p + "mix.in": ((2 * C, W), "matrix"), p + "mix.conv": ((C, K), "wide"), p + "mix.conv.b": ((C,), "small"),
                      p + "mix.x": ((R + 2 * N, C), "matrix"), p + "mix.dt": ((C, R), "matrix"), p + "mix.dt.b": ((C,), "step"),
                      p + "mix.A_log": ((C, N), "decay"), p + "mix.D": ((C,), "gamma"), p + "mix.o": ((W, C), "matrix")})
        else:
            l, r = m["left"], m["right"]
            H, G, D, Vd = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
            s.update({p + "mix.left.q": ((H * D, W), "matrix"), p + "mix.left.k": ((G * D, W), "matrix"),
                      p + "mix.left.v": ((G * Vd, W), "matrix"), p + "mix.left.q.norm": ((H * D,), "gamma"),
                      p + "mix.left.k.norm": ((G * D,), "gamma"), p + "mix.left.talk": ((H, H), "talk"),
                      p + "mix.left.o": ((W, H * Vd), "matrix"), p + "mix.left.out": ((W,), "gamma")})
            H, D, Vd = r["heads"], r["dim"], r["vdim"]
            s.update({p + "mix.right.q": ((H * D, W), "matrix"), p + "mix.right.f": ((H * D, W), "matrix"),
                      p + "mix.right.f.b": ((H * D,), "wide"), p + "mix.right.lower": ((H * D,), "unit"),
                      p + "mix.right.v": ((H * Vd, W), "matrix"), p + "mix.right.norm": ((Vd,), "gamma"),
                      p + "mix.right.o": ((W, H * Vd), "matrix"), p + "mix.right.out": ((W,), "gamma")})
        if L.get("mlp"):
            F = L["mlp"]["ff"]
            s.update({p + "norm2": ((W,), "gamma"), p + "mlp.gate": ((F, W), "matrix"), p + "mlp.up": ((F, W), "matrix"),
                      p + "mlp.down": ((W, F), "matrix")})
    return s


def draw(cfg, seed, long_memory=False, sharp=1.0):
    """Random tensors (bfloat16) for ``cfg``.  ``long_memory``: forget gates near one, slow decays and
    high lower bounds, so that a state still holds tokens from hundreds of positions back.  ``sharp``:
    factor on the attention's query and key norm weights, so that the softmax settles on few keys and
    one key more or less, or one position off, changes the output."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, (shape, kind) in sorted(tensor_shapes(cfg).items()):
        z = torch.randn(shape, generator=g)
        if kind == "matrix":
            t = z * (1.0 / shape[-1] ** 0.5)
        elif kind == "embed":
            t = z
        elif kind == "gamma":
            t = 1.0 + 0.1 * z
            if sharp != 1.0 and (name.endswith("q.norm") or name.endswith("k.norm")):
                t = t * sharp
        elif kind == "small":
            t = 0.1 * z
        elif kind == "wide":
            t = z
        elif kind == "forget":
            t = z + (6.0 if long_memory else 1.0)
        elif kind == "step":
            t = z - (4.0 if long_memory else 1.0)
        elif kind == "decay":
            t = 0.5 * z - (2.0 if long_memory else 0.0)
        elif kind == "unit":
            t = torch.sigmoid(z + (5.0 if long_memory else 0.0))
        elif kind == "talk":
            t = torch.eye(shape[0]) + 0.5 * z
        else:
            raise ValueError(kind)
        out[name] = t.to(torch.bfloat16)
    return out


def write_folder(cfg, tensors, folder=None):
    from gopherllm_b200.weights.safetensors_io import write_file
    folder = folder or tempfile.mkdtemp(prefix="gl_vopedra_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(folder, "model.safetensors"), sorted(tensors.items()), metadata={"format": "pt"})
    return folder
