"""Small Gozolix configurations for the tests, with weights made by the tests themselves.

The tensors are drawn here by name (the design's naming rules, restated), written with the library's
container writer and read back by the library and by the plain implementation, so a wrong name or shape
on either side shows.  The configurations differ in every respect: widths (one a multiple of nothing),
head counts (one head, as many key/value heads as query heads, nine query heads on one key/value head,
ten key/value heads), key sizes that are no multiples of 16, value sizes other than key sizes, memories
wider than one block of columns, filters of one to four taps, temperatures whose period is shorter than
the prompts, soft caps that bite, layers without a feed-forward, a delta layer first, a layer that reads
the keys of a layer that is not its neighbour, two readers of one layer, routers with groups of one
expert, with several groups kept and without groups, mixtures with and without a shared expert, an
embedding with and without the hashed pair table.
"""
import json
import os
import tempfile

import torch

ALPHA = dict(
    architecture="Gozolix", vocab=300, width=64, norm={"eps": 1e-5},
    embedding={"scale": 3.0, "bigram": {"buckets": 101, "mul_prev": 13, "mul_cur": 5}},
    layers=[
        {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 3},
         "mlp": {"kind": "dense", "ff": 96}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.2, "softcap": 5.0,
                                        "q_temp": {"coef": 0.5, "every": 7}},
         "mlp": {"kind": "moe", "expert": {"ff": 40}, "shared": {"ff": 24},
                 "router": {"experts": 8, "top": 3, "scale": 2.5, "groups": {"count": 4, "keep": 2}}}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.3, "softcap": 8.0,
                                        "q_temp": {"coef": 0.2, "every": 50}, "kv_from": 1}, "mlp": None},
        {"type": "delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 8, "conv": 2},
         "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 6, "top": 2, "scale": 1.0}}},
    ])

BETA = dict(
    architecture="Gozolix", vocab=257, width=96, norm={"eps": 1e-6},
    embedding={"scale": 1.0},
    layers=[
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 3, "dim": 16, "vdim": 48, "scale": 0.25},
         "mlp": {"kind": "dense", "ff": 64}},
        {"type": "delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 72, "vdim": 130, "conv": 1}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 1, "dim": 24, "vdim": 24, "scale": 0.2, "softcap": 30.0,
                                        "q_temp": {"coef": 0.1, "every": 64}},
         "mlp": {"kind": "moe", "expert": {"ff": 32}, "shared": {"ff": 48},
                 "router": {"experts": 4, "top": 2, "scale": 1.0, "groups": {"count": 4, "keep": 3}}}},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 3, "dim": 16, "vdim": 48, "scale": 0.5, "kv_from": 0},
         "mlp": {"kind": "dense", "ff": 40}},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 3, "dim": 16, "vdim": 48, "scale": 0.125, "softcap": 2.0,
                                        "kv_from": 0}, "mlp": None},
    ])

# sizes that are multiples of nothing convenient
GAMMA = dict(
    architecture="Gozolix", vocab=91, width=36, norm={"eps": 3e-6},
    embedding={"scale": 0.7, "bigram": {"buckets": 17, "mul_prev": 2000000011, "mul_cur": 1}},
    layers=[
        {"type": "delta", "mixer": {"heads": 3, "kv_heads": 1, "dim": 5, "vdim": 7, "conv": 4},
         "mlp": {"kind": "moe", "expert": {"ff": 11}, "shared": {"ff": 5},
                 "router": {"experts": 9, "top": 2, "scale": 0.5, "groups": {"count": 3, "keep": 1}}}},
        {"type": "attention", "mixer": {"heads": 9, "kv_heads": 1, "dim": 6, "vdim": 10, "scale": 0.4, "softcap": 3.0,
                                        "q_temp": {"coef": 1.0, "every": 3}}, "mlp": {"kind": "dense", "ff": 20}},
        {"type": "attention", "mixer": {"heads": 20, "kv_heads": 10, "dim": 16, "vdim": 16, "scale": 0.25}, "mlp": None},
    ])


def only(cfg, index, mlp=True):
    """A model of one layer of ``cfg`` (a mechanism alone), with or without its feed-forward."""
    layer = json.loads(json.dumps(cfg["layers"][index]))
    layer["mixer"].pop("kv_from", None)
    if not mlp:
        layer["mlp"] = None
    elif layer["mlp"] is None:
        layer["mlp"] = {"kind": "dense", "ff": 32}
    out = {k: v for k, v in cfg.items() if k != "layers"}
    out["layers"] = [layer]
    return out


def tensor_shapes(cfg):
    """name -> (shape, how it is drawn)."""
    W, V = cfg["width"], cfg["vocab"]
    s = {"embed": ((V, W), "embed"), "final.norm": ((W,), "gamma"), "head": ((V, W), "matrix")}
    if cfg["embedding"].get("bigram"):
        s["bigram"] = ((cfg["embedding"]["bigram"]["buckets"] + 1, W), "embed")
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s[p + "norm1"] = ((W,), "gamma")
        H, G, D, Vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if L["type"] == "delta":
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * Vd)):
                s[p + "mix." + n] = ((rows, W), "matrix")
                s[p + "mix." + n + ".conv"] = ((rows, m["conv"]), "taps")
            s.update({p + "mix.b": ((H, W), "matrix"), p + "mix.a": ((H, W), "matrix"), p + "mix.A_log": ((H,), "decay"),
                      p + "mix.dt_bias": ((H,), "step"), p + "mix.g": ((H * Vd, W), "matrix"),
                      p + "mix.norm": ((Vd,), "gamma"), p + "mix.o": ((W, H * Vd), "matrix")})
        else:
            s.update({p + "mix.q": ((H * D, W), "query"), p + "mix.q.b": ((H * D,), "small"), p + "mix.o": ((W, H * Vd), "matrix")})
            if m.get("kv_from") is None:
                s.update({p + "mix.k": ((G * D, W), "query"), p + "mix.k.b": ((G * D,), "small"),
                          p + "mix.v": ((G * Vd, W), "matrix"), p + "mix.v.b": ((G * Vd,), "small")})
        mlp = L.get("mlp")
        if mlp and mlp.get("kind", "dense") == "dense":
            s.update({p + "mlp.up": ((mlp["ff"], W), "matrix"), p + "mlp.down": ((W, mlp["ff"]), "matrix")})
        elif mlp:
            F = mlp["expert"]["ff"]
            s[p + "mlp.router"] = ((mlp["router"]["experts"], W), "router")
            units = [(f"e{e}", F) for e in range(mlp["router"]["experts"])]
            if mlp.get("shared"):
                units.append(("shared", mlp["shared"]["ff"]))
            for name, f in units:
                s.update({f"{p}mlp.{name}.gate": ((f, W), "matrix"), f"{p}mlp.{name}.up": ((f, W), "matrix"),
                          f"{p}mlp.{name}.down": ((W, f), "matrix")})
    return s


def draw(cfg, seed, long_memory=False, sharp=1.0):
    """Random tensors (bfloat16) for ``cfg``.  ``long_memory``: decays near one, so that a memory still holds
    tokens from hundreds of positions back.  ``sharp``: factor on the attention's query and key weights, so
    that the softmax settles on few keys and one key more or less, or one position off, changes the output."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, (shape, kind) in sorted(tensor_shapes(cfg).items()):
        z = torch.randn(shape, generator=g)
        if kind == "matrix":
            t = z * (1.0 / shape[-1] ** 0.5)
        elif kind == "query":
            t = z * (sharp / shape[-1] ** 0.5)
        elif kind == "router":
            t = z * (2.0 / shape[-1] ** 0.5)
        elif kind == "embed":
            t = z
        elif kind == "gamma":
            t = 1.0 + 0.1 * z
        elif kind == "small":
            t = 0.1 * z
        elif kind == "taps":
            t = 0.6 * z
        elif kind == "decay":
            t = 0.5 * z - (3.0 if long_memory else 0.0)
        elif kind == "step":
            t = z - (3.0 if long_memory else 0.0)
        else:
            raise ValueError(kind)
        out[name] = t.to(torch.bfloat16)
    return out


def write_folder(cfg, tensors, folder=None):
    from gopherllm_b200.weights.safetensors_io import write_file
    folder = folder or tempfile.mkdtemp(prefix="gl_gozolix_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(folder, "model.safetensors"), sorted(tensors.items()), metadata={"format": "pt"})
    return folder


def read_folder(folder):
    """(config dict, name -> 64-bit tensor) with a reader of the tests' own: 8 bytes of length, a JSON header,
    the data."""
    import struct
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    raw = open(os.path.join(folder, "model.safetensors"), "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16}
    tensors = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        a, b = e["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + a:8 + n + b]), dtype=kinds[e["dtype"]])
        tensors[name] = t.reshape(e["shape"]).to(torch.float64)
    return cfg, tensors
