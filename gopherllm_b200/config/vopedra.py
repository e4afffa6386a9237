"""The Vopedra design: a decoder whose layers mix tokens in different ways and may run in a loop.

config.json lists the layers one by one (``layers[i].type`` is ``mlstm``, ``mamba1`` or ``parallel``,
``layers[i].mixer`` the mixer's sizes, ``layers[i].mlp`` a gated feed-forward or null) and may name
a range of layers that runs several times in a row with the same weights (``loop``: start, stop,
times).  A layer is x <- x + (mixer(norm1(x)) + ff(norm2(x))) with RMS norms; the embedding is
normalised before the first layer, and the output head has no bias.

  mlstm     a matrix memory per head with exponential input and forget gates, a normaliser and a
            running maximum of the log gates (the mLSTM of xLSTM); log gates are soft-capped
  mamba1    a selective state-space scan behind a short causal convolution (Mamba)
  parallel  softmax attention (grouped keys/values, queries and keys normalised over the whole
            projection, partial rotation, head weights mixed by a learned table after the softmax) beside
            a gated linear attention whose bounded forget gate also sets what is written (HGRN2); each
            output normalised over the width, the two averaged

Every size and constant comes from config.json; constants the design fixes are in the parts.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Optional

from .registry import Architecture, register_architecture
from .specs import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                    default_schedule, looped_schedule)

# the design sets no longest sequence; the cache's size bounds one
UNBOUNDED_POSITIONS = 1 << 20


def _positive_int(where: str, d: dict, key: str) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ValueError(f"config.json: {where}.{key} must be a positive integer, is {v!r}")
    return v


def _positive(where: str, d: dict, key: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not (v > 0 and math.isfinite(v)):
        raise ValueError(f"config.json: {where}.{key} must be a positive number, is {v!r}")
    return float(v)


@dataclass
class VopedraConfig:
    """Typed view of a Vopedra config.json (key names are the file's own)."""
    vocab: int
    width: int
    layers: list
    norm_eps: float
    loop: Optional[dict] = None
    architecture: str = "Vopedra"
    torch_dtype: str = "bfloat16"
    initializer_range: float = 0.05

    @classmethod
    def from_dict(cls, d: dict) -> "VopedraConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm") if k not in d]
        if missing:
            raise ValueError(f"config.json lacks required keys: {', '.join(missing)}")
        if not isinstance(d["norm"], dict):
            raise ValueError("config.json: norm must be an object with eps")
        cfg = cls(vocab=_positive_int("config", d, "vocab"), width=_positive_int("config", d, "width"),
                  layers=copy.deepcopy(d["layers"]), norm_eps=_positive("norm", d["norm"], "eps"),
                  loop=copy.deepcopy(d.get("loop")) or None,
                  architecture=str(d.get("architecture", "Vopedra")),
                  torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
                  initializer_range=float(d.get("initializer_range", 0.05)))
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "layers": copy.deepcopy(self.layers), "norm": {"eps": self.norm_eps},
             "torch_dtype": self.torch_dtype, "initializer_range": self.initializer_range}
        if self.loop:
            d["loop"] = dict(self.loop)
        return d

    def validate(self) -> None:
        if not isinstance(self.layers, list) or not self.layers:
            raise ValueError("config.json: layers must be a non-empty list")
        for i, L in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(L, dict) or L.get("type") not in _MIXERS:
                raise ValueError(f"config.json: {where}.type must be one of {', '.join(sorted(_MIXERS))}")
            if not isinstance(L.get("mixer"), dict):
                raise ValueError(f"config.json: {where}.mixer must be an object")
            _MIXERS[L["type"]](self, L["mixer"], where + ".mixer")        # raises on a bad size
            mlp = L.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind", "dense") != "dense":
                    raise ValueError(f"config.json: {where}.mlp.kind must be dense (or mlp null)")
                _positive_int(where + ".mlp", mlp, "ff")
        if self.loop:
            lp = self.loop
            for k in ("start", "stop", "times"):
                if isinstance(lp.get(k), bool) or not isinstance(lp.get(k), int):
                    raise ValueError(f"config.json: loop.{k} must be an integer")
            if not (0 <= lp["start"] <= lp["stop"] <= len(self.layers)) or lp["times"] < 1:
                raise ValueError(f"config.json: loop {lp} does not fit {len(self.layers)} layers")


def _mlstm(cfg: VopedraConfig, m: dict, where: str) -> MixerSpec:
    return MixerSpec(kind="mlstm", hidden=cfg.width, num_heads=_positive_int(where, m, "heads"),
                     head_dim=_positive_int(where, m, "dim"), value_dim=_positive_int(where, m, "vdim"),
                     q_scale=float(m["dim"]) ** -0.5, bias=False,
                     extra=(("gate_cap", _positive(where, m, "gate_cap")), ("norm_eps", cfg.norm_eps)))


def _mamba1(cfg: VopedraConfig, m: dict, where: str) -> MixerSpec:
    return MixerSpec(kind="mamba1", hidden=cfg.width, bias=False,
                     extra=(("inner", _positive_int(where, m, "inner")), ("state", _positive_int(where, m, "state")),
                            ("dt_rank", _positive_int(where, m, "dt_rank")), ("conv", _positive_int(where, m, "conv"))))


def _talking_attention(cfg: VopedraConfig, m: dict, where: str) -> MixerSpec:
    heads, kv = _positive_int(where, m, "heads"), _positive_int(where, m, "kv_heads")
    dim = _positive_int(where, m, "dim")
    if heads % kv:
        raise ValueError(f"config.json: {where}.heads {heads} is not a multiple of kv_heads {kv}")
    rot = m.get("rot") or {}
    dims = rot.get("dims", 0)
    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > dim:
        raise ValueError(f"config.json: {where}.rot.dims must be even and at most dim, is {dims!r}")
    position = (PositionSpec("rope", dims, _positive(where + ".rot", rot, "base"), interleaved=False,
                             extra=(("exact_angles", True),))
                if dims > 0 else PositionSpec("none"))
    return MixerSpec(kind="attention_mixed", hidden=cfg.width, num_heads=heads, num_kv_heads=kv, head_dim=dim,
                     value_dim=_positive_int(where, m, "vdim"), q_scale=_positive(where, m, "scale"), bias=False,
                     position=position, extra=(("norm_eps", cfg.norm_eps), ("qk_norm", "projection"), ("talk", True)))


def _hgrn2(cfg: VopedraConfig, m: dict, where: str) -> MixerSpec:
    return MixerSpec(kind="hgrn2", hidden=cfg.width, num_heads=_positive_int(where, m, "heads"),
                     head_dim=_positive_int(where, m, "dim"), value_dim=_positive_int(where, m, "vdim"), bias=False,
                     extra=(("norm_eps", cfg.norm_eps),))


def _parallel(cfg: VopedraConfig, m: dict, where: str) -> MixerSpec:
    for side in ("left", "right"):
        if not isinstance(m.get(side), dict):
            raise ValueError(f"config.json: {where}.{side} must be an object")
    return MixerSpec(kind="normed_pair", hidden=cfg.width, bias=False,
                     extra=(("left", _talking_attention(cfg, m["left"], where + ".left")),
                            ("right", _hgrn2(cfg, m["right"], where + ".right")),
                            ("norm_eps", cfg.norm_eps), ("weight", 0.5)))


_MIXERS = {"mlstm": _mlstm, "mamba1": _mamba1, "parallel": _parallel}


def vopedra_model_spec(cfg: VopedraConfig) -> ModelSpec:
    norm = NormSpec("rmsnorm", cfg.width, cfg.norm_eps, bias=False)
    layers = []
    for i, L in enumerate(cfg.layers):
        mixer = _MIXERS[L["type"]](cfg, L["mixer"], f"layers[{i}].mixer")
        mlp = L.get("mlp")
        ffn = (FeedForwardSpec(kind="gated", hidden=cfg.width, intermediate=int(mlp["ff"]),
                               activation="gelu_pytorch_tanh", bias=False) if mlp is not None else None)
        layers.append(BlockSpec(arrangement="parallel_two_norms", norm=norm, mixer=mixer, ffn=ffn,
                                norm2=norm if ffn is not None else None))
    if cfg.loop:
        schedule = looped_schedule(len(layers), cfg.loop["start"], cfg.loop["stop"], cfg.loop["times"])
        passes = cfg.loop["times"]
    else:
        schedule, passes = default_schedule(len(layers)), 0
    return ModelSpec(hidden=cfg.width, vocab=cfg.vocab, max_positions=UNBOUNDED_POSITIONS, layers=tuple(layers),
                     schedule=schedule, final_norm=norm, tie_embeddings=False, head_bias=False,
                     embedding_norm=norm, pass_vectors=passes)


class VopedraTensorNames:
    """Names of the tensors in a Vopedra safetensors file: ``embed``, ``embed.norm``, ``loop.step``,
    ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``; a linear
    layer's weight carries no suffix, its bias ``.b``."""
    _top = {"embedding": "embed", "embedding_norm/weight": "embed.norm", "pass_vectors": "loop.step",
            "final_norm/weight": "final.norm", "head/weight": "head"}
    _slots = {"norm": "norm1", "norm2": "norm2", "mixer": "mix", "ffn": "mlp"}

    def __init__(self, cfg: VopedraConfig):
        self.cfg = cfg

    def top(self, key: str) -> str:
        return self._top[key]

    def layer(self, i: int, slot: str, key: str) -> str:
        """Parts spell a parameter "q.weight", "i.bias", "norm.weight", "left.q_norm.weight"; the file
        spells them "q", "i.b", "norm", "left.q.norm"."""
        base = f"l{i}.{self._slots[slot]}"
        if slot in ("norm", "norm2"):
            return base
        words = key.split(".")
        if words[-1] == "weight":
            words = words[:-1]
        elif words[-1] == "bias":
            words[-1] = "b"
        words = [w.replace("q_norm", "q.norm").replace("k_norm", "k.norm") for w in words]
        return ".".join([base] + words)


register_architecture(
    Architecture(name="vopedra", config_class=VopedraConfig, build_spec=vopedra_model_spec,
                 tensor_names=VopedraTensorNames),
)
