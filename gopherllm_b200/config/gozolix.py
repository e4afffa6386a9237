"""The Gozolix design: a decoder whose layers mix tokens by softmax attention or by a gated delta rule, and
whose feed-forwards are dense or mixtures of experts.

config.json lists the layers one by one: ``layers[i].type`` is ``attention`` or ``delta``, ``layers[i].mixer``
the mixer's sizes and constants, ``layers[i].mlp`` a feed-forward (``kind`` ``dense`` or ``moe``) or null.  A
layer is x <- x + (mixer(n) + ff(n)) with n = RMS norm of x: one norm feeds both branches.  The embedding is
scaled, and a hashed embedding of the pair (token before, token) is added to it.  Final RMS norm, a head
without bias.

  attention  grouped keys and values with biases on q, k and v; no rotation: positions enter through a query
             temperature 1 + coef ln(floor((p + 1) / every) + 1) and through a penalty slope_h (i - j) on the
             scores, slope_h = 2^(-8 (h + 1) / heads); scores are scaled and soft-capped before the penalty.
             A mixer with ``kv_from: j`` has no key and value projections and reads layer j's cache entry.
  delta      the gated delta rule behind short causal convolutions (see parts/recurrent.py)
  dense      down(relu(up x)^2)
  moe        sigmoid router with groups of experts, gated silu experts, a shared expert

Every size and every constant that differs between models comes from config.json; what the design fixes
(the slopes' exponent 8, the 1e-6 under the unit norms, the 1e-20 in the router's sum) is in the parts.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Optional

from .registry import Architecture, register_architecture
from .specs import (BlockSpec, FeedForwardSpec, HashedPairSpec, MixerSpec, ModelSpec, NormSpec, ScheduleEntry)

# the design sets no longest sequence; the cache's size bounds one
UNBOUNDED_POSITIONS = 1 << 20
# head h's penalty per position of distance is 2^(-SLOPE_SPAN (h + 1) / heads)
SLOPE_SPAN = 8.0


def _int(where: str, d: dict, key: str, least: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < least:
        raise ValueError(f"config.json: {where}.{key} must be an integer of at least {least}, is {v!r}")
    return v


def _number(where: str, d: dict, key: str, positive: bool = True) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or (positive and not v > 0):
        raise ValueError(f"config.json: {where}.{key} must be a {'positive ' if positive else ''}number, is {v!r}")
    return float(v)


@dataclass
class GozolixConfig:
    """Typed view of a Gozolix config.json (key names are the file's own)."""
    vocab: int
    width: int
    layers: list
    norm_eps: float
    embedding: dict
    architecture: str = "Gozolix"
    torch_dtype: str = "bfloat16"
    initializer_range: float = 0.05

    @classmethod
    def from_dict(cls, d: dict) -> "GozolixConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm", "embedding") if k not in d]
        if missing:
            raise ValueError(f"config.json lacks required keys: {', '.join(missing)}")
        if not isinstance(d["norm"], dict) or not isinstance(d["embedding"], dict):
            raise ValueError("config.json: norm and embedding must be objects")
        cfg = cls(vocab=_int("config", d, "vocab"), width=_int("config", d, "width"),
                  layers=copy.deepcopy(d["layers"]), norm_eps=_number("norm", d["norm"], "eps"),
                  embedding=copy.deepcopy(d["embedding"]),
                  architecture=str(d.get("architecture", "Gozolix")),
                  torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
                  initializer_range=float(d.get("initializer_range", 0.05)))
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "embedding": copy.deepcopy(self.embedding), "layers": copy.deepcopy(self.layers),
                "norm": {"eps": self.norm_eps}, "torch_dtype": self.torch_dtype,
                "initializer_range": self.initializer_range}

    def validate(self) -> None:
        if not isinstance(self.layers, list) or not self.layers:
            raise ValueError("config.json: layers must be a non-empty list")
        gozolix_model_spec(self)            # raises on anything a part or the schedule cannot take


def _pair_embedding(cfg: GozolixConfig) -> Optional[HashedPairSpec]:
    bg = cfg.embedding.get("bigram")
    if bg is None:
        return None
    if not isinstance(bg, dict):
        raise ValueError("config.json: embedding.bigram must be an object")
    return HashedPairSpec(buckets=_int("embedding.bigram", bg, "buckets"),
                          mul_prev=_int("embedding.bigram", bg, "mul_prev", least=0),
                          mul_cur=_int("embedding.bigram", bg, "mul_cur", least=0))


def _attention(cfg: GozolixConfig, m: dict, where: str) -> MixerSpec:
    heads, kv = _int(where, m, "heads"), _int(where, m, "kv_heads")
    if heads % kv:
        raise ValueError(f"config.json: {where}.heads {heads} is not a multiple of kv_heads {kv}")
    extra = [("score_scale", _number(where, m, "scale")), ("distance_bias", SLOPE_SPAN)]
    if m.get("softcap") is not None:
        extra.append(("softcap", _number(where, m, "softcap")))
    qt = m.get("q_temp")
    if qt is not None:
        if not isinstance(qt, dict):
            raise ValueError(f"config.json: {where}.q_temp must be an object")
        extra.append(("q_temp", (_number(where + ".q_temp", qt, "coef", positive=False),
                                 _number(where + ".q_temp", qt, "every"))))
    if m.get("kv_from") is not None:
        extra.append(("shared_kv", True))
    return MixerSpec(kind="attention_mixed", hidden=cfg.width, num_heads=heads, num_kv_heads=kv,
                     head_dim=_int(where, m, "dim"), value_dim=_int(where, m, "vdim"), q_scale=1.0, bias=True,
                     extra=tuple(extra))


def _delta(cfg: GozolixConfig, m: dict, where: str) -> MixerSpec:
    heads, kv = _int(where, m, "heads"), _int(where, m, "kv_heads")
    if heads % kv:
        raise ValueError(f"config.json: {where}.heads {heads} is not a multiple of kv_heads {kv}")
    dim = _int(where, m, "dim")
    return MixerSpec(kind="gated_delta", hidden=cfg.width, num_heads=heads, num_kv_heads=kv, head_dim=dim,
                     value_dim=_int(where, m, "vdim"), q_scale=float(dim) ** -0.5, bias=False,
                     extra=(("conv", _int(where, m, "conv")), ("norm_eps", cfg.norm_eps)))


_MIXERS = {"attention": _attention, "delta": _delta}


def _feed_forward(cfg: GozolixConfig, mlp: Optional[dict], where: str) -> Optional[FeedForwardSpec]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ValueError(f"config.json: {where} must be an object or null")
    kind = mlp.get("kind", "dense")
    if kind == "dense":
        return FeedForwardSpec(kind="dense", hidden=cfg.width, intermediate=_int(where, mlp, "ff"),
                               activation="relu2", bias=False)
    if kind != "moe":
        raise ValueError(f"config.json: {where}.kind must be dense or moe, is {kind!r}")
    r, ex = mlp.get("router"), mlp.get("expert")
    if not isinstance(r, dict) or not isinstance(ex, dict):
        raise ValueError(f"config.json: {where}.router and {where}.expert must be objects")
    experts = _int(where + ".router", r, "experts")
    groups = r.get("groups")
    count = keep = 1
    if groups is not None:
        if not isinstance(groups, dict):
            raise ValueError(f"config.json: {where}.router.groups must be an object")
        count, keep = _int(where + ".router.groups", groups, "count"), _int(where + ".router.groups", groups, "keep")
        if experts % count or keep > count:
            raise ValueError(f"config.json: {where}.router: {experts} experts do not form {count} equal groups "
                             f"of which {keep} stay")
    shared = mlp.get("shared")
    if shared is not None and not isinstance(shared, dict):
        raise ValueError(f"config.json: {where}.shared must be an object or null")
    return FeedForwardSpec(kind="moe", hidden=cfg.width, intermediate=_int(where + ".expert", ex, "ff"),
                           activation="silu", bias=False,
                           extra=(("experts", experts), ("top", _int(where + ".router", r, "top")),
                                  ("groups", count), ("keep", keep),
                                  ("router_scale", _number(where + ".router", r, "scale") if r.get("scale") is not None else 1.0),
                                  ("shared", _int(where + ".shared", shared, "ff") if shared is not None else 0)))


def gozolix_model_spec(cfg: GozolixConfig) -> ModelSpec:
    norm = NormSpec("rmsnorm", cfg.width, cfg.norm_eps, bias=False)
    layers, schedule = [], []
    entry_of = {}                    # layer -> the cache entry its run writes
    for i, L in enumerate(cfg.layers):
        where = f"layers[{i}]"
        if not isinstance(L, dict) or L.get("type") not in _MIXERS:
            raise ValueError(f"config.json: {where}.type must be one of {', '.join(sorted(_MIXERS))}")
        if not isinstance(L.get("mixer"), dict):
            raise ValueError(f"config.json: {where}.mixer must be an object")
        mixer = _MIXERS[L["type"]](cfg, L["mixer"], where + ".mixer")
        layers.append(BlockSpec(arrangement="parallel", norm=norm, mixer=mixer,
                                ffn=_feed_forward(cfg, L.get("mlp"), where + ".mlp")))
        source = L["mixer"].get("kv_from") if L["type"] == "attention" else None
        if source is None:
            entry_of[i] = len(entry_of)
            schedule.append(ScheduleEntry(layer=i, cache=entry_of[i]))
            continue
        if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < i:
            raise ValueError(f"config.json: {where}.mixer.kv_from must name an earlier layer, is {source!r}")
        theirs = cfg.layers[source]
        if theirs.get("type") != "attention" or theirs["mixer"].get("kv_from") is not None:
            raise ValueError(f"config.json: {where}.mixer.kv_from names layer {source}, which has no keys and "
                             f"values of its own")
        if any(theirs["mixer"].get(k) != L["mixer"].get(k) for k in ("kv_heads", "dim", "vdim")):
            raise ValueError(f"config.json: {where}.mixer reads layer {source}'s keys and values but its kv_heads, "
                             f"dim or vdim differ")
        schedule.append(ScheduleEntry(layer=i, cache=entry_of[source], writes=False))
    return ModelSpec(hidden=cfg.width, vocab=cfg.vocab, max_positions=UNBOUNDED_POSITIONS, layers=tuple(layers),
                     schedule=tuple(schedule), final_norm=norm, tie_embeddings=False, head_bias=False,
                     embedding_scale=_number("embedding", cfg.embedding, "scale") if cfg.embedding.get("scale") is not None else 1.0,
                     pair_embedding=_pair_embedding(cfg))


class GozolixTensorNames:
    """Names of the tensors in a Gozolix safetensors file: ``embed``, ``bigram``, ``l<i>.norm1``,
    ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``; a linear layer's weight carries no suffix, its
    bias ``.b``, a convolution's taps ``.conv``."""
    _top = {"embedding": "embed", "pair_embedding": "bigram", "final_norm/weight": "final.norm", "head/weight": "head"}
    _slots = {"norm": "norm1", "mixer": "mix", "ffn": "mlp"}

    def __init__(self, cfg: GozolixConfig):
        self.cfg = cfg

    def top(self, key: str) -> str:
        return self._top[key]

    def layer(self, i: int, slot: str, key: str) -> str:
        """Parts spell a parameter "q.weight", "q.bias", "q.conv", "norm.weight", "e3.gate.weight"; the file
        spells them "q", "q.b", "q.conv", "norm", "e3.gate"."""
        base = f"l{i}.{self._slots[slot]}"
        if slot == "norm":
            return base
        words = key.split(".")
        if words[-1] == "weight":
            words = words[:-1]
        elif words[-1] == "bias":
            words[-1] = "b"
        return ".".join([base] + words)


register_architecture(
    Architecture(name="gozolix", config_class=GozolixConfig, build_spec=gozolix_model_spec,
                 tensor_names=GozolixTensorNames),
)
