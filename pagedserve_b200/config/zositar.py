"""Typed Zositar configuration, read from the design's own config.json keys.

A Zositar model is a stack of pre-norm attention layers, listed one by one in ``layers``.  Attention has grouped
queries with biased projections, a norm of every query and key head, rotary positions on the first dimensions of
a head (halves paired), a chunked causal mask, and values of a size of their own; a layer may read the keys and
values that an earlier layer cached (``kv_from``) instead of making its own.  The feed-forward is a gated dense
one, a mixture of experts with a sigmoid router and a shared expert, or absent.  Every size and constant comes
from the file; nothing here depends on the values of a particular model.

    {"architecture": "Zositar", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}, "rot": {"base", "dims"},
                           "kv_from": j (optional)},
                 "mlp": {"kind": "dense", "ff": F}
                      | {"kind": "moe", "router": {"experts", "top"}, "expert": {"ff", "limit"},
                         "shared": {"ff", "limit"} (optional)}
                      | null}]}
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import List, Optional

from pagedserve_b200.config.registry import ConfigError, ModelConfig

# The design has no position table: a request may grow until the cache is full.  The engine needs some bound
# for its block tables; its configuration may set another (EngineConfig.max_model_len).
UNBOUNDED = 1 << 30
# the slope of the sigmoid in an expert's activation: fixed by the design
EXPERT_SIGMOID_SLOPE = 1.702


def _positive_int(value, what):
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ConfigError(f"Zositar: {what} must be a positive integer, got {value!r}")
    return value


def _number(value, what):
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not value > 0:
        raise ConfigError(f"Zositar: {what} must be a positive number, got {value!r}")
    return float(value)


@dataclass
class ZositarConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    layers: List[dict] = field(default_factory=list)

    def __post_init__(self):
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        self.norm_eps = _number(self.norm_eps, "norm.eps")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("Zositar: 'layers' must be a non-empty list")
        self.layers = [self._check_layer(index, layer) for index, layer in enumerate(self.layers)]
        for index, layer in enumerate(self.layers):
            lender = layer["mixer"].get("kv_from")
            if lender is None:
                continue
            if not isinstance(lender, int) or isinstance(lender, bool) or not (0 <= lender < index):
                raise ConfigError(f"Zositar: layer {index}: kv_from must name an earlier layer")
            other = self.layers[lender]["mixer"]
            if other.get("kv_from") is not None:
                raise ConfigError(f"Zositar: layer {index} reads the cache of layer {lender}, which has none itself")
            mine = layer["mixer"]
            for key in ("kv_heads", "dim", "vdim", "rot"):
                if mine[key] != other[key]:
                    raise ConfigError(f"Zositar: layer {index} reads the cache of layer {lender} but differs in {key}")

    @staticmethod
    def _check_layer(index: int, layer) -> dict:
        where = f"layer {index}"
        if not isinstance(layer, dict) or layer.get("type") != "attention":
            raise ConfigError(f"Zositar: {where}: 'type' must be 'attention'")
        layer = copy.deepcopy(layer)
        mixer = layer.get("mixer")
        if not isinstance(mixer, dict):
            raise ConfigError(f"Zositar: {where}: no 'mixer'")
        for key in ("heads", "kv_heads", "dim"):
            _positive_int(mixer.get(key), f"{where}: mixer.{key}")
        mixer["vdim"] = _positive_int(mixer.get("vdim", mixer["dim"]), f"{where}: mixer.vdim")
        if mixer["heads"] % mixer["kv_heads"]:
            raise ConfigError(f"Zositar: {where}: heads must be a multiple of kv_heads")
        if max(mixer["dim"], mixer["vdim"]) > 256:
            raise ConfigError(f"Zositar: {where}: head sizes above 256 are not supported")
        mixer["scale"] = _number(mixer.get("scale"), f"{where}: mixer.scale")
        mask = mixer.get("mask")
        if mask is not None:
            if not isinstance(mask, dict):
                raise ConfigError(f"Zositar: {where}: mixer.mask must be an object")
            _positive_int(mask.get("size"), f"{where}: mixer.mask.size")
        mixer["mask"] = mask
        rot = mixer.get("rot")
        if rot is not None:
            if not isinstance(rot, dict):
                raise ConfigError(f"Zositar: {where}: mixer.rot must be an object")
            rot["base"] = _number(rot.get("base"), f"{where}: mixer.rot.base")
            dims = rot.get("dims")
            if not isinstance(dims, int) or isinstance(dims, bool) or dims < 0 or dims % 2 or dims > mixer["dim"]:
                raise ConfigError(f"Zositar: {where}: mixer.rot.dims must be even and at most dim")
        mixer["rot"] = rot
        mlp = layer.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                raise ConfigError(f"Zositar: {where}: mlp.kind must be 'dense' or 'moe' (or mlp null)")
            if mlp["kind"] == "dense":
                _positive_int(mlp.get("ff"), f"{where}: mlp.ff")
            else:
                router, expert, shared = mlp.get("router"), mlp.get("expert"), mlp.get("shared")
                if not isinstance(router, dict) or not isinstance(expert, dict):
                    raise ConfigError(f"Zositar: {where}: a mixture of experts needs mlp.router and mlp.expert")
                _positive_int(router.get("experts"), f"{where}: mlp.router.experts")
                _positive_int(router.get("top"), f"{where}: mlp.router.top")
                if router["top"] > router["experts"] or router["experts"] > 256:
                    raise ConfigError(f"Zositar: {where}: top <= experts <= 256")
                _positive_int(expert.get("ff"), f"{where}: mlp.expert.ff")
                expert["limit"] = _number(expert.get("limit"), f"{where}: mlp.expert.limit")
                if shared is not None:
                    if not isinstance(shared, dict):
                        raise ConfigError(f"Zositar: {where}: mlp.shared must be an object")
                    _positive_int(shared.get("ff"), f"{where}: mlp.shared.ff")
                    shared["limit"] = _number(shared.get("limit"), f"{where}: mlp.shared.limit")
                mlp["shared"] = shared
        layer["mlp"] = mlp
        return layer

    # ---- ModelConfig interface ----------------------------------------
    @property
    def architecture(self) -> str:
        return "Zositar"

    @property
    def vocabulary_size(self) -> int:
        return self.vocab

    @property
    def max_model_len(self) -> int:
        return UNBOUNDED

    @classmethod
    def from_dict(cls, values: dict) -> "ZositarConfig":
        norm = values.get("norm")
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError("Zositar: config.json needs norm.eps")
        return cls(vocab=values.get("vocab"), width=values.get("width"), norm_eps=norm["eps"],
                   layers=values.get("layers"))

    def to_dict(self) -> dict:
        layers = copy.deepcopy(self.layers)
        for layer in layers:                       # optional keys that are absent stay absent
            for key in ("mask", "rot"):
                if layer["mixer"].get(key) is None:
                    layer["mixer"].pop(key, None)
            if layer["mlp"] is not None and layer["mlp"].get("kind") == "moe" and layer["mlp"].get("shared") is None:
                layer["mlp"].pop("shared", None)
        return {"architecture": self.architecture, "layers": layers, "norm": {"eps": self.norm_eps},
                "vocab": self.vocab, "width": self.width}


def attention_layer(heads: int, kv_heads: int, dim: int, chunk: Optional[int], mlp: Optional[dict],
                    vdim: Optional[int] = None, rot_dims: Optional[int] = None, base: float = 10000.0,
                    scale: Optional[float] = None, kv_from: Optional[int] = None) -> dict:
    """A layer entry as config.json writes it (for random models: benchmarks, tests, the command line)."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim if vdim is None else vdim,
             "scale": dim ** -0.5 if scale is None else scale,
             "rot": {"base": base, "dims": (dim // 4) * 2 if rot_dims is None else rot_dims}}
    if chunk is not None:
        mixer["mask"] = {"size": chunk}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": copy.deepcopy(mlp)}


def dense_mlp(ff: int) -> dict:
    return {"kind": "dense", "ff": ff}


def moe_mlp(experts: int, top: int, ff: int, limit: float = 7.0, shared_ff: Optional[int] = None,
            shared_limit: float = 7.0) -> dict:
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared_ff:
        mlp["shared"] = {"ff": shared_ff, "limit": shared_limit}
    return mlp


def repeating_config(width: int, heads: int, kv_heads: int, head_dim: int, ff: int, layers: int, chunk: int, vocab: int,
                     experts: int = 8, top: int = 2, expert_ff: Optional[int] = None, shared_ff: Optional[int] = None,
                     every: int = 4, eps: float = 1e-6) -> ZositarConfig:
    """A model for random weights: spans of ``every`` layers in which the first has a dense feed-forward and keys
    and values of its own, the second experts and its own keys and values, and the others experts and the second
    layer's keys and values."""
    entries = []
    for index in range(layers):
        place = index % every
        mlp = dense_mlp(ff) if place == 0 else moe_mlp(experts, top, expert_ff or ff // 4, shared_ff=shared_ff or ff // 2)
        kv_from = index - place + 1 if place >= 2 else None
        entries.append(attention_layer(heads, kv_heads, head_dim, chunk, mlp, kv_from=kv_from))
    return ZositarConfig(vocab=vocab, width=width, norm_eps=eps, layers=entries)


# sizes that the command line and the benchmark know by name (random weights)
NAMED_CONFIGS = {
    "zositar-tiny": dict(width=64, heads=4, kv_heads=2, head_dim=16, ff=128, layers=4, chunk=24, vocab=512, experts=4,
                         top=2, expert_ff=32, shared_ff=48),
    "zositar-w1024": dict(width=1024, heads=16, kv_heads=16, head_dim=64, ff=4096, layers=8, chunk=1024, vocab=32000,
                          experts=8, top=2, expert_ff=1024, shared_ff=2048),
    "zositar-w2048": dict(width=2048, heads=16, kv_heads=16, head_dim=128, ff=8192, layers=8, chunk=1024, vocab=32000,
                          experts=8, top=2, expert_ff=2048, shared_ff=4096),
}


def named_config(name: str) -> ZositarConfig:
    if name not in NAMED_CONFIGS:
        raise ConfigError(f"unknown named configuration {name!r}; known: {sorted(NAMED_CONFIGS)}")
    return repeating_config(**NAMED_CONFIGS[name])
