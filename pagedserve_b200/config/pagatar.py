"""Typed Pagatar configuration, read from the design's own config.json keys.

A Pagatar model norms its embedded tokens, runs layers listed one by one in ``layers``, and ends every layer with a
learned average over the embedded rows and the results of all layers so far.  A layer adds the *normed* result of
its mixer, then of its feed-forward, to the residual rows (the sublayers read the rows themselves); every norm is
an RMS norm over ``norm.groups`` equal runs of the row.  Mixers: ``mingru`` (a gated recurrence whose gates read
only the current token), ``latent_attention`` (queries through a normed latent, keys and values of all heads from
one cached latent, a sigmoid gate per head) and ``attention`` (grouped queries with biased projections, a short
causal convolution on q, k and v, head norms, a halves-paired rotation that may be stretched, a chunked causal
mask, values blended with those of the first such layer, a sigmoid gate on the joined heads).  The feed-forward is
a mixture of experts with sigmoid scores, a correction that moves the election only and unnormalised weights, or
absent.  Logits are taken against the token table.  Every size and constant comes from the file.

    {"architecture": "Pagatar", "vocab": V, "width": W, "norm": {"eps": e, "groups": g},
     "layers": [{"type": "mingru", "mixer": {"width"}, "mlp": ...},
                {"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot": {"base", "dims"}},
                 "mlp": ...},
                {"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "conv": taps, "mask": {"size"},
                           "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}},
                           "v_mix": true},
                 "mlp": {"kind": "moe", "router": {"experts", "top"}, "expert": {"ff"}} | null}]}
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import List, Optional

from pagedserve_b200.config.registry import ConfigError, ModelConfig

LAYER_TYPES = ("mingru", "latent_attention", "attention")
# No position table: a request may grow until the cache is full (the engine's own setting bounds it).
UNBOUNDED = 1 << 30


def _positive_int(value, what):
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ConfigError(f"Pagatar: {what} must be a positive integer, got {value!r}")
    return value


def _number(value, what):
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not value > 0:
        raise ConfigError(f"Pagatar: {what} must be a positive number, got {value!r}")
    return float(value)


def _rotation(rot, limit, where, scaling_allowed):
    if not isinstance(rot, dict):
        raise ConfigError(f"Pagatar: {where}: mixer.rot must be an object")
    rot = dict(rot)
    rot["base"] = _number(rot.get("base"), f"{where}: mixer.rot.base")
    dims = rot.get("dims")
    if not isinstance(dims, int) or isinstance(dims, bool) or dims < 0 or dims % 2 or dims > limit:
        raise ConfigError(f"Pagatar: {where}: mixer.rot.dims must be even and at most {limit}")
    scaling = rot.get("scaling")
    if scaling is not None:
        if not scaling_allowed or not isinstance(scaling, dict):
            raise ConfigError(f"Pagatar: {where}: mixer.rot.scaling is an object, and only attention layers have one")
        rot["scaling"] = {key: _number(scaling.get(key), f"{where}: mixer.rot.scaling.{key}")
                          for key in ("factor", "original", "fast", "slow")}
        if rot["base"] == 1.0:
            raise ConfigError(f"Pagatar: {where}: a stretched rotation needs a base other than 1")
    return rot


@dataclass
class PagatarConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    norm_groups: int = 1
    layers: List[dict] = field(default_factory=list)

    def __post_init__(self):
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        self.norm_eps = _number(self.norm_eps, "norm.eps")
        _positive_int(self.norm_groups, "norm.groups")
        if self.width % self.norm_groups or self.norm_groups > 64:
            raise ConfigError("Pagatar: norm.groups must divide the width (at most 64 groups)")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("Pagatar: 'layers' must be a non-empty list")
        self.layers = [self._check_layer(index, layer) for index, layer in enumerate(self.layers)]
        mixing = [layer["mixer"] for layer in self.layers if layer["type"] == "attention" and layer["mixer"]["v_mix"]]
        for mixer in mixing[1:]:
            if mixer["kv_heads"] * mixer["vdim"] != mixing[0]["kv_heads"] * mixing[0]["vdim"]:
                raise ConfigError("Pagatar: layers that mix values must have values of one size")

    @staticmethod
    def _check_layer(index: int, layer) -> dict:
        where = f"layer {index}"
        if not isinstance(layer, dict) or layer.get("type") not in LAYER_TYPES:
            raise ConfigError(f"Pagatar: {where}: 'type' must be one of {LAYER_TYPES}")
        layer = copy.deepcopy(layer)
        mixer = layer.get("mixer")
        if not isinstance(mixer, dict):
            raise ConfigError(f"Pagatar: {where}: no 'mixer'")
        kind = layer["type"]
        if kind == "mingru":
            _positive_int(mixer.get("width"), f"{where}: mixer.width")
        elif kind == "latent_attention":
            for key in ("heads", "dim", "vdim", "kv_rank", "q_rank"):
                _positive_int(mixer.get(key), f"{where}: mixer.{key}")
            rot_dim = mixer.get("rot_dim")
            if not isinstance(rot_dim, int) or isinstance(rot_dim, bool) or rot_dim < 0 or rot_dim % 2:
                raise ConfigError(f"Pagatar: {where}: mixer.rot_dim must be an even integer")
            mixer["scale"] = _number(mixer.get("scale"), f"{where}: mixer.scale")
            mixer["rot"] = _rotation(mixer.get("rot") or {"base": 10000.0, "dims": rot_dim}, rot_dim, where, False)
            if mixer["rot"]["dims"] != rot_dim:
                raise ConfigError(f"Pagatar: {where}: the turning part is turned whole (rot.dims = rot_dim)")
            if mixer["kv_rank"] + rot_dim > 1024:
                raise ConfigError(f"Pagatar: {where}: kv_rank + rot_dim above 1024 is not supported")
        else:
            mixer.setdefault("kv_heads", mixer.get("heads"))          # absent: every query head has its own
            for key in ("heads", "kv_heads", "dim"):
                _positive_int(mixer.get(key), f"{where}: mixer.{key}")
            mixer["vdim"] = _positive_int(mixer.get("vdim", mixer["dim"]), f"{where}: mixer.vdim")
            if mixer["heads"] % mixer["kv_heads"]:
                raise ConfigError(f"Pagatar: {where}: heads must be a multiple of kv_heads")
            if max(mixer["dim"], mixer["vdim"]) > 256:
                raise ConfigError(f"Pagatar: {where}: head sizes above 256 are not supported")
            mixer["scale"] = _number(mixer.get("scale"), f"{where}: mixer.scale")
            # absent: no convolution and no '.conv' tensors (one tap is a convolution: a factor per channel)
            if mixer.get("conv") is not None:
                mixer["conv"] = _positive_int(mixer["conv"], f"{where}: mixer.conv")
                if mixer["conv"] > 16:
                    raise ConfigError(f"Pagatar: {where}: more than 16 taps are not supported")
            else:
                mixer["conv"] = None
            mask = mixer.get("mask")
            if mask is not None:
                if not isinstance(mask, dict):
                    raise ConfigError(f"Pagatar: {where}: mixer.mask must be an object")
                _positive_int(mask.get("size"), f"{where}: mixer.mask.size")
            mixer["mask"] = mask
            rot = mixer.get("rot")
            mixer["rot"] = _rotation(rot, mixer["dim"], where, True) if rot is not None else None
            mixer["v_mix"] = bool(mixer.get("v_mix", False))
        mlp = layer.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                raise ConfigError(f"Pagatar: {where}: mlp.kind must be 'moe' (or mlp null)")
            router, expert = mlp.get("router"), mlp.get("expert")
            if not isinstance(router, dict) or not isinstance(expert, dict):
                raise ConfigError(f"Pagatar: {where}: a mixture of experts needs mlp.router and mlp.expert")
            _positive_int(router.get("experts"), f"{where}: mlp.router.experts")
            _positive_int(router.get("top"), f"{where}: mlp.router.top")
            if router["top"] > router["experts"] or router["experts"] > 256:
                raise ConfigError(f"Pagatar: {where}: top <= experts <= 256")
            _positive_int(expert.get("ff"), f"{where}: mlp.expert.ff")
        layer["mlp"] = mlp
        return layer

    # ---- ModelConfig interface ----------------------------------------
    @property
    def architecture(self) -> str:
        return "Pagatar"

    @property
    def vocabulary_size(self) -> int:
        return self.vocab

    @property
    def max_model_len(self) -> int:
        return UNBOUNDED

    @classmethod
    def from_dict(cls, values: dict) -> "PagatarConfig":
        norm = values.get("norm")
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError("Pagatar: config.json needs norm.eps")
        return cls(vocab=values.get("vocab"), width=values.get("width"), norm_eps=norm["eps"],
                   norm_groups=norm.get("groups", 1), layers=values.get("layers"))

    def to_dict(self) -> dict:
        layers = copy.deepcopy(self.layers)
        for layer in layers:                       # optional keys that are absent stay absent
            if layer["type"] == "attention":
                for key in ("mask", "rot", "conv"):
                    if layer["mixer"].get(key) is None:
                        layer["mixer"].pop(key, None)
                if not layer["mixer"]["v_mix"]:
                    layer["mixer"].pop("v_mix")
        return {"architecture": self.architecture, "layers": layers,
                "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "vocab": self.vocab, "width": self.width}


# ---- layer entries as config.json writes them (for random models: benchmarks, tests, the command line)
def moe_mlp(experts: int, top: int, ff: int) -> dict:
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def mingru_layer(width: int, mlp: Optional[dict]) -> dict:
    return {"type": "mingru", "mixer": {"width": width}, "mlp": copy.deepcopy(mlp)}


def latent_layer(heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, q_rank: int, mlp: Optional[dict],
                 base: float = 10000.0, scale: Optional[float] = None) -> dict:
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
             "scale": (dim + rot_dim) ** -0.5 if scale is None else scale, "rot": {"base": base, "dims": rot_dim}}
    return {"type": "latent_attention", "mixer": mixer, "mlp": copy.deepcopy(mlp)}


def attention_layer(heads: int, kv_heads: int, dim: int, chunk: Optional[int], mlp: Optional[dict],
                    vdim: Optional[int] = None, taps: Optional[int] = 3, rot_dims: Optional[int] = None, base: float = 10000.0,
                    scaling: Optional[dict] = None, v_mix: bool = True, scale: Optional[float] = None) -> dict:
    rot = {"base": base, "dims": dim if rot_dims is None else rot_dims}
    if scaling is not None:
        rot["scaling"] = dict(scaling)
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim if vdim is None else vdim,
             "scale": dim ** -0.5 if scale is None else scale, "rot": rot}
    if taps is not None:
        mixer["conv"] = taps
    if chunk is not None:
        mixer["mask"] = {"size": chunk}
    if v_mix:
        mixer["v_mix"] = True
    return {"type": "attention", "mixer": mixer, "mlp": copy.deepcopy(mlp)}


def repeating_config(width: int, heads: int, head_dim: int, layers: int, chunk: int, vocab: int, experts: int = 8,
                     top: int = 2, expert_ff: Optional[int] = None, kv_heads: Optional[int] = None,
                     kv_rank: Optional[int] = None, q_rank: Optional[int] = None, rot_dim: Optional[int] = None,
                     groups: int = 2, eps: float = 1e-6, pattern=("mingru", "latent_attention", "attention")) -> PagatarConfig:
    """A model for random weights: the layer kinds of ``pattern`` in turn, all with experts."""
    mlp = moe_mlp(experts, top, expert_ff or width)
    rot_dim = rot_dim if rot_dim is not None else max(2, head_dim // 4 * 2)
    stretch = {"factor": 8.0, "original": max(64, 4 * chunk), "fast": 32.0, "slow": 1.0}
    entries = []
    for index in range(layers):
        kind = pattern[index % len(pattern)]
        if kind == "mingru":
            entries.append(mingru_layer(width, mlp))
        elif kind == "latent_attention":
            entries.append(latent_layer(heads, head_dim, rot_dim, head_dim, kv_rank or max(16, width // 4),
                                        q_rank or max(16, width // 2), mlp))
        else:
            entries.append(attention_layer(heads, kv_heads or heads, head_dim, chunk, mlp, scaling=stretch))
    return PagatarConfig(vocab=vocab, width=width, norm_eps=eps, norm_groups=groups, layers=entries)


# sizes that the command line and the benchmark know by name (random weights)
NAMED_CONFIGS = {
    "pagatar-tiny": dict(width=64, heads=4, head_dim=16, layers=3, chunk=24, vocab=512, experts=4, top=2, expert_ff=32,
                         kv_heads=2, kv_rank=32, q_rank=48, rot_dim=8),
    "pagatar-w1024": dict(width=1024, heads=16, head_dim=64, layers=8, chunk=1024, vocab=32000, experts=8, top=2,
                          expert_ff=1024, kv_rank=96, q_rank=512, rot_dim=32,
                          pattern=("latent_attention", "attention", "latent_attention", "mingru")),
    "pagatar-w2048": dict(width=2048, heads=16, head_dim=128, layers=8, chunk=1024, vocab=32000, experts=8, top=2,
                          expert_ff=2048, kv_rank=96, q_rank=1024, rot_dim=32,
                          pattern=("latent_attention", "attention", "latent_attention", "mingru")),
}


def named_config(name: str) -> PagatarConfig:
    if name not in NAMED_CONFIGS:
        raise ConfigError(f"unknown named configuration {name!r}; known: {sorted(NAMED_CONFIGS)}")
    return repeating_config(**NAMED_CONFIGS[name])
