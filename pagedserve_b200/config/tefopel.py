"""Typed Tefopel configuration, read from the design's own config.json keys.

A Tefopel model is a stack of pre-norm layers of two kinds, listed one by one in ``layers``: ``attention``
(windowed, rotary, grouped queries, values that are the unturned keys, a softmax with a learned sink per head
and a cap on the scores) and ``wkv`` (a linear recurrence with a matrix state per head).  A layer may borrow
another layer's tensors (``weights_of``) while keeping a cache or state of its own.  Every size and constant
comes from the file; nothing here depends on the values of a particular model.

    {"architecture": "Tefopel", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap",
                                                "mask": {"size"}, "rot": {"base", "dims"}},
                 "mlp": {"kind": "dense", "ff": F} | null},
                {"type": "wkv", "mixer": {"heads", "dim"}, "mlp": ..., "weights_of": j}]}
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import List, Optional

from pagedserve_b200.config.registry import ConfigError, ModelConfig

LAYER_TYPES = ("attention", "wkv")
# The design has no position table: a request may grow until the cache is full.  The engine needs some bound
# for its block tables; its configuration may set another (EngineConfig.max_model_len).
UNBOUNDED = 1 << 30


def _positive_int(value, what):
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ConfigError(f"Tefopel: {what} must be a positive integer, got {value!r}")
    return value


def _number(value, what, positive=True):
    if isinstance(value, bool) or not isinstance(value, (int, float)) or (positive and not value > 0):
        raise ConfigError(f"Tefopel: {what} must be a{' positive' if positive else ''} number, got {value!r}")
    return float(value)


@dataclass
class TefopelConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-5
    layers: List[dict] = field(default_factory=list)
    # inner size of the decay's pair of matrices when random weights are drawn (a file's own size is read from
    # its tensors; config.json does not carry it)
    random_decay_rank: int = 16

    def __post_init__(self):
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        self.norm_eps = _number(self.norm_eps, "norm.eps")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("Tefopel: 'layers' must be a non-empty list")
        self.layers = [self._check_layer(index, layer) for index, layer in enumerate(self.layers)]
        for index, layer in enumerate(self.layers):
            owner = layer.get("weights_of")
            if owner is None:
                continue
            if not isinstance(owner, int) or isinstance(owner, bool) or not (0 <= owner < len(self.layers)) \
                    or owner == index:
                raise ConfigError(f"Tefopel: layer {index}: weights_of names no other layer")
            other = self.layers[owner]
            if "weights_of" in other:
                raise ConfigError(f"Tefopel: layer {index} borrows from layer {owner}, which has no tensors itself")
            if (other["type"], other["mixer"], other["mlp"]) != (layer["type"], layer["mixer"], layer["mlp"]):
                raise ConfigError(f"Tefopel: layer {index} borrows from layer {owner} but is described differently")

    @staticmethod
    def _check_layer(index: int, layer) -> dict:
        where = f"layer {index}"
        if not isinstance(layer, dict) or layer.get("type") not in LAYER_TYPES:
            raise ConfigError(f"Tefopel: {where}: 'type' must be one of {LAYER_TYPES}")
        layer = copy.deepcopy(layer)
        mixer = layer.get("mixer")
        if not isinstance(mixer, dict):
            raise ConfigError(f"Tefopel: {where}: no 'mixer'")
        _positive_int(mixer.get("heads"), f"{where}: mixer.heads")
        _positive_int(mixer.get("dim"), f"{where}: mixer.dim")
        if layer["type"] == "attention":
            _positive_int(mixer.get("kv_heads"), f"{where}: mixer.kv_heads")
            if mixer["heads"] % mixer["kv_heads"]:
                raise ConfigError(f"Tefopel: {where}: heads must be a multiple of kv_heads")
            if mixer.get("vdim", mixer["dim"]) != mixer["dim"]:
                # the values are the keys as projected: they cannot have another size
                raise ConfigError(f"Tefopel: {where}: vdim must equal dim (the values are the unturned keys)")
            mixer["scale"] = _number(mixer.get("scale"), f"{where}: mixer.scale")
            mixer["softcap"] = _number(mixer.get("softcap"), f"{where}: mixer.softcap")
            mask, rot = mixer.get("mask"), mixer.get("rot")
            if not isinstance(mask, dict) or not isinstance(rot, dict):
                raise ConfigError(f"Tefopel: {where}: mixer.mask and mixer.rot must be objects")
            _positive_int(mask.get("size"), f"{where}: mixer.mask.size")
            rot["base"] = _number(rot.get("base"), f"{where}: mixer.rot.base")
            dims = rot.get("dims")
            if not isinstance(dims, int) or isinstance(dims, bool) or dims < 0 or dims % 2 or dims > mixer["dim"]:
                raise ConfigError(f"Tefopel: {where}: mixer.rot.dims must be even and at most dim")
        mlp = layer.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                raise ConfigError(f"Tefopel: {where}: mlp.kind must be 'dense' (or mlp null)")
            _positive_int(mlp.get("ff"), f"{where}: mlp.ff")
        layer["mlp"] = mlp
        return layer

    # ---- ModelConfig interface ----------------------------------------
    @property
    def architecture(self) -> str:
        return "Tefopel"

    @property
    def vocabulary_size(self) -> int:
        return self.vocab

    @property
    def max_model_len(self) -> int:
        return UNBOUNDED

    def owner(self, index: int) -> int:
        """The layer whose tensors layer ``index`` uses."""
        return self.layers[index].get("weights_of", index)

    @classmethod
    def from_dict(cls, values: dict) -> "TefopelConfig":
        norm = values.get("norm")
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError("Tefopel: config.json needs norm.eps")
        return cls(vocab=values.get("vocab"), width=values.get("width"), norm_eps=norm["eps"],
                   layers=values.get("layers"))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "layers": copy.deepcopy(self.layers),
                "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}


def attention_layer(heads: int, kv_heads: int, dim: int, window: int, ff: Optional[int], rot_dims: Optional[int] = None,
                    base: float = 10000.0, scale: Optional[float] = None, softcap: float = 50.0) -> dict:
    """A layer entry as config.json writes it (for random models: benchmarks, tests, the command line)."""
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
                      "scale": dim ** -0.5 if scale is None else scale, "softcap": softcap, "mask": {"size": window},
                      "rot": {"base": base, "dims": dim if rot_dims is None else rot_dims}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def wkv_layer(heads: int, dim: int, ff: Optional[int] = None, weights_of: Optional[int] = None) -> dict:
    layer = {"type": "wkv", "mixer": {"heads": heads, "dim": dim},
             "mlp": None if ff is None else {"kind": "dense", "ff": ff}}
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


def repeating_config(width: int, heads: int, head_dim: int, ff: int, layers: int, wkv_heads: int, window: int,
                     vocab: int, wkv_dim: int = 64, every: int = 4, eps: float = 1e-5) -> TefopelConfig:
    """A model for random weights: attention layers with every ``every``-th layer a wkv layer, a feed-forward in
    each, rotation on half of every head."""
    entries = []
    for index in range(layers):
        if index % every == every - 1:
            entries.append(wkv_layer(wkv_heads, wkv_dim, ff=ff))
        else:
            entries.append(attention_layer(heads, heads, head_dim, window, ff, rot_dims=(head_dim // 4) * 2))
    return TefopelConfig(vocab=vocab, width=width, norm_eps=eps, layers=entries)


# sizes that the command line and the benchmark know by name (random weights)
NAMED_CONFIGS = {
    "tefopel-tiny": dict(width=64, heads=4, head_dim=16, ff=128, layers=4, wkv_heads=2, window=24, vocab=512, wkv_dim=16),
    "tefopel-w1024": dict(width=1024, heads=16, head_dim=64, ff=4096, layers=8, wkv_heads=16, window=1024, vocab=32000),
    "tefopel-w2048": dict(width=2048, heads=16, head_dim=128, ff=8192, layers=8, wkv_heads=32, window=1024, vocab=32000),
}


def named_config(name: str) -> TefopelConfig:
    if name not in NAMED_CONFIGS:
        raise ConfigError(f"unknown named configuration {name!r}; known: {sorted(NAMED_CONFIGS)}")
    return repeating_config(**NAMED_CONFIGS[name])
