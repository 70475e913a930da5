"""Typed Gozunex configuration, read from the design's own config.json keys.

A Gozunex model embeds a token as its table row times a constant plus a row of a second table chosen by a hash
of the token and its predecessor; runs pre-norm layers listed one by one (``latent_attention``: windowed
attention over a cached latent with a sigmoid output gate, or ``wkv``: a linear recurrence with a matrix state
per head), each with a feed-forward of routed experts or none; may run a span of its layers several times in a
row with the same tensors (``loop``), each pass on a cache or state of its own; and may carry several residual
streams through the layers (``streams``).  Every size and constant comes from the file.

    {"architecture": "Gozunex", "vocab": V, "width": W, "norm": {"eps": e}, "streams": S,
     "embedding": {"scale": a, "bigram": {"buckets": B, "mul_prev": m, "mul_cur": n}},
     "loop": {"start": i, "stop": j, "times": n},
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "mask": {"size"},
                           "rot": {"base", "dims"}},
                 "mlp": {"kind": "moe", "expert": {"ff"}, "shared": {"ff"},
                         "router": {"experts", "top", "groups": {"count", "keep"}}} | null},
                {"type": "wkv", "mixer": {"heads", "dim"}, "mlp": ...}]}
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import List, Optional

from pagedserve_b200.config.registry import ConfigError, ModelConfig

LAYER_TYPES = ("latent_attention", "wkv")
# No position table: a request may grow until the cache is full (the engine's own setting bounds it).
UNBOUNDED = 1 << 30


def _positive_int(value, what):
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ConfigError(f"Gozunex: {what} must be a positive integer, got {value!r}")
    return value


def _number(value, what, positive=True):
    if isinstance(value, bool) or not isinstance(value, (int, float)) or (positive and not value > 0):
        raise ConfigError(f"Gozunex: {what} must be a{' positive' if positive else ''} number, got {value!r}")
    return float(value)


@dataclass
class GozunexConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-5
    layers: List[dict] = field(default_factory=list)
    streams: Optional[int] = None               # None: one residual row and plain residual sums
    embedding: dict = field(default_factory=dict)
    loop: Optional[dict] = None
    # inner size of the wkv decay's pair of matrices when random weights are drawn (a file's own size is read
    # from its tensors; config.json does not carry it)
    random_decay_rank: int = 16

    def __post_init__(self):
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        self.norm_eps = _number(self.norm_eps, "norm.eps")
        if self.streams is not None:
            _positive_int(self.streams, "streams")
            if self.streams > 8:
                raise ConfigError("Gozunex: at most 8 streams are supported")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("Gozunex: 'layers' must be a non-empty list")
        self.layers = [self._check_layer(index, layer) for index, layer in enumerate(self.layers)]
        self.embedding = self._check_embedding(self.embedding)
        if self.loop is not None:
            loop = self.loop
            if not isinstance(loop, dict):
                raise ConfigError("Gozunex: 'loop' must be an object")
            for key in ("start", "stop", "times"):
                if not isinstance(loop.get(key), int) or isinstance(loop.get(key), bool):
                    raise ConfigError(f"Gozunex: loop.{key} must be an integer")
            if not (0 <= loop["start"] <= loop["stop"] <= len(self.layers)) or loop["times"] < 1:
                raise ConfigError("Gozunex: loop must name a span of the layers and a count of at least 1")
            self.loop = {key: loop[key] for key in ("start", "stop", "times")}

    @staticmethod
    def _check_embedding(embedding) -> dict:
        if embedding is None:
            embedding = {}
        if not isinstance(embedding, dict):
            raise ConfigError("Gozunex: 'embedding' must be an object")
        out = {"scale": _number(embedding.get("scale", 1.0), "embedding.scale", positive=False)}
        pair = embedding.get("bigram")
        if pair is not None:
            if not isinstance(pair, dict):
                raise ConfigError("Gozunex: embedding.bigram must be an object")
            _positive_int(pair.get("buckets"), "embedding.bigram.buckets")
            for key in ("mul_prev", "mul_cur"):
                if not isinstance(pair.get(key), int) or isinstance(pair.get(key), bool):
                    raise ConfigError(f"Gozunex: embedding.bigram.{key} must be an integer")
            out["bigram"] = {key: pair[key] for key in ("buckets", "mul_cur", "mul_prev")}
        return out

    @staticmethod
    def _check_layer(index: int, layer) -> dict:
        where = f"layer {index}"
        if not isinstance(layer, dict) or layer.get("type") not in LAYER_TYPES:
            raise ConfigError(f"Gozunex: {where}: 'type' must be one of {LAYER_TYPES}")
        layer = copy.deepcopy(layer)
        mixer = layer.get("mixer")
        if not isinstance(mixer, dict):
            raise ConfigError(f"Gozunex: {where}: no 'mixer'")
        _positive_int(mixer.get("heads"), f"{where}: mixer.heads")
        _positive_int(mixer.get("dim"), f"{where}: mixer.dim")
        if layer["type"] == "latent_attention":
            for key in ("rot_dim", "vdim", "kv_rank"):
                _positive_int(mixer.get(key), f"{where}: mixer.{key}")
            mixer["scale"] = _number(mixer.get("scale"), f"{where}: mixer.scale")
            mask, rot = mixer.get("mask"), mixer.get("rot")
            if mask is not None:
                if not isinstance(mask, dict):
                    raise ConfigError(f"Gozunex: {where}: mixer.mask must be an object")
                _positive_int(mask.get("size"), f"{where}: mixer.mask.size")
            if not isinstance(rot, dict):
                raise ConfigError(f"Gozunex: {where}: mixer.rot must be an object")
            rot["base"] = _number(rot.get("base"), f"{where}: mixer.rot.base")
            dims = rot.get("dims")
            if not isinstance(dims, int) or isinstance(dims, bool) or dims < 0 or dims % 2 or dims > mixer["rot_dim"]:
                raise ConfigError(f"Gozunex: {where}: mixer.rot.dims must be even and at most rot_dim")
        mlp = layer.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                raise ConfigError(f"Gozunex: {where}: mlp.kind must be 'moe' (or mlp null)")
            router, expert = mlp.get("router"), mlp.get("expert")
            if not isinstance(router, dict) or not isinstance(expert, dict):
                raise ConfigError(f"Gozunex: {where}: mlp.router and mlp.expert must be objects")
            _positive_int(expert.get("ff"), f"{where}: mlp.expert.ff")
            _positive_int(router.get("experts"), f"{where}: mlp.router.experts")
            _positive_int(router.get("top"), f"{where}: mlp.router.top")
            if router["top"] > router["experts"]:
                raise ConfigError(f"Gozunex: {where}: mlp.router.top exceeds the number of experts")
            groups = router.get("groups")
            if groups is not None:
                if not isinstance(groups, dict):
                    raise ConfigError(f"Gozunex: {where}: mlp.router.groups must be an object")
                _positive_int(groups.get("count"), f"{where}: mlp.router.groups.count")
                _positive_int(groups.get("keep"), f"{where}: mlp.router.groups.keep")
                if router["experts"] % groups["count"] or groups["keep"] > groups["count"]:
                    raise ConfigError(f"Gozunex: {where}: groups must divide the experts and keep at most all")
                if groups["keep"] * (router["experts"] // groups["count"]) < router["top"]:
                    raise ConfigError(f"Gozunex: {where}: the kept groups hold fewer experts than are chosen")
            shared = mlp.get("shared")
            if shared is not None:
                if not isinstance(shared, dict):
                    raise ConfigError(f"Gozunex: {where}: mlp.shared must be an object")
                _positive_int(shared.get("ff"), f"{where}: mlp.shared.ff")
        layer["mlp"] = mlp
        return layer

    # ---- ModelConfig interface ----------------------------------------
    @property
    def architecture(self) -> str:
        return "Gozunex"

    @property
    def vocabulary_size(self) -> int:
        return self.vocab

    @property
    def max_model_len(self) -> int:
        return UNBOUNDED

    def layer_runs(self) -> List[int]:
        """The layers in the order they run: the looped span ``times`` times in a row."""
        count = len(self.layers)
        if not self.loop:
            return list(range(count))
        start, stop, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, count))

    @classmethod
    def from_dict(cls, values: dict) -> "GozunexConfig":
        norm = values.get("norm")
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError("Gozunex: config.json needs norm.eps")
        return cls(vocab=values.get("vocab"), width=values.get("width"), norm_eps=norm["eps"],
                   layers=values.get("layers"), streams=values.get("streams"),
                   embedding=values.get("embedding") or {}, loop=values.get("loop"))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "embedding": copy.deepcopy(self.embedding),
               "layers": copy.deepcopy(self.layers), "norm": {"eps": self.norm_eps}, "vocab": self.vocab,
               "width": self.width}
        if self.streams is not None:
            out["streams"] = self.streams
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        return out


def moe_entry(experts: int, top: int, ff: int, shared_ff: Optional[int] = None, groups: Optional[int] = None,
              keep: Optional[int] = None) -> dict:
    """A feed-forward entry as config.json writes it."""
    router = {"experts": experts, "top": top}
    if groups:
        router["groups"] = {"count": groups, "keep": keep}
    entry = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared_ff:
        entry["shared"] = {"ff": shared_ff}
    return entry


def latent_layer(heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, window: Optional[int],
                 mlp: Optional[dict], base: float = 10000.0, scale: Optional[float] = None,
                 rot_dims: Optional[int] = None) -> dict:
    """A layer entry as config.json writes it (for random models: benchmarks, tests, the command line)."""
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
             "scale": (dim + rot_dim) ** -0.5 if scale is None else scale,
             "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if window is not None:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def wkv_layer(heads: int, dim: int, mlp: Optional[dict] = None) -> dict:
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}, "mlp": mlp}


def repeating_config(width: int, heads: int, dim: int, rot_dim: int, kv_rank: int, experts: int, top: int, ff: int,
                     layers: int, wkv_heads: int, window: int, vocab: int, wkv_dim: int = 64, every: int = 4,
                     streams: Optional[int] = 2, groups: Optional[int] = None, keep: Optional[int] = None,
                     shared_ff: Optional[int] = None, buckets: int = 4093, eps: float = 1e-5) -> GozunexConfig:
    """A model for random weights: latent-attention layers with every ``every``-th layer a wkv layer, routed
    experts in each."""
    entries = []
    for index in range(layers):
        mlp = moe_entry(experts, top, ff, shared_ff=shared_ff, groups=groups, keep=keep)
        if index % every == every - 1:
            entries.append(wkv_layer(wkv_heads, wkv_dim, mlp))
        else:
            entries.append(latent_layer(heads, dim, rot_dim, dim, kv_rank, window, mlp))
    return GozunexConfig(vocab=vocab, width=width, norm_eps=eps, layers=entries, streams=streams,
                         embedding={"scale": 1.0, "bigram": {"buckets": buckets, "mul_prev": 31, "mul_cur": 17}})


# sizes that the command line and the benchmark know by name (random weights)
NAMED_CONFIGS = {
    "gozunex-tiny": dict(width=64, heads=4, dim=16, rot_dim=16, kv_rank=32, experts=4, top=2, ff=32, layers=4,
                         wkv_heads=2, window=24, vocab=512, wkv_dim=16, shared_ff=32, buckets=251),
    "gozunex-w1024": dict(width=1024, heads=16, dim=64, rot_dim=32, kv_rank=96, experts=8, top=2, ff=1024, layers=8,
                          wkv_heads=16, window=1024, vocab=32000, shared_ff=2048, groups=4, keep=2),
    "gozunex-w2048": dict(width=2048, heads=16, dim=128, rot_dim=32, kv_rank=96, experts=8, top=2, ff=2048, layers=8,
                          wkv_heads=32, window=1024, vocab=32000, shared_ff=4096, groups=4, keep=2),
}


def named_config(name: str) -> GozunexConfig:
    if name not in NAMED_CONFIGS:
        raise ConfigError(f"unknown named configuration {name!r}; known: {sorted(NAMED_CONFIGS)}")
    return repeating_config(**NAMED_CONFIGS[name])
