"""Gozunex as a ModelSpec.

Token table (times a constant) plus a hashed table of token pairs -> layers in the listed order, a span of them
possibly several times in a row -> the model's norm -> logits against the token table.  Every layer is pre-norm
with an RMS norm and a plain gain; with ``streams`` the layers run over several residual streams
(:class:`HyperPreNormBlock`), otherwise over one row with plain residual sums.  ``latent_attention`` layers are
:class:`LatentAttention`, ``wkv`` layers :class:`WkvMixer`, the feed-forward :class:`RoutedExperts` or none.
A layer inside the looped span appears once per pass in the schedule, each time with a cache layer of its own.

Tensor names in a checkpoint: ``embed``, ``bigram``, ``final.norm``, and per layer i ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.hc1.*``, ``l<i>.hc2.*``; matrices are stored ``[out, in]``.
"""

from __future__ import annotations

import re
from typing import Optional

from pagedserve_b200.config.gozunex import GozunexConfig
from pagedserve_b200.config.registry import register_architecture
from pagedserve_b200.models.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# parts shared with other models name their tensors "<name>.weight"; this design stores the bare name
_BARE = re.compile(r"^(embed|final\.norm|l\d+\.(norm1|norm2))$")
_SUFFIX = ".weight"


def _normalise_name(name: str) -> Optional[str]:
    return name + _SUFFIX if _BARE.match(name) else name


def _checkpoint_name(name: str) -> str:
    if name.endswith(_SUFFIX) and _BARE.match(name[:-len(_SUFFIX)]):
        return name[:-len(_SUFFIX)]
    return name


def build_gozunex_spec(config: GozunexConfig) -> ModelSpec:
    width = config.width
    norm = dict(width=width, eps=config.norm_eps, has_mean=False, has_bias=False, init_std=0.1)
    width_std = width ** -0.5
    layers = []
    for index, entry in enumerate(config.layers):
        prefix = f"l{index}."
        mixer = entry["mixer"]
        if entry["type"] == "latent_attention":
            inner = mixer["heads"] * mixer["vdim"]
            mixer_spec = PartSpec("latent_attention", dict(
                hidden_size=width, n_heads=mixer["heads"], flat_dim=mixer["dim"], rot_dim=mixer["rot_dim"],
                v_dim=mixer["vdim"], kv_rank=mixer["kv_rank"], scale=mixer["scale"],
                window=mixer["mask"]["size"] if mixer.get("mask") else None, eps=config.norm_eps,
                rotary=dict(dims=mixer["rot"]["dims"], base=mixer["rot"]["base"]),
                init_std=width_std, out_init_std=inner ** -0.5), prefix + "mix.")
        else:
            mixer_spec = PartSpec("wkv", dict(
                hidden_size=width, n_heads=mixer["heads"], head_dim=mixer["dim"], eps=config.norm_eps,
                decay_rank=None, random_decay_rank=config.random_decay_rank, init_std=width_std,
                out_init_std=(mixer["heads"] * mixer["dim"]) ** -0.5), prefix + "mix.")
        norms = {"pre_mixer": PartSpec("layernorm", dict(norm, name="norm1"), prefix)}
        mlp = entry["mlp"]
        if mlp is not None:
            router = mlp["router"]
            groups = router.get("groups") or {}
            shared = mlp.get("shared") or {}
            feed_forward = PartSpec("routed_experts", dict(
                hidden_size=width, n_experts=router["experts"], expert_ff=mlp["expert"]["ff"], top=router["top"],
                groups=groups.get("count"), group_keep=groups.get("keep"), shared_ff=shared.get("ff"),
                init_std=width_std, out_init_std=mlp["expert"]["ff"] ** -0.5), prefix + "mlp.")
            norms["pre_feed_forward"] = PartSpec("layernorm", dict(norm, name="norm2"), prefix)
        else:
            feed_forward = PartSpec("none")
        if config.streams is not None:
            block = PartSpec("hyper_pre_norm", dict(streams=config.streams,
                                                    names={"mixer": "hc1", "feed_forward": "hc2"}), prefix)
        else:
            block = PartSpec("pre_norm")
        layers.append(LayerSpec(block, mixer_spec, feed_forward, norms))
    # run n of the schedule uses cache layer n: every pass of the looped span has its own pages and state
    schedule = [ScheduleEntry(layer, run) for run, layer in enumerate(config.layer_runs())]
    pair = config.embedding.get("bigram")
    return ModelSpec(
        architecture=config.architecture,
        hidden_size=width,
        vocab_size=config.vocab,
        max_model_len=config.max_model_len,
        embedding=PartSpec("token_pair_embedding", dict(
            vocab_size=config.vocab, hidden_size=width, name="embed", init_std=1.0,
            scale=config.embedding.get("scale", 1.0),
            pair=None if pair is None else dict(name="bigram", buckets=pair["buckets"], mul_prev=pair["mul_prev"],
                                                mul_cur=pair["mul_cur"], init_std=0.5))),
        positions=PartSpec("none"),
        layers=layers,
        schedule=schedule,
        final_norm=PartSpec("layernorm", dict(norm, name="final.norm")),
        head=PartSpec("lm_head", dict(vocab_size=config.vocab, hidden_size=width, tied=True, tied_to="embed.weight",
                                      name="lm_head", init_std=1.0)),
        normalise_name=_normalise_name,
        checkpoint_name=_checkpoint_name,
    )


register_architecture("Gozunex", GozunexConfig, build_gozunex_spec, replace=True)
