"""Tefopel as a ModelSpec.

Token table -> layers in the listed order -> the model's norm -> logits against the token table.  Every layer
is pre-norm (h += mixer(norm(h)); h += feed_forward(norm(h)), the second half only where the layer has a
feed-forward); the norm is the RMS form with a gain stored as its distance from one; the feed-forward is
W_down relu(W_up h)^2 without biases.  ``attention`` layers are :class:`RotaryAttention` (window, cap, sink,
values = unturned keys), ``wkv`` layers :class:`WkvMixer`.  A layer that borrows another's tensors is a second
run of that layer in the schedule, on a cache layer of its own.

Tensor names in a checkpoint: ``embed``, ``final.norm``, and per layer i ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.*``, ``l<i>.mlp.up``, ``l<i>.mlp.down``; matrices are stored ``[out, in]``.
"""

from __future__ import annotations

import re
from typing import Optional

from pagedserve_b200.config.registry import register_architecture
from pagedserve_b200.config.tefopel import TefopelConfig
from pagedserve_b200.models.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# parts shared with other models name their tensors "<name>.weight"; this design stores the bare name
_BARE = re.compile(r"^(embed|final\.norm|l\d+\.(norm1|norm2|mlp\.up|mlp\.down))$")
_SUFFIX = ".weight"


def _normalise_name(name: str) -> Optional[str]:
    return name + _SUFFIX if _BARE.match(name) else name


def _checkpoint_name(name: str) -> str:
    if name.endswith(_SUFFIX) and _BARE.match(name[:-len(_SUFFIX)]):
        return name[:-len(_SUFFIX)]
    return name


def build_tefopel_spec(config: TefopelConfig) -> ModelSpec:
    width = config.width
    norm = dict(width=width, eps=config.norm_eps, has_mean=False, has_bias=False, weight_offset=1.0, init_std=0.1)
    width_std = width ** -0.5
    layers, layer_index = [], {}
    for index, entry in enumerate(config.layers):
        if "weights_of" in entry:
            continue
        prefix = f"l{index}."
        mixer = entry["mixer"]
        if entry["type"] == "attention":
            mixer_spec = PartSpec("rotary_attention", dict(
                hidden_size=width, n_heads=mixer["heads"], n_kv_heads=mixer["kv_heads"], head_dim=mixer["dim"],
                scale=mixer["scale"], window=mixer["mask"]["size"], softcap=mixer["softcap"],
                rotary=dict(dims=mixer["rot"]["dims"], base=mixer["rot"]["base"], interleaved=True),
                q_name="mix.q", k_name="mix.k", v_name=None, out_name="mix.o", sink_name="mix.sink",
                init_std=width_std, out_init_std=(mixer["heads"] * mixer["dim"]) ** -0.5), prefix)
        else:
            mixer_spec = PartSpec("wkv", dict(
                hidden_size=width, n_heads=mixer["heads"], head_dim=mixer["dim"], eps=config.norm_eps,
                decay_rank=None, random_decay_rank=config.random_decay_rank, init_std=width_std,
                out_init_std=(mixer["heads"] * mixer["dim"]) ** -0.5), prefix + "mix.")
        norms = {"pre_mixer": PartSpec("layernorm", dict(norm, name="norm1"), prefix)}
        if entry["mlp"] is not None:
            feed_forward = PartSpec("dense_mlp", dict(
                hidden_size=width, inner_size=entry["mlp"]["ff"], activation="relu_squared", has_bias=False,
                stored_in_out=False, up_name="mlp.up", down_name="mlp.down", init_std=width_std,
                out_init_std=entry["mlp"]["ff"] ** -0.5), prefix)
            norms["pre_feed_forward"] = PartSpec("layernorm", dict(norm, name="norm2"), prefix)
        else:
            feed_forward = PartSpec("none")
        layer_index[index] = len(layers)
        layers.append(LayerSpec(PartSpec("pre_norm"), mixer_spec, feed_forward, norms))
    # run i uses the tensors of its owner and cache layer i
    schedule = [ScheduleEntry(layer_index[config.owner(index)], index) for index in range(len(config.layers))]
    return ModelSpec(
        architecture=config.architecture,
        hidden_size=width,
        vocab_size=config.vocab,
        max_model_len=config.max_model_len,
        embedding=PartSpec("token_embedding", dict(vocab_size=config.vocab, hidden_size=width, name="embed",
                                                   init_std=1.0)),
        positions=PartSpec("none"),
        layers=layers,
        schedule=schedule,
        final_norm=PartSpec("layernorm", dict(norm, name="final.norm")),
        head=PartSpec("lm_head", dict(vocab_size=config.vocab, hidden_size=width, tied=True, tied_to="embed.weight",
                                      name="lm_head", init_std=1.0)),
        normalise_name=_normalise_name,
        checkpoint_name=_checkpoint_name,
    )


register_architecture("Tefopel", TefopelConfig, build_tefopel_spec, replace=True)
