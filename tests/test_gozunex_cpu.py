"""Gozunex on the CPU: configuration, model spec, tensor names and properties of the plain mechanisms."""

import copy

import pytest
import torch

import plain_gozunex as plain
from pagedserve_b200.config.gozunex import GozunexConfig, named_config
from pagedserve_b200.config.registry import ConfigError, resolve_architecture
from pagedserve_b200.models.gozunex import build_gozunex_spec
from pagedserve_b200.models.model import Model
from pagedserve_b200.parts.base import PartEnv

L, W, X = plain.latent_layer, plain.wkv_layer, plain.experts_entry
CONFIG = plain.make_config(
    [L(4, 16, 8, 16, 24, window=12, mlp=X(4, 2, 24, shared_ff=16, groups=2, keep=1)), W(2, 16, mlp=X(6, 3, 16)),
     L(2, 8, 16, 24, 16, window=None, rot_dims=8), W(1, 24)],
    width=64, vocab=97, streams=3, loop=(1, 3, 2), scale=2.0)


def test_config_round_trip_and_registry():
    name, config_class, builder = resolve_architecture(CONFIG)
    assert name == "Gozunex" and config_class is GozunexConfig and builder is build_gozunex_spec
    config = GozunexConfig.from_dict(CONFIG)
    assert GozunexConfig.from_dict(config.to_dict()).to_dict() == config.to_dict()
    assert config.layer_runs() == plain.layer_runs(CONFIG) == [0, 1, 2, 1, 2, 3]
    assert config.vocabulary_size == 97


@pytest.mark.parametrize("change", [
    lambda c: c.update(vocab=0), lambda c: c.update(streams=9), lambda c: c["layers"][0].update(type="attention"),
    lambda c: c["layers"][0]["mixer"].pop("kv_rank"), lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10),
    lambda c: c["layers"][0]["mlp"]["router"].update(top=5), lambda c: c["layers"][0]["mlp"].update(kind="dense"),
    lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), lambda c: c["loop"].update(stop=9),
    lambda c: c["loop"].update(times=0), lambda c: c["embedding"]["bigram"].update(buckets=0),
    lambda c: c.pop("norm")])
def test_inconsistent_configurations_are_refused(change):
    values = copy.deepcopy(CONFIG)
    change(values)
    with pytest.raises(ConfigError):
        GozunexConfig.from_dict(values)


def test_spec_schedule_needs_and_tensor_names():
    spec = build_gozunex_spec(GozunexConfig.from_dict(CONFIG))
    assert [(entry.layer, entry.cache_layer) for entry in spec.schedule] == [(0, 0), (1, 1), (2, 2), (1, 3), (2, 4), (3, 5)]
    model = Model(spec, PartEnv(ops=None, dtype=torch.float32, device="cpu"))
    needs = model.kv_needs()
    assert [need is not None for need in needs] == [True, False, True, False, True, False]
    assert (needs[0].n_kv_heads, needs[0].head_dim, needs[0].window, needs[0].planes) == (1, 32, 12, 1)
    assert needs[2] == needs[4] and needs[2].window is None
    states = model.state_needs()
    assert len(states) == 7 and states[-1].dtype == "int32"             # the token before, behind the layers' state
    assert states[1].shape == (2 * 16 * 16 + 64,) and states[5].shape == (24 * 24 + 64,)
    names = {spec.checkpoint_name(param.name) for param in model.param_specs()} - {"lm_head.weight"}
    assert names == set(plain.random_model(CONFIG, 0))
    assert model.graph_safe


def test_a_model_without_streams_pairs_or_loop():
    values = plain.make_config([W(1, 8), L(1, 8, 8, 8, 8, window=4)], width=16, vocab=11, pair=None)
    spec = build_gozunex_spec(GozunexConfig.from_dict(values))
    assert spec.layers[0].block.kind == "pre_norm" and spec.embedding.params["pair"] is None
    model = Model(spec, PartEnv(ops=None, dtype=torch.float32, device="cpu"))
    assert len(model.state_needs()) == 2
    assert {spec.checkpoint_name(p.name) for p in model.param_specs()} - {"lm_head.weight"} == set(plain.random_model(values, 0))


def test_named_sizes_draw_random_models():
    from pagedserve_b200.weights.random_init import random_tensors

    config = named_config("gozunex-tiny")
    tensors = random_tensors(config, seed=1)
    logits = plain.forward(tensors, config.to_dict(), [1, 2, 3, 4, 5, 6, 7])
    assert logits.shape == (7, config.vocab) and torch.isfinite(logits).all()
    mix = tensors["l0.hc1.mix"].float()
    assert (mix - torch.eye(mix.shape[0])).abs().max() < 0.6             # drawn near the identity


# ------------------------------------------------------------------ the plain mechanisms themselves
def test_plain_route_properties():
    g = torch.Generator().manual_seed(0)
    scores = torch.softmax(torch.randn(50, 12, generator=g, dtype=torch.float64), -1)
    chosen, weights = plain.route(scores, 3, 4, 2)
    assert torch.allclose(weights.sum(-1), torch.ones(50, dtype=torch.float64))
    groups = chosen // 3
    assert all(len(set(row.tolist())) <= 2 for row in groups)            # at most two groups supply the experts
    marks = scores.reshape(50, 4, 3).max(-1).values
    best = marks.argmax(-1)
    assert all(int(best[t]) in set(groups[t].tolist()) for t in range(50))
    free, _ = plain.route(scores, 3)
    assert torch.equal(free.sort(-1).values, scores.topk(3).indices.sort(-1).values)


def test_plain_pair_rows_and_loop():
    assert plain.bigram_rows([4, 9, 2], 61, 5, 3) == [61, (4 * 5 + 9 * 3) % 61, (9 * 5 + 2 * 3) % 61]
    assert plain.layer_runs({"layers": [0] * 5, "loop": {"start": 1, "stop": 3, "times": 3}}) == [0, 1, 2, 1, 2, 1, 2, 3, 4]


def test_plain_latent_attention_is_causal_and_windowed():
    tensors = plain.random_model(CONFIG, 3)
    m = CONFIG["layers"][0]["mixer"]
    g = torch.Generator().manual_seed(1)
    h = torch.randn(40, 64, generator=g, dtype=torch.float64)
    out = plain.latent_attention(tensors, "l0.", m, h, torch.arange(40), 1e-5)
    changed = h.clone()
    changed[20] += 1.0
    moved = (plain.latent_attention(tensors, "l0.", m, changed, torch.arange(40), 1e-5) - out).abs().max(-1).values
    assert float(moved[:20].max()) == 0.0 and float(moved[20:32].min()) > 0.0 and float(moved[32:].max()) == 0.0


def test_plain_streams_reduce_to_a_residual_sum():
    """One stream with in = out = mix = 1 is the plain pre-norm layer."""
    values = plain.make_config([W(1, 8, mlp=X(2, 1, 8))], width=16, vocab=11, streams=1, pair=None)
    tensors = plain.random_model(values, 2)
    for name in ("l0.hc1.in", "l0.hc1.out", "l0.hc2.in", "l0.hc2.out"):
        tensors[name] = torch.ones(1)
    tensors["l0.hc1.mix"] = tensors["l0.hc2.mix"] = torch.ones(1, 1)
    with_streams = plain.forward(tensors, values, [3, 1, 4, 1, 5])
    values.pop("streams")
    assert torch.allclose(with_streams, plain.forward(tensors, values, [3, 1, 4, 1, 5]), atol=1e-12)
