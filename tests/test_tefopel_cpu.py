"""Tefopel without a GPU: its configuration, the model spec built from it, tensor names and shapes, and the plain
implementation's own mechanisms (tests/plain_tefopel.py) against properties that follow from the equations."""

import copy
import json

import pytest
import torch

import plain_tefopel as plain
from pagedserve_b200.config import ConfigError, load_model_config, resolve_architecture
from pagedserve_b200.config.tefopel import TefopelConfig, attention_layer, wkv_layer

A, W = plain.attention_layer, plain.wkv_layer
CONFIG = plain.make_config([W(2, 16), A(4, 2, 16, window=12, rot_dims=8, ff=48), W(3, 8, ff=40),
                            W(2, 16, weights_of=0), A(4, 2, 16, window=12, rot_dims=8, ff=48) | {"weights_of": 1},
                            A(1, 1, 32, window=5, rot_dims=32, ff=None)], width=64, vocab=97, eps=3e-6)


# ------------------------------------------------------------------ configuration
def test_config_is_read_from_its_own_keys(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(CONFIG))
    config = load_model_config(str(tmp_path))
    assert isinstance(config, TefopelConfig)
    assert (config.vocab, config.width, config.norm_eps, len(config.layers)) == (97, 64, 3e-6, 6)
    assert [config.owner(i) for i in range(6)] == [0, 1, 2, 0, 1, 5]
    assert config.to_dict() == CONFIG
    name, cls, _ = resolve_architecture({"architecture": "Tefopel"})
    assert name == "Tefopel" and cls is TefopelConfig


def test_layer_helpers_write_what_the_reader_reads():
    layers = [attention_layer(6, 3, 32, window=100, ff=256, rot_dims=16, base=5000.0, scale=0.2, softcap=12.0),
              wkv_layer(4, 32), wkv_layer(4, 32, weights_of=1), attention_layer(2, 2, 64, window=9, ff=None)]
    config = TefopelConfig(vocab=300, width=128, norm_eps=1e-5, layers=layers)
    assert config.layers[0]["mixer"]["rot"] == {"base": 5000.0, "dims": 16}
    assert config.layers[3]["mixer"]["rot"]["dims"] == 64 and config.layers[3]["mlp"] is None
    assert TefopelConfig.from_dict(config.to_dict()).to_dict() == config.to_dict()


def test_named_sizes_are_valid_configurations():
    from pagedserve_b200.config import tefopel

    for name in tefopel.NAMED_CONFIGS:
        config = tefopel.named_config(name)
        assert [layer["type"] for layer in config.layers[:4]] == ["attention"] * 3 + ["wkv"]
        assert TefopelConfig.from_dict(config.to_dict()).to_dict() == config.to_dict()
    with pytest.raises(ConfigError):
        tefopel.named_config("tefopel-huge")


def broken(change):
    values = copy.deepcopy(CONFIG)
    change(values)
    return values


@pytest.mark.parametrize("change", [
    lambda c: c["layers"][1]["mixer"].update(kv_heads=3),                   # 4 heads over 3 key heads
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7),                # odd
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18),               # more than the head has
    lambda c: c["layers"][1]["mixer"].update(vdim=8),                       # values are keys: same size
    lambda c: c["layers"][1]["mixer"]["mask"].update(size=0),
    lambda c: c["layers"][1]["mixer"].update(softcap=-1.0),
    lambda c: c["layers"][2].update(type="conv"),
    lambda c: c["layers"][2]["mlp"].update(kind="experts"),
    lambda c: c["layers"][3].update(weights_of=3),                          # itself
    lambda c: c["layers"][3].update(weights_of=4),                          # a layer without tensors of its own
    lambda c: c["layers"][3].update(weights_of=2),                          # described differently
    lambda c: c["layers"][3].update(weights_of=9),
    lambda c: c.update(layers=[]),
    lambda c: c.update(width=0),
    lambda c: c.pop("norm"),
])
def test_config_errors_are_reported(change):
    with pytest.raises(ConfigError):
        TefopelConfig.from_dict(broken(change))


# ------------------------------------------------------------------ spec, tensors, needs
def cpu_model(config_dict):
    from pagedserve_b200.models.model import Model
    from pagedserve_b200.parts.base import PartEnv

    _, cls, builder = resolve_architecture(config_dict)
    spec = builder(cls.from_dict(config_dict))
    return spec, Model(spec, PartEnv(ops=None, dtype=torch.float32, device="cpu"))


def test_spec_runs_borrowed_layers_on_caches_of_their_own():
    spec, model = cpu_model(CONFIG)
    assert len(spec.layers) == 4                                            # layers with tensors
    assert [(e.layer, e.cache_layer) for e in spec.schedule] == [(0, 0), (1, 1), (2, 2), (0, 3), (1, 4), (3, 5)]
    kv, state = model.kv_needs(), model.state_needs()
    assert [need is not None for need in kv] == [False, True, False, False, True, True]
    assert [need is not None for need in state] == [True, False, True, True, False, False]
    assert (kv[1].n_kv_heads, kv[1].head_dim, kv[1].window) == (2, 16, 12) and kv[1] == kv[4]
    assert (kv[5].n_kv_heads, kv[5].head_dim, kv[5].window) == (1, 32, 5)
    assert state[0].shape == (2 * 16 * 16 + 64,) and state[2].shape == (3 * 8 * 8 + 64,)
    assert spec.layers[3].feed_forward.kind == "none" and "pre_feed_forward" not in spec.layers[3].norms


@pytest.mark.parametrize("rank", [16, 5])
def test_tensor_names_and_a_decay_rank_that_only_the_file_gives(rank):
    from pagedserve_b200.weights.loader import WeightError, place_tensors
    from pagedserve_b200.weights.random_init import random_tensors

    spec, model = cpu_model(CONFIG)
    drawn = random_tensors(TefopelConfig.from_dict(CONFIG), seed=3)
    assert {n: tuple(t.shape) for n, t in drawn.items()} == plain.tensor_shapes(CONFIG, rank=16)
    stored = plain.random_model(CONFIG, seed=1, rank=rank)
    placed = place_tensors(model.param_specs(), stored, torch.float32, "cpu", spec.normalise_name)
    model.bind(placed)
    assert model.blocks[0].mixer.w1.shape == (rank, 64) and model.blocks[0].mixer.w2.shape == (32, rank)
    assert model.blocks[1].mixer.w_in.shape == (4 * 16 + 2 * 16, 64)        # queries and keys, no values
    stored["l3.norm1"] = stored["l0.norm1"]                                 # a borrowing layer stores nothing
    with pytest.raises(WeightError):
        place_tensors(model.param_specs(), stored, torch.float32, "cpu", spec.normalise_name)


# ------------------------------------------------------------------ the plain mechanisms themselves
def test_plain_rotation_is_relative_and_leaves_the_rest():
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, 12, generator=g, dtype=torch.float64), torch.randn(1, 1, 12, generator=g, dtype=torch.float64)
    def dot(pq, pk):
        a = plain.rotate_interleaved(q, torch.tensor([pq]), 8, 100.0)
        b = plain.rotate_interleaved(k, torch.tensor([pk]), 8, 100.0)
        return float((a * b).sum())
    assert abs(dot(40, 33) - dot(7, 0)) < 1e-12 and abs(dot(40, 33) - dot(40, 30)) > 1e-3
    turned = plain.rotate_interleaved(q, torch.tensor([9]), 8, 100.0)
    assert torch.equal(turned[..., 8:], q[..., 8:]) and not torch.equal(turned[..., :8], q[..., :8])
    # the first pair turns by the position itself (its frequency is one)
    want0 = q[0, 0, 0] * torch.cos(torch.tensor(9.0, dtype=torch.float64)) - q[0, 0, 1] * torch.sin(torch.tensor(9.0, dtype=torch.float64))
    assert abs(float(turned[0, 0, 0] - want0)) < 1e-12
    assert torch.equal(plain.rotate_interleaved(q, torch.tensor([0]), 8, 100.0), q)


def test_plain_window_and_sink():
    mask = plain.window_mask(6, 3)
    assert mask[5].tolist() == [False, False, False, True, True, True] and mask[1].tolist() == [True, True] + [False] * 4
    scores = torch.zeros(2, 6, 6, dtype=torch.float64)
    p = plain.sink_softmax(scores, mask, torch.tensor([0.0, -1e9], dtype=torch.float64))
    # three visible keys of score 0 and a sink of 0: each key gets 1/4; without a sink 1/3
    assert torch.allclose(p[0, 5, 3:], torch.full((3,), 0.25, dtype=torch.float64))
    assert torch.allclose(p[1, 5, 3:], torch.full((3,), 1 / 3, dtype=torch.float64))
    assert float(p[0, 0, 0]) == 0.5 and float(p[:, :, :].masked_select(~mask[None].expand(2, 6, 6)).abs().max()) == 0.0
    capped = plain.attention_scores(torch.full((1, 1, 4), 10.0, dtype=torch.float64),
                                    torch.full((1, 1, 4), 10.0, dtype=torch.float64), 0.5, 7.0)
    assert abs(float(capped) - 7.0 * torch.tanh(torch.tensor(200.0 / 7.0)).item()) < 1e-12 and float(capped) <= 7.0


def test_plain_recurrence_continues_from_its_state():
    g = torch.Generator().manual_seed(2)
    T, heads, d = 11, 2, 5
    r, k, v = (torch.randn(T, heads, d, generator=g, dtype=torch.float64) for _ in range(3))
    w = torch.rand(T, heads, d, generator=g, dtype=torch.float64)
    u = torch.randn(heads, d, generator=g, dtype=torch.float64)
    whole, S = plain.wkv_recurrence(r, k, v, w, u)
    first, S1 = plain.wkv_recurrence(r[:4], k[:4], v[:4], w[:4], u)
    second, S2 = plain.wkv_recurrence(r[4:], k[4:], v[4:], w[4:], u, state=S1)
    assert torch.allclose(torch.cat([first, second]), whole, atol=1e-13) and torch.allclose(S2, S, atol=1e-13)
    # the first token sees only itself, through the bonus: o_0 = (r_0 . (u * k_0)) v_0
    want = (r[0] * u * k[0]).sum(-1, keepdim=True) * v[0]
    assert torch.allclose(whole[0], want, atol=1e-13)
    # the second token sees the first without decay (the decay of a token acts from the token after it)
    want1 = (r[1] * k[0]).sum(-1, keepdim=True) * v[0] + (r[1] * u * k[1]).sum(-1, keepdim=True) * v[1]
    assert torch.allclose(whole[1], want1, atol=1e-13)
    x = torch.randn(4, 6, generator=g, dtype=torch.float64)
    mu = torch.rand(6, generator=g, dtype=torch.float64)
    shifted = plain.token_shift(x, mu)
    assert torch.allclose(shifted[0], x[0] * (1 - mu)) and torch.allclose(shifted[2], x[2] + (x[1] - x[2]) * mu)
    assert torch.allclose(plain.token_shift(x[2:], mu, first=x[1]), shifted[2:])


def test_plain_model_is_causal_and_windows_forget():
    """Changing a token changes nothing before it; a model of attention layers alone forgets a token once it has
    left every window's reach, a model with a recurrent layer does not."""
    tensors = plain.random_model(CONFIG, seed=4)
    tokens = [(7 * i + 3) % 97 for i in range(40)]
    base = plain.forward(tensors, CONFIG, tokens)
    other = list(tokens)
    other[20] = (tokens[20] + 1) % 97
    changed = plain.forward(tensors, CONFIG, other)
    assert torch.equal(changed[:20], base[:20]) and not torch.equal(changed[20], base[20])
    only_attention = plain.make_config([A(2, 1, 16, window=4, rot_dims=8, ff=24), A(2, 2, 16, window=3, rot_dims=16, ff=None)],
                                       width=32, vocab=50)
    tensors = plain.random_model(only_attention, seed=5)
    tokens = [(5 * i + 1) % 50 for i in range(16)]
    base = plain.forward(tensors, only_attention, tokens)
    other = [(tokens[0] + 9) % 50] + tokens[1:]
    changed = plain.forward(tensors, only_attention, other)
    # reach of two layers: (4 - 1) + (3 - 1) = 5 tokens back
    assert torch.allclose(changed[6:], base[6:], atol=1e-12) and not torch.allclose(changed[5], base[5], atol=1e-9)
