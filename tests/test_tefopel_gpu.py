"""Tefopel in the engine against the plain implementation (tests/plain_tefopel.py): every mechanism alone, then whole
models through the step function, the trace replay and the scheduler, in float32 and bfloat16.

The configurations are made here, with random weights; sizes differ from model to model so that nothing rests on a
value that happens to be 1 or on two sizes that happen to be equal."""

import json
import os
import tempfile

import numpy as np
import pytest
import torch

import helpers
import plain_tefopel as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TORCH_DTYPE = {"float32": torch.float32, "bfloat16": torch.bfloat16}

A = plain.attention_layer
W = plain.wkv_layer
# small heads (CUDA-core attention in both precisions), grouped queries, a layer run twice, a wkv layer with a feed-forward
CONFIG_A = plain.make_config([A(4, 2, 16, window=12, rot_dims=8, ff=48), W(2, 16), A(2, 1, 32, window=40, rot_dims=32,
                              base=500.0, scale=0.3, softcap=8.0, ff=None), W(2, 16, weights_of=1),
                              A(4, 2, 16, window=12, rot_dims=8, ff=48, ) | {"weights_of": 0}, W(1, 24, ff=40)],
                             width=64, vocab=97)
# head sizes of the tensor-core attention kernels (64, 128), windows that span several key tiles, no rotation at all
CONFIG_B = plain.make_config([A(2, 1, 64, window=70, rot_dims=64, ff=96, softcap=15.0, scale=0.2),
                              W(3, 32, ff=64), A(1, 1, 128, window=200, rot_dims=0, ff=None, scale=0.05, softcap=50.0),
                              A(2, 2, 64, window=129, rot_dims=16, base=250000.0, ff=72)],
                             width=128, vocab=211, eps=1e-6)
# sizes that are no multiple of 8 or 16, a window of one token, single heads
CONFIG_C = plain.make_config([W(1, 40), A(1, 1, 24, window=1, rot_dims=24, ff=52, scale=0.25, softcap=5.0),
                              A(3, 3, 24, window=7, rot_dims=4, ff=None, scale=0.2, softcap=22.0), W(2, 12, ff=36)],
                             width=72, vocab=53, eps=1e-4)
# one kind of layer only: a model without any pages, and one without any slot state
CONFIG_D = plain.make_config([W(2, 32, ff=48), W(1, 20), W(2, 32, ff=48) | {"weights_of": 0}], width=48, vocab=61)
CONFIG_E = plain.make_config([A(3, 1, 16, window=9, rot_dims=6, ff=40, scale=0.3, softcap=9.0),
                              A(2, 2, 48, window=33, rot_dims=48, ff=None, base=300.0, softcap=25.0)], width=40, vocab=77)
CONFIGS = {"a": (CONFIG_A, 1, 8, 16), "b": (CONFIG_B, 2, 4, 16), "c": (CONFIG_C, 3, 6, 8),     # config, seed, rank, page
           "d": (CONFIG_D, 4, 3, 16), "e": (CONFIG_E, 5, 8, 32)}

_FOLDERS, _TENSORS, _LOGITS = {}, {}, {}


def folder_of(which):
    if which not in _FOLDERS:
        from pagedserve_b200.weights.safetensors_io import write_safetensors

        config, seed, rank, _ = CONFIGS[which]
        holder = tempfile.TemporaryDirectory(prefix=f"ps_tefopel_{which}_")
        _TENSORS[which] = plain.random_model(config, seed, rank)
        with open(os.path.join(holder.name, "config.json"), "w") as handle:
            json.dump(config, handle)
        write_safetensors(os.path.join(holder.name, "model.safetensors"), _TENSORS[which])
        _FOLDERS[which] = holder
    return _FOLDERS[which].name


def plain_logits(which, sequences):
    folder_of(which)
    out = {}
    for name, tokens in sequences.items():
        key = (which, tuple(tokens))
        if key not in _LOGITS:
            _LOGITS[key] = plain.forward(_TENSORS[which], CONFIGS[which][0], tokens).numpy()
        out[name] = _LOGITS[key]
    return out


def build_engine(which, dtype, **options):
    from pagedserve_b200.config.engine_config import EngineConfig
    from pagedserve_b200.engine.engine import Engine

    defaults = dict(dtype=dtype, block_size=CONFIGS[which][3], num_blocks=96, max_num_seqs=4, max_model_len=512)
    defaults.update(options)
    return Engine.from_folder(folder_of(which), EngineConfig(**defaults))


def sequences_for(which, lengths, seed=0):
    vocab = CONFIGS[which][0]["vocab"]
    return {f"s{i}": helpers.random_tokens(vocab, n, seed=seed + i) for i, n in enumerate(lengths)}


def rel_err(got, want):
    want = want.double()
    return float((got.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-30))


# ------------------------------------------------------------------ the replay program on whole models
def run_replay(which, dtype, steps, slots=4):
    from types import SimpleNamespace
    import io
    from pagedserve_b200.engine import replay as replay_module

    with tempfile.TemporaryDirectory(prefix="ps_out_") as out:
        args = SimpleNamespace(model=folder_of(which), dtype=dtype, out=out, max_tokens=helpers.peak_tokens(steps),
                               block_size=CONFIGS[which][3], max_num_seqs=slots, disable_cuda_graphs=False)
        stdin = io.StringIO("".join(json.dumps(step) + "\n" for step in steps))
        assert replay_module.run(args, stdin=stdin, stdout=io.StringIO()) == 0
        return helpers.collect(out, steps)


def check_replay(which, dtype, steps, sequences, what):
    got = run_replay(which, dtype, steps)
    want = plain_logits(which, sequences)
    for name in sequences:
        # The first token's wkv output is one value row times a single number, the second token's a mix of two
        # rows; the head norm divides by their size, so where those numbers come out small, bfloat16 rounding of
        # r, k, v is magnified (seen: up to 3.5e-3 x scale in the mean over 30 two-token sequences, float32 1e-7).
        # Sequences of a few tokens get twice the mean bound; everything longer the usual one.
        factor = 2.0 if len(sequences[name]) < 4 else 1.0
        helpers.assert_close(got[name], want[name], dtype, f"{what}/{which}/{name}", mean_factor=factor)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b", "c"])
def test_whole_prompts_and_decoded_tails(which, dtype):
    """Each request alone: whole in one step, and most of it in one step with its tail token by token, so that
    prefill and decoding through cache and state give the same logits."""
    sequences = sequences_for(which, [1, 2, 37, 150, 301], seed=10)
    check_replay(which, dtype, helpers.trace_whole(sequences), sequences, "whole")
    check_replay(which, dtype, helpers.trace_tail(sequences, tail=48), sequences, "tail")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b", "c"])
def test_portions_of_every_size(which, dtype):
    """Portions down to two tokens, cut inside pages, windows and key tiles."""
    sequences = sequences_for(which, [61, 143, 260], seed=20)
    check_replay(which, dtype, helpers.trace_chunks(sequences, seed=1), sequences, "portions")
    check_replay(which, dtype, helpers.trace_chunks(sequences, seed=2, sizes=(2, 2, 17, 64, 3, 130, 2, 31)), sequences,
                 "portions-2")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b", "c"])
def test_mixed_batches_reuse_pages_and_slots(which, dtype):
    """Nine unequal requests through four slots: portions of some beside single tokens of others, requests left
    out of steps, pages and state slots handed out again; every request must equal itself alone."""
    sequences = sequences_for(which, [90, 33, 200, 5, 61, 148, 17, 75, 2], seed=30)
    steps = helpers.trace_mixed(sequences, seed=3, live=4, decode_tail=20, max_portion=40)
    assert helpers.peak_tokens(steps) < sum(len(t) for t in sequences.values())
    check_replay(which, dtype, steps, sequences, "mixed")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["d", "e"])
def test_models_of_one_kind_of_layer(which, dtype):
    sequences = sequences_for(which, [70, 3, 131, 29, 64, 1], seed=70)
    check_replay(which, dtype, helpers.trace_whole(sequences), sequences, "whole")
    steps = helpers.trace_mixed(sequences, seed=5, live=4, decode_tail=16, max_portion=30)
    check_replay(which, dtype, steps, sequences, "mixed")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_prompt_longer_than_the_usual_step(dtype):
    """2,100 tokens in one step (more than the engine's default token budget of a step), and the same prompt in
    portions with a decoded tail: keys thousands of positions back, angles of thousands of radians, a recurrent
    state that has seen thousands of tokens."""
    sequences = sequences_for("a", [2100], seed=80)
    wanted = list(range(0, 2100, 97)) + list(range(2040, 2100))
    whole = [{"step": 0, "entries": [{"id": "s0", "tokens": sequences["s0"], "want": wanted}], "end": ["s0"]}]
    got = run_replay("a", dtype, whole)
    want = plain_logits("a", sequences)["s0"][wanted]
    helpers.assert_close(got["s0"], want, dtype, "long prompt in one step")
    steps, number, done = [], 0, 0
    for size in [1000, 700, 340] + [1] * 60:
        places = [i for i in range(size) if done + i in wanted]
        steps.append({"step": number, "entries": [{"id": "s0", "tokens": sequences["s0"][done:done + size],
                                                   "want": places}], "end": []})
        number, done = number + 1, done + size
    steps[-1]["end"] = ["s0"]
    got = run_replay("a", dtype, steps)
    helpers.assert_close(got["s0"], want, dtype, "long prompt in portions")


def test_long_decoding_float32():
    """A short prompt, then 330 tokens one by one: windows, pages that are released behind them and the
    recurrent state over hundreds of single steps."""
    sequences = sequences_for("a", [340], seed=40)
    check_replay("a", "float32", helpers.trace_tail(sequences, tail=330), sequences, "long decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_layers_give_pages_back(dtype):
    engine = build_engine("a", dtype, num_blocks=24)
    tokens = sequences_for("a", [300], seed=50)["s0"]
    from pagedserve_b200.engine.batch import StepEntry

    got = []
    for lo in range(0, 300, 50):
        got.append(engine.step([StepEntry("r", tokens[lo:lo + 50], list(range(50)))]).cpu().numpy())
    # 300 tokens would need 19 pages of 16 in each group; the widest window (40) keeps at most 4 + 4
    assert all(group.allocator.used_pages <= 8 for group in engine.cache.groups)
    helpers.assert_close(np.concatenate(got), plain_logits("a", {"r": tokens})["r"], dtype, "window pages")
    engine.finish("r")
    engine.cache.check_invariants()


# ------------------------------------------------------------------ generation through the scheduler
@pytest.mark.parametrize("strategy", ["orca", "sarathi"])
def test_greedy_generation_equals_the_plain_model(strategy):
    from pagedserve_b200.engine.engine import generate

    engine = build_engine("a", "float32", strategy=strategy, prefill_chunk_size=7, max_num_seqs=3)
    prompts = list(sequences_for("a", [9, 30, 3, 55, 1], seed=60).values())
    got = generate(engine, prompts, max_new_tokens=12)
    config, tensors = CONFIGS["a"][0], _TENSORS["a"]
    for prompt, tokens in zip(prompts, got):
        sequence = list(prompt)
        for _ in range(12):
            logits = plain.forward(tensors, config, sequence)[-1]
            top = torch.topk(logits, 2).values
            if float(top[0] - top[1]) < 1e-3 * float(logits.abs().max()):
                break                                        # a near tie: either token is a correct greedy choice
            sequence.append(int(logits.argmax()))
        made = len(sequence) - len(prompt)
        assert tokens[:made] == sequence[len(prompt):]
    engine.check_status()


def test_command_line_runs_a_model_folder(capsys):
    from pagedserve_b200.main import main

    assert main(["--model", folder_of("c"), "--dtype", "bfloat16", "--max-new-tokens", "4", "--block-size", "8",
                 "--num-blocks", "64", "--max-batch-size", "2", "--prompt-ids", "1 2 3 4 5"]) == 0
    assert "request 0:" in capsys.readouterr().out
    # a named size with random weights
    assert main(["--model", "tefopel-tiny", "--seed", "3", "--dtype", "float32", "--max-new-tokens", "5",
                 "--num-blocks", "32", "--max-batch-size", "2", "--prompt-ids", "7 8 9"]) == 0
    assert "request 0:" in capsys.readouterr().out


# ------------------------------------------------------------------ each part alone
def make_ctx(engine, entries):
    from pagedserve_b200.engine.batch import StepEntry

    ctx = engine.runner.prepare([StepEntry(*entry) for entry in entries])
    engine.runner.begin(ctx)
    return ctx


def layer_context(engine, schedule_index):
    from pagedserve_b200.parts.base import LayerContext

    entry = engine.spec.schedule[schedule_index]
    layer = LayerContext(entry.layer, entry.cache_layer, engine.model.positions)
    cache = engine.cache
    group_index = cache.group_of_layer.get(entry.cache_layer)
    if group_index is not None:
        group = cache.groups[group_index]
        layer.k_pool, layer.v_pool = group.layer_views(entry.cache_layer)
        layer.page_stride, layer.page_size = group.page_stride, group.page_size
        layer.pool, layer.pool_layer = group.pool, group.cache_layers.index(entry.cache_layer)
        layer.block_table = cache.slots.table_views[group_index]
    layer.state = cache.state.get(entry.cache_layer)
    return engine.model.blocks[entry.layer], layer


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-6), ("bfloat16", 1.2e-2)])
@pytest.mark.parametrize("which", ["a", "b", "c"])
def test_each_part_alone(which, dtype, tol):
    """Norm, both mixers, the feed-forward and the head, each fed with the plain implementation's own values.
    The mixers run a prompt in two portions, so the second one starts from pages and state."""
    engine = build_engine(which, dtype)
    config, tensors = CONFIGS[which][0], _TENSORS[which]
    eps, compute = config["norm"]["eps"], engine.dtype
    count, cut = 45, 29
    tokens = helpers.random_tokens(config["vocab"], count, seed=9)
    g = torch.Generator().manual_seed(5)
    stream = torch.randn(count, config["width"], generator=g, dtype=torch.float64) * 2.0
    for index, entry in enumerate(config["layers"]):
        prefix = "l%d." % plain.weight_owner(config, index)
        block, layer = layer_context(engine, index)
        t = lambda name: tensors[prefix + name].double()
        normed = plain.offset_rms_norm(stream, t("norm1"), eps)
        got_normed = block.norms["pre_mixer"].forward(stream.float().to(DEV))
        assert rel_err(got_normed, normed) < max(tol, 1e-6) / 2
        fed = normed.to(compute)                       # what the mixer is given, as the plain side sees it too
        if entry["type"] == "attention":
            want = plain.attention_mixer(tensors, prefix, entry["mixer"], fed.double(), torch.arange(count))
        else:
            want = plain.wkv_mixer(tensors, prefix, entry["mixer"], fed.double(), eps)
        residual = torch.zeros(count, config["width"], dtype=torch.float32, device=DEV)
        for name, lo, hi in (("x", 0, cut), ("x", cut, count)):
            ctx = make_ctx(engine, [(name, tokens[lo:hi], [])])
            block.mixer.forward(fed[lo:hi].to(DEV).contiguous(), residual[lo:hi], ctx, layer)
            engine.cache.commit_many([name])
        assert rel_err(residual, want) < tol, (which, index, entry["type"])
        engine.cache.free("x")
        if entry["mlp"] is not None:
            normed2 = plain.offset_rms_norm(stream, t("norm2"), eps).to(compute)
            want = plain.squared_relu_ff(tensors, prefix, normed2.double())
            residual.zero_()
            ctx = make_ctx(engine, [("y", tokens, [])])
            block.feed_forward.forward(normed2.to(DEV), residual, ctx)
            engine.cache.rollback("y")
            engine.cache.free("y")
            assert rel_err(residual, want) < tol
    # the model's norm on chosen rows, and the head against the token table
    ctx = make_ctx(engine, [("z", tokens, [0, 7, 44])])
    picked = engine.model.final_norm.forward(stream.float().to(DEV), rows=ctx.logit_rows)
    logits = engine.model.head.forward(picked, engine.model.embedding)
    want = plain.offset_rms_norm(stream, tensors["final.norm"].double(), eps)[[0, 7, 44]] @ tensors["embed"].double().T
    assert rel_err(logits, want) < tol
    hidden = engine.model.embedding.forward(ctx, engine.model.positions)
    assert torch.equal(hidden.cpu(), tensors["embed"].float()[torch.tensor(tokens)])
    engine.cache.rollback("z")
    engine.cache.free("z")
    engine.check_status()


# ------------------------------------------------------------------ kernels alone
def ops_for(dtype):
    from pagedserve_b200.kernels.ops import Ops

    return Ops(dtype)


def plain_attention_rows(case, scale, softcap, window, sink):
    """float64 attention of every sequence of a PagedCase with the plain implementation's pieces."""
    rows, start = [], 0
    rep = case.n_heads // case.n_kv_heads
    for length in case.lengths:
        sl = slice(start, start + length)
        q = case.q[sl].double().reshape(length, case.n_heads, case.head_dim)
        k = case.k[sl].double().reshape(length, case.n_kv_heads, case.head_dim).repeat_interleave(rep, 1)
        v = case.v[sl].double().reshape(length, case.n_kv_heads, case.head_dim).repeat_interleave(rep, 1)
        s = plain.attention_scores(q, k, scale, softcap)
        p = plain.sink_softmax(s, plain.window_mask(length, window), sink.double())
        rows.append(torch.einsum("hij,jhd->ihd", p, v).reshape(length, -1))
        start += length
    return torch.cat(rows)


def run_attention_kernel(kernel, ops, case, lengths, window, scale, softcap, sink):
    heads, kv_heads, head_dim, page = case.n_heads, case.n_kv_heads, case.head_dim, case.page_size
    total = sum(lengths)
    out = torch.full((total, heads * head_dim), float("nan"), dtype=case.dtype, device=DEV)
    q = case.q.to(DEV)
    starts = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]), dtype=torch.int32, device=DEV)
    kv_len = torch.tensor(lengths, dtype=torch.int32, device=DEV)
    if kernel == "simt":
        ops.paged_attention_simt(q, out, case.k_pool, case.v_pool, case.page_stride, case.token_item, case.positions,
                                 case.table, heads, kv_heads, head_dim, page, window, scale, softcap=softcap, sink=sink)
    elif kernel == "decode":
        ops.paged_attention_decode(q, out, case.k_pool, case.v_pool, case.page_stride, case.token_item, case.positions,
                                   case.table, heads, kv_heads, head_dim, page, window, scale, max(lengths),
                                   softcap=softcap, sink=sink)
    elif kernel == "decode-one-split":
        ops.paged_attention_decode(q, out, case.k_pool, case.v_pool, case.page_stride, case.token_item, case.positions,
                                   case.table, heads, kv_heads, head_dim, page, window, scale, max(lengths),
                                   target_ctas=1, softcap=softcap, sink=sink)
    elif kernel == "prefill":
        ops.prefill_attention(q, out, case.k_pool, case.v_pool, case.page_stride, starts, kv_len, case.table, 0,
                              len(lengths), sum(-(-n // 64) for n in lengths), heads, kv_heads, head_dim, page, window,
                              scale, softcap=softcap, sink=sink)
    else:
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops.prefill_attention_tc(q, out, case.pool, 0, starts, kv_len, case.table, 0, len(lengths),
                                 sum(-(-n // 128) for n in lengths), heads, kv_heads, head_dim, page, window, scale,
                                 status=status, row_threads=2 if kernel == "tcgen05-two" else 1, softcap=softcap,
                                 sink=sink)
        assert int(status.item()) == 0
    return out


ATTENTION_KERNELS = [("simt", torch.float32, 24, 3e-6), ("simt", torch.bfloat16, 40, 8e-3),
                     ("decode", torch.bfloat16, 64, 8e-3), ("decode-one-split", torch.bfloat16, 32, 8e-3),
                     ("prefill", torch.bfloat16, 48, 8e-3), ("tcgen05", torch.bfloat16, 64, 8e-3),
                     ("tcgen05-two", torch.bfloat16, 128, 8e-3), ("decode", torch.bfloat16, 256, 8e-3),
                     ("prefill", torch.bfloat16, 96, 8e-3)]


@pytest.mark.parametrize("kernel,dtype,head_dim,tol", ATTENTION_KERNELS)
@pytest.mark.parametrize("window", [1, 19, 141, 5000])
def test_attention_kernels_with_cap_sink_and_window(kernel, dtype, head_dim, tol, window):
    """Every attention kernel with capped scores, a sink per head and a window, on contexts around page, tile and
    window edges.  Large sinks (most of the weight goes nowhere) and very negative ones (no effect) are both there."""
    from test_kernels_gpu import PagedCase

    ops = ops_for(dtype)
    heads, kv_heads, page = 4, 2, 16
    lengths = [1, 2, 18, 19, 20, 127, 140, 141, 142, 300]
    case = PagedCase(ops, dtype, lengths, heads, kv_heads, head_dim, page, seed=head_dim + window)
    sink = torch.tensor([4.0, -30.0, 0.5, -1.0])
    scale, softcap = 0.37, 3.0                       # raw scores reach far beyond the cap
    want = plain_attention_rows(case, scale, softcap, window, sink)
    got = run_attention_kernel(kernel, ops, case, lengths, window, scale, softcap, sink.to(DEV))
    assert torch.isfinite(got.float()).all()
    assert rel_err(got, want) < tol
    # without the sink the result differs clearly: the comparison above is not blind to it
    assert rel_err(plain_attention_rows(case, scale, softcap, window, torch.full((4,), -1e9)), want) > 0.05


@pytest.mark.parametrize("kernel,dtype,head_dim,tol", ATTENTION_KERNELS)
def test_attention_window_edge_and_far_key_stand_out(kernel, dtype, head_dim, tol):
    """Two keys are made to dominate the last query of a sequence: the oldest one the window still holds and the
    one just before it.  The first must carry the output, the second must not be seen at all."""
    from test_kernels_gpu import PagedCase

    ops = ops_for(dtype)
    heads, kv_heads, page, window, length = 2, 1, 16, 141, 700
    for inside in (True, False):
        case = PagedCase(ops, dtype, [length, 40], heads, kv_heads, head_dim, page, seed=head_dim)
        g = torch.Generator().manual_seed(1)
        direction = torch.randn(head_dim, generator=g)
        direction = direction / direction.norm()
        last = length - 1
        key = last - window + 1 if inside else last - window
        case.q[last, head_dim:2 * head_dim] = (direction * 20).to(dtype)
        case.k[key, :head_dim] = (direction * 20).to(dtype)
        ops.kv_append(case.k.to(DEV), case.v.to(DEV), case.token_item, case.positions, case.table, case.k_pool,
                      case.v_pool, case.page_stride, kv_heads, head_dim, page)
        sink = torch.tensor([0.0, 1.0])
        want = plain_attention_rows(case, 1.0, 50.0, window, sink)
        got = run_attention_kernel(kernel, ops, case, [length, 40], window, 1.0, 50.0, sink.to(DEV))
        assert rel_err(got, want) < tol
        row = got[last, head_dim:2 * head_dim].double().cpu()
        seen = float((row - case.v[key, :head_dim].double()).abs().max()) < 0.05
        assert seen == inside


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,rot_dims,page", [(4, 2, 16, 8, 16), (3, 3, 24, 24, 8), (2, 1, 64, 0, 4),
                                                                   (1, 1, 10, 6, 2), (2, 1, 9, 4, 4), (3, 1, 7, 6, 8)])
@pytest.mark.parametrize("own_values", [False, True])
def test_rotary_kernel_turns_queries_and_fills_pages(dtype, heads, kv_heads, head_dim, rot_dims, page, own_values):
    from test_kernels_gpu import PagedCase
    from types import SimpleNamespace

    ops = ops_for(dtype)
    lengths = [5, 33, 70]
    case = PagedCase(ops, dtype, lengths, heads, kv_heads, head_dim, page, seed=rot_dims + page)
    case.pool.fill_(float("nan"))
    base = 777.0
    positions = case.positions.cpu() + 1000 * (case.token_item.cpu() == 2)        # far positions too
    # pages for those positions: sequence 2 gets a table of its own that reaches them
    table = torch.full((3, 1100 // page + 2), -1, dtype=torch.int32)
    table[:, :case.table.shape[1]] = case.table.cpu()
    spare = int(case.table.max()) + 1
    extra = -(-(1000 + lengths[2]) // page)
    pool = torch.full((spare + extra + 1, 1, 2, kv_heads, page, head_dim), float("nan"), dtype=dtype, device=DEV)
    table[2, :extra] = torch.arange(spare, spare + extra, dtype=torch.int32)
    layer = SimpleNamespace(k_pool=pool[:, 0, 0], v_pool=pool[:, 0, 1], page_stride=case.page_stride, page_size=page,
                            block_table=table.to(DEV))
    ctx = SimpleNamespace(token_slot=case.token_item, positions=positions.to(torch.int32).to(DEV))
    q, k = case.q.to(DEV).clone(), case.k.to(DEV).clone()
    v = case.v.to(DEV) if own_values else None
    inv_freq = (base ** (-2.0 * torch.arange(rot_dims // 2, dtype=torch.float64) / max(rot_dims, 1))).float().to(DEV)
    ops.rotary_cache_write(q, k, v, inv_freq if rot_dims else None, rot_dims, True, ctx, layer, heads, kv_heads,
                           head_dim)
    T = sum(lengths)
    want_q = plain.rotate_interleaved(case.q.double().reshape(T, heads, head_dim), positions, rot_dims, base)
    want_k = plain.rotate_interleaved(case.k.double().reshape(T, kv_heads, head_dim), positions, rot_dims, base)
    tol = 2e-4 if dtype == torch.float32 else 8e-3                                # float32 angles at position 1,000
    assert rel_err(q.reshape(T, heads, head_dim), want_q) < tol
    assert torch.equal(k.cpu(), case.k)                                           # the projection's keys stay
    host = pool.cpu()
    values = case.v if own_values else case.k
    for t in range(T):
        item, p = int(case.token_item[t]), int(positions[t])
        page_id = int(table[item, p // page])
        got_k = host[page_id, 0, 0, :, p % page, :]
        got_v = host[page_id, 0, 1, :, p % page, :]
        assert rel_err(got_k, want_k[t]) < tol
        assert torch.equal(got_v.reshape(-1), values[t])
    assert int(torch.isnan(host).sum()) > 0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 6e-6), (torch.bfloat16, 8e-3)])     # float32: sums of up to 128 terms
@pytest.mark.parametrize("heads,dim,width", [(2, 16, 64), (1, 40, 72), (3, 64, 200), (2, 128, 96), (5, 12, 36),
                                             (2, 96, 64), (1, 80, 40), (3, 30, 48)])
def test_wkv_kernels_alone(dtype, tol, heads, dim, width):
    """Token shift and the recurrence on three entries at once (one of a single token, one that continues stored
    state), against the plain recurrence; the state left in the slots is checked too."""
    from types import SimpleNamespace

    ops = ops_for(dtype)
    g = torch.Generator().manual_seed(heads * dim)
    inner = heads * dim
    lengths, slots = [7, 1, 30], [2, 0, 3]
    T = sum(lengths)
    x = torch.randn(T, width, generator=g).to(dtype)
    mu = torch.rand(5, width, generator=g)
    r, k, v = (torch.randn(T, inner, generator=g) for _ in range(3))
    gate = torch.randn(T, inner, generator=g)
    decay_arg = -1.0 + 1.5 * torch.randn(T, inner, generator=g)
    u, gain = 0.5 * torch.randn(heads, dim, generator=g), 1.0 + 0.1 * torch.randn(inner, generator=g)
    matrix = heads * dim * dim
    state = torch.zeros(5, matrix + width)
    state[3, :matrix] = torch.randn(matrix, generator=g)                   # entry 2 continues a request
    state[3, matrix:] = torch.randn(width, generator=g)
    state_dev = state.to(DEV)
    starts = np.concatenate([[0], np.cumsum(lengths)])
    ctx = SimpleNamespace(token_item=torch.tensor(np.repeat(np.arange(3), lengths), dtype=torch.int32, device=DEV),
                          q_start=torch.tensor(starts, dtype=torch.int32, device=DEV),
                          item_slot=torch.tensor(slots, dtype=torch.int32, device=DEV), num_items=3)
    blends = torch.empty(5, T, width, dtype=dtype, device=DEV)
    ops.token_shift_mix(x.to(DEV), mu.to(DEV), state_dev, matrix, ctx, blends)
    out = torch.empty(T, inner, dtype=dtype, device=DEV)
    ops.wkv_recurrence(r.to(DEV), k.to(DEV), v.to(DEV), decay_arg.to(DEV), gate.to(DEV), u.reshape(-1).to(DEV),
                       gain.to(DEV), 1e-5, x.to(DEV), state_dev, matrix, ctx, out, heads, dim)
    after = state_dev.cpu()
    for item, (length, slot) in enumerate(zip(lengths, slots)):
        sl = slice(starts[item], starts[item + 1])
        xs = x[sl].double()
        for s in range(5):
            want = plain.token_shift(xs, mu[s].double(), first=state[slot, matrix:].double())
            assert rel_err(blends[s, sl], want) < tol
        shape = (length, heads, dim)
        w = torch.exp(-torch.exp(decay_arg[sl].double())).reshape(shape)
        want, S = plain.wkv_recurrence(r[sl].double().reshape(shape), k[sl].double().reshape(shape),
                                       v[sl].double().reshape(shape), w, u.double(),
                                       state[slot, :matrix].double().reshape(heads, dim, dim))
        want = plain.rms_unit(want, 1e-5).reshape(length, inner) * gain.double() * gate[sl].double()
        assert rel_err(out[sl], want) < tol
        assert rel_err(after[slot, :matrix].reshape(heads, dim, dim), S) < 1e-5
        assert torch.equal(after[slot, matrix:], x[sl][-1].float())
    assert torch.equal(after[[1, 4]], state[[1, 4]])                          # other slots are left alone


@pytest.mark.parametrize("act", ["relu_squared", "silu", "tanh"])
@pytest.mark.parametrize("dtype,M,N,K", [(torch.float32, 9, 40, 24), (torch.bfloat16, 8, 96, 64),
                                         (torch.bfloat16, 40, 2304, 768), (torch.bfloat16, 200, 336, 128)])
def test_product_epilogues(act, dtype, M, N, K):
    """The activations this design adds, in the epilogue of every kind of matrix product the dispatch picks."""
    ops = ops_for(dtype)
    g = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=g).to(dtype)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(dtype)
    out = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.linear(a.to(DEV), w.to(DEV), None, out, act=act)
    z = a.double() @ w.double().T
    want = {"relu_squared": torch.relu(z) ** 2, "silu": torch.nn.functional.silu(z), "tanh": torch.tanh(z)}[act]
    assert rel_err(out, want) < (1e-5 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("dtype,M,groups,cols,K", [(torch.bfloat16, 1, 4, 32, 64), (torch.bfloat16, 8, 4, 96, 200),
                                                   (torch.bfloat16, 32, 3, 1024, 1024), (torch.bfloat16, 40, 4, 64, 128),
                                                   (torch.bfloat16, 5, 2, 24, 64), (torch.float32, 6, 4, 32, 48)])
def test_grouped_products(dtype, M, groups, cols, K):
    """Several products of equal shape, each on rows of its own, as one call: the one-launch form for few bfloat16
    rows and the product-by-product form elsewhere give what separate products give; the activation touches only
    the groups it is asked for."""
    ops = ops_for(dtype)
    g = torch.Generator().manual_seed(M + cols)
    a = torch.randn(groups, M, K, generator=g).to(dtype)
    w = (torch.randn(groups * cols, K, generator=g) / K ** 0.5).to(dtype)
    out = torch.full((groups + 1, M, cols), float("nan"), dtype=torch.float32, device=DEV)
    before = ops.launches
    ops.linear_grouped(a.to(DEV), w.to(DEV), out[:groups], act="silu", act_from_group=groups - 1)
    one_launch = dtype == torch.bfloat16 and M <= ops.GROUPED_ROWS and cols % 16 == 0
    assert ops.launches - before == (1 if one_launch else groups)
    for index in range(groups):
        z = a[index].double() @ w[index * cols:(index + 1) * cols].double().T
        want = torch.nn.functional.silu(z) if index == groups - 1 else z
        assert rel_err(out[index], want) < (1e-5 if dtype == torch.float32 else 5e-3)
    assert torch.isnan(out[groups]).all()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 5e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("width,inner,rank", [(64, 32, 8), (72, 40, 5), (1024, 512, 16), (200, 192, 3)])
def test_wkv_first_kernel_norms_blends_and_decays(dtype, tol, width, inner, rank):
    """The mixer's first kernel alone: RMS norm of the residual rows, blends with the row before (the slot's
    stored row for an entry's first token), and the decay's argument, against the plain functions."""
    from types import SimpleNamespace

    ops = ops_for(dtype)
    g = torch.Generator().manual_seed(width + rank)
    lengths, slots = [6, 1, 19], [1, 3, 0]
    T = sum(lengths)
    hidden = 3.0 * torch.randn(T, width, generator=g)
    gain = 1.0 + 0.2 * torch.randn(width, generator=g)
    mu = torch.rand(5, width, generator=g)
    w1 = (torch.randn(rank, width, generator=g) / width ** 0.5).to(dtype)
    w2 = torch.randn(inner, rank, generator=g).to(dtype)
    w0 = torch.randn(inner, generator=g)
    matrix = 7
    state = torch.zeros(4, matrix + width)
    state[0, matrix:] = torch.randn(width, generator=g).to(dtype).float()      # entry 2 continues a request
    starts = np.concatenate([[0], np.cumsum(lengths)])
    ctx = SimpleNamespace(token_item=torch.tensor(np.repeat(np.arange(3), lengths), dtype=torch.int32, device=DEV),
                          q_start=torch.tensor(starts, dtype=torch.int32, device=DEV),
                          item_slot=torch.tensor(slots, dtype=torch.int32, device=DEV), num_items=3)
    blends = torch.full((5, T, width), float("nan"), dtype=dtype, device=DEV)
    decay = torch.full((T, inner), float("nan"), dtype=torch.float32, device=DEV)
    eps = 1e-5
    ops.wkv_prepare(hidden.to(DEV), gain.to(DEV), eps, mu.to(DEV), state.to(DEV), matrix, ctx, w1.to(DEV), w2.to(DEV),
                    w0.to(DEV), blends, decay)
    normed = plain.rms_unit(hidden.double(), eps) * gain.double()
    assert rel_err(blends[4], normed) < tol
    x = blends[4].cpu().double()                           # the kernel's own rounding of the normed rows
    for item, (length, slot) in enumerate(zip(lengths, slots)):
        sl = slice(starts[item], starts[item + 1])
        for s in range(4):
            want = plain.token_shift(x[sl], mu[s].double(), first=state[slot, matrix:].double())
            assert rel_err(blends[s, sl], want) < tol
        m_w = plain.token_shift(x[sl], mu[4].double(), first=state[slot, matrix:].double())
        want = torch.tanh(m_w @ w1.double().T) @ w2.double().T + w0.double()
        assert rel_err(decay[sl], want) < 2 * tol
