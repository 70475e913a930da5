"""Causal self-attention over the paged cache."""

from __future__ import annotations

import torch

from pagedserve_b200.cache.manager import KVNeed
from pagedserve_b200.parts.base import Mixer, register_part
from pagedserve_b200.weights.loader import ParamSpec


@register_part("mixer", "causal_attention")
class CausalSelfAttention(Mixer):
    """Packed QKV projection, causal attention over the request's pages, output projection.

    qkv = x W + b, split q|k|v in that order, head j = columns [j*hd, (j+1)*hd)
    (reference: src/model/paged_decoder.py:49-53, 63-69);
    s = (q.k) * scale, keys after the query masked, softmax in float32, o = p v
    (reference: src/model/paged_attention.py:262-295);
    residual += o W_o + b_o (reference: src/model/paged_decoder.py:135, 184).

    The step's keys and values are written to the pages first; queries then read
    everything, old and new, from the pages.  A token's result therefore does not
    depend on how its prompt was cut into steps.

    params: hidden_size, n_heads, n_kv_heads, head_dim, scale, window (None = all keys),
    has_bias, stored_in_out (True: matrices stored [in, out]), qkv_name, out_name,
    init_std, out_init_std, write_cache (False: this run only reads a cache layer that another
    run of the schedule has written in the same step).
    """

    graph_safe = True
    accepts_deferred_norm = True       # x goes straight into ops.linear_qkv

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = self.params
        if p["n_heads"] % p["n_kv_heads"] != 0:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if not (0 < p["head_dim"] <= 256):
            # multiples of 16 run on the tensor-core kernels in bfloat16; other sizes on the CUDA-core ones
            raise ValueError(f"head_dim {p['head_dim']} is not supported: at most 256")
        self.q_width = p["n_heads"] * p["head_dim"]
        self.kv_width = p["n_kv_heads"] * p["head_dim"]

    def cache_need(self):
        p = self.params
        return KVNeed(p["n_kv_heads"], p["head_dim"], p.get("window"))

    def _matrix(self, name, n_out, n_in, std):
        stored = (n_in, n_out) if self.params.get("stored_in_out", False) else (n_out, n_in)
        return (ParamSpec(self._n(name + ".weight"), stored, "matmul",
                          transpose=self.params.get("stored_in_out", False)), ("normal", std))

    def param_specs(self):
        p = self.params
        total = self.q_width + 2 * self.kv_width
        specs = [self._matrix(p["qkv_name"], total, p["hidden_size"], p.get("init_std", 0.02)),
                 self._matrix(p["out_name"], p["hidden_size"], self.q_width, p.get("out_init_std", 0.02))]
        if p.get("has_bias", True):
            specs.append((ParamSpec(self._n(p["qkv_name"] + ".bias"), (total,), "vector"),
                          ("normal", p.get("init_std", 0.02))))
            specs.append((ParamSpec(self._n(p["out_name"] + ".bias"), (p["hidden_size"],), "vector"),
                          ("normal", p.get("init_std", 0.02))))
        return specs

    def bind(self, tensors):
        p = self.params
        self.w_qkv = tensors[self._n(p["qkv_name"] + ".weight")]       # [q+2kv, H]
        self.w_out = tensors[self._n(p["out_name"] + ".weight")]       # [H, q]
        has_bias = p.get("has_bias", True)
        self.b_qkv = tensors[self._n(p["qkv_name"] + ".bias")] if has_bias else None
        self.b_out = tensors[self._n(p["out_name"] + ".bias")] if has_bias else None

    def forward(self, x, residual, ctx, layer):
        p = self.params
        ops = self.env.ops
        tokens = x.shape[0]
        from pagedserve_b200.parts.base import PositionEncoding

        qkv = ops.empty((tokens, self.q_width + 2 * self.kv_width), self.env.dtype, x.device)
        write_cache = p.get("write_cache", True)
        # keys may go from the projection straight into the pages unless the position encoding
        # still has to transform them
        no_rotation = type(layer.positions).rotate is PositionEncoding.rotate
        written = ops.linear_qkv(x, self.w_qkv, self.b_qkv, qkv, ctx, layer, self.q_width, self.kv_width,
                                 p["head_dim"], scatter=write_cache and no_rotation)
        q = qkv[:, :self.q_width]
        k = qkv[:, self.q_width:self.q_width + self.kv_width]
        v = qkv[:, self.q_width + self.kv_width:]
        if not no_rotation:
            layer.positions.rotate(q, k, ctx)
        context = ops.empty((tokens, self.q_width), self.env.dtype, x.device)
        ops.attention(q, k, v, context, ctx, layer, p["n_heads"], p["n_kv_heads"], p["head_dim"],
                      p.get("window"), float(p["scale"]), write_cache=write_cache and not written)
        ops.linear(context, self.w_out, self.b_out, residual, accumulate=True)


@register_part("mixer", "rotary_attention")
class RotaryAttention(Mixer):
    """Attention with separate projections, rotary positions of its own, and optional extras of the softmax.

    q = x W_q, k = x W_k, v = x W_v, or, without ``v_name``, v = k as projected (before it is turned): such a
    layer has no value projection.  Queries and keys turn by position (``rotary``: dims, base, interleaved);
    s = (q . k) * scale; with ``softcap`` c: s <- c * tanh(s / c); query i sees keys j with
    0 <= i - j < ``window`` (all earlier keys without a window); with ``sink_name`` every query head has a
    learned number whose exponential is added to the softmax's denominator and to nothing else;
    residual += o W_o.  Scores, softmax, angles: float32.

    The projections run as one product over the stacked matrices; one kernel then turns the queries in place
    and sends the turned keys and the values into the pages; attention reads only pages.

    params: hidden_size, n_heads, n_kv_heads, head_dim, scale, window, softcap, rotary (dict or None),
    q_name, k_name, v_name (None: values are the unturned keys), out_name, sink_name (None: no sinks),
    init_std, out_init_std.
    """

    graph_safe = True
    accepts_deferred_norm = True       # x goes straight into ops.linear

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = self.params
        if p["n_heads"] % p["n_kv_heads"] != 0:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        if not (0 < p["head_dim"] <= 256):
            raise ValueError(f"head_dim {p['head_dim']} is not supported: at most 256")
        if p.get("window") is not None and p["window"] <= 0:
            raise ValueError("window must be positive")
        self.q_width = p["n_heads"] * p["head_dim"]
        self.kv_width = p["n_kv_heads"] * p["head_dim"]
        self.has_v = p.get("v_name") is not None
        rotary = p.get("rotary") or dict(dims=0, base=10000.0)
        from pagedserve_b200.parts.positions import RotaryPositions

        self.rotary = RotaryPositions(dict(dims=rotary["dims"], base=rotary["base"],
                                           interleaved=rotary.get("interleaved", True), head_dim=p["head_dim"]),
                                      prefix, env)

    def cache_need(self):
        p = self.params
        return KVNeed(p["n_kv_heads"], p["head_dim"], p.get("window"))

    def param_specs(self):
        p = self.params
        std = p.get("init_std", 0.02)
        specs = [(ParamSpec(self._n(p["q_name"]), (self.q_width, p["hidden_size"]), "matmul"), ("normal", std)),
                 (ParamSpec(self._n(p["k_name"]), (self.kv_width, p["hidden_size"]), "matmul"), ("normal", std))]
        if self.has_v:
            specs.append((ParamSpec(self._n(p["v_name"]), (self.kv_width, p["hidden_size"]), "matmul"),
                          ("normal", std)))
        specs.append((ParamSpec(self._n(p["out_name"]), (p["hidden_size"], self.q_width), "matmul"),
                      ("normal", p.get("out_init_std", std))))
        if p.get("sink_name"):
            specs.append((ParamSpec(self._n(p["sink_name"]), (p["n_heads"],), "vector"), ("normal", 1.0)))
        return specs

    def bind(self, tensors):
        p = self.params
        pieces = [tensors[self._n(p["q_name"])], tensors[self._n(p["k_name"])]]
        if self.has_v:
            pieces.append(tensors[self._n(p["v_name"])])
        self.w_in = torch.cat(pieces, dim=0).contiguous()              # [q + k (+ v), H]
        self.w_out = tensors[self._n(p["out_name"])]
        self.sink = tensors[self._n(p["sink_name"])].contiguous() if p.get("sink_name") else None

    def forward(self, x, residual, ctx, layer):
        p = self.params
        ops = self.env.ops
        tokens = x.shape[0]
        projected = ops.empty((tokens, self.w_in.shape[0]), self.env.dtype, residual.device)
        ops.linear(x, self.w_in, None, projected)
        q = projected[:, :self.q_width]
        k = projected[:, self.q_width:self.q_width + self.kv_width]
        v = projected[:, self.q_width + self.kv_width:] if self.has_v else None
        self.rotary.turn_and_store(q, k, v, ctx, layer, p["n_heads"], p["n_kv_heads"],
                                   write_cache=p.get("write_cache", True))
        context = ops.empty((tokens, self.q_width), self.env.dtype, residual.device)
        ops.attention(q, k, v, context, ctx, layer, p["n_heads"], p["n_kv_heads"], p["head_dim"], p.get("window"),
                      float(p["scale"]), write_cache=False, softcap=p.get("softcap"), sink=self.sink)
        ops.linear(context, self.w_out, None, residual, accumulate=True)


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    """Attention whose keys and values of all heads are made from one small vector per token, which is all the
    cache holds.

    With H heads, per head ``flat_dim`` unturned and ``rot_dim`` turning query/key numbers, values of size
    ``v_dim``, and a latent of size ``kv_rank``:
    q = x W_q, head by head [flat | turning];  down = x W_dkv (kv_rank + rot_dim numbers): c = its first kv_rank,
    divided by their root mean square and multiplied by a gain; k_turn = its last rot_dim, one for all heads.
    Head h has k_flat = W_uk(h) c and v = W_uv(h) c.  Turning parts turn by position (neighbouring pairs, the
    first ``rotary.dims`` of the rot_dim numbers);  s = (q_flat . k_flat + q_turn . k_turn) * scale over the keys
    j with 0 <= i - j < ``window``; softmax; the joined heads are multiplied by sigmoid(x W_g) and W_o adds the
    result into the residual row.

    Since q_flat . W_uk(h) c = (W_uk(h)^T q_flat) . c and sum_j p_j W_uv(h) c_j = W_uv(h) sum_j p_j c_j, attention
    runs over the cached rows [c | k_turn] themselves: one key/value head of size kv_rank + rot_dim shared by all
    query heads, queries [W_uk(h)^T q_flat | q_turn], values the same rows (a cache of one plane), and W_uv(h)
    applied to the first kv_rank numbers of each head's result.  Prompt portions and single tokens take the same
    path, so a position's result does not depend on how the prompt was cut.

    Launches: the stacked projection (q | down | gate), ``latent_prepare`` (norm of c, turns, cache write), the
    per-head products with W_uk^T, attention, the per-head products with W_uv, the gate, the output product.
    Norm statistics, angles, scores and softmax are float32.

    params: hidden_size, n_heads, flat_dim, rot_dim, v_dim, kv_rank, scale, window, eps,
    rotary (dims, base), init_std, out_init_std; tensors q, dkv, dkv.norm, uk, uv, g, o.
    """

    graph_safe = True
    accepts_deferred_norm = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = self.params
        self.row = p["kv_rank"] + p["rot_dim"]                    # the cached row, and the attention head size
        if not (0 < self.row <= 256):
            raise ValueError(f"latent_attention: kv_rank + rot_dim = {self.row} is not supported: at most 256")
        if p.get("window") is not None and p["window"] <= 0:
            raise ValueError("window must be positive")
        rotary = p.get("rotary") or dict(dims=0, base=10000.0)
        if rotary["dims"] < 0 or rotary["dims"] % 2 or rotary["dims"] > p["rot_dim"]:
            raise ValueError("latent_attention: rotary dims must be even and at most rot_dim")
        self.q_width = p["n_heads"] * (p["flat_dim"] + p["rot_dim"])
        self.v_width = p["n_heads"] * p["v_dim"]
        from pagedserve_b200.parts.positions import RotaryPositions

        self.rotary = RotaryPositions(dict(dims=rotary["dims"], base=rotary["base"], interleaved=True,
                                           head_dim=max(p["rot_dim"], 1)), prefix, env)

    def cache_need(self):
        return KVNeed(1, self.row, self.params.get("window"), planes=1)

    def param_specs(self):
        p = self.params
        W, H, R = p["hidden_size"], p["n_heads"], p["kv_rank"]
        std = p.get("init_std", 0.02)
        return [(ParamSpec(self._n("q"), (self.q_width, W), "matmul"), ("normal", std)),
                (ParamSpec(self._n("dkv"), (self.row, W), "matmul"), ("normal", std)),
                (ParamSpec(self._n("dkv.norm"), (R,), "vector"), ("ones_plus_normal", 0.1)),
                (ParamSpec(self._n("uk"), (H * p["flat_dim"], R), "matmul"), ("normal", R ** -0.5)),
                (ParamSpec(self._n("uv"), (self.v_width, R), "matmul"), ("normal", R ** -0.5)),
                (ParamSpec(self._n("g"), (self.v_width, W), "matmul"), ("normal", std)),
                (ParamSpec(self._n("o"), (W, self.v_width), "matmul"), ("normal", p.get("out_init_std", std)))]

    def bind(self, tensors):
        p = self.params
        t = lambda name: tensors[self._n(name)]
        H, d, R = p["n_heads"], p["flat_dim"], p["kv_rank"]
        self.w_in = torch.cat([t("q"), t("dkv"), t("g")], dim=0).contiguous()          # [q | down | gate, W]
        self.gain = t("dkv.norm").contiguous()
        # W_uk(h)^T stacked head by head: [H * R, d], so that head h's product maps q_flat(h) to R numbers
        self.w_uk_t = t("uk").reshape(H, d, R).transpose(1, 2).reshape(H * R, d).contiguous()
        self.w_uv = t("uv").contiguous()                                                # [H * v_dim, R]
        self.w_o = t("o")

    def forward(self, x, residual, ctx, layer):
        p = self.params
        ops, dtype, device = self.env.ops, self.env.dtype, residual.device
        H, d, r, R, dv = p["n_heads"], p["flat_dim"], p["rot_dim"], p["kv_rank"], p["v_dim"]
        tokens = x.shape[0]
        projected = ops.empty((tokens, self.w_in.shape[0]), dtype, device)
        ops.linear(x, self.w_in, None, projected)
        q = projected[:, :self.q_width]
        down = projected[:, self.q_width:self.q_width + self.row]
        gate = projected[:, self.q_width + self.row:]
        queries = ops.empty((tokens, H * self.row), dtype, device)
        ops.latent_prepare(q, down, self.gain, float(p["eps"]), self.rotary.inv_freq_split(), self.rotary.params["dims"],
                           ctx, layer, queries, H, d, r, R, write_cache=p.get("write_cache", True))
        # per head: [T, d] x W_uk(h) -> the first R numbers of the head's attention query
        ops.linear_grouped(q.view(tokens, H, d + r)[:, :, :d].permute(1, 0, 2), self.w_uk_t,
                           queries.view(tokens, H, self.row)[:, :, :R].permute(1, 0, 2), max_rows=64)
        context = ops.empty((tokens, H * self.row), dtype, device)
        ops.attention(queries, None, None, context, ctx, layer, H, 1, self.row, p.get("window"), float(p["scale"]),
                      write_cache=False)
        heads = ops.empty((tokens, self.v_width), dtype, device)
        ops.linear_grouped(context.view(tokens, H, self.row)[:, :, :R].permute(1, 0, 2), self.w_uv,
                           heads.view(tokens, H, dv).permute(1, 0, 2), max_rows=64)
        ops.sigmoid_gate(heads, gate)
        ops.linear(heads, self.w_o, None, residual, accumulate=True)
