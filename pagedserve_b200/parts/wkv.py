"""A linear-recurrence mixer with per-channel, data-dependent decay and token shift."""

from __future__ import annotations

import torch

from pagedserve_b200.cache.manager import StateNeed
from pagedserve_b200.parts.base import Mixer, register_part
from pagedserve_b200.weights.loader import ParamSpec

MIXES = ("r", "k", "v", "g", "w")


@register_part("mixer", "wkv")
class WkvMixer(Mixer):
    """Time mixing with a matrix state per head instead of a cache of keys.

    With x' the input at the token before (zeros before a request's first token), each of r, k, v, g, w reads
    its own blend m_s = x + (x' - x) * mu_s.  r, k, v = W_r m_r, W_k m_k, W_v m_v (heads x d each),
    gate = silu(W_g m_g), and the decay of every head and key channel is
    w = exp(-exp(W_w2 tanh(W_w1 m_w) + w0)), a number in (0, 1).  Per head, with S a d x d matrix
    (key channel x value channel) that starts at zero:

        y_t = (S + diag(u) k_t v_t^T)^T r_t          (the bonus u weighs the current token only)
        S  <- diag(w_t) S + k_t v_t^T

    Each head's y is divided by its root mean square, the heads are joined, multiplied by a gain and by the
    gate, and W_o adds the result into the residual stream.

    A request keeps S (float32) and its newest input x in its slot, so a step runs only the tokens it brings:
    a prompt portion runs its tokens in order from the stored state, a decode step is a portion of one token.
    Decay, exponentials, state, the head norm and the gate's product are float32; r, k, v, the gate and the
    decay's argument leave their products as float32 too.

    Launches of a step: given an RMS norm not yet computed, one kernel norms the residual rows, makes the blends
    and the decay's argument (``wkv_prepare``); given normed rows, the blend kernel and two small products do.
    Then r, k, v and the gate as one grouped product where rows are few (four products otherwise), the
    recurrence, and the output projection.

    params: hidden_size, n_heads, head_dim, eps, decay_rank (inner size of W_w1 / W_w2; None: whatever the
    file holds), random_decay_rank (the size random weights are drawn with where decay_rank is None);
    the tensors are mu.r ... mu.w, r, k, v, g, w1, w2, w0, u, norm, o.
    """

    graph_safe = True
    accepts_deferred_norm = True       # an RMS norm in front is computed by the mixer's first kernel

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = self.params
        if not (0 < p["head_dim"] <= 128):
            raise ValueError(f"wkv: head_dim {p['head_dim']} is not supported: at most 128")
        self.width = p["hidden_size"]
        self.inner = p["n_heads"] * p["head_dim"]
        self.state_matrix = p["n_heads"] * p["head_dim"] * p["head_dim"]      # floats of S; x' follows

    def state_need(self):
        return StateNeed((self.state_matrix + self.width,), "float32")

    def param_specs(self):
        p = self.params
        W, inner, rank = self.width, self.inner, p.get("decay_rank")
        drawn = p.get("random_decay_rank", 16) if rank is None else rank
        rank = -1 if rank is None else rank
        std = p.get("init_std", 0.02)
        specs = [(ParamSpec(self._n("mu." + s), (W,), "vector"), ("normal", 0.3)) for s in MIXES]
        specs += [(ParamSpec(self._n(s), (inner, W), "matmul"), ("normal", std)) for s in ("r", "k", "v", "g")]
        specs += [(ParamSpec(self._n("w1"), (rank, W), "matmul"), ("normal", std, (drawn, W))),
                  (ParamSpec(self._n("w2"), (inner, rank), "matmul"), ("normal", 0.1, (inner, drawn))),
                  (ParamSpec(self._n("w0"), (inner,), "vector"), ("normal", 1.0)),
                  (ParamSpec(self._n("u"), (p["n_heads"], p["head_dim"]), "vector"), ("normal", 0.3)),
                  (ParamSpec(self._n("norm"), (inner,), "vector"), ("ones_plus_normal", 0.1)),
                  (ParamSpec(self._n("o"), (W, inner), "matmul"), ("normal", p.get("out_init_std", std)))]
        return specs

    def bind(self, tensors):
        t = lambda name: tensors[self._n(name)]
        self.mu = torch.stack([t("mu." + s) for s in MIXES]).contiguous()          # float32 [5, W]
        self.w_rkvg = torch.cat([t("r"), t("k"), t("v"), t("g")], dim=0).contiguous()      # [4 * inner, W]
        self.w1, self.w2, self.w0 = t("w1"), t("w2"), t("w0")
        if self.w1.shape[0] != self.w2.shape[1]:
            raise ValueError("wkv: the two matrices of the decay do not fit each other")
        self.u = t("u").reshape(-1).contiguous()
        self.gain = t("norm")
        self.w_o = t("o")

    def forward(self, x, residual, ctx, layer):
        p = self.params
        ops, dtype, device = self.env.ops, self.env.dtype, residual.device
        tokens = x.shape[0]
        state = layer.state
        blends = ops.empty((len(MIXES), tokens, self.width), dtype, device)
        # r, k, v, gate, decay argument: float32 rows of one buffer
        streams = ops.empty((5, tokens, self.inner), torch.float32, device)
        prologue = x.norm.fused_prologue() if hasattr(x, "materialize") and hasattr(x.norm, "fused_prologue") else None
        if prologue is not None and not prologue.has_mean and prologue.bias is None and x.rows is None:
            # the norm, the blends and the decay's small products in one launch; block 4 of `blends` holds the
            # normed rows, of which the recurrence keeps each entry's newest
            ops.wkv_prepare(x.x, prologue.weight, prologue.eps, self.mu, state, self.state_matrix, ctx, self.w1,
                            self.w2, self.w0, blends, streams[4])
            x = blends[4]
        else:
            if hasattr(x, "materialize"):
                x = x.materialize()
            ops.token_shift_mix(x, self.mu, state, self.state_matrix, ctx, blends)
            low = ops.empty((tokens, self.w1.shape[0]), dtype, device)
            ops.linear(blends[4], self.w1, None, low, act="tanh")
            ops.linear(low, self.w2, self.w0, streams[4])
        # four products of equal shape, each on its own blend; the last one is the gate
        ops.linear_grouped(blends[:4], self.w_rkvg, streams[:4], act="silu", act_from_group=3)
        mixed = ops.empty((tokens, self.inner), dtype, device)
        ops.wkv_recurrence(streams[0], streams[1], streams[2], streams[4], streams[3], self.u, self.gain,
                           float(p["eps"]), x, state, self.state_matrix, ctx, mixed, p["n_heads"], p["head_dim"])
        ops.linear(mixed, self.w_o, None, residual, accumulate=True)
