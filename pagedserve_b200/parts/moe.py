"""A feed-forward of routed experts."""

from __future__ import annotations

import torch

from pagedserve_b200.parts.base import FeedForward, register_part
from pagedserve_b200.weights.loader import ParamSpec


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    """residual += sum over the chosen experts e of weight_e * expert_e(x)  (+ gate * shared(x)).

    An expert is W_down (silu(W_gate x) * (W_up x)), without biases.  The router: z = W_router x, s = softmax(z)
    over all E experts, in float32; the experts stand in ``groups`` runs of E / groups neighbours, a group's mark
    is its largest s, and only experts of the ``group_keep`` groups with the largest marks can be chosen (no
    groups: all can); the ``top`` largest s among them are chosen and their weights are s over the sum of the
    chosen s (+ 1e-20).  A shared expert of the same form (its own inner size) runs for every token, multiplied by
    sigmoid(w_sg . x), one number per token.

    How it runs: the router kernel leaves a dense weight per (token, expert), zero where the expert is not
    chosen.  The gate and up matrices of all experts (and of the shared one) are stacked into one matrix, as are
    the down matrices along their inner axis, so a step is two products around one elementwise kernel:
    inner[t, c] = silu(gate) * up * weight[t, expert of c], then residual += inner W_down_all^T.  Every token
    passes through every expert's columns, with a zero weight where it was not sent there; what a token gets does
    not depend on the other tokens of the step.  The weight multiplies the inner activation in float32 before it
    is rounded, so the down product sums the weighted experts in its float32 accumulator.

    params: hidden_size, n_experts, expert_ff, top, groups, group_keep, shared_ff (None: no shared expert),
    init_std, out_init_std; tensors ``router``, ``e<i>.gate / up / down``, ``shared.gate / up / down / sg``.
    """

    graph_safe = True
    accepts_deferred_norm = False

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = self.params
        E, top = p["n_experts"], p["top"]
        if not (0 < top <= E <= 256):
            raise ValueError("routed_experts: 0 < top <= n_experts <= 256")
        groups = p.get("groups") or 0
        if groups > 1 and (E % groups or not (0 < (p.get("group_keep") or 0) <= groups)):
            raise ValueError("routed_experts: groups must divide the experts, and 0 < group_keep <= groups")
        self.columns = E * p["expert_ff"] + (p.get("shared_ff") or 0)

    def _expert_names(self):
        names = [f"e{index}." for index in range(self.params["n_experts"])]
        return names + ["shared."] if self.params.get("shared_ff") else names

    def param_specs(self):
        p = self.params
        W = p["hidden_size"]
        std, out_std = p.get("init_std", 0.02), p.get("out_init_std", 0.02)
        specs = [(ParamSpec(self._n("router"), (p["n_experts"], W), "matmul"), ("normal", 4.0 * std))]
        for name in self._expert_names():
            F = p["shared_ff"] if name == "shared." else p["expert_ff"]
            specs += [(ParamSpec(self._n(name + "gate"), (F, W), "matmul"), ("normal", std)),
                      (ParamSpec(self._n(name + "up"), (F, W), "matmul"), ("normal", std)),
                      (ParamSpec(self._n(name + "down"), (W, F), "matmul"), ("normal", out_std))]
        if p.get("shared_ff"):
            specs.append((ParamSpec(self._n("shared.sg"), (1, W), "matmul"), ("normal", std)))
        return specs

    def bind(self, tensors):
        t = lambda name: tensors[self._n(name)]
        names = self._expert_names()
        self.router = t("router").contiguous()
        self.w_gate_up = torch.cat([t(name + "gate") for name in names] + [t(name + "up") for name in names],
                                   dim=0).contiguous()                                  # [2 * columns, W]
        self.w_down = torch.cat([t(name + "down") for name in names], dim=1).contiguous()      # [W, columns]
        self.w_shared_gate = t("shared.sg").reshape(-1).contiguous() if self.params.get("shared_ff") else None

    def forward(self, x, residual, ctx):
        p = self.params
        ops, dtype, device = self.env.ops, self.env.dtype, residual.device
        if hasattr(x, "materialize"):
            x = x.materialize()
        tokens, E = x.shape[0], p["n_experts"]
        dense = ops.empty((tokens, E), torch.float32, device)
        chosen = ops.empty((tokens, p["top"]), torch.int32, device)
        chosen_w = ops.empty((tokens, p["top"]), torch.float32, device)
        shared_gate = ops.empty((tokens,), torch.float32, device) if self.w_shared_gate is not None else None
        ops.moe_route(x, self.router, self.w_shared_gate, dense, chosen, chosen_w, shared_gate, p["top"],
                      p.get("groups") or 0, p.get("group_keep") or 0)
        gate_up = ops.empty((tokens, 2 * self.columns), dtype, device)
        ops.linear(x, self.w_gate_up, None, gate_up)
        inner = ops.empty((tokens, self.columns), dtype, device)
        ops.moe_gate_mul(gate_up, dense, shared_gate, inner, E, p["expert_ff"])
        ops.linear(inner, self.w_down, None, residual, accumulate=True)
