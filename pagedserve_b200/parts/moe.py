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
    sigmoid(w_sg . x), one number per token (``shared_gate`` False: the shared expert is added as it is).

    Other forms of the same part.  ``score`` "sigmoid": s = sigmoid(z), expert by expert, instead of the softmax;
    ``normalize`` False: the weights are the chosen s themselves.  ``expert_form`` dict(kind="clamped_swish", limit,
    alpha): an expert is W_down (g sigmoid(alpha g) (u + 1)) with g = min(W_gate x', limit), u = clamp(W_up x',
    -limit, limit), and its weight multiplies its input, x' = w x, not its output; the shared expert has a limit of
    its own (``shared_limit``).  There are no biases, so W (w x) = w (W x): the weight is applied to the two
    pre-activations in float32 by the kernel that forms the inner row, in both ways of running.

    How it runs.  The gate and up matrices of all experts (and of the shared one) are stacked into one matrix,
    expert by expert, and the down matrices stand side by side along their inner axis; the weight multiplies the
    inner activation in float32 before it is rounded.
    Few tokens (decode steps, short portions; and the float32 path): the router kernel leaves a dense weight per
    (token, expert), zero where the expert is not chosen, and the step is two products around one elementwise
    kernel: inner[t, c] = silu(gate) * up * weight[t, expert of c], then residual += inner W_down_all^T.  Every
    token passes through every expert's columns: the weights stream once, which is what bounds such a step.
    Many tokens in bfloat16: the (token, expert) pairs are sorted by expert into a buffer in which every expert's
    run starts on a tile of the tcgen05 product (``moe_plan``, ``moe_gather``); the two products read, per tile of
    rows, the matrix of that tile's expert (``linear_experts``); ``moe_combine`` adds each token's rows into the
    residual in the order of its election.  The shared expert runs as two plain products beside them.
    Either way a token's result does not depend on the other tokens of the step, and both ways compute the same
    sums up to their order.

    params: hidden_size, n_experts, expert_ff, top, groups, group_keep, shared_ff (None: no shared expert),
    score ("softmax"), normalize (True), expert_form (None: silu), shared_limit, shared_gate (True),
    correction_name (None; a float32 tensor of one number per expert that is added to the scores for the election
    only: the chosen experts' weights stay their scores),
    init_std, out_init_std; tensors ``router``, ``e<i>.gate / up / down``, ``shared.gate / up / down / sg``.
    """

    graph_safe = True
    accepts_deferred_norm = True       # an RMS norm in front is computed by the router's kernel

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
        if p.get("score", "softmax") not in ("softmax", "sigmoid"):
            raise ValueError("routed_experts: score is 'softmax' or 'sigmoid'")
        form = p.get("expert_form")
        self.form = None
        if form is not None and form.get("kind", "silu") != "silu":
            if form["kind"] != "clamped_swish" or not form["limit"] > 0:
                raise ValueError("routed_experts: expert_form is silu, or clamped_swish with a positive limit")
            self.form = ("clamped_swish", float(form["limit"]), float(p.get("shared_limit") or form["limit"]),
                         float(form.get("alpha", 1.702)))
        self.has_shared_gate = bool(p.get("shared_ff")) and p.get("shared_gate", True)

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
        if self.has_shared_gate:
            specs.append((ParamSpec(self._n("shared.sg"), (1, W), "matmul"), ("normal", std)))
        if p.get("correction_name"):
            specs.append((ParamSpec(self._n(p["correction_name"]), (p["n_experts"],), "vector"), ("normal", 0.1)))
        return specs

    def bind(self, tensors):
        t = lambda name: tensors[self._n(name)]
        names = self._expert_names()
        self.router = t("router").contiguous()
        self.w_gate_up = torch.cat([t(name + which) for name in names for which in ("gate", "up")],
                                   dim=0).contiguous()           # [2 * columns, W]: per expert its gates, then its ups
        self.w_down = torch.cat([t(name + "down") for name in names], dim=1).contiguous()      # [W, columns]
        self.w_shared_gate = t("shared.sg").reshape(-1).contiguous() if self.has_shared_gate else None
        name = self.params.get("correction_name")
        self.correction = t(name).contiguous() if name else None

    def forward(self, x, residual, ctx):
        p = self.params
        ops, dtype, device = self.env.ops, self.env.dtype, residual.device
        norm = None
        if hasattr(x, "materialize"):
            prologue = x.norm.fused_prologue() if hasattr(x.norm, "fused_prologue") else None
            if (prologue is not None and not prologue.has_mean and prologue.bias is None and x.rows is None
                    and x.x.dtype == torch.float32 and x.x.stride(1) == 1):
                # the router's kernel norms the rows on its way and leaves them for the products
                norm = (x.x, prologue.weight, prologue.eps)
                x = ops.empty(x.shape, dtype, device)
            else:
                x = x.materialize()
        tokens, E = x.shape[0], p["n_experts"]
        dense = ops.empty((tokens, E), torch.float32, device)
        chosen = ops.empty((tokens, p["top"]), torch.int32, device)
        chosen_w = ops.empty((tokens, p["top"]), torch.float32, device)
        shared_gate = ops.empty((tokens,), torch.float32, device) if self.w_shared_gate is not None else None
        ops.moe_route(x, self.router, self.w_shared_gate, dense, chosen, chosen_w, shared_gate, p["top"],
                      p.get("groups") or 0, p.get("group_keep") or 0, norm=norm, score=p.get("score", "softmax"),
                      normalize=p.get("normalize", True), correction=self.correction)
        F, width = p["expert_ff"], p["hidden_size"]
        if self._sorted_rows(tokens, x):
            self._forward_sorted(x, residual, dense, chosen, chosen_w, shared_gate)
            return
        gate_up = ops.empty((tokens, 2 * self.columns), dtype, device)
        ops.linear(x, self.w_gate_up, None, gate_up)
        inner = ops.empty((tokens, self.columns), dtype, device)
        ops.moe_gate_mul(gate_up, dense, shared_gate, inner, E, F, form=self.form)
        ops.linear(inner, self.w_down, None, residual, accumulate=True)

    SORTED_FROM = 128             # tokens of a step from which the rows are sorted by expert

    def _sorted_rows(self, tokens, x):
        """Whether this step sorts its rows by expert: a rule of shapes alone (the same step always takes the
        same path).  Below SORTED_FROM tokens the weights of all experts stream once whatever the election; where
        every expert is chosen there is nothing to save."""
        p = self.params
        return (self.env.dtype == torch.bfloat16 and tokens >= self.SORTED_FROM and p["top"] < p["n_experts"]
                and p["expert_ff"] % 8 == 0 and p["hidden_size"] % 8 == 0 and x.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0)

    def _forward_sorted(self, x, residual, dense, chosen, chosen_w, shared_gate):
        p = self.params
        ops, dtype, device = self.env.ops, self.env.dtype, residual.device
        tokens, E, top, F, width = x.shape[0], p["n_experts"], p["top"], p["expert_ff"], p["hidden_size"]
        rows_cap = ops.expert_rows(tokens, top, E)
        row_of = ops.empty((tokens * top,), torch.int32, device)
        row_token = ops.empty((rows_cap,), torch.int32, device)
        row_weight = ops.empty((rows_cap,), torch.float32, device)
        tile_expert = ops.empty((rows_cap // ops.EXPERT_TILE,), torch.int32, device)
        ops.moe_plan(chosen, chosen_w, E, row_of, row_token, row_weight, tile_expert)
        rows = ops.empty((rows_cap, width), dtype, device)
        ops.moe_gather(x, row_token, rows)
        gate_up = ops.empty((rows_cap, 2 * F), dtype, device)
        ops.linear_experts(rows, self.w_gate_up[:E * 2 * F], gate_up, tile_expert, E)
        inner = ops.empty((rows_cap, F), dtype, device)
        ops.moe_gate_mul_rows(gate_up, row_weight, inner, form=self.form)
        down = ops.empty((rows_cap, width), torch.float32, device)
        ops.linear_experts(inner, self.w_down[:, :E * F], down, tile_expert, E, along_k=True)
        ops.moe_combine(down, row_of, top, residual)
        shared_ff = p.get("shared_ff") or 0
        if shared_ff:
            gate_up_shared = ops.empty((tokens, 2 * shared_ff), dtype, device)
            ops.linear(x, self.w_gate_up[E * 2 * F:], None, gate_up_shared)
            inner_shared = ops.empty((tokens, shared_ff), dtype, device)
            ops.moe_gate_mul(gate_up_shared, dense, shared_gate, inner_shared, 0, shared_ff, form=self.form)
            ops.linear(inner_shared, self.w_down[:, E * F:], None, residual, accumulate=True)
