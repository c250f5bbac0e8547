"""A gated recurrence whose gates read only the current token."""

from __future__ import annotations

import torch

from pagedserve_b200.cache.manager import StateNeed
from pagedserve_b200.parts.base import Mixer, register_part
from pagedserve_b200.weights.loader import ParamSpec


@register_part("mixer", "mingru")
class MinGRUMixer(Mixer):
    """minGRU: z = sigmoid(W_z x + b_z), u = W_x x + b_x (both ``width`` numbers); the candidate is u + 1/2 where
    u >= 0 and sigmoid(u) where u < 0; element by element

        S_t = (1 - z_t) S_(t-1) + z_t * candidate_t,        S = 0 before a sequence's first token

    and residual += W_o (S_t * silu(W_g x)).  Neither gate reads S, so the recurrence is linear in S and a prompt
    portion is folded in segments side by side (csrc/mingru.cu).

    A request keeps S (float32, ``width`` numbers) in its slot, so a step runs only the tokens it brings: a prompt
    portion runs its tokens in order from the stored state, a decode step is a portion of one token.  The three
    projections are one product with float32 output; gates, candidate, state and the output gate are float32.

    params: hidden_size, width, init_std, out_init_std; tensors z, z.b, x, x.b, g, o.
    """

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        if not (isinstance(self.params["width"], int) and self.params["width"] > 0):
            raise ValueError("mingru: width must be a positive integer")
        self.inner = self.params["width"]

    def state_need(self):
        return StateNeed((self.inner,), "float32")

    def param_specs(self):
        p = self.params
        W, inner, std = p["hidden_size"], self.inner, p.get("init_std", 0.02)
        return [(ParamSpec(self._n("z"), (inner, W), "matmul"), ("normal", std)),
                (ParamSpec(self._n("z.b"), (inner,), "vector"), ("normal", 1.0)),
                (ParamSpec(self._n("x"), (inner, W), "matmul"), ("normal", std)),
                (ParamSpec(self._n("x.b"), (inner,), "vector"), ("normal", 0.5)),
                (ParamSpec(self._n("g"), (inner, W), "matmul"), ("normal", std)),
                (ParamSpec(self._n("o"), (W, inner), "matmul"), ("normal", p.get("out_init_std", std)))]

    def bind(self, tensors):
        t = lambda name: tensors[self._n(name)]
        self.w_in = torch.cat([t("z"), t("x"), t("g")], dim=0).contiguous()             # [3 * inner, W]
        self.b_in = torch.cat([t("z.b"), t("x.b"), torch.zeros_like(t("z.b"))]).contiguous()
        self.w_o = t("o")

    def forward(self, x, residual, ctx, layer):
        ops, device = self.env.ops, residual.device
        if hasattr(x, "materialize"):
            x = x.materialize()
        tokens = x.shape[0]
        projected = ops.empty((tokens, 3 * self.inner), torch.float32, device)
        ops.linear(x, self.w_in, self.b_in, projected)
        mixed = ops.empty((tokens, self.inner), self.env.dtype, device)
        ops.mingru_scan(projected, self.inner, layer.state, ctx, mixed)
        ops.linear(mixed, self.w_o, None, residual, accumulate=True)
