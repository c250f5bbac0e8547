"""Norm parts."""

from __future__ import annotations

import torch

from pagedserve_b200.parts.base import Norm, NormPrologue, register_part
from pagedserve_b200.weights.loader import ParamSpec


class DeferredNorm:
    """A norm that has been asked for but not computed: the consumer (a matrix product) may fold it
    into its own kernel, or call :meth:`materialize` to get the normed tensor."""

    def __init__(self, norm, x, rows=None):
        self.norm = norm
        self.x = x
        self.rows = rows
        count = rows.numel() if rows is not None else x.shape[0]
        self.shape = (count, x.shape[1])
        self.device = x.device

    def materialize(self, out=None):
        return self.norm.forward(self.x, out=out, rows=self.rows)


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    """y = (x - mean) / sqrt(var + eps) * weight + bias over the last axis, in float32.

    reference: nn.LayerNorm at src/model/paged_decoder.py:170-177, 291-294 and the
    fused kernel src/kernels/triton_residual_layernorm.py:25-40.
    params: width, eps, name, has_mean (False gives the RMS form), has_bias, init_std,
    weight_offset (a constant added to the stored weight once, in float32, when it is bound: 1.0 for
    gains that are stored as their distance from one; random weights are then drawn around zero).
    """

    graph_safe = True

    def param_specs(self):
        p = self.params
        centred = bool(p.get("weight_offset"))
        specs = [(ParamSpec(self._n(p["name"] + ".weight"), (p["width"],), "vector"),
                  ("normal" if centred else "ones_plus_normal", p.get("init_std", 0.0)))]
        if p.get("has_bias", True):
            specs.append((ParamSpec(self._n(p["name"] + ".bias"), (p["width"],), "vector"),
                          ("normal", p.get("init_std", 0.0))))
        return specs

    def bind(self, tensors):
        p = self.params
        self.weight = tensors[self._n(p["name"] + ".weight")]
        if p.get("weight_offset"):
            self.weight = self.weight + float(p["weight_offset"])        # float32: the "vector" role
        self.bias = tensors[self._n(p["name"] + ".bias")] if p.get("has_bias", True) else None

    def defer(self, x, rows=None):
        return DeferredNorm(self, x, rows)

    def fused_prologue(self):
        return NormPrologue(self.weight, self.bias, float(self.params["eps"]), bool(self.params.get("has_mean", True)))

    def forward(self, x, out=None, rows=None, out_dtype=None):
        n_rows = rows.numel() if rows is not None else x.shape[0]
        if out is None:
            out = self.env.ops.empty((n_rows, x.shape[1]), out_dtype or self.env.dtype, x.device)
        return self.env.ops.layernorm(x, self.weight, self.bias, float(self.params["eps"]), out, rows=rows,
                                      has_mean=self.params.get("has_mean", True))


@register_part("norm", "group_rms_norm")
class GroupRMSNorm(Norm):
    """The row is cut into ``groups`` equal consecutive runs; each run is divided by its own
    sqrt(mean(run^2) + eps); the whole is multiplied by a plain gain of the row's width.  One group is the plain RMS
    norm.  Statistics and products are float32; the input may be float32 rows (the residual stream) or rows of the
    compute type (a product's output).

    Besides ``forward`` it closes a sublayer of a layer that norms what the sublayer returns (``add_into``):
    x += norm(y), in one kernel with what the block wants done to x afterwards.
    params: width, eps, groups, name, init_std."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = self.params
        groups = p.get("groups", 1)
        if not (isinstance(groups, int) and 0 < groups <= 64) or p["width"] % groups:
            raise ValueError("group_rms_norm: between 1 and 64 groups that divide the width")
        self.groups = groups

    def param_specs(self):
        p = self.params
        return [(ParamSpec(self._n(p["name"] + ".weight"), (p["width"],), "vector"),
                 ("ones_plus_normal", p.get("init_std", 0.0)))]

    def bind(self, tensors):
        self.weight = tensors[self._n(self.params["name"] + ".weight")].contiguous()

    def forward(self, x, out=None, rows=None, out_dtype=None):
        n_rows = rows.numel() if rows is not None else x.shape[0]
        if out is None:
            out = self.env.ops.empty((n_rows, x.shape[1]), out_dtype or self.env.dtype, x.device)
        return self.env.ops.group_rms_norm(x, self.weight, float(self.params["eps"]), self.groups, out, rows=rows)

    def add_into(self, y, x, x_cast=None, history=None, n_history=0, weight=None):
        """x += norm(y); y = 0; then, with ``history``, entry ``n_history - 1`` = x and x = the weighted sum of the
        first ``n_history`` entries; ``x_cast`` receives x in the compute type."""
        self.env.ops.post_norm_add(y, x, self.weight, float(self.params["eps"]), self.groups, x_cast=x_cast,
                                   history=history, n_history=n_history, weight=weight)
