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

    q = x W_q, k = x W_k, v = x W_v (each plus a bias with ``bias``), or, without ``v_name``, v = k as projected
    (before it is turned): such a layer has no value projection.  With ``head_norm`` every query head and every key
    head is first divided by its root mean square (eps inside the root) and multiplied by a gain of ``head_dim``
    numbers, one gain for all query heads and one for all key heads.  Queries and keys then turn by position
    (``rotary``: dims, base, interleaved);
    s = (q . k) * scale; with ``softcap`` c: s <- c * tanh(s / c); query i sees keys j <= i with
    i - j < ``window``, or, with ``chunk`` C instead, with j // C == i // C (runs of C positions counted from
    position 0 of the sequence, however the prompt was cut); neither: all earlier keys.  With ``sink_name`` every
    query head has a learned number whose exponential is added to the softmax's denominator and to nothing else;
    values may have a size of their own (``v_dim``); residual += o W_o.  Scores, softmax, norms, angles: float32.

    ``kv_source`` False: the layer has no key and value tensors (projections, biases, key gain); its run in the
    schedule names the cache layer of another layer, which has written that step's keys and values (after their
    norm and turning) before this one runs, and it brings only its own queries, mask and output projection.

    The projections run as one product over the stacked matrices; one kernel then norms and turns the queries in
    place and sends the keys and the values into the pages; attention reads only pages.  Where a layer with a value
    projection has key and value sizes that differ, or that are no multiple of 16 in bfloat16, a cached head takes
    ``slot_dim`` numbers, the larger of the two rounded up: the projections' matrices get zero rows there (zero keys add nothing to a score, zero values
    give zeros that the output projection's zero columns ignore), and every attention kernel runs unchanged.

    params: hidden_size, n_heads, n_kv_heads, head_dim, v_dim (head_dim), scale, window, chunk, softcap,
    rotary (dict or None), q_name, k_name, v_name (None: values are the unturned keys), out_name, sink_name (None: no
    sinks), bias (False; tensors ``<name>.b``), head_norm (None, or dict(q_name, k_name, eps)), kv_source (True),
    init_std, out_init_std.
    """

    graph_safe = True
    accepts_deferred_norm = True       # x goes straight into ops.linear

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = self.params
        if p["n_heads"] % p["n_kv_heads"] != 0:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        self.dim = p["head_dim"]
        self.v_dim = p.get("v_dim") or self.dim
        self.has_v = p.get("v_name") is not None
        self.kv_source = p.get("kv_source", True)
        self.head_norm = p.get("head_norm")
        if not self.has_v and self.v_dim != self.dim:
            raise ValueError("values that are the unturned keys have the keys' size")
        # what a head takes in the cache and in the attention kernels
        slot = max(self.dim, self.v_dim)
        if env.dtype == torch.bfloat16 and self.has_v:
            slot = -(-slot // 16) * 16                 # the tensor-core attention kernels take multiples of 16
        self.slot_dim = slot
        if not (0 < self.slot_dim <= 256):
            raise ValueError(f"head_dim {p['head_dim']} / v_dim {self.v_dim} is not supported: at most 256")
        if p.get("window") is not None and p["window"] <= 0:
            raise ValueError("window must be positive")
        if p.get("chunk") is not None and (p["chunk"] <= 0 or p.get("window") is not None):
            raise ValueError("chunk must be positive, and excludes a window")
        # the plain kernel turns heads as they are; norms, padded heads and borrowed keys take the other one
        self.plain = (self.head_norm is None and self.slot_dim == self.dim == self.v_dim and self.kv_source)
        if not self.plain and not self.has_v:
            raise ValueError("rotary_attention: head norms, padded heads and borrowed keys need a value projection")
        self.q_width = p["n_heads"] * self.slot_dim
        self.kv_width = p["n_kv_heads"] * self.slot_dim
        rotary = p.get("rotary") or dict(dims=0, base=10000.0)
        from pagedserve_b200.parts.positions import RotaryPositions

        self.rotary = RotaryPositions(dict(dims=rotary["dims"], base=rotary["base"],
                                           interleaved=rotary.get("interleaved", True), head_dim=p["head_dim"]),
                                      prefix, env)

    def cache_need(self):
        p = self.params
        return KVNeed(p["n_kv_heads"], self.slot_dim, p.get("window"), chunk=p.get("chunk"))

    def param_specs(self):
        p = self.params
        W, H, G = p["hidden_size"], p["n_heads"], p["n_kv_heads"]
        std = p.get("init_std", 0.02)
        names = [(p["q_name"], H * self.dim)]
        if self.kv_source:
            names.append((p["k_name"], G * self.dim))
            if self.has_v:
                names.append((p["v_name"], G * self.v_dim))
        specs = [(ParamSpec(self._n(name), (rows, W), "matmul"), ("normal", std)) for name, rows in names]
        if p.get("bias"):
            specs += [(ParamSpec(self._n(name + ".b"), (rows,), "vector"), ("normal", 0.3)) for name, rows in names]
        if self.head_norm:
            specs.append((ParamSpec(self._n(self.head_norm["q_name"]), (self.dim,), "vector"), ("ones_plus_normal", 0.1)))
            if self.kv_source:
                specs.append((ParamSpec(self._n(self.head_norm["k_name"]), (self.dim,), "vector"),
                              ("ones_plus_normal", 0.1)))
        specs.append((ParamSpec(self._n(p["out_name"]), (W, H * self.v_dim), "matmul"),
                      ("normal", p.get("out_init_std", std))))
        if p.get("sink_name"):
            specs.append((ParamSpec(self._n(p["sink_name"]), (H,), "vector"), ("normal", 1.0)))
        return specs

    def _padded_rows(self, tensor, heads, size):
        """[heads * size, ...] -> [heads * slot_dim, ...] with zero rows behind every head's own."""
        if size == self.slot_dim:
            return tensor
        shaped = tensor.reshape(heads, size, *tensor.shape[1:])
        out = shaped.new_zeros((heads, self.slot_dim) + tuple(tensor.shape[1:]))
        out[:, :size] = shaped
        return out.reshape(heads * self.slot_dim, *tensor.shape[1:])

    def bind(self, tensors):
        p = self.params
        H, G = p["n_heads"], p["n_kv_heads"]
        kinds = [(p["q_name"], H, self.dim)]
        if self.kv_source:
            kinds.append((p["k_name"], G, self.dim))
            if self.has_v:
                kinds.append((p["v_name"], G, self.v_dim))
        self.w_in = torch.cat([self._padded_rows(tensors[self._n(name)], heads, size) for name, heads, size in kinds],
                              dim=0).contiguous()                   # [q + k (+ v), W]
        self.b_in = None
        if p.get("bias"):
            self.b_in = torch.cat([self._padded_rows(tensors[self._n(name + ".b")], heads, size)
                                   for name, heads, size in kinds], dim=0).contiguous()
        w_out = tensors[self._n(p["out_name"])]
        if self.v_dim != self.slot_dim:                             # zero columns where the heads are padded
            w_out = self._padded_rows(w_out.t().contiguous(), H, self.v_dim).t().contiguous()
        self.w_out = w_out
        self.sink = tensors[self._n(p["sink_name"])].contiguous() if p.get("sink_name") else None
        self.q_gain = self.k_gain = None
        if self.head_norm:
            self.q_gain = tensors[self._n(self.head_norm["q_name"])].contiguous()
            if self.kv_source:
                self.k_gain = tensors[self._n(self.head_norm["k_name"])].contiguous()

    def forward(self, x, residual, ctx, layer):
        p = self.params
        ops = self.env.ops
        tokens = x.shape[0]
        H, G, D = p["n_heads"], p["n_kv_heads"], self.slot_dim
        projected = ops.empty((tokens, self.w_in.shape[0]), self.env.dtype, residual.device)
        ops.linear(x, self.w_in, self.b_in, projected)
        q = projected[:, :self.q_width]
        k = v = None
        if self.kv_source:
            k = projected[:, self.q_width:self.q_width + self.kv_width]
            v = projected[:, self.q_width + self.kv_width:] if self.has_v else None
        write_cache = p.get("write_cache", True) and self.kv_source
        if self.plain:
            self.rotary.turn_and_store(q, k, v, ctx, layer, H, G, write_cache=write_cache)
        else:
            rotary = self.rotary.params
            ops.head_norm_rotary_cache_write(
                q, k, v, self.q_gain, self.k_gain, float(self.head_norm["eps"]) if self.head_norm else 0.0,
                self.rotary.inv_freq_split(), rotary["dims"], rotary.get("interleaved", True), self.dim, ctx, layer,
                H, G, D, write_cache=write_cache)
        context = ops.empty((tokens, self.q_width), self.env.dtype, residual.device)
        ops.attention(q, k, v, context, ctx, layer, H, G, D, p.get("window"), float(p["scale"]), write_cache=False,
                      softcap=p.get("softcap"), sink=self.sink, chunk=p.get("chunk"))
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
