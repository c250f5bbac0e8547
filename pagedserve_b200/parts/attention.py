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

    ``conv`` = dict(taps, suffix): directly behind the projections (biases included) every channel of q, k and v
    passes a short causal convolution over time, y_t = sum_j w[:, j] u_(t - taps + 1 + j) with zeros before the
    sequence's start (tensors ``<projection><suffix>`` [channels, taps]); a request keeps its last taps - 1 projected
    rows in its slot, so a step runs only the tokens it brings.  ``rotary.scaling`` stretches the rotation
    (:class:`RotaryPositions`).  ``value_mix`` = dict(name, role, key): a layer of role "first" leaves its values (as
    convolved, float32) in the step's shared rows ``key``; a layer of role "later" caches v <- (1 - m) v + m * those
    rows of the same token, m its scalar tensor ``name`` (which a "first" layer also stores and does not use).
    ``gate_name``: the joined heads are multiplied by sigmoid(x W_g), number by number, before W_o.
    With a convolution or a gate the stacked product leaves float32 rows, and one kernel convolves, blends the
    values, passes the gate's columns through and rounds to the compute type.

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
    conv (None), value_mix (None), gate_name (None), init_std, out_init_std.
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
        rotary = p.get("rotary") or dict(dims=0, base=10000.0)
        # the plain kernel turns heads as they are; norms, padded heads, borrowed keys and stretched rotations take
        # the other one
        self.plain = (self.head_norm is None and self.slot_dim == self.dim == self.v_dim and self.kv_source
                      and not rotary.get("scaling"))
        if not self.plain and not self.has_v:
            raise ValueError("rotary_attention: head norms, padded heads and borrowed keys need a value projection")
        self.q_width = p["n_heads"] * self.slot_dim
        self.kv_width = p["n_kv_heads"] * self.slot_dim
        from pagedserve_b200.parts.positions import RotaryPositions

        self.rotary = RotaryPositions(dict(dims=rotary["dims"], base=rotary["base"],
                                           interleaved=rotary.get("interleaved", True), head_dim=p["head_dim"],
                                           scaling=rotary.get("scaling")), prefix, env)
        self.conv = p.get("conv")
        self.value_mix = p.get("value_mix")
        self.gate_name = p.get("gate_name")
        if self.conv is not None:
            taps = self.conv.get("taps")
            if not (isinstance(taps, int) and 1 <= taps <= 16):
                raise ValueError("rotary_attention: a convolution has 1 to 16 taps")
        if (self.conv is not None or self.value_mix) and not (self.kv_source and self.has_v):
            raise ValueError("rotary_attention: a convolution or mixed values need key and value projections")
        if self.value_mix and self.value_mix.get("role") not in ("first", "later"):
            raise ValueError("rotary_attention: value_mix.role is 'first' or 'later'")
        # the channels that are convolved (q, k, v as laid out in the stacked product); a gate's columns follow
        self.conv_channels = self.q_width + 2 * self.kv_width if self.conv is not None else 0
        self.staged = self.conv is not None or self.value_mix is not None or self.gate_name is not None

    def cache_need(self):
        p = self.params
        return KVNeed(p["n_kv_heads"], self.slot_dim, p.get("window"), chunk=p.get("chunk"))

    def state_need(self):
        if self.conv is None or self.conv["taps"] < 2:
            return None
        from pagedserve_b200.cache.manager import StateNeed

        return StateNeed(((self.conv["taps"] - 1) * self.conv_channels,), "float32")

    def step_shared(self):
        """Rows that live for the whole step and that several layers touch: key -> (numbers per token, dtype)."""
        if self.value_mix and self.value_mix["role"] == "first":
            return {self.value_mix["key"]: (self.params["n_kv_heads"] * self.v_dim, torch.float32)}
        return {}

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
        if self.conv is not None:
            taps = self.conv["taps"]
            specs += [(ParamSpec(self._n(name + self.conv.get("suffix", ".conv")), (rows, taps), "vector"),
                       ("normal", taps ** -0.5)) for name, rows in names]
        if self.value_mix:
            specs.append((ParamSpec(self._n(self.value_mix["name"]), (), "vector"), ("normal", 0.3)))
        if self.gate_name:
            specs.append((ParamSpec(self._n(self.gate_name), (H * self.v_dim, W), "matmul"), ("normal", std)))
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
        stacked = [self._padded_rows(tensors[self._n(name)], heads, size) for name, heads, size in kinds]
        if self.gate_name:                                          # the gate's rows ride behind, laid out like the heads
            stacked.append(self._padded_rows(tensors[self._n(self.gate_name)], H, self.v_dim))
        self.w_in = torch.cat(stacked, dim=0).contiguous()          # [q + k (+ v) (+ gate), W]
        self.b_in = None
        if p.get("bias"):
            biases = [self._padded_rows(tensors[self._n(name + ".b")], heads, size) for name, heads, size in kinds]
            if self.gate_name:
                biases.append(biases[0].new_zeros(H * self.slot_dim))
            self.b_in = torch.cat(biases, dim=0).contiguous()
        self.conv_weight = None
        if self.conv is not None:
            suffix = self.conv.get("suffix", ".conv")
            self.conv_weight = torch.cat([self._padded_rows(tensors[self._n(name + suffix)], heads, size)
                                          for name, heads, size in kinds], dim=0).contiguous()      # [channels, taps]
        self.mix = tensors[self._n(self.value_mix["name"])].reshape(1).contiguous() if self.value_mix else None
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
        gate = None
        if self.staged:
            # float32 rows out of the product; one kernel convolves q, k and v over time from the request's kept
            # rows, blends the values, passes the gate through and rounds to the compute type
            raw = ops.empty((tokens, self.w_in.shape[0]), torch.float32, residual.device)
            ops.linear(x, self.w_in, self.b_in, raw)
            projected = ops.empty(raw.shape, self.env.dtype, residual.device)
            blend = None
            if self.value_mix:
                shared = getattr(ctx, "shared", {}).get(self.value_mix["key"])
                if shared is None or shared.shape[1] != G * self.v_dim:
                    raise ValueError("rotary_attention: the layers that mix values do not have values of one size")
                blend = ("store" if self.value_mix["role"] == "first" else "mix", self.q_width + self.kv_width, G, D,
                         self.v_dim, shared, self.mix)
            taps = self.conv["taps"] if self.conv is not None else 1
            channels = self.conv_channels or (self.q_width + 2 * self.kv_width if blend else 0)
            weight = self.conv_weight
            if weight is None and channels:                       # values are mixed without a convolution: one tap of 1
                if getattr(self, "_unit_tap", None) is None:
                    self._unit_tap = torch.ones((channels, 1), dtype=torch.float32, device=residual.device)
                weight = self._unit_tap
            ops.short_conv(raw, weight, taps, channels, layer.state, ctx, projected, blend=blend)
            if self.gate_name:
                gate = projected[:, self.q_width + 2 * self.kv_width:]
        else:
            projected = ops.empty((tokens, self.w_in.shape[0]), self.env.dtype, residual.device)
            ops.linear(x, self.w_in, self.b_in, projected)
        q = projected[:, :self.q_width]
        k = v = None
        if self.kv_source:
            k = projected[:, self.q_width:self.q_width + self.kv_width]
            v = projected[:, self.q_width + self.kv_width:self.q_width + 2 * self.kv_width] if self.has_v else None
        write_cache = p.get("write_cache", True) and self.kv_source
        if self.plain:
            self.rotary.turn_and_store(q, k, v, ctx, layer, H, G, write_cache=write_cache)
        else:
            rotary = self.rotary.params
            ops.head_norm_rotary_cache_write(
                q, k, v, self.q_gain, self.k_gain, float(self.head_norm["eps"]) if self.head_norm else 0.0,
                self.rotary.inv_freq_split(), rotary["dims"], rotary.get("interleaved", True), self.dim, ctx, layer,
                H, G, D, write_cache=write_cache, amplitude=self.rotary.amplitude)
        context = ops.empty((tokens, self.q_width), self.env.dtype, residual.device)
        ops.attention(q, k, v, context, ctx, layer, H, G, D, p.get("window"), float(p["scale"]), write_cache=False,
                      softcap=p.get("softcap"), sink=self.sink, chunk=p.get("chunk"))
        if gate is not None:
            ops.sigmoid_gate(context, gate)
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

    With ``q_rank`` the queries go through a latent of their own: c_q = x W_dq divided by its root mean square and
    multiplied by a gain (tensors ``dq``, ``dq.norm``), q = c_q W_uq (``uq``), instead of the one matrix ``q``.
    ``gate`` "head": W_g has one row per head and head h's result is multiplied by sigmoid(x W_g)_h ("element", the
    default: a row per number of the joined heads).

    Launches: the stacked projection (q or c_q | down | gate), with ``q_rank`` the norm of c_q and the product with
    W_uq, ``latent_prepare`` (norm of c, turns, cache write), the per-head products with W_uk^T, attention, the
    per-head products with W_uv, the gate, the output product.  Norm statistics, angles, scores and softmax are
    float32.

    params: hidden_size, n_heads, flat_dim, rot_dim, v_dim, kv_rank, q_rank (None), gate ("element"), scale, window,
    eps, rotary (dims, base), init_std, out_init_std; tensors q (or dq, dq.norm, uq), dkv, dkv.norm, uk, uv, g, o.
    """

    graph_safe = True
    accepts_deferred_norm = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = self.params
        self.row = p["kv_rank"] + p["rot_dim"]                    # the cached row, and the attention head size
        if not (0 < self.row <= 1024):         # (above 256 the CUDA-core attention kernel runs in bfloat16 too)
            raise ValueError(f"latent_attention: kv_rank + rot_dim = {self.row} is not supported: at most 1024")
        if p.get("window") is not None and p["window"] <= 0:
            raise ValueError("window must be positive")
        rotary = p.get("rotary") or dict(dims=0, base=10000.0)
        if rotary["dims"] < 0 or rotary["dims"] % 2 or rotary["dims"] > p["rot_dim"]:
            raise ValueError("latent_attention: rotary dims must be even and at most rot_dim")
        self.q_width = p["n_heads"] * (p["flat_dim"] + p["rot_dim"])
        self.v_width = p["n_heads"] * p["v_dim"]
        self.q_rank = p.get("q_rank")
        if self.q_rank is not None and not (isinstance(self.q_rank, int) and self.q_rank > 0):
            raise ValueError("latent_attention: q_rank must be a positive integer")
        if p.get("gate", "element") not in ("element", "head"):
            raise ValueError("latent_attention: gate is 'element' or 'head'")
        self.gate_width = p["n_heads"] if p.get("gate", "element") == "head" else self.v_width
        from pagedserve_b200.parts.positions import RotaryPositions

        self.rotary = RotaryPositions(dict(dims=rotary["dims"], base=rotary["base"], interleaved=True,
                                           head_dim=max(p["rot_dim"], 1)), prefix, env)

    def cache_need(self):
        return KVNeed(1, self.row, self.params.get("window"), planes=1)

    def param_specs(self):
        p = self.params
        W, H, R = p["hidden_size"], p["n_heads"], p["kv_rank"]
        std = p.get("init_std", 0.02)
        if self.q_rank is None:
            queries = [(ParamSpec(self._n("q"), (self.q_width, W), "matmul"), ("normal", std))]
        else:
            queries = [(ParamSpec(self._n("dq"), (self.q_rank, W), "matmul"), ("normal", std)),
                       (ParamSpec(self._n("dq.norm"), (self.q_rank,), "vector"), ("ones_plus_normal", 0.1)),
                       (ParamSpec(self._n("uq"), (self.q_width, self.q_rank), "matmul"), ("normal", self.q_rank ** -0.5))]
        return queries + [
                (ParamSpec(self._n("dkv"), (self.row, W), "matmul"), ("normal", std)),
                (ParamSpec(self._n("dkv.norm"), (R,), "vector"), ("ones_plus_normal", 0.1)),
                (ParamSpec(self._n("uk"), (H * p["flat_dim"], R), "matmul"), ("normal", R ** -0.5)),
                (ParamSpec(self._n("uv"), (self.v_width, R), "matmul"), ("normal", R ** -0.5)),
                (ParamSpec(self._n("g"), (self.gate_width, W), "matmul"), ("normal", std)),
                (ParamSpec(self._n("o"), (W, self.v_width), "matmul"), ("normal", p.get("out_init_std", std)))]

    def bind(self, tensors):
        p = self.params
        t = lambda name: tensors[self._n(name)]
        H, d, R = p["n_heads"], p["flat_dim"], p["kv_rank"]
        first = t("q") if self.q_rank is None else t("dq")
        self.w_in = torch.cat([first, t("dkv"), t("g")], dim=0).contiguous()            # [q or c_q | down | gate, W]
        self.first_width = first.shape[0]
        self.q_gain = self.w_uq = None
        if self.q_rank is not None:
            self.q_gain = t("dq.norm").contiguous()
            self.w_uq = t("uq").contiguous()
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
        q = projected[:, :self.first_width]
        down = projected[:, self.first_width:self.first_width + self.row]
        gate = projected[:, self.first_width + self.row:]
        if self.q_rank is not None:
            latent = ops.empty((tokens, self.q_rank), dtype, device)
            ops.group_rms_norm(q, self.q_gain, float(p["eps"]), 1, latent)
            q = ops.empty((tokens, self.q_width), dtype, device)
            ops.linear(latent, self.w_uq, None, q)
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
        ops.sigmoid_gate(heads, gate, span=self.v_width // self.gate_width)
        ops.linear(heads, self.w_o, None, residual, accumulate=True)
