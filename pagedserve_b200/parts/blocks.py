"""Arrangements of norms, mixer and feed-forward inside a layer."""

from __future__ import annotations

import torch

from pagedserve_b200.parts.base import Block, register_part
from pagedserve_b200.weights.loader import ParamSpec


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    """h += mixer(norm(h)); h += feed_forward(norm(h))
    (reference: src/model/paged_decoder.py:181-189, 210-228).  The residual stream ``h``
    is float32 and is updated in place; the adds happen in the epilogues of the
    mixer's and the feed-forward's last matrix products.  A layer whose feed-forward is the ``none`` part has
    the first sublayer only, and no second norm."""

    graph_safe = True

    @property
    def required_norms(self):
        if getattr(self.feed_forward, "is_empty", False):
            return ("pre_mixer",)
        return ("pre_mixer", "pre_feed_forward")

    @staticmethod
    def _normed(norm, consumer, hidden):
        # a consumer whose first operation is a matrix product may take the norm unevaluated
        if getattr(consumer, "accepts_deferred_norm", False) and hasattr(norm, "defer"):
            return norm.defer(hidden)
        return norm.forward(hidden)

    def forward(self, hidden, ctx, layer):
        self.mixer.forward(self._normed(self.norms["pre_mixer"], self.mixer, hidden), hidden, ctx, layer)
        if getattr(self.feed_forward, "is_empty", False):
            return
        self.feed_forward.forward(self._normed(self.norms["pre_feed_forward"], self.feed_forward, hidden),
                                  hidden, ctx)


class StreamCarrier:
    """What runs through the layers of a model with several residual streams: the streams ``[S, T, W]``, the
    row ``u`` that the open sublayer reads, the row ``y`` it adds its result into, and the (mix, out) weights of
    a sublayer that has run but whose update of the streams is still to be done."""

    def __init__(self, streams, u, y):
        self.streams = streams
        self.u = u
        self.y = y
        self.pending = None


@register_part("block", "hyper_pre_norm")
class HyperPreNormBlock(Block):
    """A pre-norm layer over S residual streams x_1 .. x_S instead of one (all equal to the embedded rows at the
    start, summed at the end).  For each sublayer f (the mixer, then the feed-forward if the layer has one) with
    its own weights in[S], out[S], mix[S, S]:

        u = sum_s in[s] x_s;   y = f(norm(u));   x_t <- sum_s mix[s, t] x_s + out[t] y   (all t from the old x)

    Everything is float32.  The update of one sublayer and the read of the next are one pass over the streams
    (``ops.hyper_step``): a sublayer leaves its update pending and whatever comes next (the feed-forward, the
    next layer, the end of the model) does it together with its own read.  The sublayer adds its result into a
    zeroed row, exactly as it would into the residual row of a plain layer, so every mixer and feed-forward
    works here unchanged.

    params: streams, names (a dict: mixer -> prefix of its three tensors, feed_forward -> likewise), init_std;
    tensors are ``<prefix>.in``, ``<prefix>.out``, ``<prefix>.mix``."""

    graph_safe = True

    def _sublayers(self):
        names = self.params["names"]
        if getattr(self.feed_forward, "is_empty", False):
            return [names["mixer"]]
        return [names["mixer"], names["feed_forward"]]

    @property
    def required_norms(self):
        if getattr(self.feed_forward, "is_empty", False):
            return ("pre_mixer",)
        return ("pre_mixer", "pre_feed_forward")

    def param_specs(self):
        S = self.params["streams"]
        if not (isinstance(S, int) and 0 < S <= 8):
            raise ValueError("hyper_pre_norm: between 1 and 8 streams")
        std = self.params.get("init_std", 0.1)
        specs = []
        for name in self._sublayers():
            specs += [(ParamSpec(self._n(name + ".in"), (S,), "vector"), ("ones_plus_normal", std)),
                      (ParamSpec(self._n(name + ".out"), (S,), "vector"), ("ones_plus_normal", std)),
                      (ParamSpec(self._n(name + ".mix"), (S, S), "vector"), ("eye_plus_normal", std))]
        return specs

    def bind(self, tensors):
        self.weights = [tuple(tensors[self._n(f"{name}.{which}")].contiguous() for which in ("in", "out", "mix"))
                        for name in self._sublayers()]

    def begin(self, hidden, ctx):
        ops, S = self.env.ops, self.params["streams"]
        streams = ops.empty((S,) + tuple(hidden.shape), torch.float32, hidden.device)
        u = ops.empty(hidden.shape, torch.float32, hidden.device)
        y = ops.empty(hidden.shape, torch.float32, hidden.device)
        ops.hyper_begin(hidden, self.weights[0][0], streams, u, y)
        return StreamCarrier(streams, u, y)

    def _open(self, carrier, w_in):
        """Make ``carrier.u`` the input of the sublayer whose read weights are ``w_in`` (None: the plain sum)."""
        if carrier.pending is None:
            return                                 # ``begin`` of this very block has done it
        w_out, mix = carrier.pending
        self.env.ops.hyper_step(carrier.streams, carrier.y, mix, w_out, w_in, carrier.u)
        carrier.pending = None

    @staticmethod
    def _normed(norm, consumer, rows):
        if getattr(consumer, "accepts_deferred_norm", False) and hasattr(norm, "defer"):
            return norm.defer(rows)
        return norm.forward(rows)

    def forward(self, hidden, ctx, layer):
        carrier = hidden
        w_in, w_out, mix = self.weights[0]
        self._open(carrier, w_in)
        self.mixer.forward(self._normed(self.norms["pre_mixer"], self.mixer, carrier.u), carrier.y, ctx, layer)
        carrier.pending = (w_out, mix)
        if len(self.weights) > 1:
            w_in, w_out, mix = self.weights[1]
            self._open(carrier, w_in)
            self.feed_forward.forward(self._normed(self.norms["pre_feed_forward"], self.feed_forward, carrier.u),
                                      carrier.y, ctx)
            carrier.pending = (w_out, mix)

    def end(self, carrier, ctx):
        self._open(carrier, None)
        return carrier.u


class ResidualCarrier:
    """What runs through the layers of a model that norms its sublayers' results: the float32 rows ``x``, the same
    rows in the compute type (``x_cast``: what the sublayers' products read; ``x`` itself in a float32 engine), the
    zeroed float32 rows ``y`` a sublayer adds its result into, and, where the layers end with an average over
    depth, ``history`` [entries, T, W]: the embedded rows and every layer's result so far."""

    def __init__(self, x, x_cast, y, history):
        self.x = x
        self.x_cast = x_cast
        self.y = y
        self.history = history


@register_part("block", "post_norm")
class PostNormBlock(Block):
    """x <- x + norm(mixer(x)); x <- x + norm(feed_forward(x)): the sublayers read the rows themselves and the norm
    (``post_mixer``, ``post_feed_forward``: :class:`GroupRMSNorm`) is applied to what they return.  The residual rows
    and the sums are float32.  A layer whose feed-forward is the ``none`` part has the first half only.

    ``depth`` = dict(index, name, entries): the layer ends with an average over depth.  With X_0 the embedded rows and
    X_(i+1) this layer's result (``index`` = i), what goes on to the next layer (and, behind the last, to the
    model's norm) is sum_(j <= i+1) w[j] X_j with w the tensor ``name`` of i + 2 numbers; ``entries`` is the number
    of layer runs of the model plus one (the rows the history holds).

    A sublayer adds its result into a zeroed row exactly as it would into the residual row of a pre-norm layer, so
    every mixer and feed-forward works here unchanged; one kernel then norms that row, adds it, clears it, stores and
    averages over depth where the layer ends, and leaves the new rows in the compute type for the next product."""

    graph_safe = True

    @property
    def required_norms(self):
        if getattr(self.feed_forward, "is_empty", False):
            return ("post_mixer",)
        return ("post_mixer", "post_feed_forward")

    def param_specs(self):
        depth = self.params.get("depth")
        if not depth:
            return []
        if not (0 <= depth["index"] < depth["entries"] - 1):
            raise ValueError("post_norm: a layer's index lies below the number of history entries")
        return [(ParamSpec(self._n(depth["name"]), (depth["index"] + 2,), "vector"),
                 ("share_plus_normal", depth.get("init_std", 0.2)))]

    def bind(self, tensors):
        depth = self.params.get("depth")
        self.depth_weight = tensors[self._n(depth["name"])].contiguous() if depth else None

    def begin(self, hidden, ctx):
        ops, depth = self.env.ops, self.params.get("depth")
        history = ops.empty((depth["entries"],) + tuple(hidden.shape), torch.float32, hidden.device) if depth else None
        x_cast = hidden if self.env.dtype == torch.float32 else ops.empty(hidden.shape, self.env.dtype, hidden.device)
        y = ops.empty(hidden.shape, torch.float32, hidden.device)
        ops.depth_begin(hidden, history[0] if depth else None, None if x_cast is hidden else x_cast, y)
        return ResidualCarrier(hidden, x_cast, y, history)

    def _close(self, carrier, norm, ends_layer):
        depth = self.params.get("depth") if ends_layer else None
        x_cast = None if carrier.x_cast is carrier.x else carrier.x_cast
        if depth:
            norm.add_into(carrier.y, carrier.x, x_cast, carrier.history, depth["index"] + 2, self.depth_weight)
        else:
            norm.add_into(carrier.y, carrier.x, x_cast)

    def forward(self, hidden, ctx, layer):
        carrier = hidden
        alone = getattr(self.feed_forward, "is_empty", False)
        self.mixer.forward(carrier.x_cast, carrier.y, ctx, layer)
        self._close(carrier, self.norms["post_mixer"], alone)
        if not alone:
            self.feed_forward.forward(carrier.x_cast, carrier.y, ctx)
            self._close(carrier, self.norms["post_feed_forward"], True)

    def end(self, carrier, ctx):
        return carrier.x
