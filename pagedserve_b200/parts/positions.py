"""Position encodings."""

from __future__ import annotations

from pagedserve_b200.parts.base import PositionEncoding, register_part
from pagedserve_b200.weights.loader import ParamSpec


@register_part("positions", "learned_absolute")
class LearnedAbsolutePositions(PositionEncoding):
    """h0[t] += table[pos_t]; positions are bounded by the table
    (reference: src/model/paged_decoder.py:289, 306-314, 521-522).
    params: max_positions, hidden_size, name, init_std."""

    graph_safe = True

    def param_specs(self):
        p = self.params
        return [(ParamSpec(self._n(p["name"] + ".weight"), (p["max_positions"], p["hidden_size"]), "table"),
                 ("normal", p.get("init_std", 0.02)))]

    def bind(self, tensors):
        self.table = tensors[self._n(self.params["name"] + ".weight")]

    def embedding_table(self):
        return self.table

    def max_positions(self):
        return self.params["max_positions"]


@register_part("positions", "none")
class NoPositions(PositionEncoding):
    """No position information at all."""

    graph_safe = True


@register_part("positions", "rotary")
class RotaryPositions(PositionEncoding):
    """Queries and keys turn by their position: of the first ``dims`` dimensions of every head, pair i turns by
    the angle position * base^(-2i / dims); the other dimensions pass unchanged.  ``interleaved`` pairs
    neighbours (2i, 2i + 1), otherwise dimension i goes with i + dims / 2.  Angles, sines and products are
    float32; the table of frequencies is made on the host in float64 and rounded once.

    A model may name it as its position encoding (``rotate`` is then called by the attention mixers), or a
    mixer with constants of its own builds one for itself.  Keys reach the cache turned: the kernel that turns
    them also writes the pages (``turn_and_store``).

    ``scaling`` = dict(factor, original, fast, slow) stretches the rotation to contexts longer than ``original``
    positions: with index(t) = dims * ln(original / (2 pi t)) / (2 ln base), lo = max(floor(index(fast)), 0) and
    hi = min(ceil(index(slow)), dims - 1), pair i keeps its frequency f_i below lo, turns at f_i / factor above hi and
    at the blend f_i / factor * r + f_i * (1 - r), r = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), between; every
    sine and cosine is multiplied by ``amplitude`` = 0.1 ln(factor) + 1.
    params: dims, base, interleaved, head_dim, scaling (None)."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = self.params
        if p["dims"] < 0 or p["dims"] % 2 or p["dims"] > p["head_dim"]:
            raise ValueError("rotary: dims must be even and at most the head size")
        if not p["base"] > 0:
            raise ValueError("rotary: base must be positive")
        self._inv_freq = None
        scaling = p.get("scaling")
        if scaling is not None and not (scaling["factor"] > 0 and scaling["original"] > 0 and scaling["fast"] > 0
                                        and scaling["slow"] > 0):
            raise ValueError("rotary: scaling needs positive factor, original, fast and slow")

    @property
    def amplitude(self) -> float:
        """What every sine and cosine is multiplied by (1 without ``scaling``)."""
        import math

        scaling = self.params.get("scaling")
        return 0.1 * math.log(scaling["factor"]) + 1.0 if scaling else 1.0

    def _frequencies(self):
        """The frequencies of the pairs in float64."""
        import math

        import torch

        dims, base = self.params["dims"], float(self.params["base"])
        index = torch.arange(dims // 2, dtype=torch.float64)
        table = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * index / max(dims, 1))
        scaling = self.params.get("scaling")
        if scaling and dims:
            place = lambda turns: dims * math.log(scaling["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
            lo = max(math.floor(place(scaling["fast"])), 0)
            hi = min(math.ceil(place(scaling["slow"])), dims - 1)
            ramp = torch.clamp((index - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            table = table / float(scaling["factor"]) * ramp + table * (1.0 - ramp)
        return table

    def inv_freq(self):
        if self._inv_freq is None:
            import torch

            self._inv_freq = self._frequencies().to(torch.float32).to(self.env.device)
        return self._inv_freq

    def inv_freq_split(self):
        """The frequencies as pairs of floats ``[dims / 2, 2]``: the float nearest to each, and the float nearest
        to what that one misses (for kernels that form position * frequency to more than one float)."""
        if getattr(self, "_inv_freq_split", None) is None:
            import torch

            table = self._frequencies()
            high = table.to(torch.float32)
            low = (table - high.to(torch.float64)).to(torch.float32)
            self._inv_freq_split = torch.stack([high, low], dim=1).contiguous().to(self.env.device)
        return self._inv_freq_split

    def turn_and_store(self, q, k, v, ctx, layer, n_heads, n_kv_heads, write_cache=True):
        """Turn ``q`` in place; write the turned keys and the values (``v``, or the unturned keys when ``v`` is
        None) into the pages of ``layer``."""
        p = self.params
        if p.get("scaling"):
            raise ValueError("rotary: a stretched rotation runs through the kernel that takes an amplitude")
        self.env.ops.rotary_cache_write(q, k, v, self.inv_freq(), p["dims"], p.get("interleaved", True), ctx, layer,
                                        n_heads, n_kv_heads, p["head_dim"], write_cache=write_cache)
