"""Token embedding and LM head."""

from __future__ import annotations

import torch

from pagedserve_b200.parts.base import Embedding, Head, register_part
from pagedserve_b200.weights.loader import ParamSpec


@register_part("embedding", "token_embedding")
class TokenEmbedding(Embedding):
    """hidden[t] = table[id_t] (+ the position encoding's table row, fused into the same gather).

    reference: src/model/paged_decoder.py:288, 306-314.  The result is float32:
    it starts the residual stream.  params: vocab_size, hidden_size, name, init_std."""

    graph_safe = True

    def param_specs(self):
        p = self.params
        return [(ParamSpec(self._n(p["name"] + ".weight"), (p["vocab_size"], p["hidden_size"]), "table"),
                 ("normal", p.get("init_std", 0.02)))]

    def bind(self, tensors):
        self.table = tensors[self._n(self.params["name"] + ".weight")]

    def forward(self, ctx, positions):
        hidden = self.env.ops.empty((ctx.num_tokens, self.params["hidden_size"]), torch.float32, self.table.device)
        position_table = positions.embedding_table()
        self.env.ops.embed(ctx.token_ids, ctx.positions, self.table, position_table, hidden, ctx.status)
        if position_table is None:
            positions.add_to_hidden(hidden, ctx)
        return hidden


@register_part("embedding", "normed_token_embedding")
class NormedTokenEmbedding(TokenEmbedding):
    """hidden[t] = norm(table[id_t]): the token's row, then an RMS norm in groups with a gain of its own
    (:class:`pagedserve_b200.parts.norms.GroupRMSNorm`), float32, in place.
    params: vocab_size, hidden_size, name, init_std, norm (dict: name, eps, groups, init_std)."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        from pagedserve_b200.parts.norms import GroupRMSNorm

        norm = self.params["norm"]
        self.norm = GroupRMSNorm(dict(width=self.params["hidden_size"], eps=norm["eps"], groups=norm.get("groups", 1),
                                      name=norm["name"], init_std=norm.get("init_std", 0.0)), prefix, env)

    def param_specs(self):
        return super().param_specs() + self.norm.param_specs()

    def bind(self, tensors):
        super().bind(tensors)
        self.norm.bind(tensors)

    def forward(self, ctx, positions):
        hidden = super().forward(ctx, positions)
        return self.norm.forward(hidden, out=hidden)


@register_part("embedding", "token_pair_embedding")
class TokenPairEmbedding(TokenEmbedding):
    """hidden[t] = scale * table[id_t] + pair[row_t]: the token table times a constant, plus a row of a second
    table chosen by a hash of the token and the one before it, row_t = (id_{t-1} * mul_prev + id_t * mul_cur) mod
    buckets; the first token of a sequence takes the table's extra last row (index ``buckets``).  Without
    ``pair`` only the scale is left.

    The token before a step's first token of a request is part of the request's state: one int32 in its slot
    (``state_need``), read and then replaced by the kernel that embeds the entry's first token.  The sum is
    float32.  params: vocab_size, hidden_size, name, init_std, scale, pair (None or a dict: name, buckets,
    mul_prev, mul_cur, init_std)."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        pair = self.params.get("pair")
        if pair is not None and not (isinstance(pair["buckets"], int) and pair["buckets"] > 0):
            raise ValueError("token_pair_embedding: buckets must be a positive integer")

    def state_need(self):
        from pagedserve_b200.cache.manager import StateNeed

        return StateNeed((1,), "int32") if self.params.get("pair") else None

    def param_specs(self):
        specs = super().param_specs()
        pair = self.params.get("pair")
        if pair:
            specs.append((ParamSpec(self._n(pair["name"]), (pair["buckets"] + 1, self.params["hidden_size"]), "table"),
                          ("normal", pair.get("init_std", 0.02))))
        return specs

    def bind(self, tensors):
        super().bind(tensors)
        pair = self.params.get("pair")
        self.pair_table = tensors[self._n(pair["name"])].contiguous() if pair else None

    def forward(self, ctx, positions, state=None):
        p = self.params
        pair = p.get("pair") or {}
        hidden = self.env.ops.empty((ctx.num_tokens, p["hidden_size"]), torch.float32, self.table.device)
        if self.pair_table is not None and state is None:
            raise ValueError("token_pair_embedding: the cache holds no slot state for the token before")
        self.env.ops.embed_pair(ctx, self.table, float(p.get("scale", 1.0)), self.pair_table, pair.get("buckets", 0),
                                pair.get("mul_prev", 0), pair.get("mul_cur", 0), state, hidden)
        positions.add_to_hidden(hidden, ctx)
        return hidden


@register_part("head", "lm_head")
class LMHead(Head):
    """logits = x table^T in float32, no bias; ``tied`` uses the token embedding's table
    (reference: src/model/paged_decoder.py:295-301; src/model/gpt2.py:42-43, 77-78).
    A tied model may still store the head: the copy must then equal the table it is tied to
    (``tied_to``, the canonical name of that tensor), else loading fails.
    params: vocab_size, hidden_size, tied, tied_to, name, init_std."""

    graph_safe = True

    def param_specs(self):
        p = self.params
        spec = ParamSpec(self._n(p["name"] + ".weight"), (p["vocab_size"], p["hidden_size"]), "table",
                         optional=bool(p["tied"]), same_as=p.get("tied_to") if p["tied"] else None)
        if p["tied"]:
            return [(spec, ("skip", 0.0))]
        return [(spec, ("normal", p.get("init_std", 0.02)))]

    def bind(self, tensors):
        self.table = None if self.params["tied"] else tensors[self._n(self.params["name"] + ".weight")]

    def forward(self, x_rows, embedding):
        table = embedding.table if self.table is None else self.table
        logits = self.env.ops.empty((x_rows.shape[0], table.shape[0]), torch.float32, x_rows.device)
        if x_rows.shape[0] == 0:
            return logits
        return self.env.ops.linear(x_rows, table, None, logits)
