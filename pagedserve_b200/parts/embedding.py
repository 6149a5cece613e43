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
