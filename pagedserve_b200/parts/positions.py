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
