"""Interfaces of the parts and the part registry.

A part is built from a :class:`PartSpec` (its constants), declares the tensors
it needs (:meth:`Part.param_specs`), receives them (:meth:`Part.bind`) and then
runs.  No part knows which model it is in: sizes, names of tensors and every
constant are parameters.

Categories and what each must provide
-------------------------------------
``embedding``          ``forward(ctx) -> hidden``: float32 ``[T, H]`` residual stream.
``positions``          ``embedding_table()`` (a table to add to the token embedding, or None),
                       ``add_to_hidden(hidden, ctx)`` and ``rotate(q, k, ctx)`` hooks.
``norm``               ``forward(x, out=None, rows=None) -> normed`` (compute dtype).
``mixer``              ``cache_need()``, ``state_need()``,
                       ``forward(x, residual, ctx, layer)``: adds its output into ``residual``.
``feed_forward``       ``forward(x, residual, ctx)``: adds its output into ``residual``.
``block``              ``forward(hidden, ctx, layer)``: runs norms, mixer, feed-forward in its arrangement.
``head``               ``forward(x_rows) -> float32 logits [R, V]``.

``ctx`` is the :class:`pagedserve_b200.engine.batch.StepContext` of the step;
``layer`` is a :class:`LayerContext` that carries what this run of the layer
may touch of the cache (pages of its cache layer, its slot state).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch

from pagedserve_b200.cache.manager import KVNeed, StateNeed
from pagedserve_b200.weights.loader import ParamSpec

Init = Tuple[str, float]            # ("normal" | "ones_plus_normal", std)


@dataclass
class PartEnv:
    """What every part gets at construction."""

    ops: object                      # pagedserve_b200.kernels.Ops (None on a host without kernels)
    dtype: torch.dtype               # compute dtype
    device: object


@dataclass
class LayerContext:
    layer: int                       # index of the layer whose parameters run
    cache_layer: int                 # index of the cache layer it uses
    positions: "PositionEncoding"
    k_pool: Optional[torch.Tensor] = None      # [pages, kv heads, page size, head dim] view
    v_pool: Optional[torch.Tensor] = None
    page_stride: int = 0             # elements between consecutive pages
    page_size: int = 0
    pool: Optional[torch.Tensor] = None        # the group's whole pool [pages, layers, 2, kv heads, page, head dim]
    pool_layer: int = 0                        # index of this cache layer inside the pool
    block_table: Optional[torch.Tensor] = None  # int32 [slots + 1, max pages] of the layer's group, by request slot
    state: Optional[torch.Tensor] = None        # [max slots, *state shape] of this cache layer


class Part:
    category = ""
    # True when ``forward`` only launches work whose shapes and addresses depend on the batch size alone
    # and reads the batch from ``ctx``'s device arrays: such a step can be captured once as a CUDA graph
    # and replayed. A part that branches on host data (``ctx.host``) leaves this False, and a model
    # with such a part runs every step eagerly.
    graph_safe = False

    def __init__(self, params: dict, prefix: str, env: PartEnv):
        self.params = dict(params)
        self.prefix = prefix
        self.env = env

    # name helper: tensors are named prefix + local name
    def _n(self, local: str) -> str:
        return self.prefix + local

    def param_specs(self) -> List[Tuple[ParamSpec, Init]]:
        """Tensors this part needs, each with the rule by which random weights are drawn."""
        return []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receive the loaded tensors (by canonical name)."""


class Embedding(Part):
    category = "embedding"

    def forward(self, ctx, positions: "PositionEncoding") -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    category = "positions"

    def embedding_table(self) -> Optional[torch.Tensor]:
        """A ``[positions, H]`` table to be added to the token embedding, if this encoding has one."""
        return None

    def add_to_hidden(self, hidden: torch.Tensor, ctx) -> None:
        """Add a position term to the embedded tokens (absolute encodings)."""

    def rotate(self, q: torch.Tensor, k: torch.Tensor, ctx) -> None:
        """Transform queries and keys in place by position (rotary encodings)."""

    def max_positions(self) -> Optional[int]:
        return None


@dataclass
class NormPrologue:
    """What a matrix product needs to compute a norm of the form ``(x - mean?) * rsqrt(var + eps) * weight
    (+ bias)`` over the last axis inside its own kernel, in float32."""

    weight: torch.Tensor                 # float32 [width]
    bias: Optional[torch.Tensor]         # float32 [width] or None
    eps: float
    has_mean: bool                       # False: the RMS form


class Norm(Part):
    category = "norm"

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def fused_prologue(self) -> Optional[NormPrologue]:
        """A norm that a consuming product may fold into its prologue says how here (any norm of the form
        :class:`NormPrologue` describes, whatever its class); None: it has to run as its own kernel."""
        return None


class Mixer(Part):
    category = "mixer"

    def cache_need(self) -> Optional[KVNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, layer: LayerContext) -> None:
        raise NotImplementedError


class FeedForward(Part):
    category = "feed_forward"

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx) -> None:
        raise NotImplementedError


class Block(Part):
    category = "block"

    def __init__(self, params, prefix, env, mixer: Mixer, feed_forward: FeedForward, norms: Dict[str, Norm]):
        super().__init__(params, prefix, env)
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = norms

    required_norms: Tuple[str, ...] = ()

    def forward(self, hidden: torch.Tensor, ctx, layer: LayerContext) -> None:
        raise NotImplementedError


class Head(Part):
    category = "head"

    def forward(self, x_rows: torch.Tensor, embedding: Embedding) -> torch.Tensor:
        raise NotImplementedError


# ---------------------------------------------------------------------------- registry
_PARTS: Dict[Tuple[str, str], Callable] = {}
CATEGORIES = ("embedding", "positions", "norm", "mixer", "feed_forward", "block", "head")


def register_part(category: str, kind: str, replace: bool = False):
    """Class decorator: make ``kind`` available to ModelSpecs under ``category``."""
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r}; one of {CATEGORIES}")

    def decorate(cls):
        key = (category, kind)
        if key in _PARTS and not replace:
            raise ValueError(f"part {kind!r} is already registered as a {category}")
        _PARTS[key] = cls
        return cls

    return decorate


def part_kinds(category: str) -> List[str]:
    return sorted(kind for (cat, kind) in _PARTS if cat == category)


def create_part(category: str, spec, env: PartEnv, **extra) -> Part:
    key = (category, spec.kind)
    if key not in _PARTS:
        raise ValueError(f"no {category} part named {spec.kind!r}; registered: {part_kinds(category)}")
    return _PARTS[key](spec.params, spec.prefix, env, **extra)
