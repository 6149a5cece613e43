"""A model built from a ModelSpec: parts from the registry, run in the schedule's order."""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from pagedserve_b200.cache.manager import KVNeed, StateNeed
from pagedserve_b200.models.spec import ModelSpec
from pagedserve_b200.parts.base import LayerContext, PartEnv, create_part
from pagedserve_b200.weights.loader import ParamSpec, load_weights, place_tensors


class Model:
    """Embedding -> scheduled layers -> final norm on the wanted rows -> head.

    reference: ``PagedDecoderLM.forward_iteration`` (src/model/paged_decoder.py:509-619):
    embed all tokens of the step, run every layer over the flattened batch, select the
    rows that produce output, final norm and LM head only on those rows (:591-605).
    """

    def __init__(self, spec: ModelSpec, env: PartEnv):
        import pagedserve_b200.parts  # noqa: F401  (registers the built-in parts)

        self.spec = spec
        self.env = env
        self.embedding = create_part("embedding", spec.embedding, env)
        self.positions = create_part("positions", spec.positions, env)
        self.blocks = []
        for layer in spec.layers:
            mixer = create_part("mixer", layer.mixer, env)
            feed_forward = create_part("feed_forward", layer.feed_forward, env)
            norms = {role: create_part("norm", norm, env) for role, norm in layer.norms.items()}
            block = create_part("block", layer.block, env, mixer=mixer, feed_forward=feed_forward, norms=norms)
            missing = [role for role in block.required_norms if role not in norms]
            if missing:
                raise ValueError(f"block {layer.block.kind!r} needs norms {missing}")
            self.blocks.append(block)
        self.final_norm = create_part("norm", spec.final_norm, env)
        self.head = create_part("head", spec.head, env)

    # ------------------------------------------------------------------ parameters
    def parts(self):
        yield self.embedding
        yield self.positions
        for block in self.blocks:
            yield block
            yield block.mixer
            yield block.feed_forward
            yield from block.norms.values()
        yield self.final_norm
        yield self.head

    @property
    def graph_safe(self) -> bool:
        """Whether a decode-only step of this model may be captured as a CUDA graph."""
        return all(part.graph_safe for part in self.parts())

    def param_plan(self) -> List[Tuple[ParamSpec, tuple]]:
        plan = []
        for part in self.parts():
            plan.extend(part.param_specs())
        return plan

    def param_specs(self) -> List[ParamSpec]:
        return [spec for spec, _ in self.param_plan()]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.tensors = tensors
        for part in self.parts():
            part.bind(tensors)

    def load_folder(self, folder: str) -> None:
        self.bind(load_weights(folder, self.param_specs(), self.env.dtype, self.env.device,
                               self.spec.normalise_name))

    def load_tensors(self, stored: Dict[str, torch.Tensor]) -> None:
        self.bind(place_tensors(self.param_specs(), stored, self.env.dtype, self.env.device,
                                self.spec.normalise_name))

    def weight_bytes(self) -> int:
        seen = {}
        for tensor in self.tensors.values():
            seen[tensor.data_ptr()] = tensor.numel() * tensor.element_size()
        return sum(seen.values())

    # ------------------------------------------------------------------ cache needs
    def _needs(self, which: str) -> list:
        """Per cache layer, what the mixer of the run(s) that use it asks for."""
        needs = [None] * self.spec.num_cache_layers
        seen = [False] * self.spec.num_cache_layers
        for entry in self.spec.schedule:
            need = getattr(self.blocks[entry.layer].mixer, which)()
            if seen[entry.cache_layer] and needs[entry.cache_layer] != need:
                raise ValueError(f"cache layer {entry.cache_layer} is shared by runs with different needs")
            needs[entry.cache_layer] = need
            seen[entry.cache_layer] = True
        return needs

    def kv_needs(self) -> List[Optional[KVNeed]]:
        return self._needs("cache_need")

    def state_needs(self) -> List[Optional[StateNeed]]:
        return self._needs("state_need")

    # ------------------------------------------------------------------ forward
    def forward(self, ctx) -> torch.Tensor:
        """Run the tokens of ``ctx`` from the cache; return float32 logits ``[R, V]``."""
        hidden = self.embedding.forward(ctx, self.positions)
        cache = ctx.cache
        # what a layer asks of the step arena is dead when the layer is done (the residual stream came first):
        # every layer starts from the same place in it
        arena = getattr(self.env.ops, "arena", None)
        mark = arena.mark() if arena is not None else None
        for entry in self.spec.schedule:
            if arena is not None:
                arena.release(mark)
            layer = LayerContext(entry.layer, entry.cache_layer, self.positions)
            group_index = cache.group_of_layer.get(entry.cache_layer)
            if group_index is not None:
                group = cache.groups[group_index]
                layer.k_pool, layer.v_pool = group.layer_views(entry.cache_layer)
                layer.page_stride = group.page_stride
                layer.page_size = group.page_size
                layer.pool = group.pool
                layer.pool_layer = group.cache_layers.index(entry.cache_layer)
                layer.block_table = ctx.block_tables[group_index]
            layer.state = cache.state.get(entry.cache_layer)
            self.blocks[entry.layer].forward(hidden, ctx, layer)
        if arena is not None:
            arena.release(mark)
        if ctx.num_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=hidden.device)
        if hasattr(self.final_norm, "defer"):
            normed = self.final_norm.defer(hidden, rows=ctx.logit_rows)     # the head's product may fold it in
        else:
            normed = self.final_norm.forward(hidden, rows=ctx.logit_rows)
        return self.head.forward(normed, self.embedding)


def init_plan(spec: ModelSpec):
    """(ParamSpec, init rule) of every tensor a random model of ``spec`` needs."""
    model = Model(spec, PartEnv(ops=None, dtype=torch.float32, device="cpu"))
    return [(param, init) for param, init in model.param_plan() if init[0] != "skip"]
