"""The parts a model is put together from; importing this package registers the built-in ones."""

from pagedserve_b200.parts.base import (  # noqa: F401
    Block,
    Embedding,
    FeedForward,
    Head,
    LayerContext,
    Mixer,
    Norm,
    Part,
    PartEnv,
    PositionEncoding,
    create_part,
    part_kinds,
    register_part,
)
from pagedserve_b200.parts import attention, blocks, embedding, mlp, norms, positions  # noqa: F401
