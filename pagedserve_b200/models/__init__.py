"""Architectures: importing this package registers the built-in ones."""

from pagedserve_b200.models import gpt2  # noqa: F401  (registers "GPT2LMHeadModel")
from pagedserve_b200.models.model import Model, init_plan  # noqa: F401
from pagedserve_b200.models.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry  # noqa: F401
