"""pagedserve_b200: a small, whole, single-GPU paged-KV inference engine for sm_100a.

Public entry points
-------------------
``Engine``          model + cache + step function (``pagedserve_b200.engine.engine``)
``Scheduler``       continuous batching above the step function
``build_scheduler`` factory in the manner of the reference's ``main.build_scheduler``
                    (reference: main.py:136-254)
``generate``        token ids in, token ids out
"""

__version__ = "0.1.0"

_LAZY = {
    "Engine": ("pagedserve_b200.engine.engine", "Engine"),
    "Scheduler": ("pagedserve_b200.engine.scheduler", "Scheduler"),
    "build_scheduler": ("pagedserve_b200.main", "build_scheduler"),
    "generate": ("pagedserve_b200.engine.engine", "generate"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib

        module, attr = _LAZY[name]
        return getattr(importlib.import_module(module), attr)
    raise AttributeError(name)
