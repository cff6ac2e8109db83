"""Start-up shim for processes that run the unmodified reference engine.

The reference pins torch 2.13 and calls two collectives by their 2.13 names; this image has
torch 2.11, where the same functions exist under their earlier names. Worker processes the
reference spawns import this module automatically (the harness puts this directory first
on PYTHONPATH), so the aliases exist before the reference's code runs. Nothing in the
reference itself is changed.
"""

try:
    import torch.distributed as _dist

    if not hasattr(_dist, "all_gather_single"):
        _dist.all_gather_single = _dist.all_gather_into_tensor
    if not hasattr(_dist, "reduce_scatter_single"):
        _dist.reduce_scatter_single = _dist.reduce_scatter_tensor
except Exception:  # torch missing: nothing to alias
    pass
