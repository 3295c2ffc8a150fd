"""Placeholder for the reference's pure-PyTorch backend.

The reference ships an eager implementation of every operator
(comfy_kitchen/backends/eager/).  In this build that arithmetic lives outside the
package, as the test oracle, and is not a dispatch target: there is no CPU
implementation of the quantized-linear operators.  The module exists so that
``list_backends()`` keeps reporting the ``eager`` key and so that code importing the
dtype-code tables from their historical location keeps working.
"""
from comfy_kitchen.ops import DTYPE_CODE_TO_DTYPE, DTYPE_TO_CODE  # noqa: F401


def _register():
    from comfy_kitchen.registry import registry

    registry.mark_unavailable("eager", "not shipped: the pure-PyTorch path is kept only as the test oracle")


_register()
