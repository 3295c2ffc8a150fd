"""The reference's Triton backend is not part of this build (sm_100a kernels only)."""


def _register():
    from comfy_kitchen.registry import registry

    registry.mark_unavailable("triton", "removed: this build has a single hand-written sm_100a backend")


_register()
