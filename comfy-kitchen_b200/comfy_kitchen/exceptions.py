"""Exception types of the dispatch layer.

Same names, attributes and base class as the reference's
comfy_kitchen/exceptions.py:1-40: every one derives from RuntimeError because the
tensor layouts catch ``(RuntimeError, TypeError)`` around the fast matmul path.
"""
from __future__ import annotations


class BackendError(RuntimeError):
    """Root of all dispatch failures."""


class BackendNotFoundError(BackendError):
    """The named backend is not registered, failed to load, or is disabled."""

    def __init__(self, backend_name: str, reason: str | None = None):
        self.backend_name = backend_name
        text = f"Backend '{backend_name}' is not available"
        super().__init__(f"{text}: {reason}" if reason else text)


class BackendNotImplementedError(BackendError):
    """The named backend exists but has no implementation of the function."""

    def __init__(self, backend_name: str, func_name: str):
        self.backend_name = backend_name
        self.func_name = func_name
        super().__init__(f"Backend '{backend_name}' does not implement '{func_name}'")


class NoCapableBackendError(BackendError):
    """No backend accepted the call; ``failures`` maps backend name -> reason."""

    def __init__(self, func_name: str, failures: dict[str, str]):
        self.func_name = func_name
        self.failures = failures
        if failures:
            why = "; ".join(f"{k}: {v}" for k, v in failures.items())
            super().__init__(f"No backend can handle '{func_name}': {why}")
        else:
            super().__init__(f"No backend available for '{func_name}'")
