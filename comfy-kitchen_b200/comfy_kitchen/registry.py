"""Operator dispatch.

The reference (comfy_kitchen/registry.py:20-307) chooses among three backends by
priority.  This build ships exactly one implementation of the quantized-linear
operators - the sm_100a C-ABI library registered as ``cuda`` - so the selection loop
degenerates to "validate the call against that backend or raise".  There is no CPU
implementation to fall back to: a call the CUDA backend cannot take raises
``NoCapableBackendError``.  The public surface (method names, the ``eager`` / ``cuda`` /
``triton`` keys of ``list_backends()``, ``use_backend``, exception types) is unchanged so
callers and tests written against the reference keep working.
"""
from __future__ import annotations

import logging
import threading
from collections.abc import Callable, Mapping
from contextlib import contextmanager
from typing import Any

import torch

from .constraints import FunctionConstraints, ValidationResult, validate_function_call
from .exceptions import BackendNotFoundError, BackendNotImplementedError, NoCapableBackendError

logger = logging.getLogger("comfy_kitchen.dispatch")

_KNOWN = ("cuda", "triton", "eager")


class BackendRegistry:
    def __init__(self):
        self._backends: dict[str, Any] = {}
        self._capabilities: dict[str, set[str]] = {}
        self._constraints: dict[tuple[str, str], FunctionConstraints] = {}
        self._priority: list[str] = list(_KNOWN)
        self._disabled: set[str] = set()
        self._unavailable: dict[str, str] = {}
        self._lock = threading.Lock()
        self._tls = threading.local()
        self._cc: tuple[int, int] | None | bool = False  # False = not probed yet

    # -- hardware ------------------------------------------------------------------------
    @property
    def _compute_capability(self) -> tuple[int, int] | None:
        if self._cc is False:
            cc = None
            if torch.cuda.is_available():
                try:
                    p = torch.cuda.get_device_properties(torch.cuda.current_device())
                    cc = (p.major, p.minor)
                except Exception:  # noqa: BLE001 - a broken driver means "no capability"
                    cc = None
            self._cc = cc
        return self._cc  # type: ignore[return-value]

    # -- registration --------------------------------------------------------------------
    def register(self, name: str, module, capabilities: dict[str, FunctionConstraints]):
        with self._lock:
            self._backends[name] = module
            self._capabilities[name] = set(capabilities)
            for fn, fc in capabilities.items():
                self._constraints[(name, fn)] = fc
            self._unavailable.pop(name, None)

    def mark_unavailable(self, name: str, reason: str):
        with self._lock:
            self._unavailable[name] = reason

    def get_constraints(self, backend_name: str, func_name: str) -> FunctionConstraints | None:
        return self._constraints.get((backend_name, func_name))

    # -- configuration -------------------------------------------------------------------
    def disable(self, backend_name: str):
        with self._lock:
            self._disabled.add(backend_name)

    def enable(self, backend_name: str):
        with self._lock:
            self._disabled.discard(backend_name)

    def set_priority(self, priority_list: list[str]):
        with self._lock:
            self._priority = list(priority_list)

    def is_available(self, backend_name: str) -> bool:
        return backend_name in self._backends and backend_name not in self._disabled

    def list_backends(self) -> dict:
        names = set(self._priority) | set(self._backends) | set(self._unavailable) | set(_KNOWN)
        return {
            n: {
                "available": n in self._backends,
                "disabled": n in self._disabled,
                "unavailable_reason": self._unavailable.get(n),
                "capabilities": sorted(self._capabilities.get(n, ())),
            }
            for n in names
        }

    # -- selection -----------------------------------------------------------------------
    def validate_backend_for_call(self, backend_name: str, func_name: str, kwargs: Mapping[str, Any]) -> ValidationResult:
        if not self.is_available(backend_name):
            return ValidationResult.fail("__backend__", self._unavailable.get(backend_name, "not available"))
        if func_name not in self._capabilities.get(backend_name, ()):
            return ValidationResult.fail("__function__", "not implemented")
        fc = self._constraints.get((backend_name, func_name))
        if fc is None:
            return ValidationResult.ok()
        return validate_function_call(fc, kwargs, compute_capability=self._compute_capability)

    def _try(self, name: str, func_name: str, kwargs, failures: dict[str, str]) -> bool:
        if not self.is_available(name):
            failures[name] = self._unavailable.get(name, "not available")
            return False
        if func_name not in self._capabilities.get(name, ()):
            failures[name] = "not implemented"
            return False
        if kwargs:
            res = self.validate_backend_for_call(name, func_name, kwargs)
            if not res.success:
                failures[name] = f"{res.failed_param}: {res.failure_reason}"
                return False
        return True

    def get_capable_backend(self, func_name: str, kwargs: Mapping[str, Any] | None = None) -> str:
        failures: dict[str, str] = {}
        override = getattr(self._tls, "override", None)
        order = ([override] if override else []) + [n for n in self._priority if n != override]
        for name in order:
            if name != override and name not in self._backends:
                continue  # never-registered backends are not "failures", they just do not exist
            if self._try(name, func_name, kwargs, failures):
                logger.debug("Backend %s selected for %s", name, func_name)
                return name
        for name, why in self._unavailable.items():
            failures.setdefault(name, why)
        raise NoCapableBackendError(func_name, failures)

    def get_implementation(self, func_name: str, backend: str | None = None,
                           kwargs: Mapping[str, Any] | None = None) -> Callable:
        if backend:
            if backend not in self._backends:
                raise BackendNotFoundError(backend, self._unavailable.get(backend, "not registered"))
            if backend in self._disabled:
                raise BackendNotFoundError(backend, "disabled")
            if func_name not in self._capabilities.get(backend, ()):
                raise BackendNotImplementedError(backend, func_name)
            if kwargs:
                res = self.validate_backend_for_call(backend, func_name, kwargs)
                if not res.success:
                    raise NoCapableBackendError(func_name, {backend: f"{res.failed_param}: {res.failure_reason}"})
            return getattr(self._backends[backend], func_name)
        return getattr(self._backends[self.get_capable_backend(func_name, kwargs)], func_name)

    @contextmanager
    def use_backend(self, backend_name: str):
        """Force ``backend_name`` for calls made by this thread inside the ``with`` block."""
        if not self.is_available(backend_name):
            if backend_name in self._disabled:
                raise BackendNotFoundError(backend_name, "disabled")
            raise BackendNotFoundError(backend_name, self._unavailable.get(backend_name, "not registered"))
        previous = getattr(self._tls, "override", None)
        self._tls.override = backend_name
        try:
            yield
        finally:
            self._tls.override = previous


registry = BackendRegistry()
