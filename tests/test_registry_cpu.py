"""Dispatch layer on the host: shape rules, argument constraints, backend selection and its
exceptions.  The behaviours pinned here are the ones the reference pins for its registry
(tests/test_constraints.py:17-330 and tests/test_backends.py:12-115); no GPU and no kernel runs:
the backends registered below are plain Python objects."""
from __future__ import annotations

import types

import pytest
import torch

import comfy_kitchen  # noqa: F401 - puts the package on the path and registers the real backend
from comfy_kitchen.constraints import (
    DivisibleBy,
    ExactDims,
    FunctionConstraints,
    MinDims,
    ParamConstraint,
    validate_function_call,
    validate_param,
)
from comfy_kitchen.exceptions import (
    BackendError,
    BackendNotFoundError,
    BackendNotImplementedError,
    NoCapableBackendError,
)
from comfy_kitchen.registry import BackendRegistry

CPU_AND_CUDA = frozenset({"cpu", "cuda"})


# ---------------------------------------------------------------------------------- shape rules
def test_shape_rules():
    t = torch.zeros(4, 48)
    assert DivisibleBy(dim=1, factor=16).check(t)
    assert not DivisibleBy(dim=1, factor=32).check(t)
    assert not DivisibleBy(dim=2, factor=1).check(t)  # the dimension does not exist
    assert MinDims(2).check(t) and not MinDims(3).check(t)
    assert ExactDims(2).check(t) and not ExactDims(1).check(t) and not ExactDims(3).check(t)
    assert "16" in DivisibleBy(dim=1, factor=16).describe()
    assert "2" in MinDims(2).describe() and "2" in ExactDims(2).describe()


# ---------------------------------------------------------------------------------- one argument
def test_param_constraint_dtype_device_shape():
    pc = ParamConstraint(dtypes=frozenset({torch.bfloat16, torch.float16}), shape_rules=(ExactDims(2), DivisibleBy(1, 16)))
    good = torch.zeros(3, 32, dtype=torch.bfloat16)
    assert validate_param("x", good, pc, CPU_AND_CUDA).success
    r = validate_param("x", good.float(), pc, CPU_AND_CUDA)
    assert not r.success and r.failed_param == "x" and "dtype" in r.failure_reason
    r = validate_param("x", torch.zeros(3, 30, dtype=torch.bfloat16), pc, CPU_AND_CUDA)
    assert not r.success and "shape" in r.failure_reason and "divisible" in r.failure_reason
    r = validate_param("x", torch.zeros(32, dtype=torch.bfloat16), pc, CPU_AND_CUDA)
    assert not r.success and "exactly 2D" in r.failure_reason
    # None always passes; a bare dtype value is checked against the dtype set only
    assert validate_param("x", None, pc, CPU_AND_CUDA).success
    assert validate_param("out_dtype", torch.float16, pc, CPU_AND_CUDA).success
    assert not validate_param("out_dtype", torch.float32, pc, CPU_AND_CUDA).success
    # no dtype set: any dtype
    assert validate_param("x", torch.zeros(2, 16, dtype=torch.int8), ParamConstraint(), CPU_AND_CUDA).success


def test_param_constraint_devices():
    t = torch.zeros(2, 16)
    assert validate_param("x", t, ParamConstraint(), frozenset({"cpu"})).success
    r = validate_param("x", t, ParamConstraint(), frozenset({"cuda"}))
    assert not r.success and "device cpu" in r.failure_reason
    # a parameter's own device set wins over the function's default; "*" admits everything
    assert validate_param("x", t, ParamConstraint(devices=frozenset({"cpu"})), frozenset({"cuda"})).success
    assert validate_param("x", t, ParamConstraint(devices=frozenset({"*"})), frozenset({"cuda"})).success


# ---------------------------------------------------------------------------------- one call
def _fc(**kw):
    return FunctionConstraints(params={"x": ParamConstraint(dtypes=frozenset({torch.float32}), shape_rules=(ExactDims(2),))},
                               default_devices=frozenset({"cpu"}), **kw)


def test_function_constraints_first_failure_and_missing_arguments():
    fc = _fc()
    assert validate_function_call(fc, {"x": torch.zeros(2, 2)}).success
    assert validate_function_call(fc, {}).success  # an argument that is not passed is not checked
    r = validate_function_call(fc, {"x": torch.zeros(2, 2, dtype=torch.float16)})
    assert not r.success and r.failed_param == "x"


def test_compute_capability_gate():
    fc = _fc(min_compute_capability=(10, 0))
    x = {"x": torch.zeros(2, 2)}
    r = validate_function_call(fc, x, compute_capability=None)
    assert not r.success and r.failed_param == "__hardware__"
    r = validate_function_call(fc, x, compute_capability=(9, 0))
    assert not r.success and "9.0" in r.failure_reason and "10.0" in r.failure_reason
    assert validate_function_call(fc, x, compute_capability=(10, 0)).success
    assert validate_function_call(fc, x, compute_capability=(12, 1)).success
    assert validate_function_call(_fc(), x, compute_capability=None).success  # no requirement, no probe needed


# ---------------------------------------------------------------------------------- registry
def _backend(tag):
    return types.SimpleNamespace(scale=lambda x: (tag, x), only_here=lambda: tag)


@pytest.fixture()
def reg():
    r = BackendRegistry()
    fp32_2d = FunctionConstraints(params={"x": ParamConstraint(dtypes=frozenset({torch.float32}), shape_rules=(ExactDims(2),))},
                                  default_devices=frozenset({"cpu"}))
    any_cpu = FunctionConstraints(params={"x": ParamConstraint()}, default_devices=frozenset({"cpu"}))
    r.register("cuda", _backend("fast"), {"scale": fp32_2d, "only_here": FunctionConstraints()})
    r.register("eager", _backend("slow"), {"scale": any_cpu})
    r.mark_unavailable("triton", "triton is not installed")
    return r


def test_list_backends_reports_every_known_name(reg):
    info = reg.list_backends()
    assert set(info) >= {"cuda", "eager", "triton"}
    assert info["cuda"]["available"] and not info["cuda"]["disabled"] and info["cuda"]["capabilities"] == ["only_here", "scale"]
    assert not info["triton"]["available"] and info["triton"]["unavailable_reason"] == "triton is not installed"


def test_selection_follows_priority_and_constraints(reg):
    x = torch.zeros(2, 2)
    assert reg.get_capable_backend("scale", {"x": x}) == "cuda"
    assert reg.get_implementation("scale", kwargs={"x": x})(x)[0] == "fast"
    # the first backend refuses the dtype: the next one in the priority list takes the call
    half = x.half()
    assert reg.get_capable_backend("scale", {"x": half}) == "eager"
    assert reg.validate_backend_for_call("cuda", "scale", {"x": half}).failed_param == "x"
    assert reg.validate_backend_for_call("eager", "scale", {"x": half}).success
    reg.set_priority(["eager", "cuda", "triton"])
    assert reg.get_capable_backend("scale", {"x": x}) == "eager"
    assert reg.get_constraints("cuda", "scale").default_devices == frozenset({"cpu"})
    assert reg.get_constraints("cuda", "missing") is None


def test_disable_enable_and_thread_local_override(reg):
    x = torch.zeros(2, 2)
    reg.disable("cuda")
    assert reg.list_backends()["cuda"]["disabled"] and not reg.is_available("cuda")
    assert reg.get_capable_backend("scale", {"x": x}) == "eager"
    with pytest.raises(BackendNotFoundError, match="disabled"):
        reg.get_implementation("scale", backend="cuda")
    with pytest.raises(BackendNotFoundError, match="disabled"):
        with reg.use_backend("cuda"):
            pass
    reg.enable("cuda")
    assert reg.get_capable_backend("scale", {"x": x}) == "cuda"
    with reg.use_backend("eager"):
        assert reg.get_capable_backend("scale", {"x": x}) == "eager"
        with reg.use_backend("cuda"):  # nests, and restores the outer choice
            assert reg.get_capable_backend("scale", {"x": x}) == "cuda"
        assert reg.get_capable_backend("scale", {"x": x}) == "eager"
    assert reg.get_capable_backend("scale", {"x": x}) == "cuda"


def test_exceptions_carry_their_context(reg):
    with pytest.raises(BackendNotFoundError) as e:
        reg.get_implementation("scale", backend="nonexistent")
    assert e.value.backend_name == "nonexistent" and isinstance(e.value, BackendError) and isinstance(e.value, RuntimeError)
    with pytest.raises(BackendNotFoundError, match="triton is not installed"):
        reg.get_implementation("scale", backend="triton")
    with pytest.raises(BackendNotFoundError):
        with reg.use_backend("triton"):
            pass
    with pytest.raises(BackendNotImplementedError) as e:
        reg.get_implementation("only_here", backend="eager")
    assert (e.value.backend_name, e.value.func_name) == ("eager", "only_here")
    # nobody takes a 3-D half tensor on "scale"... eager does (no rules); a function nobody implements:
    with pytest.raises(NoCapableBackendError) as e:
        reg.get_capable_backend("does_not_exist", {"x": torch.zeros(1)})
    assert e.value.func_name == "does_not_exist"
    assert e.value.failures["cuda"] == "not implemented" and e.value.failures["triton"] == "triton is not installed"
    # a named backend that refuses the arguments says which one and why
    with pytest.raises(NoCapableBackendError) as e:
        reg.get_implementation("scale", backend="cuda", kwargs={"x": torch.zeros(2, 2, dtype=torch.float16)})
    assert "dtype" in e.value.failures["cuda"]
    assert "No backend available" in str(NoCapableBackendError("f", {}))


def test_the_real_registry_has_one_backend_and_no_cpu_path():
    import comfy_kitchen as ck

    info = ck.list_backends()
    assert set(info) >= {"cuda", "eager", "triton"}
    assert not info["eager"]["available"] and info["eager"]["unavailable_reason"]
    assert not info["triton"]["available"] and info["triton"]["unavailable_reason"]
    x = torch.zeros(32, 64, dtype=torch.bfloat16)
    with pytest.raises(NoCapableBackendError):  # a CPU tensor: nothing to fall back to
        ck.quantize_nvfp4(x, torch.ones((), dtype=torch.float32))
    with pytest.raises(NoCapableBackendError):
        ck.quantize_mxfp8(x)
    with pytest.raises(BackendNotFoundError):
        with ck.use_backend("eager"):
            pass
