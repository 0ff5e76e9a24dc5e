"""Discovery of the reference project's own example tests (python/examples/test_*.py of
microsoft/triton-shared) so that they can be executed, unmodified, with B200Driver in the place
of the reference's CPUDriver.

TEST INFRASTRUCTURE.  The examples are not part of this repository: the directory holding them is
named by the environment variable TSB_REFERENCE_EXAMPLES (a checkout's python/examples).  Without
it nothing is collected.  What python/examples/conftest.py does for the reference is done here:

* ``triton.backends.triton_shared.driver.CPUDriver`` resolves to ``B200Driver`` (the examples
  import that name, python/examples/conftest.py:5-7);
* the ``device`` fixture value (conftest.py:17-19) is supplied by the caller: "cuda" for the GPU
  run, "cpu" for the host stand-in run;
* ``pytest.mark.interpreter`` is the identity (conftest.py:10-14);
* on a GPU, ``torch.testing.assert_close``, ``torch.equal`` and ``torch.allclose`` compare values across
  devices, because several examples build their expected tensor on the host.
"""
import importlib.util
import inspect
import itertools
import os
import sys
import types

import pytest

ENV = "TSB_REFERENCE_EXAMPLES"


def examples_dir():
    d = os.environ.get(ENV, "")
    return d if d and os.path.isdir(d) else None


def install_driver_alias():
    import triton_shared_b200 as tsb
    if "triton.backends.triton_shared" not in sys.modules:
        pkg = types.ModuleType("triton.backends.triton_shared")
        pkg.__path__ = []
        drv = types.ModuleType("triton.backends.triton_shared.driver")
        drv.CPUDriver = tsb.B200Driver
        pkg.driver = drv
        sys.modules["triton.backends.triton_shared"] = pkg
        sys.modules["triton.backends.triton_shared.driver"] = drv
    pytest.mark.interpreter = lambda f: f


# Example tests that cannot pass with any driver but the reference's own, and why.  They are
# collected and reported as skipped with this reason; everything else must pass.
EXCLUDED = {
    "test_unstructured_mask.py": "runs the reference's triton-shared-opt tool on the TTIR and counts tts ops in its output",
    "test_reduce.py::test": "after its numeric check it compiles for GPUTarget(device, 0, 0) and prints the reference's "
                            "ttsharedir / llir / obj stages",
}

_modules = {}


def load(path):
    name = "tsb_ref_example_" + os.path.splitext(os.path.basename(path))[0]
    if os.path.dirname(path) not in sys.path:
        sys.path.insert(0, os.path.dirname(path))  # the examples import their sibling `benchmark` module
    if name not in _modules:
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        _modules[name] = mod
    return _modules[name]


def _param_sets(fn):
    """Expand @pytest.mark.parametrize marks of a test function into keyword dicts."""
    marks = [m for m in getattr(fn, "pytestmark", []) if m.name == "parametrize"]
    axes = []
    for m in marks:
        names = m.args[0]
        names = [n.strip() for n in names.split(",")] if isinstance(names, str) else list(names)
        rows = []
        for v in m.args[1]:
            v = getattr(v, "values", v)  # pytest.param(...) carries its values as a tuple
            if len(names) == 1:
                rows.append({names[0]: v[0] if hasattr(v, "_fields") or (isinstance(v, tuple) and v is not m.args[1] and
                                                                         getattr(v, "__class__", None).__name__ == "ParameterSet") else v})
            else:
                rows.append(dict(zip(names, v)))
        axes.append(rows)
    out = []
    for combo in itertools.product(*axes) if axes else [()]:
        kw = {}
        for c in combo:
            kw.update(c)
        out.append(kw)
    return out


def cases():
    """[(id, file path, function name, kwargs)] for every test function of every example file."""
    d = examples_dir()
    if d is None:
        return []
    install_driver_alias()
    out = []
    for fname in sorted(os.listdir(d)):
        if not fname.endswith(".py") or not (fname.startswith("test_") or fname == "bare_matmul.py"):
            continue
        path = os.path.join(d, fname)
        if fname in EXCLUDED:
            out.append((f"{fname}::<excluded>", path, None, {"skip": EXCLUDED[fname]}))
            continue
        try:
            mod = load(path)
        except Exception as e:  # an example that cannot even be imported is a failing case
            out.append((f"{fname}::<import>", path, None, {"error": repr(e)}))
            continue
        for name, fn in inspect.getmembers(mod, inspect.isfunction):
            if not (name.startswith("test_") or name == "test") or fn.__module__ != mod.__name__:
                continue
            for kw in _param_sets(fn):
                tag = ",".join(f"{k}={v}" for k, v in kw.items())
                out.append((f"{fname}::{name}" + (f"[{tag}]" if tag else ""), path, name, kw))
    return out


def run_case(path, name, kw, device):
    if name is None and "skip" in kw:
        pytest.skip(kw["skip"])
    if name is None:
        raise RuntimeError(f"cannot import {path}: {kw['error']}")
    key = f"{os.path.basename(path)}::{name}"
    if key in EXCLUDED:
        pytest.skip(EXCLUDED[key])
    fn = getattr(load(path), name)
    args = dict(kw)
    sig = inspect.signature(fn)
    if "device" in sig.parameters:
        args["device"] = device
    missing = [p for p in sig.parameters if p not in args and sig.parameters[p].default is inspect._empty]
    if missing:
        pytest.skip(f"needs fixtures {missing} that this runner does not provide")
    if device == "cpu":
        return fn(**args)
    # several examples build their expected tensor on the host (they were written for a CPU device
    # only): values are compared across devices, everything else about the assertion stands
    import torch
    strict = torch.testing.assert_close

    def assert_close(actual, expected, **kwargs):
        kwargs.setdefault("check_device", False)
        return strict(actual, expected, **kwargs)
    equal, allclose = torch.equal, torch.allclose
    host = lambda t: t.cpu() if isinstance(t, torch.Tensor) else t
    same = lambda a, b: not (isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor)) or a.device == b.device
    torch.testing.assert_close = assert_close
    torch.equal = lambda a, b: equal(a, b) if same(a, b) else equal(host(a), host(b))
    torch.allclose = lambda a, b, *r, **k: allclose(a, b, *r, **k) if same(a, b) else allclose(host(a), host(b), *r, **k)
    try:
        return fn(**args)
    finally:
        torch.testing.assert_close, torch.equal, torch.allclose = strict, equal, allclose
