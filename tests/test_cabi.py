"""The C-ABI shared library loads and exports every symbol declared in include/pipedream_b200.h."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "pipedream_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    return sorted(set(re.findall(r"\b(pd_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_declared_symbols():
    from pipedream_b200 import _lib, build
    path = build.build()
    lib = ctypes.CDLL(path)
    names = declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), "library does not export %s" % n
    # and the ctypes table binds exactly the declared entry points
    assert sorted(_lib.SIGNATURES) == names
    assert lib.pd_abi_version() >= 1


def test_missing_library_is_an_error(monkeypatch):
    from pipedream_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "_LIB_PATH", "/nonexistent/libpipedream_b200.so")
    try:
        _lib.load()
    except _lib.PipedreamB200Error as e:
        assert "no non-CUDA fallback" in str(e)
    else:
        raise AssertionError("loading a missing library must fail")


def test_runtime_refuses_cpu():
    import torch
    if torch.cuda.is_available():
        return
    from pipedream_b200 import runtime
    model = [(torch.nn.Linear(2, 2), ["input0"], ["out0"]), (torch.nn.MSELoss(), ["out0"], ["loss"])]
    try:
        runtime.StageRuntime(model, "gloo", False, 1, {}, {}, {}, {"input": 0}, {"target"},
                             {"module_to_stage_map": None, "stage_to_rank_map": None, "stage_to_depth_map": None},
                             None, None, 0, 1, 0, runtime.IMAGE_CLASSIFICATION)
    except RuntimeError as e:
        assert "CUDA" in str(e)
    else:
        raise AssertionError("StageRuntime must not run without a CUDA device")
