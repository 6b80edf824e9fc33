"""CPU-side checks of the C ABI: the library loads without a GPU, exports every symbol the header declares,
and fails loudly (no fallback) when no device is present."""
import ctypes as C
import os
import re

import pytest

from zllm_b200 import ffi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(zq_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    lib = ffi.load()
    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"


def test_every_declared_symbol_has_a_prototype_in_the_binding():
    assert _declared_symbols() == set(ffi.PROTOTYPES)


def test_context_creation_fails_loudly_without_a_device():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    handle = C.c_void_p()
    with pytest.raises(ffi.ZqFailure) as info:
        ffi.call("zq_ctx_create", 0, C.byref(handle))
    assert "no CPU fallback" in str(info.value)


def test_product_package_does_not_touch_the_oracle():
    pkg = os.path.join(ROOT, "zllm_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp", ".hpp")):
                text = open(os.path.join(dirpath, f), errors="replace").read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"
