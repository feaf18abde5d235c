"""Host-side checks that need no GPU: the C-ABI library builds, loads and exports every symbol the
header declares, and it refuses to run without a CUDA device instead of falling back to anything."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def kv():
    import tract_b200
    from tract_b200 import build

    build.build()
    return tract_b200


def test_header_and_library_agree(kv):
    header = open(os.path.join(ROOT, "include", "b200kv.h")).read()
    declared = set(re.findall(r"\b(b200kv_[a-z0-9_]+)\s*\(", header))
    assert declared == set(kv.EXPORTS), declared ^ set(kv.EXPORTS)
    L = kv.lib()
    for name in declared:
        assert hasattr(L, name), f"{name} is declared in include/b200kv.h but not exported"
    assert b"sm_100a" in L.b200kv_version()


def test_no_cpu_fallback(kv):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    cfg = kv.Config(0, kv.FMT_F16, 8, 128, 1, 4, 1024, 4096)
    h = C.c_void_p()
    assert kv.lib().b200kv_create(C.byref(cfg), C.byref(h)) == 1
    assert b"no CUDA device" in kv.lib().b200kv_last_error()
    with pytest.raises(kv.B200KvError, match="no CUDA device"):
        kv.KvCache("f16", 8, 128, 4, 1024)
    # argument validation comes first and is reported through the same channel
    bad = kv.Config(0, 99, 8, 128, 1, 4, 1024, 4096)
    assert kv.lib().b200kv_create(C.byref(bad), C.byref(h)) == 1
    assert b"format" in kv.lib().b200kv_last_error()


def test_product_never_touches_the_oracle():
    # the oracle is test infrastructure: nothing under the package may import, link or call it
    pkg = os.path.join(ROOT, "tract_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp", ".hpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), os.path.join(dirpath, f)
