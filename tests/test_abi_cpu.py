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


def _c_signatures(header):
    """{name: [C parameter types]} of every function the header declares."""
    text = re.sub(r"/\*.*?\*/", " ", header, flags=re.S)
    sigs = {}
    for m in re.finditer(r"\b(b200kv_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S):
        params = [p.strip() for p in m.group(2).replace("\n", " ").split(",")]
        sigs[m.group(1)] = [] if params in ([""], ["void"]) else params
    return sigs


def _rust_signatures(src):
    """{name: number of parameters} of every `pub fn` inside the extern "C" block of the Rust binding."""
    block = src[src.index('extern "C" {'):]
    block = block[:block.index("\n}\n")]
    block = re.sub(r"//.*", "", block)
    sigs = {}
    for m in re.finditer(r"pub fn (b200kv_[a-z0-9_]+)\s*\((.*?)\)\s*(?:->\s*[^;]+)?;", block, flags=re.S):
        params = [p.strip() for p in m.group(2).split(",") if p.strip()]
        sigs[m.group(1)] = len(params)
    return sigs


def test_rust_binding_declares_exactly_the_header():
    # the Rust shim a tract maintainer drops in (rust-shim/b200kv_sys.rs) and INTEGRATION.md's extern block must bind
    # every symbol of the header, no more, with the same number of arguments
    header = open(os.path.join(ROOT, "include", "b200kv.h")).read()
    c = _c_signatures(header)
    assert len(c) >= 40
    rust = _rust_signatures(open(os.path.join(ROOT, "rust-shim", "b200kv_sys.rs")).read())
    assert set(rust) == set(c), set(rust) ^ set(c)
    for name, params in c.items():
        assert rust[name] == len(params), (name, rust[name], params)
    doc = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    in_doc = set(re.findall(r"pub fn (b200kv_[a-z0-9_]+)", doc))
    assert in_doc == set(c), in_doc ^ set(c)
    # the config struct: same fields, same order
    fields_c = re.findall(r"^\s*int(?:32|64)_t\s+([a-z_]+);", header[header.index("typedef struct {"):header.index("} b200kv_config;")], flags=re.M)
    rs = open(os.path.join(ROOT, "rust-shim", "b200kv_sys.rs")).read()
    fields_rs = re.findall(r"pub ([a-z_]+): i(?:32|64),", rs[rs.index("pub struct b200kv_config"):rs.index('extern "C" {')])
    assert fields_c == fields_rs, (fields_c, fields_rs)


def test_device_memory_is_allocated_at_create_only():
    # no entry point called after b200kv_create may allocate or free device memory: cudaMalloc / cudaFree appear in the
    # create / destroy functions of the cache (cache.cu, kivi.cu) and nowhere else
    csrc = os.path.join(ROOT, "tract_b200", "csrc")
    allowed = {"cache.cu": {"b200kv_create", "b200kv_destroy"}, "kivi.cu": {"kivi_create", "kivi_destroy"}}
    for f in sorted(os.listdir(csrc)):
        text = re.sub(r"//.*", "", open(os.path.join(csrc, f)).read())
        hits = [m.start() for m in re.finditer(r"\bcuda(Malloc|Free|MallocHost|FreeHost|MallocAsync|FreeAsync)\s*\(", text)]
        if not hits:
            continue
        assert f in allowed, f"{f} allocates device memory"
        for at in hits:
            # the function the call sits in: the last function header before it
            heads = list(re.finditer(r"^(?:extern \"C\" )?(?:static )?(?:int|void|int64_t)\s+(\w+)\s*\([^;{]*\)\s*\{", text[:at], flags=re.M))
            assert heads and heads[-1].group(1) in allowed[f], (f, heads[-1].group(1) if heads else None)
