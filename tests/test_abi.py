"""CPU: the shared library builds for sm_100a, loads, and exports every symbol include/petb200.h declares.
No compute call is made here (there is no GPU in this process)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols(header="petb200.h"):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(petb200_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    from pet_b200 import build, lib
    path = build.build()
    assert os.path.exists(path)
    handle = ctypes.CDLL(path)
    names = declared_symbols()
    assert len(names) >= 35
    for name in names:
        assert hasattr(handle, name), f"{name} is declared in include/petb200.h but not exported"
    # the Python binding covers the same set
    assert sorted(lib.SYMBOLS) == names
    graph_names = declared_symbols("petb200_graph.h")
    assert len(graph_names) >= 40
    for name in graph_names:
        assert hasattr(handle, name), f"{name} is declared in include/petb200_graph.h but not exported"
    from pet_b200 import graph
    assert sorted(graph.GRAPH_SYMBOLS) == graph_names


def test_status_strings_and_ctx_create_without_gpu():
    from pet_b200 import lib
    l = lib.load()
    assert l.petb200_status_string(0) == b"ok"
    assert l.petb200_status_string(2) == b"unsupported"
    import torch
    if not torch.cuda.is_available():
        h = ctypes.c_void_p()
        rc = l.petb200_ctx_create(0, ctypes.byref(h))
        assert rc == lib.ERR_CUDA and not h.value  # fails loudly, no CPU fallback
        assert b"CUDA" in l.petb200_last_error(None) or b"device" in l.petb200_last_error(None)


def test_product_does_not_use_the_oracle():
    """The CPU oracle is test infrastructure: nothing under pet_b200/ may import, include, link or load it."""
    pkg = os.path.join(ROOT, "pet_b200")
    pat = re.compile(r"(import\s+oracle|from\s+oracle|pet_oracle|petref|libpet_oracle|#include\s+\".*oracle)")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".h", ".cuh", ".cc")):
                text = open(os.path.join(dirpath, f)).read()
                assert not pat.search(text), f"{os.path.join(dirpath, f)} reaches into oracle/"
