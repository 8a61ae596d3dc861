"""CPU-side checks of the drop-in boundary: the shared library loads and exports exactly the entry
points include/fluxb200.h declares, with matching ctypes prototypes; without a GPU every compute
path fails loudly (there is no CPU fallback)."""
import ctypes as C
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fluxb200.h")


def declared_symbols():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return re.findall(r"\b(?:int32_t|int64_t|const char\s*\*)\s+(fb_[a-z0-9_]+)\s*\(", src)


def declared_arg_counts():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    out = {}
    for m in re.finditer(r"\b(?:int32_t|int64_t|const char\s*\*)\s+(fb_[a-z0-9_]+)\s*\(([^;]*?)\)\s*;", src, flags=re.S):
        args = m.group(2).strip()
        out[m.group(1)] = 0 if args in ("", "void") else len(args.split(","))
    return out


def test_library_exports_every_declared_symbol():
    from fluxb200 import lib
    names = declared_symbols()
    assert len(names) >= 40 and len(set(names)) == len(names)
    handle = C.CDLL(lib.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} is declared in fluxb200.h but not exported"
    assert set(lib.PROTOTYPES) == set(names)


def test_prototypes_match_header_arity():
    from fluxb200 import lib
    counts = declared_arg_counts()
    for name, (_, argtypes) in lib.PROTOTYPES.items():
        assert counts[name] == len(argtypes), f"{name}: header has {counts[name]} arguments, binding has {len(argtypes)}"


def test_version_and_error_string():
    from fluxb200 import lib
    assert lib.raw().fb_version() == 100
    assert isinstance(lib.last_error(), str)


def test_null_context_is_rejected_without_touching_a_device():
    from fluxb200 import lib
    st = lib.raw().fb_sync(None, None)
    assert st == -1 and "ctx is NULL" in lib.last_error()
    st = lib.raw().fb_layernorm_fwd(None, None, None, None, None, None, None, None, 4, 4, 1e-5, 0)
    assert st == -1


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_no_cpu_fallback_without_a_gpu():
    from fluxb200 import lib
    h = C.c_void_p()
    st = lib.raw().fb_ctx_create(0, C.byref(h))
    assert st == -4 and "no CPU fallback" in lib.last_error()
    import fluxb200
    with pytest.raises(lib.FluxB200Error):
        fluxb200.context()


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "flux.jl_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".jl")):
                txt = open(os.path.join(dirpath, f), errors="replace").read()
                assert "flux_oracle" not in txt and "oracle/" not in txt, f
