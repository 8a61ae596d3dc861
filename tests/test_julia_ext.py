"""Static check of the Julia side of the boundary (flux.jl_b200/julia): every `ccall(sym(:fb_...), Ret, (types...), ...)`
must name an entry point that include/fluxb200.h declares, with the declared return type, the declared number of
arguments and a Julia C type of the right class for each of them (pointer / Int32 / Int64 / UInt64 / Float32).
The Julia sources cannot be executed here (no Julia toolchain), so this is what stands between them and a typo."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fluxb200.h")
JULIA = os.path.join(ROOT, "flux.jl_b200", "julia")


def header_signatures():
    src = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    out = {}
    for m in re.finditer(r"\b(int32_t|int64_t|const char\s*\*)\s+(fb_[a-z0-9_]+)\s*\(([^;]*?)\)\s*;", src, flags=re.S):
        ret, name, args = m.group(1), m.group(2), m.group(3).strip()
        kinds = []
        if args not in ("", "void"):
            for a in args.split(","):
                a = " ".join(a.split())
                if "*" in a:
                    kinds.append("ptr")
                elif a.startswith("int32_t"):
                    kinds.append("i32")
                elif a.startswith("int64_t"):
                    kinds.append("i64")
                elif a.startswith("uint64_t"):
                    kinds.append("u64")
                elif a.startswith("float"):
                    kinds.append("f32")
                else:
                    raise AssertionError(f"{name}: unclassified C parameter {a!r}")
        out[name] = ("cstr" if "char" in ret else ("i32" if ret == "int32_t" else "i64"), kinds)
    return out


JL_KIND = {"PV": "ptr", "Ptr{Cvoid}": "ptr", "Int32": "i32", "Int64": "i64", "UInt64": "u64", "Float32": "f32", "Cstring": "cstr"}


def julia_kind(t):
    t = t.strip()
    if t.startswith("Ptr{"):
        return "ptr"
    return JL_KIND.get(t)


def split_top(s):
    """Splits on commas that are not nested in brackets."""
    parts, depth, cur = [], 0, ""
    for ch in s:
        if ch in "({[":
            depth += 1
        elif ch in ")}]":
            depth -= 1
        if ch == "," and depth == 0:
            parts.append(cur)
            cur = ""
        else:
            cur += ch
    if cur.strip():
        parts.append(cur)
    return [p.strip() for p in parts]


def julia_ccalls():
    calls = []
    for dirpath, _, files in os.walk(JULIA):
        for f in files:
            if not f.endswith(".jl"):
                continue
            path = os.path.join(dirpath, f)
            src = open(path, encoding="utf-8").read()
            for m in re.finditer(r"ccall\(\s*sym\(\s*:?(\w+)\s*\)\s*,", src):
                name = m.group(1)
                # the text of the whole call: balance parentheses from the opening one
                i = src.index("(", m.start())
                depth, j = 0, i
                while True:
                    if src[j] == "(":
                        depth += 1
                    elif src[j] == ")":
                        depth -= 1
                        if depth == 0:
                            break
                    j += 1
                parts = split_top(src[i + 1:j])
                line = src.count("\n", 0, m.start()) + 1
                calls.append((os.path.relpath(path, ROOT), line, name, parts))
    return calls


def test_every_ccall_matches_the_header():
    sigs = header_signatures()
    calls = julia_ccalls()
    assert len(calls) >= 60, "the extension should bind the whole hot path"
    seen = set()
    for path, line, name, parts in calls:
        where = f"{path}:{line} {name}"
        if name in ("f",):     # cache_floats(f::Symbol, ...) binds the three *_cache_bytes functions by symbol
            ret, types, args = parts[1], split_top(parts[2].strip()[1:-1]), parts[3:]
            assert ret == "Int64" and [julia_kind(t) for t in types] == ["i64"] * 4 and len(args) == 4, where
            continue
        assert name in sigs, f"{where}: not declared in fluxb200.h"
        seen.add(name)
        want_ret, want = sigs[name]
        ret = parts[1]
        assert julia_kind(ret) == want_ret, f"{where}: return type {ret}, header says {want_ret}"
        tup = parts[2].strip()
        assert tup.startswith("(") and tup.endswith(")"), where
        types = split_top(tup[1:-1])
        assert len(types) == len(want), f"{where}: {len(types)} argument types, header declares {len(want)}"
        for k, (t, w) in enumerate(zip(types, want)):
            assert julia_kind(t) == w, f"{where}: argument {k + 1} is {t}, header wants {w}"
        args = parts[3:]
        assert len(args) == len(want), f"{where}: {len(args)} arguments passed, {len(want)} declared"
    # the bindings cover every layer family of the path
    for must in ("fb_dense_fwd", "fb_dense_bwd", "fb_layernorm_fwd", "fb_layernorm_bwd", "fb_batchnorm_fwd_train", "fb_batchnorm_bwd",
                 "fb_groupnorm_fwd", "fb_groupnorm_bwd", "fb_lstm_fwd", "fb_lstm_bwd", "fb_gru_fwd", "fb_gru_bwd", "fb_rnn_fwd",
                 "fb_rnn_bwd", "fb_gruv3_fwd", "fb_gruv3_bwd", "fb_attn_fwd", "fb_attn_bwd", "fb_attn_scores",
                 "fb_logitcrossentropy_dense", "fb_logitcrossentropy_labels", "fb_sumsq", "fb_adam_step", "fb_allreduce", "fb_bcast",
                 "fb_reduce", "fb_bucket_create", "fb_bucket_mark_ready", "fb_bucket_wait", "fb_embedding_fwd", "fb_embedding_bwd",
                 "fb_dropout", "fb_dense_fwd_bf16", "fb_dense_bwd_bf16", "fb_cast_f32_bf16", "fb_device_error", "fb_comm_async_error"):
        assert must in seen, f"{must} is not bound by the Julia extension"


def test_the_cache_size_symbols_exist():
    sigs = header_signatures()
    src = open(os.path.join(JULIA, "ext", "FluxB200Ext", "recurrent.jl"), encoding="utf-8").read()
    for name in re.findall(r"cache_floats\(:(\w+)", src):
        assert name in sigs and sigs[name] == ("i64", ["i64"] * 4), name


def test_every_pullback_that_writes_parameter_gradients_marks_them_ready():
    """GradientArena's overlap depends on it: a pullback that takes a gradient slice with grad_like(p) must call
    grad_done!(p) for the same parameter."""
    ext = os.path.join(JULIA, "ext", "FluxB200Ext")
    for f in os.listdir(ext):
        src = open(os.path.join(ext, f), encoding="utf-8").read()
        for fn in re.split(r"\nfunction ", src):
            taken = set(re.findall(r"grad_like\(([^)]+)\)", fn))
            done = set(re.findall(r"grad_done!\(([^)]+)\)", fn))
            taken.discard("p::B200Array")
            taken.discard("::Any")
            for p in taken:
                assert p in done, f"{f}: gradient slice of {p} is written but never marked ready"
