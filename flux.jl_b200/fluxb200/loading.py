"""`Flux.state` / `Flux.loadmodel!` for models whose arrays live on the B200, plus optimiser-state save / restore and a
single-file checkpoint (src/loading.jl:1-189).

`state(model)` returns the model's structure made of basic containers only - dicts keyed by field name, tuples, host
(numpy) arrays, numbers, strings, None; activation names and other non-state leaves become `()`, as in the reference.
`loadmodel(dst, src)` walks `dst` and `src` (a model or a state) together and copies arrays into `dst`'s device
arrays in place, with the reference's error cases: mismatched structure, mismatched sizes, array <-> non-array leaves,
tied destination parameters loaded from different sources; `False` stands for an inactive (absent) parameter and is
interchangeable with an all-zero array.
"""
from __future__ import annotations

import json

import numpy as np
import torch

from .core import B200Array, cpu
from .layers import ArgumentError, DimensionMismatch, Layer

_STATE_TYPES = (int, float, str, bool, type(None), np.integer, np.floating)


def state(x):
    """Flux.state(x) (loading.jl:112-166)."""
    if isinstance(x, B200Array):
        return cpu(x)
    if isinstance(x, np.ndarray):
        return x
    if isinstance(x, Layer):
        return {name: state(getattr(x, name, None)) for name in x._fields}
    if isinstance(x, (tuple, list)):
        return tuple(state(v) for v in x)
    if isinstance(x, dict):
        return {k: state(v) for k, v in x.items()}
    if isinstance(x, _STATE_TYPES):
        return x
    return ()


def _children(x):
    if isinstance(x, Layer):
        return {name: getattr(x, name, None) for name in x._fields}
    if isinstance(x, dict):
        return x
    if isinstance(x, (tuple, list)):
        return {i: v for i, v in enumerate(x)}
    return None


def _is_array(x):
    return isinstance(x, (B200Array, np.ndarray))


def _is_zero(x):
    if isinstance(x, B200Array):
        return not bool(torch.any(x.t != 0).item())
    return not np.any(np.asarray(x) != 0)


def _loadleaf(dst, src):
    """loadleaf! (loading.jl:1-24)."""
    if _is_array(dst) and _is_array(src):
        ssize = src.size if isinstance(src, B200Array) else src.shape
        if tuple(dst.size) != tuple(ssize):
            raise DimensionMismatch(f"Tried to load size {tuple(ssize)} array into size {tuple(dst.size)}")
        if isinstance(src, B200Array):
            dst.t.copy_(src.t)
        else:
            flat = np.ascontiguousarray(np.asarray(src, dtype=np.float32 if dst.t.dtype == torch.float32 else None).reshape(-1, order="F"))
            dst.t.copy_(torch.from_numpy(flat).to(dst.t.dtype))
        return
    if _is_array(dst) and isinstance(src, (bool, np.bool_)):
        if src:
            raise ValueError("Cannot copy boolean parameter == true to non-zero parameter.")
        dst.t.zero_()
        return
    if isinstance(dst, (bool, np.bool_)) and _is_array(src):
        if dst or not _is_zero(src):
            raise ValueError("Cannot copy non-zero parameter to boolean parameter == true.")
        return
    if _is_array(dst):
        raise ValueError(f"Tried to copy {src!r} into an array destination; this is not allowed.")
    if _is_array(src):
        raise ValueError(f"Tried to copy an array to {dst!r}; this is not allowed.")
    # non-array leaves (activation names, numbers) are not copied and need not match


def loadmodel(dst, src, _cache=None):
    """Flux.loadmodel!(dst, src) (loading.jl:90-108): `dst` is a model on the B200, `src` a model or a `state`."""
    cache = {} if _cache is None else _cache
    cd, cs = _children(dst), _children(src)
    if cd is None or cs is None:
        raise ArgumentError("loadmodel: destination and source must be models or states")
    if list(cd.keys()) != list(cs.keys()):
        raise ArgumentError(f"Tried to load {tuple(cs.keys())} into {tuple(cd.keys())} but the structures do not match.")
    for k in cs:
        ldst, lsrc = cd[k], cs[k]
        leaf = _children(ldst) is None or (isinstance(ldst, (tuple, dict)) and len(ldst) == 0)
        if isinstance(ldst, B200Array) and id(ldst) in cache:
            # a tied destination parameter: every source it is loaded from must agree (loading.jl:26-33)
            prev = cache[id(ldst)]
            same = (_is_array(lsrc) and np.array_equal(cpu(ldst), cpu(lsrc) if isinstance(lsrc, B200Array) else np.asarray(lsrc)))
            if not same and not (isinstance(lsrc, (bool, np.bool_)) and not lsrc and _is_zero(ldst)):
                raise ValueError("Encountered tied destination parameters with untied and mismatched sources.")
            continue
        if leaf:
            if isinstance(ldst, B200Array):
                cache[id(ldst)] = lsrc
            _loadleaf(ldst, lsrc)
        else:
            loadmodel(ldst, lsrc, cache)
    return dst


# ----------------------------------------------------------------------------- optimiser state ---
def opt_state(opt) -> dict:
    """The optimiser state as basic containers: per trainable array (in `Flux.trainables` order) the moments m, v and
    the running powers (β1ᵗ, β2ᵗ) of Optimisers.Adam's Leaf state."""
    leaves = []
    seen = set()
    for p in opt.params:
        if id(p) in seen:
            continue
        seen.add(id(p))
        st = opt.leaves[id(p)].state
        leaves.append(None if st is None else {"m": cpu(st[0]), "v": cpu(st[1]), "bt": (float(st[2][0]), float(st[2][1]))})
    return {"rule": type(opt.rule).__name__, "leaves": leaves}


def load_opt_state(opt, saved: dict):
    """Restores what `opt_state` saved into an optimiser state built by `setup` for a model of the same structure."""
    if saved.get("rule") != type(opt.rule).__name__:
        raise ArgumentError(f"optimiser rule mismatch: saved {saved.get('rule')}, have {type(opt.rule).__name__}")
    params, seen = [], set()
    for p in opt.params:
        if id(p) not in seen:
            seen.add(id(p))
            params.append(p)
    if len(params) != len(saved["leaves"]):
        raise ArgumentError(f"optimiser state has {len(saved['leaves'])} leaves, the model has {len(params)} trainable arrays")
    for p, s in zip(params, saved["leaves"]):
        leaf = opt.leaves[id(p)]
        if leaf.master is not None:      # BFloat16 parameter: the Float32 master copy restarts from the loaded value
            leaf.master.t.copy_(p.t.float())
        st = leaf.state
        if (st is None) != (s is None):
            raise ArgumentError("optimiser state structure mismatch")
        if s is None:
            continue
        _loadleaf(st[0], s["m"])
        _loadleaf(st[1], s["v"])
        st[2] = (float(np.float32(s["bt"][0])), float(np.float32(s["bt"][1])))
    return opt


# ----------------------------------------------------------------------------------- one file ---
def _flatten(x, prefix, arrays, meta):
    if isinstance(x, np.ndarray):
        arrays[prefix] = x
        return {"__array__": prefix}
    if isinstance(x, dict):
        return {"__dict__": {str(k): _flatten(v, f"{prefix}/{k}", arrays, meta) for k, v in x.items()}}
    if isinstance(x, (tuple, list)):
        return {"__tuple__": [_flatten(v, f"{prefix}/{i}", arrays, meta) for i, v in enumerate(x)]}
    if isinstance(x, (np.integer, np.floating)):
        return x.item()
    return x


def _unflatten(node, arrays):
    if isinstance(node, dict):
        if "__array__" in node:
            return arrays[node["__array__"]]
        if "__dict__" in node:
            return {k: _unflatten(v, arrays) for k, v in node["__dict__"].items()}
        if "__tuple__" in node:
            return tuple(_unflatten(v, arrays) for v in node["__tuple__"])
    return node


def save_checkpoint(path, model, opt=None):
    """Writes `state(model)` (and the optimiser state) to one .npz file: arrays under path-like keys, the structure as
    a JSON string."""
    arrays: dict = {}
    tree = {"model": _flatten(state(model), "model", arrays, None)}
    if opt is not None:
        tree["opt"] = _flatten(opt_state(opt), "opt", arrays, None)
    np.savez(path, __structure__=np.array(json.dumps(tree)), **arrays)


def load_checkpoint(path, model, opt=None):
    """Reads a file written by `save_checkpoint` into `model` (and `opt`) in place; returns the model state."""
    with np.load(path, allow_pickle=False) as f:
        arrays = {k: f[k] for k in f.files if k != "__structure__"}
        tree = json.loads(str(f["__structure__"]))
    ms = _unflatten(tree["model"], arrays)
    loadmodel(model, ms)
    if opt is not None:
        if "opt" not in tree:
            raise ArgumentError("the checkpoint holds no optimiser state")
        load_opt_state(opt, _unflatten(tree["opt"], arrays))
    return ms
