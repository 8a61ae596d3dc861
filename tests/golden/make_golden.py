"""Generates tests/golden/oracle_vectors.npz: seeded inputs and float64 oracle outputs for every function on the
hot path, at sizes that run in milliseconds.

    python tests/golden/make_golden.py

The reference itself (Flux.jl) cannot be run here (no Julia toolchain), so these vectors pin the *oracle* against
silent drift; the oracle in turn is pinned to the reference's own known-answer tests in tests/test_oracle_golden.py.
The GPU parity tests load the same file and compare the CUDA library against it.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import flux_oracle as O  # noqa: E402


def generate():
    rng = np.random.default_rng(20240607)
    out = {}
    # Dense: W (6,5), b, x (5,7), relu / gelu
    W, b, x, dy = rng.normal(size=(6, 5)), rng.normal(size=6), rng.normal(size=(5, 7)), rng.normal(size=(6, 7))
    out.update(dense_W=W, dense_b=b, dense_x=x, dense_dy=dy)
    for act in ("relu", "gelu_tanh"):
        out[f"dense_y_{act}"] = O.dense_fwd(W, b, x, act)
        dW, db, dx = O.dense_bwd(W, b, x, dy, act)
        out[f"dense_dW_{act}"], out[f"dense_db_{act}"], out[f"dense_dx_{act}"] = dW, db, dx
    # LayerNorm (8, 5)
    x, g, be, dy = rng.normal(size=(8, 5)), rng.normal(size=8) + 1, rng.normal(size=8), rng.normal(size=(8, 5))
    out.update(ln_x=x, ln_g=g, ln_b=be, ln_dy=dy, ln_y=O.layernorm_fwd(x, g, be))
    out["ln_dx"], out["ln_dg"], out["ln_db"] = O.layernorm_bwd(x, g, be, dy)
    # BatchNorm WHCN (3, 2, 4, 5), relu
    x, g, be, dy = rng.normal(size=(3, 2, 4, 5)) * 2 + 0.5, rng.normal(size=4) + 1.5, rng.normal(size=4), rng.normal(size=(3, 2, 4, 5))
    y, nm, nv = O.batchnorm_fwd_train(x, g, be, np.zeros(4), np.ones(4), 0.1, 1e-5, "relu")
    out.update(bn_x=x, bn_g=g, bn_b=be, bn_dy=dy, bn_y=y, bn_mean=nm, bn_var=nv)
    out["bn_dx"], out["bn_dg"], out["bn_db"] = O.batchnorm_bwd(x, g, be, dy, 1e-5, "relu")
    # LSTM / GRU: I=3, H=4, T=5, B=2
    for name, ng, fwd, bwd in (("lstm", 4, O.lstm_scan_fwd, O.lstm_scan_bwd), ("gru", 3, O.gru_scan_fwd, O.gru_scan_bwd)):
        Wi, Wh, bb = rng.normal(size=(ng * 4, 3)) * .5, rng.normal(size=(ng * 4, 4)) * .5, rng.normal(size=ng * 4) * .1
        xs = rng.normal(size=(3, 5, 2))
        o = fwd(Wi, Wh, bb, xs)[0]
        dWi, dWh, dbb, dxs = bwd(Wi, Wh, bb, xs, 2 * o)
        out.update({f"{name}_Wi": Wi, f"{name}_Wh": Wh, f"{name}_b": bb, f"{name}_x": xs, f"{name}_out": o,
                    f"{name}_dWi": dWi, f"{name}_dWh": dWh, f"{name}_db": dbb, f"{name}_dx": dxs})
    # attention: E=8, heads=2, L=6, B=2, causal
    q, k, v, do = (rng.normal(size=(8, 6, 2)) for _ in range(4))
    mask = O.make_causal_mask(6)
    o, a = O.dot_product_attention(q, k, v, None, 2, mask)
    dq, dk, dv = O.dot_product_attention_bwd(q, k, v, do, None, 2, mask)
    out.update(attn_q=q, attn_k=k, attn_v=v, attn_do=do, attn_o=o, attn_alpha=a, attn_dq=dq, attn_dk=dk, attn_dv=dv)
    # loss
    yhat, lab = rng.normal(size=(5, 9)) * 2, rng.integers(1, 6, size=9)
    y1h = O.onehotbatch(lab, 5, np.float64)
    out.update(xent_yhat=yhat, xent_labels=lab.astype(np.int64), xent_loss=np.array(O.logitcrossentropy(yhat, y1h)),
               xent_dyhat=O.logitcrossentropy_bwd(yhat, y1h))
    # Adam: 3 steps on one leaf (float32 arithmetic, as the rule runs)
    w = rng.normal(size=11).astype(np.float32)
    st = O.adam_init(w)
    gs = rng.normal(size=(3, 11)).astype(np.float32)
    w3 = w.copy()
    for gstep in gs:
        w3 = O.adam_apply(st, w3, gstep)
    out.update(adam_w0=w, adam_g=gs, adam_w3=w3, adam_m3=st[0], adam_v3=st[1])
    return {k: np.asarray(v) for k, v in out.items()}


if __name__ == "__main__":
    path = os.path.join(HERE, "oracle_vectors.npz")
    np.savez_compressed(path, **generate())
    print("wrote", path, os.path.getsize(path), "bytes")
