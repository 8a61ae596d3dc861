"""CPU checks of the host-side mirror: initialisers (test/utils.jl:53-59, 95-104), constructor dimension logic and
the gradient-bucket bookkeeping for parameters that are used more than once."""
import numpy as np
import pytest

import flux_oracle as O


def test_nfan_table():
    """test/utils.jl:53-59."""
    import fluxb200 as F
    assert F.nfan() == (1, 1)
    assert F.nfan(100) == (1, 100)
    assert F.nfan(100, 200) == (200, 100) == F.nfan((100, 200))
    assert F.nfan(2, 30, 40) == (2 * 30, 2 * 40)
    assert F.nfan(2, 3, 40, 50) == (2 * 3 * 40, 2 * 3 * 50)
    assert F.nfan(2, 3, 4, 50, 60) == (2 * 3 * 4 * 50, 2 * 3 * 4 * 60)


def test_glorot_uniform_variance_and_eltype():
    """test/utils.jl:95-104: variance within 10 % of 2 / (fan_in + fan_out); Float32 output."""
    import fluxb200 as F
    F.seed(0)
    for dims in [(1000,), (100, 100), (100, 400), (2, 3, 32, 64), (2, 3, 4, 32, 64)]:
        v = F.glorot_uniform(*dims)
        fan_in, fan_out = F.nfan(*dims)
        s2 = 2 / (fan_in + fan_out)
        assert v.shape == dims and 0.9 * s2 < v.var() < 1.1 * s2
    assert F.glorot_uniform(3, 4, gain=1.5).dtype == np.float32
    # the same stream and scale as the oracle's restatement of src/utils.jl:81-84
    a = F.glorot_uniform(np.random.default_rng(5), 7, 9, gain=2.0)
    b = O.glorot_uniform(np.random.default_rng(5), 7, 9, gain=2.0)
    assert (a == b).all()
    # glorot_uniform(rng; gain) without dims returns a bound initialiser (src/utils.jl:86)
    init = F.glorot_uniform(np.random.default_rng(5), gain=2.0)
    assert (init(7, 9) == b).all()


def test_create_bias():
    """src/utils.jl:537-543."""
    import fluxb200 as F
    w = np.zeros((3, 4), np.float32)
    assert (F.create_bias(w, True, 3) == np.zeros(3, np.float32)).all()
    assert F.create_bias(w, False, 3) is False
    assert F.create_bias(w, np.arange(3.0), 3).dtype == np.float32
    with pytest.raises(F.DimensionMismatch):
        F.create_bias(w, np.zeros(4), 3)
