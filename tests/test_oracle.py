"""Pins the CPU oracle: golden vectors produced by the reference itself, and (when it has been
compiled here) the reference's own CPU extension on fresh random inputs."""
import os

import numpy as np
import pytest

import oracle

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "scan_golden.npz"))
CASES = sorted({k.split("/")[0] for k in GOLDEN.files})
ROWS_CASES = [c for c in CASES if not c.startswith("cl_")]
CL_CASES = [c for c in CASES if c.startswith("cl_")]


def case(name):
    return {k: GOLDEN[f"{name}/{k}"] for k in ("a", "b", "g", "h", "ga", "gb")}


def test_golden_file_is_complete():
    assert len(ROWS_CASES) >= 10 and len(CL_CASES) >= 3
    assert any(GOLDEN[f"{c}/a"].dtype == np.float64 for c in CASES)
    # the "resets" case really holds exact zeros
    assert (case("resets_2x2048")["a"] == 0).mean() > 0.05


@pytest.mark.parametrize("name", ROWS_CASES)
def test_oracle_matches_reference_bit_for_bit(name):
    c = case(name)
    h = oracle.scan_forward(c["a"], c["b"])
    assert h.dtype == c["h"].dtype and np.array_equal(h, c["h"])
    ga, gb = oracle.scan_backward(c["a"], c["h"], c["g"])
    assert np.array_equal(gb, c["gb"])
    assert np.array_equal(ga, c["ga"])


@pytest.mark.parametrize("name", CL_CASES)
def test_channels_last_oracle_matches_reference(name):
    c = case(name)
    h = oracle.scan_forward_channels_last(c["a"], c["b"])
    assert np.array_equal(h, c["h"])
    ga, gb = oracle.scan_backward_channels_last(c["a"], c["h"], c["g"])
    assert np.array_equal(gb, c["gb"]) and np.array_equal(ga, c["ga"])
    # and it is the rows oracle applied to the transposed problem
    h2 = oracle.scan_forward(c["a"].transpose(0, 2, 1), c["b"].transpose(0, 2, 1)).transpose(0, 2, 1)
    assert np.array_equal(h, h2)


@pytest.mark.parametrize("splits", [[7], [1, 2, 3], [100, 613]])
def test_oracle_carries_reproduce_the_unsplit_scan(splits):
    """Splitting a sequence and threading the carries through is exact for a sequential scan."""
    rng = np.random.default_rng(5)
    a = rng.standard_normal((3, 1000)).astype(np.float32)
    b = rng.standard_normal((3, 1000)).astype(np.float32)
    g = rng.standard_normal((3, 1000)).astype(np.float32)
    h = oracle.scan_forward(a, b)
    ga, gb = oracle.scan_backward(a, h, g)
    cuts = [0] + list(np.cumsum(splits)) + [1000]
    # forward, left to right
    carry = np.zeros(3, np.float32)
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        part = oracle.scan_forward(a[:, lo:hi], b[:, lo:hi], h_in=carry)
        assert np.array_equal(part, h[:, lo:hi])
        carry = part[:, -1].copy()
    # backward, right to left: the carry is a_t*gb_t of the first step of the part to the right
    carry = np.zeros(3, np.float32)
    for lo, hi in reversed(list(zip(cuts[:-1], cuts[1:]))):
        h_prev = h[:, lo - 1].copy() if lo > 0 else None
        pga, pgb = oracle.scan_backward(a[:, lo:hi], h[:, lo:hi], g[:, lo:hi], gb_in=carry, h_prev=h_prev)
        assert np.array_equal(pgb, gb[:, lo:hi]) and np.array_equal(pga, ga[:, lo:hi])
        carry = (a[:, lo] * pgb[:, 0]).astype(np.float32)


def test_oracle_edge_shapes():
    z = np.zeros((4, 0), np.float32)
    assert oracle.scan_forward(z, z).shape == (4, 0)
    one = np.full((2, 1), 3.0, np.float32)
    assert np.array_equal(oracle.scan_forward(one, one), one)  # h_0 = a*0 + b
    ga, gb = oracle.scan_backward(one, one, one)
    assert np.array_equal(gb, one) and np.array_equal(ga, np.zeros_like(one))
    with pytest.raises(AssertionError):
        oracle.scan_forward(np.zeros(5, np.float32), np.zeros(5, np.float32))
    with pytest.raises(TypeError):
        oracle.scan_forward(np.zeros((2, 2), np.float16), np.zeros((2, 2), np.float16))


@pytest.mark.skipif(not oracle.reference_available(), reason="reference CPU extension not built here")
@pytest.mark.parametrize("shape,dtype", [((32, 5), "float32"), ((32, 1025), "float32"), ((7, 4100), "float32"),
                                         ((5, 333), "float64")])
def test_oracle_matches_compiled_reference(shape, dtype):
    import torch

    rng = np.random.default_rng(11)
    a, b, g = (rng.standard_normal(shape).astype(dtype) for _ in range(3))
    ta, tb, tg = (torch.from_numpy(x) for x in (a, b, g))
    h_ref = oracle.reference_forward(ta, tb)
    ga_ref, gb_ref = oracle.reference_backward(ta, h_ref, tg)
    h = oracle.scan_forward(a, b)
    ga, gb = oracle.scan_backward(a, h, g)
    assert np.array_equal(h, h_ref.numpy())
    assert np.array_equal(ga, ga_ref.numpy()) and np.array_equal(gb, gb_ref.numpy())
