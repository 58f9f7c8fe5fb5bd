"""The CPU restatement of the learned-grid quantize-dequantize against outputs of the reference's own backend
(tests/golden/affine_qdq.npz), and the host-side layout logic of the CUDA path."""
import importlib.util
import os

import numpy as np
import pytest

HERE = os.path.dirname(__file__)
_spec = importlib.util.spec_from_file_location("affine_qdq_oracle", os.path.join(HERE, "..", "oracle", "affine_qdq_oracle.py"))
oracle = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(oracle)

GOLDEN = np.load(os.path.join(HERE, "golden", "affine_qdq.npz"))
BLOCK_CASES = sorted(key.split("/")[0] for key in GOLDEN.files if key.endswith("/block_size"))
CASES = sorted({key.split("/")[0] for key in GOLDEN.files} - {"nan"} - set(BLOCK_CASES))


def case_arrays(name):
    g = {key.split("/", 1)[1]: GOLDEN[key] for key in GOLDEN.files if key.startswith(name + "/")}
    n = g["x"].size
    for flags in ("keep", "fast_keep"):
        if flags in g:
            g[flags] = np.unpackbits(g[flags])[:n].astype(bool).reshape(g["x"].shape)
    return g


def same_bits(a, b):
    """Equal bit for bit (signed zeros included); a NaN matches a NaN of any payload."""
    a, b = np.asarray(a, dtype=np.float32), np.asarray(b, dtype=np.float32)
    if a.shape != b.shape or not np.array_equal(np.isnan(a), np.isnan(b)):
        return False
    real = ~np.isnan(a)
    return np.array_equal(a.view(np.uint32)[real], b.view(np.uint32)[real])


@pytest.mark.parametrize("name", CASES)
def test_oracle_divide_form_matches_the_reference(name):
    g = case_arrays(name)
    qmin, qmax = (int(v) for v in g["range"])
    y, keep = oracle.divide_form(g["x"], g["scale"], g["offset"], qmin, qmax)
    assert same_bits(y, g["y"])
    assert np.array_equal(keep, g["keep"])
    dx, scale_terms, offset_terms = oracle.divide_form_backward(g["grad"], g["x"], g["scale"], g["offset"], qmin, qmax)
    assert same_bits(dx, g["grad"] * g["keep"])
    tolerance = 1e-5 * np.maximum(g["dscale_abs"], 1e-30)
    assert np.all(np.abs(oracle.reduce_to_grid(scale_terms, g["scale"].shape) - g["dscale"]) <= tolerance)
    want = g["doffset"]
    assert np.allclose(oracle.reduce_to_grid(offset_terms, g["offset"].shape), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("name", CASES)
def test_oracle_reciprocal_form_matches_the_reference(name):
    g = case_arrays(name)
    qmin, qmax = (int(v) for v in g["range"])
    y, keep = oracle.reciprocal_form(g["x"], g["scale"], g["offset"], qmin, qmax)
    assert same_bits(y, g["fast_y"])
    assert np.array_equal(keep, g["fast_keep"])


def test_oracle_nan_inputs():
    x = GOLDEN["nan/x"]
    assert np.isnan(x).sum() == 3
    y, keep = oracle.divide_form(x, np.float32(0.05), np.float32(-3.0), -128, 127)
    assert same_bits(y, GOLDEN["nan/y"]) and not keep[np.isnan(x)].any()
    y, keep = oracle.reciprocal_form(x, np.float32(0.05), np.float32(-3.0), -128, 127)
    assert same_bits(y, GOLDEN["nan/fast_y"]) and not keep[np.isnan(x)].any()


def test_the_two_forms_differ_only_by_the_rounding_of_the_quotient():
    g = case_arrays("rows_int8_vector")
    y_div, _ = oracle.divide_form(g["x"], g["scale"], g["offset"], -128, 127)
    y_rec, _ = oracle.reciprocal_form(g["x"], g["scale"], g["offset"], -128, 127)
    step = np.broadcast_to(g["scale"], g["x"].shape)
    assert np.all(np.abs(y_div - y_rec) <= step * 1.0001)


def test_grid_layout():
    from rx_met_b200.affine_qdq import grid_layout
    assert grid_layout((4, 5, 6), ()) == (1, 1, 120)
    assert grid_layout((4, 5, 6), (1,)) == (1, 1, 120)
    assert grid_layout((4, 5, 6), (6,)) == (20, 6, 1)
    assert grid_layout((4, 5, 6), (5, 1)) == (4, 5, 6)
    assert grid_layout((4, 5, 6), (4, 1, 1)) == (1, 4, 30)
    for bad in ((4, 6), (5,), (2, 1, 1), (1, 1, 1, 6)):
        with pytest.raises(RuntimeError):
            grid_layout((4, 5, 6), bad)


@pytest.mark.parametrize("name", BLOCK_CASES)
def test_oracle_blockwise_grids_match_the_reference(name):
    g = case_arrays(name)
    qmin, qmax = (int(v) for v in g["range"])
    scale, offset = oracle.expand_blocks(g["scale"], g["x"].shape), oracle.expand_blocks(g["offset"], g["x"].shape)
    y, keep = oracle.divide_form(g["x"], scale, offset, qmin, qmax)
    assert same_bits(y, g["y"]) and np.array_equal(keep, g["keep"])
    dx, scale_terms, offset_terms = oracle.divide_form_backward(g["grad"], g["x"], scale, offset, qmin, qmax)
    assert same_bits(dx, g["grad"] * g["keep"])
    size = oracle.reduce_to_blocks(np.abs(scale_terms), g["scale"].shape)
    assert np.all(np.abs(oracle.reduce_to_blocks(scale_terms, g["scale"].shape) - g["dscale"]) <= 1e-5 * size + 1e-30)
    assert np.allclose(oracle.reduce_to_blocks(offset_terms, g["offset"].shape), g["doffset"], rtol=1e-5, atol=1e-5)


def test_blocked_shapes():
    from rx_met_b200.affine_qdq import blocked_shapes, grid_layout
    assert blocked_shapes((8, 64), (8, 4), (1, 16)) == ((8, 1, 4, 16), (8, 1, 4, 1))
    assert blocked_shapes((8, 64), (8, 4), (-1, -1)) == ((8, 1, 4, 16), (8, 1, 4, 1))
    assert grid_layout(*blocked_shapes((8, 64), (8, 4), (1, 16))) == (1, 32, 16)
    assert grid_layout(*blocked_shapes((6, 32, 3, 3), (6, 2, 1, 1), (-1, 16, -1, -1))) == (1, 12, 144)
    assert grid_layout(*blocked_shapes((5, 8, 64), (8, 4), (1, 16))) == (5, 32, 16)
    assert grid_layout((4, 5, 6), (4, 5, 1)) == (1, 20, 6)
    for bad in (((8, 64), (8, 4), (1, 8)), ((8, 64), (8, 4), (16,)), ((64,), (8, 4), (1, 16))):
        with pytest.raises(RuntimeError):
            blocked_shapes(*bad)
    with pytest.raises(RuntimeError):   # blocks along the first of two dimensions: entries are not contiguous
        grid_layout(*blocked_shapes((8, 64), (2, 64), (4, 1)))
