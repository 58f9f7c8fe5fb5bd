"""CUDA path of the learned-grid quantize-dequantize: against outputs of the reference's own backend
(tests/golden/affine_qdq.npz), against the CPU restatement on larger seeded tensors, and through autograd."""
import numpy as np
import pytest
import torch

from test_affine_qdq_cpu import BLOCK_CASES, CASES, GOLDEN, case_arrays, oracle, same_bits

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run_both(x, scale, offset, grad, qmin, qmax):
    from rx_met_b200 import affine_qdq
    xt, st, ot, gt = dev(x), dev(scale), dev(offset), dev(grad)
    out = {}
    y, keep = affine_qdq.forward(xt, st, ot, qmin, qmax, reciprocal=False, want_keep=True)
    out["y"], out["keep"] = y.cpu().numpy(), keep.cpu().numpy()
    y, keep = affine_qdq.forward(xt, st, ot, qmin, qmax, reciprocal=True, want_keep=True)
    out["fast_y"], out["fast_keep"] = y.cpu().numpy(), keep.cpu().numpy()
    dx, ds, do = affine_qdq.backward(gt, xt, st, ot, qmin, qmax, reciprocal=False, want_scale_grad=True,
                                     want_offset_grad=True)
    out["dx"], out["dscale"], out["doffset"] = dx.cpu().numpy(), ds.cpu().numpy(), do.cpu().numpy()
    dx, _, _ = affine_qdq.backward(gt, xt, st, ot, qmin, qmax, reciprocal=True)
    out["fast_dx"] = dx.cpu().numpy()
    return out


@pytest.mark.parametrize("name", CASES)
def test_cuda_matches_the_reference(name):
    g = case_arrays(name)
    qmin, qmax = (int(v) for v in g["range"])
    got = run_both(g["x"], g["scale"], g["offset"], g["grad"], qmin, qmax)
    assert same_bits(got["y"], g["y"]) and np.array_equal(got["keep"], g["keep"])
    assert same_bits(got["fast_y"], g["fast_y"]) and np.array_equal(got["fast_keep"], g["fast_keep"])
    assert same_bits(got["dx"], g["grad"] * g["keep"])
    assert same_bits(got["fast_dx"], g["grad"] * g["fast_keep"])
    tolerance = 1e-5 * np.maximum(g["dscale_abs"], 1e-30)   # 1e-5 of the magnitude that was summed
    assert np.all(np.abs(got["dscale"].reshape(g["dscale"].shape) - g["dscale"]) <= tolerance)
    assert np.allclose(got["doffset"].reshape(g["doffset"].shape), g["doffset"], rtol=1e-5, atol=1e-5)


def test_cuda_nan_inputs():
    from rx_met_b200 import affine_qdq
    x = GOLDEN["nan/x"]
    s, o = dev(np.float32(0.05).reshape(())), dev(np.float32(-3.0).reshape(()))
    y, keep = affine_qdq.forward(dev(x), s, o, -128, 127, reciprocal=False, want_keep=True)
    assert same_bits(y.cpu().numpy(), GOLDEN["nan/y"]) and not keep.cpu().numpy()[np.isnan(x)].any()
    y, keep = affine_qdq.forward(dev(x), s, o, -128, 127, reciprocal=True, want_keep=True)
    assert same_bits(y.cpu().numpy(), GOLDEN["nan/fast_y"]) and not keep.cpu().numpy()[np.isnan(x)].any()


@pytest.mark.parametrize("shape,grid_shape,qmin,qmax", [
    ((3, 1 << 20), (), -128, 127),              # per tensor, many segments
    ((512, 4096), (512, 1), -128, 127),         # a weight matrix, one grid entry per output row
    ((96, 1000), (96, 1), -8, 7),               # rows that are not a multiple of four long
    ((4096, 768), (768,), 0, 255),              # activations, grid along the last axis
    ((33, 40, 50), (40, 1), -32768, 32767),     # middle axis, short rows
    ((9, 16, 300), (16, 1), -128, 127),         # middle axis, long rows, several outer slices
    ((2048, 64), (2048, 1), -128, 127),         # short rows that are whole grid entries: 16 lanes per row
    ((300, 37), (300, 1), -8, 7),               # the same with rows that are not a multiple of four long
    ((1000, 8), (1000, 1), -128, 127),          # two lanes per row
])
def test_cuda_matches_the_restatement_on_larger_tensors(shape, grid_shape, qmin, qmax):
    rng = np.random.default_rng(abs(hash((shape, grid_shape))) % (1 << 31))
    count = int(np.prod(grid_shape)) if grid_shape else 1
    scale = rng.uniform(0.005, 0.1, size=count).astype(np.float32).reshape(grid_shape)
    offset = np.zeros(grid_shape, dtype=np.float32) if count > 1 else np.float32(rng.integers(qmin // 2, 1)).reshape(())
    span = (qmax - qmin) * 0.6
    x = (rng.standard_normal(shape) * span * np.broadcast_to(scale, shape) * 0.5).astype(np.float32)
    x.reshape(-1)[:: 97] = 0.0
    grad = rng.standard_normal(shape).astype(np.float32)
    got = run_both(x, scale, offset, grad, qmin, qmax)
    y, keep = oracle.divide_form(x, scale, offset, qmin, qmax)
    assert same_bits(got["y"], y) and np.array_equal(got["keep"], keep)
    assert 0.02 < 1.0 - keep.mean() < 0.6   # the case does clip
    y, keep_fast = oracle.reciprocal_form(x, scale, offset, qmin, qmax)
    assert same_bits(got["fast_y"], y) and np.array_equal(got["fast_keep"], keep_fast)
    dx, scale_terms, offset_terms = oracle.divide_form_backward(grad, x, scale, offset, qmin, qmax)
    assert same_bits(got["dx"], dx)
    assert same_bits(got["fast_dx"], grad * keep_fast)
    want = oracle.reduce_to_grid(scale_terms, grid_shape)
    size = oracle.reduce_to_grid(np.abs(scale_terms), grid_shape)
    assert np.all(np.abs(got["dscale"].reshape(want.shape) - want) <= 1e-5 * size)
    want = oracle.reduce_to_grid(offset_terms, grid_shape)
    size = oracle.reduce_to_grid(np.abs(offset_terms), grid_shape)
    assert np.all(np.abs(got["doffset"].reshape(want.shape) - want) <= 1e-5 * size + 1e-30)


def test_gradients_are_the_same_on_every_run():
    from rx_met_b200 import affine_qdq
    rng = np.random.default_rng(3)
    x, grad = dev(rng.standard_normal((256, 3000)).astype(np.float32)), dev(rng.standard_normal((256, 3000)).astype(np.float32))
    s, o = dev(np.full((256, 1), 0.02, np.float32)), dev(np.zeros((256, 1), np.float32))
    first = affine_qdq.backward(grad, x, s, o, -128, 127, reciprocal=False, want_scale_grad=True, want_offset_grad=True)
    for _ in range(3):
        again = affine_qdq.backward(grad, x, s, o, -128, 127, reciprocal=False, want_scale_grad=True, want_offset_grad=True)
        assert all(torch.equal(a, b) for a, b in zip(first, again))


def test_autograd_function_and_form_selection():
    from rx_met_b200 import affine_qdq
    g = case_arrays("rows_int8_vector")
    x = dev(g["x"]).requires_grad_()
    s, o = dev(g["scale"]).requires_grad_(), dev(g["offset"]).requires_grad_()
    y = affine_qdq.quantize_dequantize(x, s, o, -128, 127)
    y.backward(dev(g["grad"]))
    assert same_bits(y.detach().cpu().numpy(), g["y"])
    assert same_bits(x.grad.cpu().numpy(), g["grad"] * g["keep"])
    assert s.grad.shape == s.shape and o.grad.shape == o.shape
    assert np.all(np.abs(s.grad.cpu().numpy() - g["dscale"]) <= 1e-5 * g["dscale_abs"])
    # a grid that is not trained takes the fast form, like the reference
    x2 = dev(g["x"]).requires_grad_()
    y2 = affine_qdq.quantize_dequantize(x2, dev(g["scale"]), dev(g["offset"]), -128, 127)
    y2.backward(dev(g["grad"]))
    assert same_bits(y2.detach().cpu().numpy(), g["fast_y"])
    assert same_bits(x2.grad.cpu().numpy(), g["grad"] * g["fast_keep"])
    with torch.no_grad():
        y3 = affine_qdq.quantize_dequantize(dev(g["x"]), s, o, -128, 127)
    assert same_bits(y3.cpu().numpy(), g["fast_y"])


def test_refusals():
    from rx_met_b200 import affine_qdq
    x = torch.zeros(8, 8, device="cuda")
    s, o = torch.ones(8, 1, device="cuda"), torch.zeros(8, 1, device="cuda")
    with pytest.raises(RuntimeError):
        affine_qdq.quantize_dequantize(x, s, o, -128, 127, block_size=[1, 3])
    with pytest.raises(RuntimeError):
        affine_qdq.quantize_dequantize(x, s, o, -128, 127, zero_point_shift=0.5)
    with pytest.raises(RuntimeError):
        affine_qdq.quantize_dequantize(x.double(), s, o, -128, 127)
    with pytest.raises(RuntimeError):
        affine_qdq.quantize_dequantize(x.cpu(), s.cpu(), o.cpu(), -128, 127)
    with pytest.raises((RuntimeError, ValueError)):
        affine_qdq.forward(x, s, o, 5, 5, reciprocal=False)
    with pytest.raises((RuntimeError, ValueError)):
        affine_qdq.backward(x, x, s, o, -128, 127, reciprocal=True, want_scale_grad=True)
    empty = torch.zeros(0, 8, device="cuda")
    y, _ = affine_qdq.forward(empty, torch.ones((), device="cuda"), torch.zeros((), device="cuda"), -128, 127, reciprocal=False)
    assert y.shape == empty.shape


@pytest.mark.parametrize("name", BLOCK_CASES)
def test_cuda_blockwise_grids_match_the_reference(name):
    from rx_met_b200 import affine_qdq
    g = case_arrays(name)
    qmin, qmax = (int(v) for v in g["range"])
    block_size = [int(v) for v in g["block_size"]]
    x = dev(g["x"]).requires_grad_()
    s, o = dev(g["scale"]).requires_grad_(), dev(g["offset"]).requires_grad_()
    y = affine_qdq.quantize_dequantize(x, s, o, qmin, qmax, block_size=block_size)
    y.backward(dev(g["grad"]))
    assert same_bits(y.detach().cpu().numpy(), g["y"])
    assert same_bits(x.grad.cpu().numpy(), g["grad"] * g["keep"])
    scale_full = oracle.expand_blocks(g["scale"], g["x"].shape)
    _, scale_terms, _ = oracle.divide_form_backward(g["grad"], g["x"], scale_full, np.zeros_like(scale_full), qmin, qmax)
    size = oracle.reduce_to_blocks(np.abs(scale_terms), g["scale"].shape)
    assert s.grad.shape == s.shape
    assert np.all(np.abs(s.grad.cpu().numpy() - g["dscale"]) <= 1e-5 * size + 1e-30)
    assert np.allclose(o.grad.cpu().numpy(), g["doffset"], rtol=1e-5, atol=1e-5)
    # a blockwise grid that is not trained still takes the divide form
    with torch.no_grad():
        y2 = affine_qdq.quantize_dequantize(dev(g["x"]), s, o, qmin, qmax, block_size=block_size)
    assert same_bits(y2.cpu().numpy(), g["y"])


@pytest.mark.parametrize("shape,grid_shape,block_size", [
    ((512, 1024), (512, 16), [1, 64]),
    ((96, 384), (96, 3), [-1, 128]),
    ((64, 48, 3, 3), (64, 3, 1, 1), [-1, 16, -1, -1]),
])
def test_cuda_blockwise_grids_match_the_restatement_on_larger_tensors(shape, grid_shape, block_size):
    from rx_met_b200 import affine_qdq
    rng = np.random.default_rng(sum(shape))
    scale = rng.uniform(0.005, 0.1, size=grid_shape).astype(np.float32)
    offset = np.zeros(grid_shape, dtype=np.float32)
    full = oracle.expand_blocks(scale, shape)
    x = (rng.standard_normal(shape) * 5.0 * full).astype(np.float32)
    grad = rng.standard_normal(shape).astype(np.float32)
    xt, st, ot, gt = dev(x), dev(scale), dev(offset), dev(grad)
    y, keep = affine_qdq.forward(xt, st, ot, -8, 7, reciprocal=False, want_keep=True, block_size=block_size)
    want_y, want_keep = oracle.divide_form(x, full, np.zeros_like(full), -8, 7)
    assert same_bits(y.cpu().numpy(), want_y) and np.array_equal(keep.cpu().numpy(), want_keep)
    assert 0.02 < 1.0 - want_keep.mean() < 0.6
    dx, ds, do = affine_qdq.backward(gt, xt, st, ot, -8, 7, reciprocal=False, want_scale_grad=True, want_offset_grad=True,
                                     block_size=block_size)
    want_dx, scale_terms, offset_terms = oracle.divide_form_backward(grad, x, full, np.zeros_like(full), -8, 7)
    assert same_bits(dx.cpu().numpy(), want_dx)
    for got, terms in ((ds, scale_terms), (do, offset_terms)):
        want = oracle.reduce_to_blocks(terms, grid_shape)
        size = oracle.reduce_to_blocks(np.abs(terms), grid_shape)
        assert got.shape == want.shape
        assert np.all(np.abs(got.cpu().numpy() - want) <= 1e-5 * size + 1e-30)


def test_backward_of_nan_inputs():
    """A NaN input has no gradient of its own (it is outside the grid) and makes the scale gradient NaN, as in the
    reference's expressions; the offset gradient stays finite."""
    from rx_met_b200 import affine_qdq
    x = GOLDEN["nan/x"]
    grad = np.ones_like(x)
    s, o = dev(np.float32(0.05).reshape(())), dev(np.float32(-3.0).reshape(()))
    dx, ds, do = affine_qdq.backward(dev(grad), dev(x), s, o, -128, 127, reciprocal=False, want_scale_grad=True,
                                     want_offset_grad=True)
    want_dx, scale_terms, offset_terms = oracle.divide_form_backward(grad, x, np.float32(0.05), np.float32(-3.0), -128, 127)
    assert same_bits(dx.cpu().numpy(), want_dx) and not dx.cpu().numpy()[np.isnan(x)].any()
    assert np.isnan(scale_terms).sum() == 3 and np.isnan(ds.cpu().numpy()).all()
    assert np.allclose(do.cpu().numpy().reshape(()), offset_terms.astype(np.float64).sum(), rtol=1e-5)
