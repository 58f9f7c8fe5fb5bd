"""CPU restatement of the affine quantize-dequantize with a learned grid.  Test infrastructure: only the
tests and the bench's CPU leg import it; the product never does.

Follows src/aimet_torch/v2/quantization/affine/backends/torch_builtins.py of the reference:
  * `divide_form`      - QuantDequantFunc._forward_impl (:640-669) and .backward (:675-691);
  * `reciprocal_form`  - the torch.fake_quantize fast path chosen at :217-250 (per tensor :372-402, per
                         channel :405-440), whose kernel computes rne(x * (1 / s)) + zp on integers, with
                         NaN inputs restored afterwards (:243-250).
Every operation is a float32 numpy operation, so each result is rounded where the eager reference rounds
it.  Pinned against outputs of the reference itself (tests/golden/affine_qdq.npz).
"""
import numpy as np

F = np.float32


def _broadcast(x, grid_value):
    g = np.asarray(grid_value, dtype=F)
    if g.ndim < x.ndim:
        g = g.reshape((1,) * (x.ndim - g.ndim) + g.shape)
    return np.broadcast_to(g, x.shape)


def divide_form(x, scale, offset, qmin, qmax):
    """y and the in-grid flags."""
    x = np.asarray(x, dtype=F)
    s, o = _broadcast(x, scale), _broadcast(x, offset)
    with np.errstate(invalid="ignore", over="ignore"):
        t = np.rint(x / s).astype(F) - o
        keep = (t >= F(qmin)) & (t <= F(qmax))
        clamped = np.where(np.isnan(t), t, np.minimum(np.maximum(t, F(qmin)), F(qmax))).astype(F)
        y = ((clamped + o).astype(F) * s).astype(F)
    return y, keep


def divide_form_backward(grad, x, scale, offset, qmin, qmax):
    """dx and the un-reduced terms of dscale and doffset (float32, shape of x); the caller sums them over
    the axes the grid broadcasts along."""
    x, grad = np.asarray(x, dtype=F), np.asarray(grad, dtype=F)
    s, o = _broadcast(x, scale), _broadcast(x, offset)
    with np.errstate(invalid="ignore", over="ignore"):
        xs = (x / s).astype(F)
        q = np.rint(xs).astype(F)
        t = (q - o).astype(F)
        keep = (t >= F(qmin)) & (t <= F(qmax))
        m = keep.astype(F)
        lo, hi = (o + F(qmin)).astype(F), (o + F(qmax)).astype(F)
        qc = np.where(np.isnan(q), q, np.minimum(np.maximum(q, lo), hi)).astype(F)
        scale_terms = (grad * (qc - (xs * m).astype(F)).astype(F)).astype(F)
        offset_terms = (grad * np.where(keep, F(0), s).astype(F)).astype(F)
        dx = (grad * m).astype(F)
    return dx, scale_terms, offset_terms


def reciprocal_form(x, scale, offset, qmin, qmax):
    """y and the in-grid flags of the fast path.  Values beyond the int64 range are left out of the
    contract: the reference's CPU and CUDA casts disagree there."""
    x = np.asarray(x, dtype=F)
    s, o = _broadcast(x, scale), _broadcast(x, offset)
    zp = -(o.astype(np.int32))
    inv = (F(1.0) / s).astype(F)
    nan = np.isnan(x)
    with np.errstate(invalid="ignore", over="ignore"):
        r = (np.rint((np.where(nan, F(0), x) * inv).astype(F)).astype(F) + zp.astype(F)).astype(F)
        q = np.clip(r, -9.0e18, 9.0e18).astype(np.int64)
        keep = (q >= qmin) & (q <= qmax) & ~nan
        c = np.clip(q, qmin, qmax)
        y = ((c - zp).astype(F) * s).astype(F)
    y = np.where(nan, x, y).astype(F)
    return y, keep


def reduce_to_grid(terms, grid_shape):
    """Sum of per-element terms over every axis the grid broadcasts along, accumulated in double."""
    terms = np.asarray(terms, dtype=np.float64)
    grid_shape = tuple(grid_shape)
    padded = (1,) * (terms.ndim - len(grid_shape)) + grid_shape
    axes = tuple(a for a, n in enumerate(padded) if n == 1 and terms.shape[a] != 1)
    out = terms.sum(axis=axes, keepdims=True) if axes else terms
    return out.reshape(grid_shape)


def expand_blocks(grid_value, tensor_shape):
    """A blockwise grid repeated to the tensor's shape: entry [i, j, ...] covers the block of extents
    tensor_shape[d] / grid_shape[d] (torch_builtins.py:717-754 views the tensor the other way round)."""
    full = np.asarray(grid_value, dtype=F)
    for axis, (extent, blocks) in enumerate(zip(tensor_shape, full.shape)):
        full = np.repeat(full, extent // blocks, axis=axis)
    return full


def reduce_to_blocks(terms, grid_shape):
    """Sum of per-element terms over every block, accumulated in double."""
    terms = np.asarray(terms, dtype=np.float64)
    view = []
    for extent, blocks in zip(terms.shape, grid_shape):
        view += [blocks, extent // blocks]
    return terms.reshape(view).sum(axis=tuple(range(1, 2 * len(grid_shape), 2)))
