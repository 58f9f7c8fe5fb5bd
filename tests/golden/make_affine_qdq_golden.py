"""Writes tests/golden/affine_qdq.npz from the reference's own backend, run on the CPU.

    python tests/golden/make_affine_qdq_golden.py /path/to/reference

src/aimet_torch/v2/quantization/affine/backends/torch_builtins.py is loaded as a single module (its parent
packages are entered as empty namespaces and its ONNX-symbolic registry, which only decorates, is a stand-in, so
that the package's heavy imports are not needed); `quantize_dequantize` is then called the way a quantizer calls
it: once without gradients on the grid (the fake-quantize fast path) and once with a trained grid
(QuantDequantFunc), and outputs and gradients are stored.  Inputs hold ties, clipped values on both sides,
signed zeros and (fast form only where the CPU and CUDA casts agree) NaN.
"""
import importlib
import os
import sys
import types

import numpy as np
import torch


def load_backend(reference_root):
    src = os.path.join(reference_root, "src")

    def namespace(name):
        module = types.ModuleType(name)
        module.__path__ = [os.path.join(src, *name.split("."))]
        sys.modules[name] = module

    for name in ("aimet_torch", "aimet_torch.v2", "aimet_torch.v2.experimental", "aimet_torch.v2.experimental.onnx",
                 "aimet_torch.v2.quantization", "aimet_torch.v2.quantization.affine",
                 "aimet_torch.v2.quantization.affine.backends"):
        namespace(name)
    registry = types.ModuleType("aimet_torch.v2.experimental.onnx._export")
    registry.register_symbolic = lambda symbolic: (lambda fn: fn)
    registry.__getattr__ = lambda name: None
    sys.modules[registry.__name__] = registry
    sys.modules["aimet_torch.v2.experimental.onnx"]._export = registry
    return importlib.import_module("aimet_torch.v2.quantization.affine.backends.torch_builtins")


def make_input(rng, shape, scale, offset, qmin, qmax, with_nan):
    s = np.broadcast_to(scale, shape).astype(np.float32)
    o = np.broadcast_to(offset, shape).astype(np.float32)
    codes = rng.uniform(qmin - 6, qmax + 6, size=shape)
    x = ((codes + o) * s).astype(np.float32)
    flat = x.reshape(-1)
    flat_s, flat_o = s.reshape(-1), o.reshape(-1)
    n = flat.size
    ties = rng.choice(n, size=n // 8, replace=False)
    flat[ties] = ((np.floor(codes.reshape(-1)[ties]) + 0.5 + flat_o[ties]) * flat_s[ties]).astype(np.float32)
    flat[rng.choice(n, size=max(1, n // 50), replace=False)] = 0.0
    flat[rng.choice(n, size=max(1, n // 50), replace=False)] = -0.0
    flat[rng.choice(n, size=max(1, n // 60), replace=False)] *= 1e4
    if with_nan:
        flat[rng.choice(n, size=3, replace=False)] = np.nan
    return x


def packed_keep(dx, grad):
    """dx is grad where the value was inside the grid and 0 elsewhere; the flags are stored, one bit each."""
    keep = dx != 0
    assert np.array_equal(dx, grad * keep) and not np.any(grad == 0)
    return np.packbits(keep.reshape(-1))


def main(reference_root):
    backend = load_backend(reference_root)
    rng = np.random.default_rng(7)
    specs = [  # name, tensor shape, grid shape, qmin, qmax
        ("per_tensor_int8_ragged", (1031,), (), -128, 127),
        ("per_tensor_uint4", (16, 64), (1,), 0, 15),
        ("per_tensor_int16", (3, 400), (), -32768, 32767),
        ("rows_int8_vector", (6, 260), (6, 1), -128, 127),
        ("rows_int8_scalar", (7, 257), (7, 1), -127, 127),
        ("rows_two_segments", (2, 8200), (2, 1), -8, 7),
        ("columns_last_axis", (70, 24), (24,), -128, 127),
        ("columns_middle_axis", (5, 6, 7), (6, 1), 0, 255),
        ("rows_middle_axis_long", (3, 4, 256), (4, 1), -128, 127),
    ]
    out = {}
    for name, shape, grid_shape, qmin, qmax in specs:
        count = int(np.prod(grid_shape)) if grid_shape else 1
        scale = rng.uniform(0.01, 0.2, size=count).astype(np.float32).reshape(grid_shape)
        offset = rng.integers(qmin // 4 - 3, 4, size=count).astype(np.float32).reshape(grid_shape)
        if count > 1:
            offset[...] = 0.0   # the fast path of a per-channel grid wants its zero point inside the code range
            if qmin == 0:
                offset[...] = 0.0
        elif qmin == 0:
            offset[...] = -float(rng.integers(0, qmax))
        x = make_input(rng, shape, scale, offset, qmin, qmax, with_nan=False)
        grad = rng.standard_normal(shape).astype(np.float32)
        if np.prod(shape) > 8192:   # the long case draws from a small pool so that the archive stays small
            x = rng.choice(x.reshape(-1)[:97], size=shape).astype(np.float32)
            grad = rng.choice(grad.reshape(-1)[:31], size=shape).astype(np.float32)

        xt = torch.tensor(x, requires_grad=True)
        st, ot = torch.tensor(scale), torch.tensor(offset)
        y = backend.quantize_dequantize(xt, st, ot, qmin, qmax)
        y.backward(torch.tensor(grad))
        out[f"{name}/fast_y"] = y.detach().numpy()
        out[f"{name}/fast_keep"] = packed_keep(xt.grad.numpy(), grad)

        xt = torch.tensor(x, requires_grad=True)
        st, ot = torch.tensor(scale, requires_grad=True), torch.tensor(offset, requires_grad=True)
        y = backend.quantize_dequantize(xt, st, ot, qmin, qmax)
        y.backward(torch.tensor(grad))
        out[f"{name}/y"] = y.detach().numpy()
        out[f"{name}/keep"] = packed_keep(xt.grad.numpy(), grad)
        out[f"{name}/dscale"], out[f"{name}/doffset"] = st.grad.numpy().copy(), ot.grad.numpy().copy()
        # size of the terms behind each sum, for the tolerance of the float reductions
        xs = torch.tensor(x) / torch.tensor(scale)
        keep = ((xs.round() - torch.tensor(offset)) >= qmin) & ((xs.round() - torch.tensor(offset)) <= qmax)
        terms = torch.tensor(grad) * (xs.round().clamp(torch.tensor(offset) + qmin, torch.tensor(offset) + qmax) - xs * keep)
        out[f"{name}/dscale_abs"] = terms.abs().sum_to_size(st.shape).numpy() if st.dim() else terms.abs().sum().numpy()
        out[f"{name}/x"], out[f"{name}/grad"], out[f"{name}/scale"], out[f"{name}/offset"] = x, grad, scale, offset
        out[f"{name}/range"] = np.array([qmin, qmax], dtype=np.int64)

    # blockwise grids: the tensor is cut into blocks along the blocked dimensions, one grid entry per block
    for name, shape, grid_shape, block_size, qmin, qmax in [
            ("blocks_of_16", (8, 64), (8, 4), [1, 16], -8, 7),
            ("blocks_conv_weight", (6, 32, 3, 3), (6, 2, 1, 1), [-1, 16, -1, -1], -128, 127)]:
        scale = rng.uniform(0.01, 0.2, size=grid_shape).astype(np.float32)
        offset = np.zeros(grid_shape, dtype=np.float32)
        full = scale
        for axis, (extent, blocks) in enumerate(zip(shape, grid_shape)):
            full = np.repeat(full, extent // blocks, axis=axis)
        x = make_input(rng, shape, full, np.zeros(shape, np.float32), qmin, qmax, with_nan=False)
        grad = rng.standard_normal(shape).astype(np.float32)
        xt = torch.tensor(x, requires_grad=True)
        st, ot = torch.tensor(scale, requires_grad=True), torch.tensor(offset, requires_grad=True)
        y = backend.quantize_dequantize(xt, st, ot, qmin, qmax, block_size=block_size)
        y.backward(torch.tensor(grad))
        out[f"{name}/y"] = y.detach().numpy()
        out[f"{name}/keep"] = packed_keep(xt.grad.numpy(), grad)
        out[f"{name}/dscale"], out[f"{name}/doffset"] = st.grad.numpy().copy(), ot.grad.numpy().copy()
        out[f"{name}/x"], out[f"{name}/grad"], out[f"{name}/scale"], out[f"{name}/offset"] = x, grad, scale, offset
        out[f"{name}/range"] = np.array([qmin, qmax], dtype=np.int64)
        out[f"{name}/block_size"] = np.array(block_size, dtype=np.int64)

    # NaN inputs: the divide form propagates them; the fast form restores them after the kernel
    x = make_input(rng, (1030,), np.float32(0.05), np.float32(-3.0), -128, 127, with_nan=True)
    st, ot = torch.tensor(0.05), torch.tensor(-3.0)
    with torch.no_grad():
        out["nan/fast_y"] = backend.quantize_dequantize(torch.tensor(x), st, ot, -128, 127).numpy()
    y = backend.quantize_dequantize(torch.tensor(x), st.clone().requires_grad_(), ot, -128, 127)
    out["nan/y"], out["nan/x"] = y.detach().numpy(), x

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "affine_qdq.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1])
