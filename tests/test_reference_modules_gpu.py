"""The reference's OWN Python modules - `QuantGRU` (operators/quant-gru/pytorch/quant_gru.py) and `QuantLSTM`
(operators/quant-lstm/pytorch/quant_lstm.py) - and two of its own unit-test files, run unmodified on the GPU with
this repository's drop-in modules registered under the extension names they import.  The copies live under the
git-ignored baseline/_ref/ (`make -f oracle/Makefile refpy`); without them the tests skip."""
from __future__ import annotations

import importlib
import sys
import types
import unittest
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not (REF / "quant_gru" / "quant_gru.py").exists(),
                                                  reason="reference Python modules not installed under baseline/_ref")]


@pytest.fixture(scope="module")
def reference():
    """quant_gru / quant_lstm of the reference, importing the drop-ins as their native extensions."""
    from rx_met_b200 import _quant_lstm, gru_interface_binding
    sys.modules["gru_interface_binding"] = gru_interface_binding
    sys.modules["_quant_lstm"] = _quant_lstm
    if "onnx" not in sys.modules:
        try:
            importlib.import_module("onnx")
        except ImportError:  # only the ONNX helpers of the reference's test support need it; they are not run here
            stub = types.ModuleType("onnx")
            stub.TensorProto = stub.helper = stub.numpy_helper = types.SimpleNamespace()
            sys.modules["onnx"] = stub
    for path in (REF, REF / "quant_gru", REF / "quant_lstm"):
        if str(path) not in sys.path:
            sys.path.insert(0, str(path))
    for name in ("tests", "tests.support", "tests.recurrent"):   # this repository's own test folder is not a package
        sys.modules.pop(name, None)
    return importlib.import_module("quant_gru"), importlib.import_module("quant_lstm")


def run_reference_unittests(module_name):
    suite = unittest.defaultTestLoader.loadTestsFromModule(importlib.import_module(module_name))
    result = unittest.TestResult()
    suite.run(result)
    problems = [f"{test}: {text.splitlines()[-1]}" for test, text in result.errors + result.failures]
    assert result.testsRun > 0 and not problems, "\n".join(problems)
    return result.testsRun


def test_reference_gru_autograd_tests_pass_on_the_drop_in(reference):
    """tests/recurrent/test_gru_autograd.py: clamp derivatives against an autograd surrogate built from the
    positional saved tensors of GRUFunction, train / eval backward, gate origins."""
    assert run_reference_unittests("tests.recurrent.test_gru_autograd") >= 3


def test_reference_gru_storage_tests_pass_on_the_drop_in(reference):
    """tests/recurrent/test_gru_storage.py: float32 / int32 code carriers keep caches, masks and backward."""
    assert run_reference_unittests("tests.recurrent.test_gru_storage") >= 1


@pytest.mark.parametrize("bidirectional", [False, True])
@pytest.mark.parametrize("method", ["minmax", "sqnr"])
def test_quant_gru_module_end_to_end(reference, bidirectional, method):
    quant_gru, _ = reference
    torch.manual_seed(5)
    model = quant_gru.QuantGRU(12, 16, batch_first=True, bidirectional=bidirectional).cuda()
    model.calibration_method = method
    batches = [torch.randn(6, 9, 12, device="cuda") for _ in range(3)]
    with model.calibration_context():
        with torch.no_grad():
            for x in batches:
                model(x)
    assert model.is_calibrated()
    model.use_quantization = True
    model.train()
    x = batches[0].clone().requires_grad_()
    y, h_n = model(x)
    assert y.shape == (6, 9, 16 * (2 if bidirectional else 1)) and h_n.shape == (2 if bidirectional else 1, 6, 16)
    (y.square().mean() + h_n.sum()).backward()
    grads = [x.grad] + [p.grad for p in model.parameters()]
    assert all(g is not None and torch.isfinite(g).all() and g.abs().sum() > 0 for g in grads)
    # inference on the same input: same codes, hence the same outputs
    model.eval()
    with torch.no_grad():
        y2, _ = model(batches[0])
    assert torch.equal(y.detach(), y2)
    # float reference of the module itself stays close
    model.use_quantization = False
    with torch.no_grad():
        y_float, _ = model(batches[0])
    assert (y2 - y_float).abs().max() < 0.1


@pytest.mark.parametrize("bidirectional", [False, True])
def test_quant_lstm_module_end_to_end(reference, bidirectional):
    _, quant_lstm = reference
    torch.manual_seed(6)
    model = quant_lstm.QuantLSTM(10, 16, batch_first=True, bidirectional=bidirectional).cuda()
    batches = [torch.randn(5, 8, 10, device="cuda") for _ in range(2)]
    with model.calibration_context():
        with torch.no_grad():
            for x in batches:
                model(x)
    model.use_quantization = True
    model.train()
    x = batches[0].clone().requires_grad_()
    y, (h_n, c_n) = model(x)
    directions = 2 if bidirectional else 1
    assert y.shape == (5, 8, 16 * directions) and h_n.shape == (directions, 5, 16) and c_n.shape == h_n.shape
    (y.square().mean() + h_n.sum() + c_n.sum()).backward()
    grads = [x.grad] + [p.grad for p in model.parameters()]
    assert all(g is not None and torch.isfinite(g).all() for g in grads)
    model.eval()
    with torch.no_grad():
        y2, _ = model(batches[0])
    assert torch.equal(y.detach(), y2)
