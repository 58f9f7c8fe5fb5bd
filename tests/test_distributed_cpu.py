"""World-size-2 gloo test of the data-parallel host logic (no GPU involved).

Each rank calibrates on its own batch shard with the CPU checker, packs the observed ranges in
the layout the CUDA calibration forward produces ([mins | maxs], 17 scalar slots then the
per-channel blocks of W, R, bw, br), all-reduces the halves with MIN / MAX and folds them with the
shipped library's host function.  The result must equal a single process calibrating on the
concatenated batch bit for bit, and so must the encodings every rank derives from it.  The
gradient exchange is checked the same way: the mean over ranks of per-shard gradients of a loss
normalised over the global batch equals the full-batch gradient."""
import ctypes as C
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_lib as ol
from rx_met_b200 import _cabi as cabi

T, B, I, H = 6, 4, 5, 8  # global batch 4, two ranks of 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _pack(ranges: ol.RangesBox) -> np.ndarray:
    half = (cabi.NUM_OPS + 12 * H)
    out = np.empty(2 * half, np.float32)
    d = ranges.as_dict()
    out[:cabi.NUM_OPS] = d["min"]
    out[half:half + cabi.NUM_OPS] = d["max"]
    for k, name in enumerate(("W", "R", "bw", "br")):
        out[cabi.NUM_OPS + k * 3 * H: cabi.NUM_OPS + (k + 1) * 3 * H] = d[f"min_{name}"]
        out[half + cabi.NUM_OPS + k * 3 * H: half + cabi.NUM_OPS + (k + 1) * 3 * H] = d[f"max_{name}"]
    return out


def _worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lib = cabi.load_library()
        assert lib.rxmet_gru_stats_floats(H) == 2 * (cabi.NUM_OPS + 12 * H)
        W, R, bw, br, x, _ = ol.gru_problem(17, T, B, I, H)
        shard = np.ascontiguousarray(x[:, rank * (B // world):(rank + 1) * (B // world)])
        local = ol.RangesBox(H)
        ol.forward_calibrate_minmax("orc", W, R, bw, br, shard, None, local)
        stats = torch.from_numpy(_pack(local))
        half = stats.numel() // 2
        dist.all_reduce(stats[:half], op=dist.ReduceOp.MIN)
        dist.all_reduce(stats[half:], op=dist.ReduceOp.MAX)
        merged = ol.RangesBox(H)
        host = stats.numpy()
        assert lib.rxmet_gru_ranges_fold_stats(C.byref(merged.c), host.ctypes.data_as(C.POINTER(C.c_float))) == 0
        cfg = ol.make_config(bits=8, symmetric=False)
        params = ol.ParamsBox(H, cfg)
        assert lib.rxmet_gru_params_from_ranges(C.byref(merged.c), C.byref(cfg), C.byref(params.c)) == 0

        # gradient exchange: loss = sum over the GLOBAL batch of <h, g> / B
        fwd = ol.forward_quant("orc", W, R, bw, br, shard, None, params)
        g = np.random.default_rng(5).standard_normal((T, B, H)).astype(np.float32)
        dh_new = np.zeros((T + 1, B // world, H), np.float32)
        dh_new[1:] = g[:, rank * (B // world):(rank + 1) * (B // world)] / B
        grads = ol.backward_quant(fwd, dh_new, fwd["h"], fwd["v"], params, fwd["masks"])
        flat = torch.from_numpy(np.concatenate([grads[k].reshape(-1) for k in ("dW", "dR", "dbw", "dbr")]))
        dist.all_reduce(flat)  # per-shard losses were already divided by the global batch
        np.savez(os.path.join(result_dir, f"rank{rank}.npz"), flat=flat.numpy(),
                 **{f"r_{k}": v for k, v in merged.as_dict().items()}, **{f"p_{k}": v for k, v in params.as_dict().items()})
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_single_process_calibration_and_gradients(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    for k in r0.files:
        assert np.array_equal(r0[k], r1[k]), f"ranks disagree on {k}"

    W, R, bw, br, x, _ = ol.gru_problem(17, T, B, I, H)
    single = ol.RangesBox(H)
    ol.forward_calibrate_minmax("orc", W, R, bw, br, x, None, single)
    for k, v in single.as_dict().items():
        assert np.array_equal(r0[f"r_{k}"], v), k
    cfg = ol.make_config(bits=8, symmetric=False)
    params = ol.params_from_ranges("orc", single, cfg)
    for k, v in params.as_dict().items():
        assert np.array_equal(r0[f"p_{k}"], v), k

    fwd = ol.forward_quant("orc", W, R, bw, br, x, None, params)
    g = np.random.default_rng(5).standard_normal((T, B, H)).astype(np.float32)
    dh_new = np.zeros((T + 1, B, H), np.float32)
    dh_new[1:] = g / B
    grads = ol.backward_quant(fwd, dh_new, fwd["h"], fwd["v"], params, fwd["masks"])
    want = np.concatenate([grads[k].reshape(-1) for k in ("dW", "dR", "dbw", "dbr")])
    assert np.abs(r0["flat"] - want).max() <= 1e-6 * max(np.abs(want).max(), 1e-30)
