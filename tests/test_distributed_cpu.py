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


# ---- histogram calibration under data parallelism -------------------------------------------------
#
# A batch sharded over ranks must leave every collector in the state one process reaches on the
# concatenated batch: all-reduce the finite extremes, bin on the common range, all-reduce the bin counts,
# commit / merge with the global element count.  Both operators' collectors, several batches (growing
# and shifted ranges, a constant batch, non-finite values), host entry points of the shipped library.

def _hist_batches():
    rng = np.random.default_rng(23)
    b = [rng.standard_normal(4000).astype(np.float32), (rng.standard_normal(4000) * 3 + 1).astype(np.float32),
         np.full(4000, 0.25, np.float32), (rng.standard_normal(4000) * 0.1 - 6).astype(np.float32)]
    b[1][::97] = np.inf
    b[3][5] = np.nan
    return b


def _gru_collector(bins):
    counts = np.zeros(bins, np.float32)
    h = cabi.Histogram()
    h.counts = counts.ctypes.data_as(C.POINTER(C.c_float))
    h.num_bins = bins
    assert cabi.load_library().rxmet_histogram_reset(C.byref(h)) == 0
    return h, counts


def _lstm_collector(bins):
    from rx_met_b200 import _cabi_lstm as L
    counts = np.zeros(bins, np.float64)
    h = L.Histogram()
    h.counts = counts.ctypes.data_as(C.POINTER(C.c_double))
    h.num_bins = bins
    return h, counts


def _finite_extremes(x):
    f = x[np.isfinite(x)]
    return (np.float32(f.min()), np.float32(f.max())) if f.size else (np.float32(np.inf), np.float32(-np.inf))


def _hist_worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lib = cabi.load_library()
        bins = 256
        gh, gcounts = _gru_collector(bins)
        lh, lcounts = _lstm_collector(bins)
        f32p, u32p, u64p = C.POINTER(C.c_float), C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)
        for batch in _hist_batches():
            shard = np.ascontiguousarray(batch[rank::world])
            lo, hi = _finite_extremes(shard)
            ext = torch.tensor([lo, -hi])
            dist.all_reduce(ext, op=dist.ReduceOp.MIN)
            glo, ghi = float(ext[0]), float(-ext[1])
            total = torch.tensor([shard.size], dtype=torch.int64)
            dist.all_reduce(total)
            # QuantGRU collector: plan, count, sum, commit
            plan = cabi.HistogramPlan()
            assert lib.rxmet_histogram_plan_batch(C.byref(gh), C.c_float(glo), C.c_float(ghi), C.byref(plan)) == 0
            counts = np.zeros(bins, np.uint32)
            assert lib.rxmet_histogram_count_host(C.byref(plan), bins, shard.ctypes.data_as(f32p), C.c_uint64(shard.size),
                                                  counts.ctypes.data_as(u32p)) == 0
            summed = torch.from_numpy(counts.astype(np.int64))
            dist.all_reduce(summed)
            counts = summed.numpy().astype(np.uint32)
            assert lib.rxmet_histogram_commit_counts(C.byref(gh), C.byref(plan), counts.ctypes.data_as(u32p),
                                                     C.c_uint64(int(total))) == 0
            # QuantLSTM collector: range, count, sum, merge
            rlo, rhi = C.c_float(), C.c_float()
            assert lib.rxmet_lstm_histogram_batch_range(C.c_float(glo), C.c_float(ghi), C.byref(rlo), C.byref(rhi)) == 0
            c64, finite = np.zeros(bins, np.uint64), C.c_uint64(0)
            assert lib.rxmet_lstm_histogram_count_host(rlo, rhi, bins, shard.ctypes.data_as(f32p), C.c_uint64(shard.size),
                                                       c64.ctypes.data_as(u64p), C.byref(finite)) == 0
            packed = torch.from_numpy(np.concatenate([c64.astype(np.int64), [finite.value]]))
            dist.all_reduce(packed)
            c64 = packed.numpy()[:-1].astype(np.uint64)
            assert lib.rxmet_lstm_histogram_merge_counts(C.byref(lh), c64.ctypes.data_as(u64p), rlo, rhi,
                                                         C.c_uint64(int(packed[-1]))) == 0
        np.savez(os.path.join(result_dir, f"hist{rank}.npz"), g=gcounts, l=lcounts,
                 gstate=np.array([gh.min_val, gh.max_val, gh.observed_min, gh.observed_max, gh.total_count], np.float64),
                 lstate=np.array([lh.minimum, lh.maximum, lh.total_count], np.float64))
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_single_process_histograms(tmp_path):
    world = 2
    mp.spawn(_hist_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r0, r1 = np.load(tmp_path / "hist0.npz"), np.load(tmp_path / "hist1.npz")
    for k in r0.files:
        assert np.array_equal(r0[k], r1[k]), f"ranks disagree on {k}"
    lib = cabi.load_library()
    bins = 256
    gh, gcounts = _gru_collector(bins)
    lh, lcounts = _lstm_collector(bins)
    for batch in _hist_batches():
        ptr = batch.ctypes.data_as(C.POINTER(C.c_float))
        assert lib.rxmet_histogram_collect_host(C.byref(gh), ptr, C.c_uint64(batch.size)) == 0
        assert lib.rxmet_lstm_histogram_collect_host(C.byref(lh), ptr, C.c_uint64(batch.size)) == 0
    assert np.array_equal(r0["g"], gcounts) and np.array_equal(r0["l"], lcounts)
    assert np.array_equal(r0["gstate"], np.array([gh.min_val, gh.max_val, gh.observed_min, gh.observed_max, gh.total_count],
                                                 np.float64))
    assert np.array_equal(r0["lstate"], np.array([lh.minimum, lh.maximum, lh.total_count], np.float64))
    # and the encodings derived from them
    for h, fn in ((gh, "rxmet_histogram_calibrate"),):
        out = [C.c_float(), C.c_float(), C.c_float()]
        assert getattr(lib, fn)(C.byref(h), 8, 0, 0, 0, C.c_float(99.9), *[C.byref(o) for o in out]) == 0
        assert out[0].value > 0

