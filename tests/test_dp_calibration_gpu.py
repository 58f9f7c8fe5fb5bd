"""Histogram calibration with the batch sharded over two GPUs (NCCL through the library's exchange hook):
every rank must end with the collectors and the parameters one process derives from the concatenated batches.
Needs two GPUs; skipped otherwise."""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

T, B, I, H = 9, 12, 10, 32  # global batch 12, two ranks of 6


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem():
    rng = np.random.default_rng(31)
    k = 1.0 / np.sqrt(H)
    u = lambda *s: rng.uniform(-k, k, s).astype(np.float32)  # noqa: E731
    batches = [rng.standard_normal((T, B, I)).astype(np.float32) * s for s in (1.0, 1.7, 0.4)]
    return dict(gW=u(I, 3 * H), gR=u(H, 3 * H), gbw=u(3 * H), gbr=u(3 * H), lw_ih=u(4 * H, I), lw_hh=u(4 * H, H),
                lb_ih=u(4 * H), lb_hh=u(4 * H), batches=batches)


def _calibrate(rank, world, group):
    """Returns the GRU collector states + parameters and the LSTM bundle of this rank."""
    from rx_met_b200 import _cabi_lstm as L
    from rx_met_b200 import _quant_lstm as lstm
    from rx_met_b200 import gru_interface_binding as gru
    p = _problem()
    dev = torch.device("cuda", torch.cuda.current_device())
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
    shard = lambda x: x if world == 1 else x[:, rank * (B // world):(rank + 1) * (B // world)]  # noqa: E731
    gru.set_calibration_process_group(group)
    collectors = gru.GRUHistogramCollectors(H, 512)
    cfg = gru.OperatorQuantConfig()
    ranges = gru.GRUQuantizationRanges(H)
    for x in p["batches"]:
        xs = shard(x)
        gru.forward_calibrate(True, T, xs.shape[1], I, H, t(p["gW"]), t(p["gR"]), t(p["gbw"]), t(p["gbr"]), t(xs),
                              torch.empty(0, device=dev), "sqnr", cfg, None, collectors)
        gru.forward_calibrate(True, T, xs.shape[1], I, H, t(p["gW"]), t(p["gR"]), t(p["gbw"]), t(p["gbr"]), t(xs),
                              torch.empty(0, device=dev), "minmax", cfg, ranges, None)
    gru.set_calibration_process_group(None)
    gparams = gru.calculate_gru_quantitative_parameters_from_histograms(collectors, cfg, False, 99.99)
    gminmax = gru.calculate_gru_quantitative_parameters(ranges, cfg)
    c_params, _keep = gparams._to_c()
    c_minmax, _keep2 = gminmax._to_c()
    out = dict(g_counts=collectors._set.counts.copy(),
               g_scale=np.array(list(c_params.scale), np.float32), g_zp=np.array(list(c_params.zero_point), np.int32),
               m_scale=np.array(list(c_minmax.scale), np.float32), m_zp=np.array(list(c_minmax.zero_point), np.int32))
    session = lstm.CalibrationSession(lstm._config_to_json(L.default_config()), I, H, True, "sqnr")
    session.process_group = group
    for x in p["batches"]:
        session.collect(t(shard(x)), t(p["lw_ih"]), t(p["lw_hh"]), t(p["lb_ih"]), t(p["lb_hh"]))
    out["l_counts"] = session._hists.counts.copy()
    out["l_bundle"] = np.frombuffer(session.finalize(False)["bundle_json"].encode(), np.uint8).copy()
    return out


def _worker(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    import torch.distributed as dist
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        np.savez(os.path.join(result_dir, f"dp{rank}.npz"), **_calibrate(rank, world, dist.group.WORLD))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_histogram_calibration_equals_single_process(tmp_path):
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "dp0.npz"), np.load(tmp_path / "dp1.npz")
    torch.cuda.set_device(0)
    single = _calibrate(0, 1, None)
    problems = []

    def differs(a, b):
        if a.shape != b.shape:
            n = min(a.size, b.size)
            first = int(np.argmax(a[:n] != b[:n])) if np.any(a[:n] != b[:n]) else n
            return f"shapes {a.shape} / {b.shape}, first difference at {first}"
        return None if np.array_equal(a, b) else f"{int(np.sum(a != b))} of {a.size} entries"

    for k, v in single.items():
        between, against = differs(r0[k], r1[k]), differs(r0[k], v)
        if between:
            problems.append(f"ranks disagree on {k}: {between}")
        if against:
            problems.append(f"sharded calibration differs from one process on {k}: {against}")
        if k == "l_bundle" and (between or against):
            text = [bytes(a).decode() for a in (r0[k], r1[k], v)]
            at = next((i for i, (x, y, z) in enumerate(zip(*text)) if not (x == y == z)), 0)
            problems.append(" | ".join(t[max(0, at - 120):at + 60] for t in text))
    assert not problems, "; ".join(problems)
