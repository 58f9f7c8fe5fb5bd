#!/usr/bin/env python
"""Benchmark of the QuantGRU QAT step (the workload the headline metric is quoted on).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload "gru_qat_step": QuantGRU I=40, H=128, T=100, batch 256 per GPU (weak scaling), W8/A8
fake-quant with straight-through masks; one step = quantized training forward + MSE gradient +
BPTT + gradient all-reduce + SGD update.  Synthetic N(0,1) inputs and targets, U(-1/sqrt(H),
1/sqrt(H)) weights, min/max calibration once before timing.

value : seq-timesteps/s with inputs resident in HBM (preallocated buffers, C ABI called directly).
e2e   : the same step through the reference-facing module ``rx_met_b200.gru_interface_binding``
        with host->device copies of x / target from pinned memory and the loss read back.
The reference arm (--impl reference) times the reference's CPU quantized forward (it has no CPU
training path) on all host cores over a bounded sample of the same shapes.
"""
import argparse
import ctypes as C
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

WORKLOAD = dict(T=100, B=256, I=40, H=128)
METRIC = "QuantGRU QAT seq-timesteps/sec"
UNIT = "seq-timesteps/s"
# Algorithmic HBM bytes per sequence-timestep of the two recurrent kernels: the module-boundary
# fp32 tensors (4*I in or out, 4*H out or in) plus the minimal saved state S = 5 code bytes per
# hidden unit + the 13H+I mask bits, once written (forward) and once read (backward).
def _algo_bytes_per_st(I, H):
    S = 5 * H + (13 * H + I + 7) // 8
    return 4 * I + 4 * H + S


# DRAM traffic per launch of the recurrent kernels at this workload, from the ncu captures
# summarised under profiles/ (dram__bytes_read.sum + dram__bytes_write.sum, one launch).
NCU_TRAFFIC_BYTES = {"recurrentForward": 19.80e6 + 42.90e6, "recurrentBackward": 85.42e6 + 40.81e6}


def _peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """SM clock and throttle reasons of one GPU during the timed region: an in-process NVML poll every
    millisecond (read-only queries), because the region lasts a few tens of milliseconds, less than an
    nvidia-smi process needs to start.  nvidia-smi in loop mode is the fallback when NVML cannot be loaded."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None
        self.thread = None
        self.samples = []      # (sm MHz, reason bits)
        self.sm_max = None
        self._stop = False

    def _nvml_index(self):
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            entries = [e.strip() for e in visible.split(",") if e.strip()]
            if self.gpu_index < len(entries) and entries[self.gpu_index].isdigit():
                return int(entries[self.gpu_index])
        return self.gpu_index

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self._nvml_index())
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons",
                              getattr(pynvml, "nvmlDeviceGetCurrentClocksThrottleReasons", None))

            def poll():
                while not self._stop:
                    try:
                        sm = float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                        bits = int(reasons(handle)) if reasons is not None else 0
                        self.samples.append((sm, bits))
                    except pynvml.NVMLError:
                        pass
                    time.sleep(0.001)

            self._pynvml = pynvml
            self.thread = threading.Thread(target=poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        if shutil.which("nvidia-smi") is None:
            return
        fd, self.path = tempfile.mkstemp(suffix=".csv")
        os.close(fd)
        self.proc = subprocess.Popen(
            ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
             "-lms", "20"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)

    @staticmethod
    def _summary(sm, smax, reasons, source):
        # samples under load = upper half of the observed SM clocks
        sm_sorted = sorted(sm)
        load = sm_sorted[len(sm_sorted) // 2:] if sm_sorted else []
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm), "source": source}

    def stop(self):
        if self.thread is not None:
            self._stop = True
            self.thread.join(timeout=2)
            nv = self._pynvml
            names = {"hw_slowdown": "HwSlowdown", "hw_thermal_slowdown": "HwThermalSlowdown",
                     "sw_thermal_slowdown": "SwThermalSlowdown", "sw_power_cap": "SwPowerCap"}
            reasons = set()
            for _, bits in self.samples:
                for name, suffix in names.items():
                    mask = getattr(nv, "nvmlClocksEventReason" + suffix, getattr(nv, "nvmlClocksThrottleReason" + suffix, 0))
                    if bits & mask:
                        reasons.add(name)
            return self._summary([sm for sm, _ in self.samples], self.sm_max, reasons, "nvml")
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "source": None}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        for line in Path(self.path).read_text().splitlines():
            f = [s.strip() for s in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return self._summary(sm, max(smax) if smax else None, reasons, "nvidia-smi")


# --------------------------------------------------------------------------
# CPU arm: the reference's own CPU quantized path (or its C restatement)
# --------------------------------------------------------------------------

def cpu_forward_throughput(seconds_target=12.0, shard_batch=8):
    """Calibration-free timing of the CPU quantized (PTQ) forward at the workload's T/I/H on all
    host cores: independent batch shards run on a thread pool (ctypes releases the GIL).  Returns
    (seq-timesteps/s, cores, kind, description)."""
    import numpy as np
    import oracle_lib as ol
    T, I, H = WORKLOAD["T"], WORKLOAD["I"], WORKLOAD["H"]
    kind = "reference" if ol.ref() is not None else "port"
    prefix = "ref" if kind == "reference" else "orc"
    cores = os.cpu_count() or 1
    W, R, bw, br, x, _ = ol.gru_problem(0, T, shard_batch, I, H)
    cfg = ol.make_config(bits=8, symmetric=False)
    ranges = ol.RangesBox(H)
    ol.forward_calibrate_minmax("orc", W, R, bw, br, x, None, ranges)
    params = ol.params_from_ranges("orc", ranges, cfg)

    def shard(seed):
        xs = np.random.default_rng(seed).standard_normal((T, shard_batch, I)).astype(np.float32)
        ol.forward_quant(prefix, W, R, bw, br, xs, None, params, training=False, want_float=False)

    t0 = time.perf_counter()
    shard(1)
    one = time.perf_counter() - t0
    rounds = max(1, int(seconds_target / max(one, 1e-3)))
    n_shards = cores * rounds
    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=cores) as pool:
        list(pool.map(shard, range(n_shards)))
    dt = time.perf_counter() - t0
    st = n_shards * shard_batch * T
    desc = (f"{n_shards} shards of {shard_batch} sequences x T={T} (I={I}, H={H}), quantized inference forward only "
            f"(the reference has no CPU training path), {cores} threads, {dt:.1f} s")
    return st / dt, cores, kind, desc, dt


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times, values = [], []
    desc = kind = None
    cores = 1
    for i in range(args.warmup + args.steps):
        v, cores, kind, desc, dt = cpu_forward_throughput(
            seconds_target=min(3.0, 150.0 / max(1, args.warmup + args.steps)))
        if i >= args.warmup:
            values.append(v)
            times.append(dt)
    value = statistics.mean(values)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 codes / int64 accumulate",
        "data": "synthetic", "config": {"workload": "gru_qat_step", **WORKLOAD, "note": "CPU reference arm: forward only"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------

def reference_cuda_step(torch, device, eng, x, reps=5):
    """The reference's OWN CUDA kernels for the same step (its integer-carrier training forward and its QAT
    backward, compiled for sm_100a into oracle/_ref/libgru_ref_cuda.so by oracle/Makefile), timed on this GPU with
    the product's weights and quantization parameters: the kernel-to-beat beside the CPU baseline.  Follows the
    reference binding's order of work: forward; float copies of the saved codes, its dequantization, transposes,
    zeroed weight gradients; backward.  The loss and the optimizer step are not included."""
    so = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle", "_ref", "libgru_ref_cuda.so")
    if not os.path.exists(so):
        return {"unavailable": "oracle/_ref/libgru_ref_cuda.so not built"}
    ref = C.CDLL(so)
    ref.refcuda_last_error.restype = C.c_char_p
    from rx_met_b200 import _cabi as cabi
    T, B, I, H = eng.T, eng.B, eng.I, eng.H
    f32, i32 = dict(dtype=torch.float32, device=device), dict(dtype=torch.int32, device=device)
    h, v = torch.zeros((T + 1, B, H), **f32), torch.zeros((T, B, 4 * H), **f32)
    W_q, R_q = torch.zeros((I, 3 * H), **i32), torch.zeros((H, 3 * H), **i32)
    bw_q, br_q, x_q = torch.zeros(3 * H, **i32), torch.zeros(3 * H, **i32), torch.zeros((T, B, I), **i32)
    shapes = {"x": (T, B, I), "W": (I, 3 * H), "R": (H, 3 * H), "bw": (3 * H,), "br": (3 * H,),
              "weight_ih_linear": (T, B, 3 * H), "weight_hh_linear": (T, B, 3 * H), "gate_input": (T, B, 3 * H),
              "gate_output": (T, B, 3 * H), "h": (T, B, H)}
    masks, ms = {}, cabi.Masks()
    for name, shape in shapes.items():
        masks[name] = torch.zeros(shape, dtype=torch.uint8, device=device)
        setattr(ms, name, masks[name].data_ptr())
    P = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    dh_new = torch.randn((T + 1, B, H), generator=torch.Generator(device="cpu").manual_seed(3)).to(device) * 1e-3

    def check(rc, what):
        if rc != 0:
            raise RuntimeError(f"{what}: {ref.refcuda_last_error().decode(errors='replace')}")

    def forward():
        check(ref.refcuda_gru_forward_quant_int(1, T, B, I, H, P(eng.W), P(eng.R), P(eng.bw), P(eng.br), P(x), None,
                                                C.byref(eng._c_params), P(h), P(v), C.byref(ms), P(W_q), P(R_q), P(bw_q),
                                                P(br_q), P(x_q)), "reference CUDA forward")

    def backward():
        Wf, Rf, bwf, brf, xf = [t.to(torch.float32) for t in (W_q, R_q, bw_q, br_q, x_q)]
        check(ref.refcuda_gru_dequantize_saved(I, H, C.c_longlong(xf.numel()), P(Wf), P(Rf), P(bwf), P(brf), P(xf),
                                               C.byref(eng._c_params)), "reference CUDA dequantize")
        x_t, W_t, R_t = xf.permute(2, 0, 1).contiguous(), Wf.t().contiguous(), Rf.t().contiguous()
        dx, dW, dR = torch.empty((T, B, I), **f32), torch.zeros((I, 3 * H), **f32), torch.zeros((H, 3 * H), **f32)
        dbw, dbr, dh0 = torch.zeros(3 * H, **f32), torch.zeros(3 * H, **f32), torch.zeros((B, H), **f32)
        check(ref.refcuda_gru_backward_quant(T, B, I, H, P(W_t), P(R_t), P(bwf), P(brf), P(x_t), P(dh_new), P(h), P(v),
                                             C.byref(eng._c_params), C.byref(ms), P(dx), P(dW), P(dR), P(dbw), P(dbr), P(dh0)),
              "reference CUDA backward")

    try:
        times = {"forward": [], "backward": []}
        for i in range(reps + 2):
            for name, fn in (("forward", forward), ("backward", backward)):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                fn()
                torch.cuda.synchronize()   # the adapter synchronises the device itself before it returns
                if i >= 2:
                    times[name].append((time.perf_counter() - t0) * 1e3)
    except Exception as e:  # noqa: BLE001
        return {"unavailable": str(e)[:200]}
    fwd, bwd = statistics.median(times["forward"]), statistics.median(times["backward"])
    return {"forward_ms": fwd, "backward_ms": bwd, "step_ms": fwd + bwd, "value": T * B / ((fwd + bwd) * 1e-3), "unit": UNIT,
            "what": "the reference's own CUDA kernels (integer carrier, training forward + QAT backward) compiled for "
                    "sm_100a, same weights, inputs and quantization parameters; host clock around synchronous calls; "
                    "loss and optimizer step not included"}


def serial_chain_bound(lib, torch, device, cfg, T, I, H, full_kernel_ms, rows=2):
    """T x the minimal per-step latency of each recurrent kernel: the same two kernels timed on a batch that is ONE
    CTA's rows, where nothing but the dependent chain of a time step (barrier, shared-memory exchange of h, the dot
    products of one row block, the write of the step's caches) is left.  `frac` = that bound / the kernels' time
    at the full batch: 1.0 means that the full-size launch is no slower than its own chain of T steps."""
    from rx_met_b200.qat import GruQatStep
    eng = GruQatStep(T, rows, I, H, device, cfg, seed=99)
    gen = torch.Generator(device="cpu").manual_seed(7)
    x = torch.randn((T, rows, I), generator=gen).to(device)
    y = torch.randn((T, rows, H), generator=gen).to(device)
    eng.calibrate([x])
    for _ in range(3):
        eng.step(x, y, 1e-3)
    torch.cuda.synchronize()
    lib.rxmet_reset_kernel_timing()
    lib.rxmet_set_kernel_timing(1)
    reps = 10
    for _ in range(reps):
        eng.step(x, y, 1e-3)
    torch.cuda.synchronize()
    out = {"rows": rows, "T": T}
    bound = 0.0
    for name in ("recurrentForward", "recurrentBackward"):
        ms, cnt = C.c_double(), C.c_longlong()
        lib.rxmet_get_kernel_timing(name.encode(), C.byref(ms), C.byref(cnt))
        one = ms.value / max(cnt.value, 1)
        out[f"{name}_us_per_step"] = one * 1e3 / T
        out[f"{name}_ms"] = one
        bound += one
    lib.rxmet_set_kernel_timing(0)
    lib.rxmet_reset_kernel_timing()
    achieved = full_kernel_ms.get("recurrentForward", 0.0) + full_kernel_ms.get("recurrentBackward", 0.0)
    out.update({"bound_ms": bound, "achieved_ms": achieved, "frac": bound / achieved if achieved else None,
                "how": "both recurrent kernels on a batch of one CTA's rows; CUDA events around each launch"})
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    from rx_met_b200 import _cabi as cabi
    from rx_met_b200 import gru_interface_binding as ops
    from rx_met_b200.qat import GruQatStep
    from rx_met_b200.losses import mse_loss_grad, workspace as loss_workspace
    from rx_met_b200.staging import stage_from_pinned_host

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"   # keeps the library's version banner off stdout: one JSON line only
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD
    lib = cabi.load_library()
    if args.profile_only and args.workload == "aimet":
        # the AIMET native kernels on a 256 MiB tensor (larger than L2) for captures under a profiler
        out = aimet_kernel_bandwidth(lib, torch, device, _peaks()[0], elements=1 << 26, reps=2)
        print(json.dumps({"profile_only": True, "workload": "aimet", "result": out}), flush=True)
        return
    if args.profile_only and args.workload == "affine":
        # the learned-grid quantize-dequantize on 256 MiB tensors (larger than L2) for captures under a profiler
        out = affine_qdq_bandwidth(torch, device, _peaks()[0], reps=max(args.steps, 1) if args.affine_log2 > 26 else 2,
                                   elements=1 << args.affine_log2)
        print(json.dumps({"profile_only": True, "workload": "affine", "result": out}), flush=True)
        return
    if args.profile_only and args.workload == "lstm":
        # small LSTM training loop for captures under a profiler; prints no bench line
        lstm_secondary(lib, torch, device, torch.empty(1, dtype=torch.uint8, device=device), profile_steps=args.steps,
                       T_override=args.lstm_T)
        print(json.dumps({"profile_only": True, "workload": "lstm"}), flush=True)
        return
    if args.workload == "kws_body":
        run_kws_body(args, torch, dist, lib, device, group, rank, world, local_rank)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.profile_only and args.workload == "lstm_sweep":
        # one small inference forward of the configs[4] layer (T = --lstm-T or 50, B = 256) for captures under a profiler
        from rx_met_b200 import _cabi_lstm as L
        from rx_met_b200 import _quant_lstm as m
        T, B, I, H = args.lstm_T or 50, 256, 256, 512
        w = _lstm_weights(torch, device, I, H, 200)
        gen = torch.Generator(device="cpu").manual_seed(78)
        session = m.CalibrationSession(m._config_to_json(L.mixed_config(4, 16)), I, H, True, "minmax")
        session.collect(torch.randn((50, 64, I), generator=gen).to(device), *w)
        bundle = session.finalize(False)["bundle_json"]
        x = torch.randn((T, B, I), generator=gen).to(device)
        order = ("input", "weight_ih", "weight_hh", "bias_ih", "bias_hh", "h_0", "c_0")
        g = [torch.randn(s, generator=gen).to(device) for s in [(T, B, H), (B, H), (B, H)]]
        for _ in range(max(args.steps, 1) + args.warmup):
            if not args.lstm_qat:
                m.lstm_forward_quantized(x, *w, None, None, False, bundle)
                continue
            ck = m.lstm_forward_quantized(x, *w, None, None, False, bundle, "pedantic", False, True)[3]
            m.lstm_backward_qat([ck["quantized_master"][n] for n in order], False, bundle,
                                [ck["values"][n] for n in ("gate_outputs", "cell_states", "cell_tanh_outputs", "hidden_outputs")],
                                *g, [ck["master_clamp_masks"][n] for n in order], [ck["clamp_masks"][n] for n in L.TRACE_VALUES])
        torch.cuda.synchronize()
        print(json.dumps({"profile_only": True, "workload": "lstm_sweep", "T": T, "B": B, "qat": bool(args.lstm_qat)}), flush=True)
        return
    if args.workload in ("lstm_sweep", "lstm_bi"):
        flush_ = torch.empty(256 << 20, dtype=torch.uint8, device=device)
        fn = lstm_w4a16_sweep if args.workload == "lstm_sweep" else lstm_bidirectional_a16
        print(json.dumps({"workload": args.workload, "result": fn(lib, torch, device, flush_, _peaks()[0], args)}), flush=True)
        return
    T, B, I, H = (WORKLOAD[k] for k in "TBIH")
    cfg = ops.OperatorQuantConfig()
    for name in cabi.OP_NAMES:
        if name not in ("W", "R", "bw", "br"):
            setattr(cfg, f"{name}_symmetric_", False)  # W8 symmetric, A8 asymmetric
    eng = GruQatStep(T, B, I, H, device, cfg, process_group=group, seed=1234)
    gen = torch.Generator(device="cpu").manual_seed(1000 + rank)
    n_sets = 4
    xs_host = [torch.randn((T, B, I), generator=gen).pin_memory() for _ in range(n_sets)]
    ys_host = [torch.randn((T, B, H), generator=gen).pin_memory() for _ in range(n_sets)]
    xs = [t.to(device) for t in xs_host]
    ys = [t.to(device) for t in ys_host]
    eng.calibrate(xs[:2])
    lr = 1e-3
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)  # > 126 MB L2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for i in range(warmup):
            fn(i)
            flush.zero_()
        barrier()
        timed.launches0 = lib.rxmet_kernel_launch_count()
        start = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        stop = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        host0 = time.perf_counter()
        for i in range(steps):
            start[i].record()
            fn(i)
            stop[i].record()
            flush.zero_()
        timed.host_ms = (time.perf_counter() - host0) * 1e3 / steps  # host time to enqueue one step
        barrier()
        timed.launches = lib.rxmet_kernel_launch_count() - timed.launches0
        ms = sum(s.elapsed_time(e) for s, e in zip(start, stop))
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # --- device-resident leg
    replays = None
    if args.graph == "on":
        # one captured graph per resident input set: a replay is one launch for the whole step
        replays = [eng.capture_step(xs[k], ys[k], lr)[0] for k in range(n_sets)]

    def resident(i):
        if replays is not None:
            replays[i % n_sets]()
        else:
            eng.step(xs[i % n_sets], ys[i % n_sets], lr)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    total_ms = timed(resident, args.steps, args.warmup)
    launches = timed.launches if replays is None else args.steps * eng.captured_launches
    resident_host_ms = timed.host_ms
    clocks = sampler.stop() if rank == 0 else None
    st_per_step = T * B * world
    value = st_per_step * args.steps / (total_ms * 1e-3)

    if args.profile_only:
        if rank == 0:
            print(json.dumps({"profile_only": True, "ms_per_step": total_ms / args.steps, "value": value}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # --- per-kernel durations of the same step (second pass, CUDA events around every kernel)
    lib.rxmet_reset_kernel_timing()
    lib.rxmet_set_kernel_timing(1)
    k_steps = min(args.steps, 10)
    timed(lambda i: eng.step(xs[i % n_sets], ys[i % n_sets], lr), k_steps, 1)   # eager: events sit between launches
    names = ["recurrentForward", "recurrentBackward", "inputLinear", "quantizeTensor", "gemmTN", "gemmNT", "inputGradUmma", "packRecurrentBf16", "weightGradMma", "weightGradUmma", "reduceWeightGrad", "fillCodes", "packStepMasks",
             "reduceSplits", "columnSums", "channelPrep", "prepareWeights", "dequantCodes", "transposeMatrix"]
    per_kernel = {}
    for n in names:
        ms, cnt = C.c_double(), C.c_longlong()
        lib.rxmet_get_kernel_timing(n.encode(), C.byref(ms), C.byref(cnt))
        if cnt.value:
            per_kernel[n] = (ms.value, cnt.value)
    lib.rxmet_set_kernel_timing(0)
    top = max(per_kernel, key=lambda n: per_kernel[n][0])
    top_ms = per_kernel[top][0] / per_kernel[top][1]
    peak, peak_kind = _peaks()
    algo = _algo_bytes_per_st(I, H) * T * B
    achieved = algo / (top_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_kind": f"of {peak_kind}", "traffic": NCU_TRAFFIC_BYTES.get(top),
                "kernel_ms": top_ms, "algorithmic_bytes": algo,
                "kernel_ms_per_step": {n: v[0] / k_steps for n, v in per_kernel.items()}}

    roofline["serial_chain_bound"] = serial_chain_bound(lib, torch, device, cfg, T, I, H, roofline["kernel_ms_per_step"])

    # --- end-to-end leg through the reference-facing module
    W, R, bw, br = eng.W, eng.R, eng.bw, eng.br
    qp = eng.params
    # Two device buffers per input: the copy of step i+1 runs on a side stream while step i computes,
    # so every step still copies its own inputs from pinned host memory inside the timed region.
    x_buf = [torch.empty((T, B, I), device=device) for _ in range(2)]
    y_buf = [torch.empty((T, B, H), device=device) for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=device)
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    loss_host = torch.zeros(2, dtype=torch.float32).pin_memory()
    loss_dev = [torch.zeros((), dtype=torch.float32, device=device) for _ in range(2)]
    loss_ws = loss_workspace(device)
    loss_ready = [torch.cuda.Event() for _ in range(2)]
    losses = []
    state = {"primed": -1}

    def stage(i):
        slot = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[slot])
            if args.e2e_copy == "kernel":
                # the library's staging kernel: a few CTAs read the pinned buffers over PCIe
                stage_from_pinned_host(x_buf[slot], xs_host[i % n_sets], ctas=args.e2e_ctas, stream=copy_stream)
                stage_from_pinned_host(y_buf[slot], ys_host[i % n_sets], ctas=args.e2e_ctas, stream=copy_stream)
            else:
                x_buf[slot].copy_(xs_host[i % n_sets], non_blocking=True)
                y_buf[slot].copy_(ys_host[i % n_sets], non_blocking=True)
            copied[slot].record(copy_stream)

    def e2e(i):
        slot = i % 2
        if state["primed"] != i:  # first step of a timed region: nothing was staged ahead
            stage(i)
        stage(i + 1)
        state["primed"] = i + 1
        torch.cuda.current_stream(device).wait_event(copied[slot])
        x_dev, y_dev = x_buf[slot], y_buf[slot]
        out = ops.forward_quant_int_storage(True, T, B, I, H, W, R, bw, br, x_dev, None, qp)
        h, v = out[0], out[1]
        dh_new = torch.empty_like(h)
        dh_new[0].zero_()
        loss, _ = mse_loss_grad(h[1:], y_dev, dh_new[1:], loss_dev[slot], loss_ws)   # loss and its gradient, one pass
        dx, dW, dR, dbw, dbr, _ = ops.backward_quant_int_storage(T, B, I, H, *out[2:7], dh_new, h, v, qp, *out[7:])
        consumed[slot].record()
        grads = [dW, dR, dbw, dbr]
        if world > 1:
            # one NCCL group call for the four gradient tensors the module returned (no packing copy)
            with coalesced(group=group, device=device, async_ops=False):
                for g in grads:
                    dist.all_reduce(g)
        torch._foreach_add_([W, R, bw, br], grads, alpha=-lr / world)   # mean over ranks and SGD in one multi-tensor kernel
        # device -> host read of the step's result: asynchronous copy into pinned memory, collected one
        # step later so that the host never stalls the queue
        loss_host[slot:slot + 1].copy_(loss.reshape(1), non_blocking=True)
        loss_ready[slot].record()
        if i > 0:
            loss_ready[1 - slot].synchronize()
            losses.append(float(loss_host[1 - slot]))

    if world > 1:
        from torch.distributed.distributed_c10d import _coalescing_manager as coalesced
    e2e_steps = min(args.steps, 20)
    for ev in consumed:
        ev.record()
    e2e_ms = timed(e2e, e2e_steps, min(args.warmup, 3))
    e2e_host_ms = timed.host_ms
    e2e_value = st_per_step * e2e_steps / (e2e_ms * 1e-3)
    torch.cuda.synchronize()
    losses.append(float(loss_host[(e2e_steps - 1) % 2]))

    # --- the same end-to-end step through the preallocated engine (C ABI) as captured graphs: the inputs of
    # step i + 1 are staged from pinned host memory into the second buffer pair while the graph of step i runs
    engine_e2e = None
    if args.graph == "on":
        e_replay = [eng.capture_step(x_buf[k], y_buf[k], lr)[0] for k in range(2)]
        e_loss = eng.loss
        state["primed"] = -1

        def e2e_engine(i):
            slot = i % 2
            if state["primed"] != i:
                stage(i)
            stage(i + 1)
            state["primed"] = i + 1
            torch.cuda.current_stream(device).wait_event(copied[slot])
            e_replay[slot]()
            consumed[slot].record()
            loss_host[slot:slot + 1].copy_(e_loss.reshape(1), non_blocking=True)
            loss_ready[slot].record()
            if i > 0:
                loss_ready[1 - slot].synchronize()

        for ev in consumed:
            ev.record()
        eng_ms = timed(e2e_engine, e2e_steps, min(args.warmup, 3))
        torch.cuda.synchronize()
        engine_e2e = {"value": st_per_step * e2e_steps / (eng_ms * 1e-3), "unit": UNIT, "ms_per_step": eng_ms / e2e_steps,
                      "host_enqueue_ms_per_step": timed.host_ms, "final_loss": float(loss_host[(e2e_steps - 1) % 2]),
                      "what": "GruQatStep (C ABI) replayed as one captured graph per buffer pair, inputs staged from pinned "
                              "host memory by the staging kernel one step ahead, loss read back every step"}

    if rank == 0:
        cpu = None
        secondary = None
        reference_cuda = None
        if world == 1:
            secondary = {"aimet_native_kernels": aimet_kernel_bandwidth(lib, torch, device, peak),
                         "affine_qdq": affine_qdq_bandwidth(torch, device, peak),
                         "lstm_w8a8": lstm_secondary(lib, torch, device, flush),
                         "lstm_bidirectional_w8a16": lstm_bidirectional_a16(lib, torch, device, flush, peak, args),
                         "lstm_h512_w4a16_sweep": lstm_w4a16_sweep(lib, torch, device, flush, peak, args),
                         "kws_body_qat": kws_body_secondary(torch, device, flush, peak)}
            v_cpu, cores, kind, desc, _ = cpu_forward_throughput()
            cpu = {"value": v_cpu, "unit": UNIT, "cores": cores, "kind": kind, "sample": desc}
            reference_cuda = reference_cuda_step(torch, device, eng, xs[0])
        binding = {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms / e2e_steps, "host_enqueue_ms_per_step": e2e_host_ms,
                   "final_loss": losses[-1] if losses else None,
                   "through": "gru_interface_binding (the reference's module surface), eager launches"}
        # headline end-to-end figure: the preallocated engine over the C ABI when it ran (graph replay), else the binding
        head = engine_e2e if engine_e2e is not None else binding
        e2e_line = {"value": head["value"], "unit": UNIT, "steps": e2e_steps, "ms_per_step": head["ms_per_step"],
                    "h2d_bytes_per_step": 4 * T * B * (I + H) * world, "d2h_bytes_per_step": 4 * world,
                    "final_loss": head["final_loss"], "host_enqueue_ms_per_step": head["host_enqueue_ms_per_step"],
                    "copy": args.e2e_copy,
                    "through": engine_e2e["what"] if engine_e2e is not None else binding["through"],
                    "binding": binding}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 codes / int32 accumulate fwd, fp32 bwd",
            "data": "synthetic",
            "config": {"workload": "gru_qat_step", **WORKLOAD, "global_batch": B * world, "parallelism": f"dp{world}",
                       "quant": "W8 symmetric per-channel, A8 asymmetric, integer carrier", "l2": "flushed between steps",
                       "kernel_timing": "second pass of the same step with CUDA events around every kernel",
                       "launch": "cuda graph replay" if args.graph == "on" else "eager launches"},
            "roofline": roofline, "cpu_baseline": cpu, "reference_cuda": reference_cuda,
            "e2e": e2e_line,
            "host_enqueue_ms_per_step": resident_host_ms,
            "gpu_launches": int(launches), "clocks": clocks, "secondary": secondary,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def aimet_kernel_bandwidth(lib, torch, device, peak_gbs, elements=1 << 28, reps=10):
    """HBM-bound AIMET native kernels on a float32 tensor larger than L2 (1 GiB by default): GB/s of
    algorithmic traffic (QDQ 8 B/element, min/max and histogram 4 B/element) from CUDA events."""
    n = elements
    x = torch.randn(n, device=device)
    y = torch.empty_like(x)
    lib.rxmet_aimet_minmax_workspace_bytes.restype = C.c_size_t
    ws = torch.empty(lib.rxmet_aimet_minmax_workspace_bytes(), dtype=torch.uint8, device=device)
    mm = torch.empty(2, device=device)
    hist = torch.empty(lib.rxmet_aimet_pdf_size(), dtype=torch.int32, device=device)
    st = C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    calls = {
        "qdq": (8, lambda: lib.rxmet_aimet_qdq(p(x), C.c_uint64(n), 0, C.c_double(-4.0), C.c_double(3.96875),
                                                C.c_double(0.03125), 0, C.c_uint64(0), p(y), st)),
        "minmax": (4, lambda: lib.rxmet_aimet_minmax(p(x), C.c_uint64(n), C.c_uint64(n), 0, p(mm), p(mm[1:]), p(ws),
                                                      C.c_size_t(ws.numel()), st)),
        "histogram": (4, lambda: lib.rxmet_aimet_histogram(p(x), C.c_uint64(n), 0, C.c_double(0.01), -768, p(hist), st)),
    }
    out = {}
    for name, (bytes_per, fn) in calls.items():
        for _ in range(3):
            assert fn() == 0, lib.rxmet_last_error()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        gbs = bytes_per * n * reps / (e0.elapsed_time(e1) * 1e-3) / 1e9
        out[name] = {"GB/s": gbs, "frac_of_measured_hbm": gbs / peak_gbs, "bytes_per_element": bytes_per}
    out["elements"] = n
    return out


def affine_qdq_bandwidth(torch, device, peak_gbs, reps=10, elements=1 << 28):
    """Learned-grid quantize-dequantize (aimet_torch.v2 affine quantizers) on float32 tensors larger than L2:
    GB/s of algorithmic traffic from CUDA events: forward 8 B/element (read x, write y), backward 12 B/element
    (read x and the incoming gradient, write dx; the scale and offset sums ride along)."""
    from rx_met_b200 import affine_qdq
    shapes = {"per_tensor": ((elements,), ()), "rows_of_16384": ((elements >> 14, 16384), (elements >> 14, 1)),
              "columns_1024": ((elements >> 10, 1024), (1024,)),
              "blocks_of_64": ((elements >> 12, 4096), (elements >> 12, 64))}   # blockwise weights: block_size [1, 64]
    out = {}
    for name, (shape, grid_shape) in shapes.items():
        x = torch.randn(shape, device=device)
        g = torch.randn(shape, device=device)
        scale = torch.full(grid_shape, 0.02, device=device)
        offset = torch.zeros(grid_shape, device=device)
        n = x.numel()
        blocks = [1, 64] if name.startswith("blocks") else None
        calls = {
            "forward": (8, lambda: affine_qdq.forward(x, scale, offset, -128, 127, reciprocal=False, block_size=blocks)),
            "forward_fast": (8, lambda: affine_qdq.forward(x, scale, offset, -128, 127, reciprocal=True, block_size=blocks)),
            "backward": (12, lambda: affine_qdq.backward(g, x, scale, offset, -128, 127, reciprocal=False,
                                                         want_scale_grad=True, want_offset_grad=True, block_size=blocks)),
        }
        entry = {}
        for kind, (bytes_per, fn) in calls.items():
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            gbs = bytes_per * n * reps / (e0.elapsed_time(e1) * 1e-3) / 1e9
            entry[kind] = {"GB/s": gbs, "frac_of_measured_hbm": gbs / peak_gbs, "bytes_per_element": bytes_per}
        out[name] = entry
        del x, g
    return out



# --------------------------------------------------------------------------
# Roofline time of a recurrent workload: the slower of (GEMM flops / measured dense tensor peak) and
# (module-boundary + saved-state bytes / measured HBM copy rate).  The int8 tensor peak is not measured on
# this pool; the measured bf16 figure stands in for it (conservative for int8).
# --------------------------------------------------------------------------

def _tensor_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["bf16_tflops_sustained"]) * 1e12, "measured bf16 sustained"
    return 1.4e15, "fallback bf16 sustained"


def _roofline_frac(st_per_s, flops_per_st, bytes_per_st, hbm_gbs):
    tc, tc_kind = _tensor_peak()
    t_flops = flops_per_st / tc
    t_bytes = bytes_per_st / (hbm_gbs * 1e9)
    bound = "tensor" if t_flops >= t_bytes else "hbm"
    roof_st_per_s = 1.0 / max(t_flops, t_bytes)
    return {"bound": bound, "frac": st_per_s / roof_st_per_s, "roofline_st_per_s": roof_st_per_s,
            "flops_per_st": flops_per_st, "bytes_per_st": bytes_per_st, "tensor_peak": tc_kind}


def _event_ms(torch, fn, flush, reps, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(reps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / reps


def _lstm_weights(torch, device, I, H, seed):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    k = 1.0 / (H ** 0.5)
    u = lambda *s: ((torch.rand(s, generator=gen) * 2 - 1) * k).to(device)  # noqa: E731  PyTorch-default uniform init
    return [u(4 * H, I), u(4 * H, H), u(4 * H), u(4 * H)]


def _kernel_ms(lib, names, per=1):
    out = {}
    for n in names:
        ms, cnt = C.c_double(), C.c_longlong()
        lib.rxmet_get_kernel_timing(n.encode(), C.byref(ms), C.byref(cnt))
        if cnt.value:
            out[n] = ms.value / per
    return out


_LSTM_WIDE_KERNELS = ["lstmQuantizePlanes", "lstmQuantizeCodes", "lstmPrepChannelsWide", "lstmInputLinearWide", "lstmRecurrentWide",
                      "lstmRecurrentFloatWide", "lstmRecurrentFloat", "lstmInputLinearFloat", "lstmJobMinMax", "lstmJobHistogram",
                      "lstmRecurrentBackwardWide", "lstmRecurrentBackward", "lstmGemmNN", "lstmGemmRowsTN", "lstmReduceSplits",
                      "lstmColumnSums", "lstmDequantWeights", "lstmPackStepMasks", "inputGradUmma", "weightGradUmma",
                      "lstmReduceWeightGradT", "lstmInputGradNarrow", "lstmPackBackwardTiles"]


def lstm_bidirectional_a16(lib, torch, device, flush, peak_gbs, args):
    """Bidirectional QuantLSTM I=80, H=128, T=200, batch 128, W8 per-channel symmetric / A16 asymmetric:
    histogram (SQNR) calibration of two seeded batches through the product's CalibrationSession, then the
    quantized inference forward of both directions (two streams).  One seq-timestep = one batch element x one
    time step of BOTH directions."""
    from rx_met_b200 import _cabi_lstm as L
    from rx_met_b200 import _quant_lstm as m
    T, B, I, H = 200, 128, 80, 128
    cfg = L.mixed_config(8, 16)
    gen = torch.Generator(device="cpu").manual_seed(77)
    batches = [torch.randn((T, B, I), generator=gen).to(device) for _ in range(2)]
    x = torch.randn((T, B, I), generator=gen).to(device)
    x_rev = x.flip(0).contiguous()
    dirs = [_lstm_weights(torch, device, I, H, 100 + d) for d in range(2)]
    sessions = [m.CalibrationSession(m._config_to_json(cfg), I, H, True, "sqnr") for _ in range(2)]
    t0 = time.perf_counter()
    for xb in batches:
        for d, (s, w) in enumerate(zip(sessions, dirs)):
            s.collect(xb if d == 0 else xb.flip(0).contiguous(), *w)
    torch.cuda.synchronize()
    calib_s = time.perf_counter() - t0
    bundles = [s.finalize(False)["bundle_json"] for s in sessions]
    side = torch.cuda.Stream(device)

    def forward():
        main = torch.cuda.current_stream(device)
        side.wait_stream(main)
        m.lstm_forward_quantized(x, *dirs[0], None, None, False, bundles[0])
        with torch.cuda.stream(side):
            m.lstm_forward_quantized(x_rev, *dirs[1], None, None, False, bundles[1])
        main.wait_stream(side)

    ms = _event_ms(torch, forward, flush, reps=5)
    lib.rxmet_reset_kernel_timing(); lib.rxmet_set_kernel_timing(1)
    m.lstm_forward_quantized(x, *dirs[0], None, None, False, bundles[0])
    torch.cuda.synchronize()
    kernels = _kernel_ms(lib, _LSTM_WIDE_KERNELS)
    lib.rxmet_set_kernel_timing(0)
    st = T * B
    st_s = st / (ms * 1e-3)
    return {"workload": {"T": T, "B": B, "I": I, "H": H, "directions": 2, "quant": "W8 per-channel symmetric, A16 asymmetric"},
            "calibration": {"method": "sqnr histograms, 2048 bins", "batches": len(batches), "seconds": calib_s,
                            "seq_timesteps_per_s": len(batches) * st / calib_s},
            "quantized_forward": {"ms": ms, "seq_timesteps_per_s": st_s,
                                  "roofline": _roofline_frac(st_s, 425984, 1344, peak_gbs)},
            "kernel_ms_one_direction": kernels}


def lstm_w4a16_sweep(lib, torch, device, flush, peak_gbs, args):
    """QuantLSTM I=256, H=512, T=1000, W4 per-channel / A16, batch 1, 16, 256, 4096: quantized inference
    forward at every batch size; QAT forward + backward at 1, 16 and 256 (at 4096 the seven float checkpoint
    tensors and 14 masks the reference's training interface hands to the backward take more than one GPU's
    memory: 4,096,000 rows x (4 x 2048 + 3 x 512) x 5 bytes = 199 GB)."""
    from rx_met_b200 import _cabi_lstm as L
    from rx_met_b200 import _quant_lstm as m
    T, I, H = 1000, 256, 512
    cfg = L.mixed_config(4, 16)
    w = _lstm_weights(torch, device, I, H, 200)
    gen = torch.Generator(device="cpu").manual_seed(78)
    session = m.CalibrationSession(m._config_to_json(cfg), I, H, True, "minmax")
    session.collect(torch.randn((50, 64, I), generator=gen).to(device), *w)
    bundle = session.finalize(False)["bundle_json"]
    out = {"workload": {"T": T, "I": I, "H": H, "quant": "W4 per-channel symmetric, A16 asymmetric"}, "batch": {}}
    order = ("input", "weight_ih", "weight_hh", "bias_ih", "bias_hh", "h_0", "c_0")
    for B in (1, 16, 256, 4096):
        x = torch.randn((T, B, I), generator=gen).to(device)
        reps = 3 if B <= 256 else 2
        ms = _event_ms(torch, lambda: m.lstm_forward_quantized(x, *w, None, None, False, bundle), flush, reps, warmup=1)
        st = T * B
        entry = {"inference_forward": {"ms": ms, "seq_timesteps_per_s": st / (ms * 1e-3),
                                       "roofline": _roofline_frac(st / (ms * 1e-3), 3145728, 3072, peak_gbs)}}
        if B <= 256:
            g = [torch.randn(s, generator=gen).to(device) for s in [(T, B, H), (B, H), (B, H)]]
            saved = {}

            def qat():
                saved.clear()   # the previous step's checkpoints go back to the allocator before the next forward asks
                saved["o"] = m.lstm_forward_quantized(x, *w, None, None, False, bundle, "pedantic", False, True)
                ck = saved["o"][3]
                m.lstm_backward_qat([ck["quantized_master"][n] for n in order], False, bundle,
                                    [ck["values"][n] for n in ("gate_outputs", "cell_states", "cell_tanh_outputs", "hidden_outputs")],
                                    *g, [ck["master_clamp_masks"][n] for n in order], [ck["clamp_masks"][n] for n in L.TRACE_VALUES])

            ms_q = _event_ms(torch, qat, flush, reps=2, warmup=2)

            def training_forward():
                saved.clear()
                saved["o"] = m.lstm_forward_quantized(x, *w, None, None, False, bundle, "pedantic", False, True)

            ms_f = _event_ms(torch, training_forward, flush, reps=2, warmup=1)
            entry["qat_forward_backward"] = {"ms": ms_q, "training_forward_ms": ms_f, "backward_ms": ms_q - ms_f,
                                             "seq_timesteps_per_s": st / (ms_q * 1e-3),
                                             "roofline": _roofline_frac(st / (ms_q * 1e-3), 9437184, 23000, peak_gbs)}
            if B == 256:
                lib.rxmet_reset_kernel_timing(); lib.rxmet_set_kernel_timing(1)
                qat()
                torch.cuda.synchronize()
                entry["kernel_ms_qat_step"] = _kernel_ms(lib, _LSTM_WIDE_KERNELS)
                lib.rxmet_set_kernel_timing(0)
            del saved, g
        out["batch"][str(B)] = entry
        del x
        torch.cuda.empty_cache()
    return out


KWS = dict(T=100, B=128, I=40, H=256, layers=3, classes=12)


def _kws_engine(torch, device, group, rank):
    from rx_met_b200.stacked_qat import StackedGruQat, a16_config
    T, B, I, H = KWS["T"], KWS["B"], KWS["I"], KWS["H"]
    eng = StackedGruQat(T, B, I, H, KWS["layers"], KWS["classes"], device, a16_config(8, 16), process_group=group, seed=4321)
    gen = torch.Generator(device="cpu").manual_seed(2000 + rank)
    xs_host = [torch.randn((T, B, I), generator=gen).clamp_(-4, 4).pin_memory() for _ in range(4)]
    ys_host = [torch.randint(0, KWS["classes"], (B,), generator=gen).pin_memory() for _ in range(4)]
    xs = [t.to(device) for t in xs_host]
    ys = [t.to(device) for t in ys_host]
    eng.calibrate(xs[:2])
    return eng, xs_host, ys_host, xs, ys


_GRU_KERNELS = ["recurrentForward", "recurrentBackward", "inputLinear", "quantizeTensor", "gemmTN", "gemmNT", "inputGradUmma",
                "packRecurrentBf16", "weightGradMma", "weightGradUmma", "reduceWeightGrad", "fillCodes", "packStepMasks",
                "reduceSplits", "columnSums", "channelPrep", "prepareWeights", "dequantCodes", "transposeMatrix"]
KWS_FLOPS_PER_ST, KWS_BYTES_PER_ST = 16883712, 57000


def kws_body_secondary(torch, device, flush, peak_gbs):
    """The stacked bidirectional QuantGRU QAT step (3 x bi-GRU H=256, 40 -> 512 -> 512, T=100, batch 128 per
    GPU, W8 per-channel / A16, linear head + cross-entropy) on one GPU."""
    from rx_met_b200 import _cabi as cabi
    lib = cabi.load_library()
    eng, _, _, xs, ys = _kws_engine(torch, device, None, 0)
    state = {"i": 0}

    def step():
        eng.step(xs[state["i"] % 4], ys[state["i"] % 4], 1e-3)
        state["i"] += 1

    ms = _event_ms(torch, step, flush, reps=5)
    lib.rxmet_reset_kernel_timing(); lib.rxmet_set_kernel_timing(1)
    step()
    torch.cuda.synchronize()
    kernels = _kernel_ms(lib, _GRU_KERNELS)
    lib.rxmet_set_kernel_timing(0)
    st = KWS["T"] * KWS["B"]
    return {"workload": {**KWS, "quant": "W8 per-channel symmetric, A16"}, "ms_per_step": ms, "seq_timesteps_per_s": st / (ms * 1e-3),
            "roofline": _roofline_frac(st / (ms * 1e-3), KWS_FLOPS_PER_ST, KWS_BYTES_PER_ST, peak_gbs),
            "kernel_ms_per_step": kernels, "gradient_floats": int(eng.flat_g.numel())}


def run_kws_body(args, torch, dist, lib, device, group, rank, world, local_rank):
    """Bench line of the stacked bidirectional QuantGRU QAT step, batch 128 per GPU (weak scaling)."""
    eng, xs_host, ys_host, xs, ys = _kws_engine(torch, device, group, rank)
    T, B = KWS["T"], KWS["B"]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    lr = 1e-3
    if args.profile_only:   # a few plain steps for captures under a profiler; prints no bench line
        for i in range(args.warmup + args.steps):
            eng.step(xs[i % 4], ys[i % 4], lr)
        torch.cuda.synchronize()
        if rank == 0:
            print(json.dumps({"profile_only": True, "workload": "kws_body"}), flush=True)
        return

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for i in range(warmup):
            fn(i)
            flush.zero_()
        barrier()
        l0 = lib.rxmet_kernel_launch_count()
        start = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        stop = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        for i in range(steps):
            start[i].record(); fn(i); stop[i].record()
            flush.zero_()
        barrier()
        timed.launches = lib.rxmet_kernel_launch_count() - l0
        t = torch.tensor([sum(s.elapsed_time(e) for s, e in zip(start, stop))], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if args.graph == "on":
        # one captured graph per resident input set: a replay is one launch for the whole step
        replays = [eng.capture_step(xs[k], ys[k], lr)[0] for k in range(4)]
        total_ms = timed(lambda i: replays[i % 4](), args.steps, args.warmup)
        launches = args.steps * eng.captured_launches
    else:
        total_ms = timed(lambda i: eng.step(xs[i % 4], ys[i % 4], lr), args.steps, args.warmup)
        launches = timed.launches
    clocks = sampler.stop() if rank == 0 else None
    st_per_step = T * B * world
    value = st_per_step * args.steps / (total_ms * 1e-3)

    # end to end: this step's inputs come from pinned host memory, the loss goes back to the host
    x_buf, y_buf = torch.empty_like(xs[0]), torch.empty_like(ys[0])
    loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()

    x_buf.copy_(xs[0]); y_buf.copy_(ys[0])   # the capture's warm-up steps read the buffers: valid features and labels
    e2e_replay = eng.capture_step(x_buf, y_buf, lr)[0] if args.graph == "on" else None

    def e2e(i):
        x_buf.copy_(xs_host[i % 4], non_blocking=True)
        y_buf.copy_(ys_host[i % 4], non_blocking=True)
        loss = e2e_replay() if e2e_replay is not None else eng.step(x_buf, y_buf, lr)
        loss_host.copy_(loss.reshape(1), non_blocking=True)

    e2e_steps = min(args.steps, 10)
    e2e_ms = timed(e2e, e2e_steps, 3)
    torch.cuda.synchronize()
    # per-kernel durations of one more step; every rank runs it (the step holds the gradient all-reduce)
    lib.rxmet_reset_kernel_timing(); lib.rxmet_set_kernel_timing(1)
    eng.step(xs[0], ys[0], 0.0)
    torch.cuda.synchronize()
    kernels = _kernel_ms(lib, _GRU_KERNELS)
    lib.rxmet_set_kernel_timing(0)
    if rank != 0:
        return
    peak, peak_kind = _peaks()
    roof = _roofline_frac(value / world, KWS_FLOPS_PER_ST, KWS_BYTES_PER_ST, peak)
    top = max(kernels, key=kernels.get)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 weight codes x int16 activation codes / int64 accumulate fwd, fp32 bwd", "data": "synthetic",
        "config": {"workload": "kws_body", **KWS, "global_batch": B * world, "parallelism": f"dp{world}",
                   "quant": "W8 per-channel symmetric, A16, integer carrier", "l2": "flushed between steps",
                   "launch": "cuda graph replay" if args.graph == "on" else "eager launches"},
        "roofline": {"bound": roof["bound"], "kernel": top, "achieved": value / world * (KWS_BYTES_PER_ST if roof["bound"] == "hbm" else KWS_FLOPS_PER_ST) / (1e9 if roof["bound"] == "hbm" else 1e12),
                     "peak": peak if roof["bound"] == "hbm" else _tensor_peak()[0] / 1e12,
                     "unit": "GB/s" if roof["bound"] == "hbm" else "TFLOP/s", "frac": roof["frac"],
                     "peak_kind": f"of {peak_kind}", "traffic": None, "scope": "whole step",
                     "kernel_ms_per_step": kernels},
        "cpu_baseline": None,
        "e2e": {"value": st_per_step * e2e_steps / (e2e_ms * 1e-3), "unit": UNIT, "steps": e2e_steps,
                "h2d_bytes_per_step": (4 * T * B * KWS["I"] + 8 * B) * world, "d2h_bytes_per_step": 4 * world,
                "final_loss": float(loss_host[0]), "ms_per_step": e2e_ms / e2e_steps},
        "gpu_launches": int(launches), "clocks": clocks, "gradient_allreduce_bytes": int(eng.flat_g.numel()) * 4,
    }
    print(json.dumps(line), flush=True)


def lstm_secondary(lib, torch, device, flush, profile_steps=0, T_override=None):
    """QuantLSTM at the same shape as the headline GRU workload (T=100, B=256, I=40, H=128, all
    points 8 bit symmetric, per-channel weights): seq-timesteps/s of the quantized inference
    forward, the training forward (7 checkpoints + masks saved) and the QAT backward, the
    per-kernel milliseconds, and the reference's CPU quantized forward on the host cores."""
    import numpy as np
    import lstm_lib as ll
    from rx_met_b200 import _cabi_lstm as L
    from rx_met_b200 import _quant_lstm as m
    T, B, I, H = (WORKLOAD[k] for k in "TBIH")
    T = T_override or T
    p = ll.problem(T, 16, I, H, seed=5, wscale=0.15)
    cfg = L.default_config(symmetric_activations=True)
    to_dev = lambda a: torch.from_numpy(a).to(device)  # noqa: E731
    session = m.CalibrationSession(m._config_to_json(cfg), I, H, True, "minmax")   # the product's calibration
    session.collect(to_dev(p["x"]), to_dev(p["w_ih"]), to_dev(p["w_hh"]), to_dev(p["b_ih"]), to_dev(p["b_hh"]),
                    to_dev(p["h0"])[None], to_dev(p["c0"])[None])
    bundle = session.finalize(False)["bundle_json"]
    box = m._bundle_to_params(bundle)
    gen = torch.Generator(device="cpu").manual_seed(99)
    x = torch.randn((T, B, I), generator=gen).to(device)
    h0 = (torch.randn((1, B, H), generator=gen) * 0.5).to(device)
    c0 = (torch.randn((1, B, H), generator=gen) * 0.5).to(device)
    w = [torch.from_numpy(p[k]).to(device) for k in ("w_ih", "w_hh", "b_ih", "b_hh")]
    g = [torch.randn(s, generator=gen).to(device) for s in [(T, B, H), (B, H), (B, H)]]
    saved = {}

    def infer():
        m.lstm_forward_quantized(x, *w, h0, c0, False, bundle)

    def train_fwd():
        saved["out"] = m.lstm_forward_quantized(x, *w, h0, c0, False, bundle, "pedantic", False, True)

    def qat_bwd():
        ck = saved["out"][3]
        order = ("input", "weight_ih", "weight_hh", "bias_ih", "bias_hh", "h_0", "c_0")
        m.lstm_backward_qat([ck["quantized_master"][n] for n in order], False, bundle,
                            [ck["values"][n] for n in ("gate_outputs", "cell_states", "cell_tanh_outputs", "hidden_outputs")],
                            *g, [ck["master_clamp_masks"][n] for n in order], [ck["clamp_masks"][n] for n in L.TRACE_VALUES])

    def time_it(fn, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / reps

    if profile_steps:
        for _ in range(profile_steps):
            train_fwd(); qat_bwd()
        torch.cuda.synchronize()
        return None
    out = {"workload": {"T": T, "B": B, "I": I, "H": H, "quant": "W8 per-channel symmetric, A8 symmetric, float-carrier semantics"}}
    ms_inf, ms_fwd = time_it(infer), time_it(train_fwd)
    ms_bwd = time_it(qat_bwd)
    st = T * B
    out["inference_forward"] = {"ms": ms_inf, "seq_timesteps_per_s": st / (ms_inf * 1e-3)}
    out["training_forward"] = {"ms": ms_fwd, "seq_timesteps_per_s": st / (ms_fwd * 1e-3)}
    out["qat_backward"] = {"ms": ms_bwd, "seq_timesteps_per_s": st / (ms_bwd * 1e-3)}
    out["qat_forward_backward"] = {"ms": ms_fwd + ms_bwd, "seq_timesteps_per_s": st / ((ms_fwd + ms_bwd) * 1e-3)}
    lib.rxmet_reset_kernel_timing()
    lib.rxmet_set_kernel_timing(1)
    for _ in range(3):
        train_fwd(); qat_bwd()
    torch.cuda.synchronize()
    per = {}
    for n in ["lstmQuantizeCodes", "lstmPrepChannels", "lstmInputLinearQ", "lstmRecurrentQ", "lstmDequantWeights",
              "lstmPackStepMasks", "lstmRecurrentBackward", "lstmRecurrentBackwardMma", "lstmGemmNN", "lstmInputGradNarrow", "inputGradUmma", "lstmGemmRowsTN", "lstmReduceSplits",
              "lstmColumnSums", "weightGradMma", "weightGradUmma", "lstmReduceWeightGradT"]:
        ms, cnt = C.c_double(), C.c_longlong()
        lib.rxmet_get_kernel_timing(n.encode(), C.byref(ms), C.byref(cnt))
        if cnt.value:
            per[n] = ms.value / 3
    lib.rxmet_set_kernel_timing(0)
    out["kernel_ms_per_step"] = per
    # per-kernel HBM roofline of the training step: algorithmic bytes per sequence-step (C = 4H gate channels; the
    # training forward writes 7 float checkpoints and 14 byte masks, the backward reads them once)
    C4 = 4 * H
    algorithmic = {"lstmQuantizeCodes": 5 * I, "lstmInputLinearQ": I + C4 * 4 + C4 * 5,
                   "lstmRecurrentQ": C4 * 4 + H + (4 * C4 + 3 * H) * 5 - C4 * 5, "lstmPackStepMasks": (4 * C4 + 3 * H) + 4 * H,
                   "lstmRecurrentBackwardMma": (C4 + 3 * H + H) * 4 + 4 * H + 2 * C4 * 4,
                   "lstmRecurrentBackward": (C4 + 3 * H + H) * 4 + 4 * H + 2 * C4 * 4,
                   "inputGradUmma": C4 * 4 + I * 5, "weightGradUmma": 2 * C4 * 4 + (I + H) * 4}
    peak, peak_kind = _peaks()
    out["kernel_roofline"] = {n: {"bytes_per_st": algorithmic[n], "GB/s": algorithmic[n] * st / (ms * 1e-3) / 1e9,
                                  "frac": algorithmic[n] * st / (ms * 1e-3) / 1e9 / peak, "peak_kind": f"of {peak_kind}"}
                              for n, ms in per.items() if n in algorithmic}
    # the reference's CPU quantized forward (its only CPU path) on all host cores, bounded sample
    prefix = "ref" if ll.have_ref() else "orc"
    q = ll.quantize_masters("orc", p, box)
    cores = os.cpu_count() or 1

    def shard(_):
        ll.forward_quantized(prefix, box, T, 16, q)

    t0 = time.perf_counter(); shard(0); one = time.perf_counter() - t0
    n_shards = cores * max(1, int(4.0 / max(one, 1e-3)))
    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=cores) as pool:
        list(pool.map(shard, range(n_shards)))
    dt = time.perf_counter() - t0
    out["cpu_baseline"] = {"value": n_shards * 16 * T / dt, "unit": UNIT, "cores": cores,
                           "kind": "reference" if prefix == "ref" else "port",
                           "sample": f"{n_shards} shards of 16 sequences x T={T}, q-carrier forward only, {dt:.1f} s"}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["gru", "lstm", "aimet", "affine", "kws_body", "lstm_sweep", "lstm_bi"], default="gru",
                    help="gru (default): the headline QAT step.  kws_body: the stacked bidirectional QuantGRU QAT step "
                         "(its own bench line, any --gpus).  lstm_sweep / lstm_bi: print the QuantLSTM W4/A16 batch sweep or "
                         "the bidirectional W8/A16 calibration + forward as a JSON object (1 GPU).  With --profile-only: "
                         "which loop to run under a profiler")
    ap.add_argument("--e2e-ctas", type=int, default=4, help="CTAs of the staging kernel in the end-to-end leg")
    ap.add_argument("--lstm-T", type=int, default=20, help="sequence length of the --profile-only lstm loop")
    ap.add_argument("--lstm-qat", action="store_true",
                    help="--profile-only lstm_sweep loop: training forward + QAT backward instead of the inference forward")
    ap.add_argument("--e2e-copy", choices=["kernel", "dma"], default="kernel",
                    help="how the end-to-end leg moves a step's inputs from pinned host memory: the library's staging "
                         "kernel (rxmet_stage_from_pinned_host) or copy-engine transfers")
    ap.add_argument("--affine-log2", type=int, default=26,
                    help="log2 of the element count of the --profile-only affine tensors (26: a small case for captures)")
    ap.add_argument("--graph", choices=["on", "off"], default="on",
                    help="device-resident leg: replay the step as one captured CUDA graph per input set")
    ap.add_argument("--profile-only", action="store_true",
                    help="run only the device-resident leg (for captures under a profiler); prints no bench line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        if args.warmup < 3:
            args.warmup = 3
        run_ours(args)


if __name__ == "__main__":
    main()
