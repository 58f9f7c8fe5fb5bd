"""Preallocated QuantGRU calibration + QAT step over the C ABI (one direction, one layer).

``gru_interface_binding`` mirrors the reference's call-by-call interface and allocates its
outputs on every call, as the reference does.  A training loop that runs the same shapes every
step does not need that: this class allocates every buffer once (weights and their gradients as
views of two flat tensors, so that the data-parallel all-reduce and the SGD update are one
operation each) and then only launches kernels.  Batches shard over ranks; the only exchanges
are the calibration min/max all-reduce and the gradient all-reduce.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from . import _cabi as cabi
from .gru_interface_binding import GRUQuantParams, OperatorQuantConfig


def _p(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else None


class GruQatStep:
    def __init__(self, T: int, B: int, I: int, H: int, device: torch.device,
                 config: Optional[OperatorQuantConfig] = None, process_group=None, seed: int = 0,
                 weights: Optional[torch.Tensor] = None, grads: Optional[torch.Tensor] = None):
        """`weights` / `grads`: optional flat float32 device tensors of `parameter_count(I, H)` elements that
        this object uses as its master weights and gradient buffer (slices of a larger flat buffer, so that a
        stack of layers all-reduces and updates in one operation); the caller initialises `weights`."""
        self.lib = cabi.load_library()
        self.T, self.B, self.I, self.H = T, B, I, H
        self.device = torch.device(device)
        self.group = process_group
        self.world = torch.distributed.get_world_size(process_group) if process_group is not None else 1
        self.config = config or OperatorQuantConfig()
        C3 = 3 * H
        f32 = dict(dtype=torch.float32, device=self.device)
        # master weights (gate order z,r,n; W [I,3H], R [H,3H]) and their gradients, flat
        sizes = [I * C3, H * C3, C3, C3]
        if weights is not None:
            if weights.numel() != sum(sizes) or grads is None or grads.numel() != sum(sizes):
                raise ValueError("weights and grads must both hold parameter_count(I, H) elements")
            self.flat_w, self.flat_g = weights, grads
        else:
            self.flat_w = torch.empty(sum(sizes), **f32)
            self.flat_g = torch.zeros(sum(sizes), **f32)
            gen = torch.Generator(device="cpu").manual_seed(seed)
            k = 1.0 / (H ** 0.5)
            self.flat_w.copy_((torch.rand(sum(sizes), generator=gen) * 2 - 1) * k)  # same on every rank
        offs = [0]
        for s in sizes:
            offs.append(offs[-1] + s)
        view = lambda flat, i, shape: flat[offs[i]:offs[i + 1]].view(shape)  # noqa: E731
        self.W, self.R = view(self.flat_w, 0, (I, C3)), view(self.flat_w, 1, (H, C3))
        self.bw, self.br = view(self.flat_w, 2, (C3,)), view(self.flat_w, 3, (C3,))
        self.dW, self.dR = view(self.flat_g, 0, (I, C3)), view(self.flat_g, 1, (H, C3))
        self.dbw, self.dbr = view(self.flat_g, 2, (C3,)), view(self.flat_g, 3, (C3,))
        # activations, caches, masks
        i32 = dict(dtype=torch.int32, device=self.device)
        u8 = dict(dtype=torch.uint8, device=self.device)
        self.h = torch.empty((T + 1, B, H), **f32)
        self.v = torch.empty((T, B, 4 * H), **f32)
        self.W_q, self.R_q = torch.empty((I, C3), **i32), torch.empty((H, C3), **i32)
        self.bw_q, self.br_q = torch.empty((C3,), **i32), torch.empty((C3,), **i32)
        self.x_q = torch.empty((T, B, I), **i32)
        shapes = {"x": (T, B, I), "W": (I, C3), "R": (H, C3), "bw": (C3,), "br": (C3,),
                  "weight_ih_linear": (T, B, C3), "weight_hh_linear": (T, B, C3), "gate_input": (T, B, C3),
                  "gate_output": (T, B, C3), "h": (T, B, H)}
        self.masks = {k_: torch.empty(s, **u8) for k_, s in shapes.items()}
        self.mask_struct = cabi.Masks()
        for k_, t in self.masks.items():
            setattr(self.mask_struct, k_, t.data_ptr())
        # compact save-for-backward of the clamp flags: one 16-bit word per element and step instead of 13 mask bytes,
        # written by the forward itself (used when the library supports it for the parameters in force)
        self.step_flags = torch.empty((T, B, H), dtype=torch.int16, device=self.device)
        self.packed_mask_struct = cabi.Masks()
        for k_ in ("x", "W", "R", "bw", "br", "weight_ih_linear"):
            setattr(self.packed_mask_struct, k_, self.masks[k_].data_ptr())
        self._packed = False
        self.dh_new = torch.zeros((T + 1, B, H), **f32)
        self.dx = torch.empty((T, B, I), **f32)
        self.dh0 = torch.empty((B, H), **f32)
        nbytes = max(self.lib.rxmet_gru_workspace_bytes(op, T, B, I, H) for op in (0, 1, 2))
        self.ws = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.stats = torch.empty(self.lib.rxmet_gru_stats_floats(H), **f32)
        self.lib.rxmet_mse_loss_workspace_bytes.restype = C.c_size_t
        self.lib.rxmet_mse_loss_grad.restype = C.c_int
        self.lib.rxmet_mse_loss_grad.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p,
                                                 C.c_size_t, C.c_void_p]
        self.loss = torch.zeros((), **f32)
        self.loss_ws = torch.empty(self.lib.rxmet_mse_loss_workspace_bytes(), dtype=torch.uint8, device=self.device)
        self.params: Optional[GRUQuantParams] = None
        self._c_params = None
        self._keep = None

    @staticmethod
    def parameter_count(I: int, H: int) -> int:
        """Elements of W [I,3H], R [H,3H], bw [3H] and br [3H] together."""
        return (I + H + 2) * 3 * H

    # ---- calibration -----------------------------------------------------
    def calibrate(self, batches) -> GRUQuantParams:
        """min/max calibration over an iterable of [T,B,I] device tensors.  With a process group
        the per-batch statistics are all-reduced (MIN / MAX), so every rank derives the same
        encodings as one process would on the concatenated batch."""
        self.begin_calibration()
        for x in batches:
            self.observe(x)
        return self.finish_calibration()

    def begin_calibration(self) -> None:
        from .gru_interface_binding import GRUQuantizationRanges
        self._ranges = GRUQuantizationRanges(self.H)
        self._c_ranges, self._ranges_keep = self._ranges._to_c()

    def observe(self, x: torch.Tensor) -> torch.Tensor:
        """Float forward of one calibration batch that folds the ranges of all quantization points into the
        running calibration; returns the float output sequence h[1:] (a view that the next call overwrites)."""
        half = self.stats.numel() // 2
        with torch.cuda.device(self.device):
            cabi.check(self.lib.rxmet_gru_forward_calibrate_stats(
                self.T, self.B, self.I, self.H, _p(self.W), _p(self.R), _p(self.bw), _p(self.br), _p(x), None,
                _p(self.h), _p(self.v), _p(self.stats), _p(self.ws), C.c_size_t(self.ws.numel()), self._stream()),
                "forward_calibrate_stats")
        if self.group is not None:
            torch.distributed.all_reduce(self.stats[:half], op=torch.distributed.ReduceOp.MIN, group=self.group)
            torch.distributed.all_reduce(self.stats[half:], op=torch.distributed.ReduceOp.MAX, group=self.group)
        host = self.stats.cpu().contiguous()
        cabi.check(self.lib.rxmet_gru_ranges_fold_stats(
            C.byref(self._c_ranges), C.cast(host.data_ptr(), C.POINTER(C.c_float))), "ranges_fold_stats")
        return self.h[1:]

    def finish_calibration(self) -> GRUQuantParams:
        from .gru_interface_binding import calculate_gru_quantitative_parameters
        self._ranges._from_c(self._c_ranges, self._ranges_keep)
        self.set_params(calculate_gru_quantitative_parameters(self._ranges, self.config))
        return self.params

    def set_params(self, params: GRUQuantParams) -> None:
        self.params = params
        self._c_params, self._keep = params._to_c()
        self._packed = (os.environ.get("RXMET_QAT_BYTE_MASKS") is None and
                        bool(self.lib.rxmet_gru_packed_flags_supported(C.byref(self._c_params), self.B, self.I, self.H)))

    # ---- one training step -------------------------------------------------
    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Quantized training forward; returns the output sequence h[1:] (a view)."""
        with torch.cuda.device(self.device):
            if self._packed:
                cabi.check(self.lib.rxmet_gru_forward_quant_packed(
                    self.T, self.B, self.I, self.H, _p(self.W), _p(self.R), _p(self.bw), _p(self.br), _p(x), None,
                    C.byref(self._c_params), _p(self.h), _p(self.v), _p(self.W_q), _p(self.R_q), _p(self.bw_q),
                    _p(self.br_q), _p(self.x_q), C.byref(self.packed_mask_struct), _p(self.step_flags), _p(self.ws),
                    C.c_size_t(self.ws.numel()), self._stream()), "forward_quant_packed")
                return self.h[1:]
            cabi.check(self.lib.rxmet_gru_forward_quant(
                1, self.T, self.B, self.I, self.H, _p(self.W), _p(self.R), _p(self.bw), _p(self.br), _p(x), None,
                C.byref(self._c_params), _p(self.h), _p(self.v), _p(self.W_q), _p(self.R_q), _p(self.bw_q),
                _p(self.br_q), _p(self.x_q), None, None, C.byref(self.mask_struct), _p(self.ws),
                C.c_size_t(self.ws.numel()), self._stream()), "forward_quant")
        return self.h[1:]

    def backward(self) -> None:
        """BPTT from self.dh_new ([T+1,B,H], row 0 unused) into the flat gradient buffer."""
        with torch.cuda.device(self.device):
            if self._packed:
                cabi.check(self.lib.rxmet_gru_backward_quant_packed(
                    self.T, self.B, self.I, self.H, _p(self.W_q), _p(self.R_q), _p(self.x_q), _p(self.dh_new), _p(self.h),
                    _p(self.v), C.byref(self._c_params), C.byref(self.packed_mask_struct), _p(self.step_flags),
                    _p(self.dx), _p(self.dW), _p(self.dR), _p(self.dbw), _p(self.dbr), _p(self.dh0), _p(self.ws),
                    C.c_size_t(self.ws.numel()), self._stream()), "backward_quant_packed")
                return
            cabi.check(self.lib.rxmet_gru_backward_quant(
                self.T, self.B, self.I, self.H, _p(self.W_q), _p(self.R_q), _p(self.bw_q), _p(self.br_q), _p(self.x_q),
                _p(self.dh_new), _p(self.h), _p(self.v), C.byref(self._c_params), C.byref(self.mask_struct),
                _p(self.dx), _p(self.dW), _p(self.dR), _p(self.dbw), _p(self.dbr), _p(self.dh0), _p(self.ws),
                C.c_size_t(self.ws.numel()), self._stream()), "backward_quant")

    def mse_loss(self, target: torch.Tensor) -> torch.Tensor:
        """Mean-squared error of the output sequence against `target` ([T,B,H] float32, contiguous) and its gradient
        into self.dh_new[1:], one fused pass.  Returns self.loss, the device scalar every call overwrites."""
        if target.dtype != torch.float32 or not target.is_contiguous() or tuple(target.shape) != (self.T, self.B, self.H):
            raise ValueError("target must be a contiguous float32 tensor of shape [T, B, H]")
        out, grad = self.h[1:], self.dh_new[1:]
        with torch.cuda.device(self.device):
            cabi.check(self.lib.rxmet_mse_loss_grad(_p(out), _p(target), out.numel(), _p(grad), _p(self.loss),
                                                    _p(self.loss_ws), self.loss_ws.numel(), self._stream()), "mse_loss_grad")
        return self.loss

    def step(self, x: torch.Tensor, target: torch.Tensor, lr: float) -> torch.Tensor:
        """forward, MSE loss and its gradient, backward, gradient all-reduce, SGD update.  Returns the loss
        (self.loss: a device scalar, not synchronised, overwritten by the next step)."""
        self.forward(x)
        loss = self.mse_loss(target)
        self.backward()
        if self.group is not None:
            torch.distributed.all_reduce(self.flat_g, group=self.group)
        self.flat_w.add_(self.flat_g, alpha=-lr / self.world)   # mean over ranks folded into the update
        return loss

    # ---- the same step as one graph launch ----------------------------------
    def capture_step(self, x: torch.Tensor, target: torch.Tensor, lr: float, warmup: int = 3):
        """Captures `step` on fixed buffers into a CUDA graph and returns `(replay, loss)`: `replay()` launches
        the whole step (about ten kernels, two small copies, the loss and the update) as one graph on the
        current stream; `loss` is the device scalar it refreshes.  `x` and `target` are read at replay time, so
        the caller fills them in place (for example with `staging.stage_from_pinned_host`) before each replay.
        With a process group only the local part is captured; the gradient all-reduce and the update follow
        the graph launch.  The quantization parameters in force at capture are baked in: capture again after
        `set_params`.  `warmup` eager steps run first (they do train), so that every lazy initialisation of the
        library has happened before the capture begins."""
        if self._c_params is None:
            raise RuntimeError("calibrate or set_params before capturing a step")
        local = self.group is None

        def body():
            self.forward(x)
            loss_ = self.mse_loss(target)
            self.backward()
            if local:
                self.flat_w.add_(self.flat_g, alpha=-lr)
            return loss_

        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(max(warmup, 1)):
                self.step(x, target, lr)
        torch.cuda.current_stream(self.device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        before = self.lib.rxmet_kernel_launch_count()
        with torch.cuda.graph(graph, stream=side):
            loss = body()
        self.captured_launches = int(self.lib.rxmet_kernel_launch_count() - before)  # library kernels per replay

        def replay():
            graph.replay()
            if not local:
                torch.distributed.all_reduce(self.flat_g, group=self.group)
                self.flat_w.add_(self.flat_g, alpha=-lr / self.world)   # mean over ranks folded into the update
            return loss

        self._graph = graph   # keeps the captured buffers alive with the object
        return replay, loss
