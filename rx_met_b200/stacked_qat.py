"""QAT step of a stack of bidirectional QuantGRU layers with a linear classification head.

The reference builds such a body from `QuantGRU(bidirectional=True)` modules
(operators/quant-gru/pytorch/quant_gru.py:1120-1260; the reverse direction runs on the time-flipped
input and its output is flipped back and concatenated, quant_gru.py:2273-2288) under a classifier, as
in examples/quick_start_kws.py:669-719.  Every direction of every layer is one `GruQatStep` (C ABI,
preallocated buffers); this class owns what lies between them:

* ONE flat weight buffer and ONE flat gradient buffer for all layers, directions and the head, so the
  data-parallel exchange is a single all-reduce and the SGD update a single operation;
* the two directions of a layer on two CUDA streams, so their recurrences overlap;
* min/max calibration layer by layer (layer k+1 observes the float outputs of layer k), statistics
  all-reduced across ranks before they are folded;
* the head: mean over time, linear layer, cross-entropy with its gradient written straight into the
  buffer the top layer's backward reads.

Torch supplies device memory, streams, the (tiny) head arithmetic and the collectives; the recurrent
layers run in the library.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .gru_interface_binding import OperatorQuantConfig
from .qat import GruQatStep


def a16_config(weight_bits: int = 8, activation_bits: int = 16) -> OperatorQuantConfig:
    """W8 per-channel weights and biases, every activation point on `activation_bits`."""
    cfg = OperatorQuantConfig()
    from . import _cabi as cabi
    for name in cabi.OP_NAMES:
        setattr(cfg, f"{name}_", weight_bits if name in ("W", "R", "bw", "br") else activation_bits)
    return cfg


class StackedGruQat:
    def __init__(self, T: int, B: int, I: int, H: int, layers: int, classes: int, device,
                 config: Optional[OperatorQuantConfig] = None, process_group=None, seed: int = 0):
        self.T, self.B, self.I, self.H, self.layers, self.classes = T, B, I, H, layers, classes
        self.device = torch.device(device)
        self.group = process_group
        self.world = torch.distributed.get_world_size(process_group) if process_group is not None else 1
        self.config = config or a16_config()
        from . import _cabi as cabi
        self._lib = cabi.load_library()
        f32 = dict(dtype=torch.float32, device=self.device)
        inputs = [I] + [2 * H] * (layers - 1)
        counts = [GruQatStep.parameter_count(i, H) for i in inputs for _ in range(2)]
        head = classes * 2 * H + classes
        total = sum(counts) + head
        self.flat_w = torch.empty(total, **f32)
        self.flat_g = torch.zeros(total, **f32)
        gen = torch.Generator(device="cpu").manual_seed(seed)
        init = torch.empty(total)
        off = 0
        k = 1.0 / (H ** 0.5)
        for n in counts:  # U(-1/sqrt(H), 1/sqrt(H)) as in the reference's reset_parameters (quant_gru.py:1352-1356)
            init[off:off + n] = (torch.rand(n, generator=gen) * 2 - 1) * k
            off += n
        kh = 1.0 / ((2 * H) ** 0.5)
        init[off:] = (torch.rand(head, generator=gen) * 2 - 1) * kh
        self.flat_w.copy_(init)  # same on every rank
        self.dirs: List[List[GruQatStep]] = []
        off = 0
        for li, i_size in enumerate(inputs):
            pair = []
            for _ in range(2):
                n = GruQatStep.parameter_count(i_size, H)
                pair.append(GruQatStep(T, B, i_size, H, self.device, self.config, process_group,
                                       weights=self.flat_w[off:off + n], grads=self.flat_g[off:off + n]))
                off += n
            self.dirs.append(pair)
        self.head_w = self.flat_w[off:off + classes * 2 * H].view(classes, 2 * H)
        self.head_b = self.flat_w[off + classes * 2 * H:]
        self.head_dw = self.flat_g[off:off + classes * 2 * H].view(classes, 2 * H)
        self.head_db = self.flat_g[off + classes * 2 * H:]
        # layer outputs [T,B,2H], their gradients, the time-flipped inputs of the reverse directions
        self.y = [torch.empty((T, B, 2 * H), **f32) for _ in range(layers)]
        self.dy = torch.empty((T, B, 2 * H), **f32)
        self.x_rev = [torch.empty((T, B, i), **f32) for i in inputs]
        self.dx = [torch.empty((T, B, i), **f32) for i in inputs]
        self.side = torch.cuda.Stream(self.device)
        self.loss = torch.zeros((), **f32)

    # ---- helpers -----------------------------------------------------------
    def _both(self, fn_forward, fn_reverse):
        """Runs the two callables on the current and the side stream and joins them."""
        main = torch.cuda.current_stream(self.device)
        self.side.wait_stream(main)
        self._lib.rxmet_set_concurrent_passes(2)   # the two directions share the SMs: their CTAs are resident together
        fn_forward()
        with torch.cuda.stream(self.side):
            fn_reverse()
        main.wait_stream(self.side)

    def _layer_input(self, li: int, x: torch.Tensor) -> torch.Tensor:
        return x if li == 0 else self.y[li - 1]

    # ---- calibration ---------------------------------------------------------
    def calibrate(self, batches) -> None:
        """min/max calibration: every batch runs through the float layers (layer k+1 observes the float
        output of layer k, as the reference's calibration context does), ranges all-reduced across ranks."""
        for pair in self.dirs:
            for d in pair:
                d.begin_calibration()
        H = self.H
        for x in batches:
            for li, (fw, bw) in enumerate(self.dirs):
                xin = self._layer_input(li, x)
                self.y[li][..., :H].copy_(fw.observe(xin))
                self.x_rev[li].copy_(xin.flip(0))
                self.y[li][..., H:].copy_(bw.observe(self.x_rev[li]).flip(0))
        for pair in self.dirs:
            for d in pair:
                d.finish_calibration()

    # ---- one training step ------------------------------------------------------
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Quantized training forward of all layers; returns the top layer's output [T,B,2H]."""
        H = self.H
        for li, (fw, bw) in enumerate(self.dirs):
            xin = self._layer_input(li, x)
            y = self.y[li]

            def run_forward():
                y[..., :H].copy_(fw.forward(xin))

            def run_reverse():
                self.x_rev[li].copy_(xin.flip(0))
                y[..., H:].copy_(bw.forward(self.x_rev[li]).flip(0))

            self._both(run_forward, run_reverse)
        return self.y[-1]

    def head(self, y: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        """Mean over time, linear layer, mean cross-entropy over the local batch; writes the gradient with respect
        to `y` into self.dy and the head gradients into the flat gradient buffer."""
        feat = y.mean(0)                                             # [B, 2H]
        logits = torch.addmm(self.head_b, feat, self.head_w.t())     # [B, classes]
        logp = torch.log_softmax(logits, dim=1)
        self.loss.copy_(-logp.gather(1, labels.view(-1, 1)).mean())
        dlogits = logp.exp()
        dlogits.scatter_add_(1, labels.view(-1, 1), torch.full((self.B, 1), -1.0, device=self.device))
        dlogits.div_(self.B)
        torch.mm(dlogits.t(), feat, out=self.head_dw)
        torch.sum(dlogits, 0, out=self.head_db)
        dfeat = torch.mm(dlogits, self.head_w).div_(self.T)          # d loss / d y[t] for every t
        self.dy.copy_(dfeat.unsqueeze(0).expand(self.T, self.B, 2 * self.H))
        return self.loss

    def backward(self) -> None:
        """BPTT of all layers from self.dy down to the input; gradients land in the flat gradient buffer."""
        H = self.H
        dy = self.dy
        for li in range(self.layers - 1, -1, -1):
            fw, bw = self.dirs[li]

            def run_forward():
                fw.dh_new[1:].copy_(dy[..., :H])
                fw.backward()

            def run_reverse():
                bw.dh_new[1:].copy_(dy[..., H:].flip(0))
                bw.backward()

            self._both(run_forward, run_reverse)
            if li > 0:  # gradient of the layer below: both directions read the same input
                torch.add(fw.dx, bw.dx.flip(0), out=self.dx[li])
                dy = self.dx[li]

    def capture_step(self, x: torch.Tensor, labels: torch.Tensor, lr: float, warmup: int = 2):
        """Captures `step` on fixed buffers into ONE CUDA graph - about 600 kernel launches on two streams per
        step at three layers - and returns `(replay, loss)`: `replay()` launches the whole step and returns `loss`,
        the device scalar it refreshes.  `x` and `labels` are read at replay time, so the caller refills them in
        place.  With a process group the gradient all-reduce and the update follow the graph launch.  The
        quantization parameters in force at capture are baked in.  `warmup` eager steps run first (they do
        train), so that every lazy initialisation has happened before the capture begins."""
        local = self.group is None
        stream = torch.cuda.Stream(self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            for _ in range(max(warmup, 1)):
                self.step(x, labels, lr)
        torch.cuda.current_stream(self.device).wait_stream(stream)
        graph = torch.cuda.CUDAGraph()
        before = self._lib.rxmet_kernel_launch_count()
        with torch.cuda.graph(graph, stream=stream):
            loss = self.head(self.forward(x), labels)
            self.backward()
            if local:
                self.flat_w.add_(self.flat_g, alpha=-lr)
        self.captured_launches = int(self._lib.rxmet_kernel_launch_count() - before)   # library kernels per replay

        def replay():
            graph.replay()
            if not local:
                torch.distributed.all_reduce(self.flat_g, group=self.group)
                self.flat_w.add_(self.flat_g, alpha=-lr / self.world)
            return loss

        self._graph = graph   # keeps the captured buffers alive with the engine
        return replay, loss

    def step(self, x: torch.Tensor, labels: torch.Tensor, lr: float) -> torch.Tensor:
        """forward, head + loss, backward, ONE gradient all-reduce, SGD update.  Returns the loss (device scalar)."""
        y = self.forward(x)
        loss = self.head(y, labels)
        self.backward()
        if self.group is not None:
            torch.distributed.all_reduce(self.flat_g, group=self.group)
            self.flat_w.add_(self.flat_g, alpha=-lr / self.world)
        else:
            self.flat_w.add_(self.flat_g, alpha=-lr)
        return loss
