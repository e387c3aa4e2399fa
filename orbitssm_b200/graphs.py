"""CUDA-graph capture of a step of this package's layers: one training step (forward + backward) or one decode step.

The layers launch 40-90 kernels per step and return without ever synchronising with the host, so for small problems a
step is bound by launch and Python time, not by the GPU (a 16k-token step of the d_model-1024 layer spends about 40 % of
its wall time between kernels).  A captured step replays the same launches from one graph.  Mirrors the reference's
`graphed_step` (src/orbit_ssm/graphs.py:449: static input and gradient buffers, warm-up on the capture stream, no silent
eager fallback) and, for decoding, its fixed-address State (src/orbit_ssm/ssm/ssd_mimo_torch.py:460-470, `step_inplace`).
"""
from __future__ import annotations

import contextlib

import torch


class CaptureError(RuntimeError):
    """The step could not be captured; `reason` is a short tag (``no-cuda``, ``capture-failed``)."""

    def __init__(self, reason, msg):
        super().__init__(f"[{reason}] {msg}")
        self.reason = reason


def _amp(dtype):
    if dtype is None:
        return contextlib.nullcontext
    # autocast's weight-cast cache would hand the replay casts made for the warm-up: keep it off inside a capture
    return lambda: torch.autocast("cuda", dtype=dtype, cache_enabled=False)


class GraphedStep:
    """One captured training step ``y = module(x); y.backward(dy)`` with static buffers.

    ``step(x, dy)`` copies its arguments into the static buffers, replays the graph and returns the static output `y`;
    after it `x_grad` holds the input gradient and every parameter's ``.grad`` the parameter gradients of THIS step (they are
    overwritten, not accumulated, by the next replay)."""

    def __init__(self, module, x, dy=None, *, amp_dtype=None, warmup=3):
        if not torch.cuda.is_available():
            raise CaptureError("no-cuda", "CUDA graphs need a CUDA device")
        if not x.is_cuda:
            raise CaptureError("not-on-cuda", "the example input must be a CUDA tensor")
        self.module = module
        self.x = x.detach().clone().requires_grad_(True)
        self.dy = None if dy is None else dy.detach().clone()
        ctx = _amp(amp_dtype)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        try:
            with torch.cuda.stream(side):
                for _ in range(max(1, int(warmup))):
                    self._zero_grads()
                    with ctx():
                        y = module(self.x)
                    if self.dy is None:
                        self.dy = torch.randn_like(y)
                    y.backward(self.dy)
            torch.cuda.current_stream().wait_stream(side)
            self._zero_grads()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):     # the stream the warm-up made the gradient accumulators on
                with ctx():
                    self.y = module(self.x)
                self.y.backward(self.dy)
        except Exception as e:                                  # noqa: BLE001 - reported by name, never a silent eager run
            raise CaptureError("capture-failed", f"{type(e).__name__}: {e}") from e
        self.x_grad = self.x.grad
        #: the static gradient buffers the replay writes: (parameter, gradient) pairs
        self.param_grads = [(p, p.grad) for p in module.parameters() if p.grad is not None]

    def _zero_grads(self):
        self.x.grad = None
        for p in self.module.parameters():
            p.grad = None

    def step(self, x, dy=None):
        self.x.data.copy_(x)
        if dy is not None:
            self.dy.copy_(dy)
        self.graph.replay()
        for p, g in self.param_grads:                          # a caller may have cleared or replaced .grad since the last step
            p.grad = g
        return self.y

    __call__ = step


class GraphedDecode:
    """One captured decode step of a layer or a `BlockStack`: ``y_t, state = module.step(x_t, state)`` under `no_grad` with the
    State kept at fixed addresses (the new carries are copied over the old ones inside the graph).

    ``step(x_t)`` returns the static output `y_t [B, d_model]` (valid until the next call); `state` is the live State."""

    def __init__(self, module, batch_size, *, device="cuda", dtype=torch.bfloat16, state=None, warmup=2):
        if not torch.cuda.is_available():
            raise CaptureError("no-cuda", "CUDA graphs need a CUDA device")
        self.module = module
        d_model = getattr(module, "d_model", None) or module.layers[0].mixer.d_model
        self.x = torch.zeros((batch_size, d_model), device=device, dtype=dtype)
        self.state = state if state is not None else module.init_state(batch_size, device=device)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        try:
            with torch.no_grad():
                saved = self._snapshot()
                with torch.cuda.stream(side):
                    for _ in range(max(1, int(warmup))):
                        self._one()
                torch.cuda.current_stream().wait_stream(side)
                self._restore(saved)                              # the warm-up steps must not advance the caller's State
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph, stream=side):
                    self.y = self._one()
                self._restore(saved)
        except Exception as e:                                  # noqa: BLE001
            raise CaptureError("capture-failed", f"{type(e).__name__}: {e}") from e

    def _carries(self):
        states = self.state if isinstance(self.state, (list, tuple)) else [self.state]
        return [v for s in states for v in s.values() if torch.is_tensor(v)]

    def _snapshot(self):
        return [v.clone() for v in self._carries()]

    def _restore(self, saved):
        for v, s in zip(self._carries(), saved):
            v.copy_(s)

    def _one(self):
        y, new = self.module.step(self.x, self.state)
        old = self.state if isinstance(self.state, (list, tuple)) else [self.state]
        new = new if isinstance(new, (list, tuple)) else [new]
        for so, sn in zip(old, new):
            for k, v in so.items():
                if torch.is_tensor(v):
                    v.copy_(sn[k])                                # fixed addresses: the next replay reads what this one wrote
        return y

    @torch.no_grad()
    def step(self, x_t):
        self.x.copy_(x_t)
        self.graph.replay()
        return self.y

    __call__ = step
