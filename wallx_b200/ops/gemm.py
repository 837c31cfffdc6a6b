"""Low-level Python face of the tcgen05 GEMM core.

``D[m, n] = epilogue(sum_k A(m, k) * B(n, k))`` with bf16 operands and fp32 accumulation.
Operand memory layouts:

* ``a_mn=False``: ``A`` is a ``[M, K]`` tensor (k contiguous);  ``a_mn=True``: ``A`` is ``[K, M]``.
* ``b_mn=False``: ``B`` is a ``[N, K]`` tensor (k contiguous);  ``b_mn=True``: ``B`` is ``[K, N]``.

So ``x @ w.T`` is ``(False, False)``, ``dy @ w`` is ``(False, True)`` and ``dy.T @ x`` is
``(True, True)`` -- no transposed copies are made (reference: the NN/NT/TN/TT instantiations of
csrc/dual_asym_grouped_gemm.cu:49-136).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import _ext

OUT_FP32 = 1
ACCUMULATE = 2
ACT_GELU = 4
ACT_SWIGLU = 8
ZERO_PAD_ROWS = 16
SWIGLU_BWD = 32  # accumulator = dL/dh; out2 = saved raw gate/up (input); out = dL/d(gate|up), 2N wide


class GemmSpec:
    """One problem of a (possibly grouped) launch."""

    __slots__ = ("a", "a_mn", "b", "b_mn", "out", "M", "N", "K", "bias", "residual", "row_map", "dyn", "out2",
                 "flags", "m0", "k0")

    def __init__(self, a, b, out, *, a_mn=False, b_mn=False, M=None, N=None, K=None, bias=None, residual=None,
                 row_map=None, dyn=None, out2=None, flags=0, m0=0, k0=0):
        self.a, self.b, self.out = a, b, out
        self.a_mn, self.b_mn = bool(a_mn), bool(b_mn)
        self.M = int(M if M is not None else (a.shape[1] if a_mn else a.shape[0]))
        self.N = int(N if N is not None else (b.shape[1] if b_mn else b.shape[0]))
        self.K = int(K if K is not None else (a.shape[0] if a_mn else a.shape[1]))
        self.bias, self.residual, self.row_map, self.dyn, self.out2 = bias, residual, row_map, dyn, out2
        self.flags, self.m0, self.k0 = int(flags), int(m0), int(k0)

    def as_tuple(self):
        return (self.a, self.a_mn, self.b, self.b_mn, self.out, self.M, self.N, self.K, self.bias, self.residual,
                self.row_map, self.dyn, self.out2, self.flags, self.m0, self.k0)


INFERENCE_AUTO = 18  # "choose the tile shape, inference": also allows K-splitting clusters for prefix-sized problems


import threading as _threading

_region = _threading.local()  # per thread: an inference region of one thread says nothing about another thread's launches


class inference_kernels:
    """Context manager (re-entrant) around inference-only code: launches inside it may use kernels whose results are
    deterministic but not bit-identical to the training kernels' (K-splitting clusters for prefix-sized problems).
    Grad mode cannot serve as the signal: autograd functions run both their forward and their backward with it off."""

    def __enter__(self):
        _region.depth = getattr(_region, "depth", 0) + 1
        return self

    def __exit__(self, *exc):
        _region.depth = getattr(_region, "depth", 1) - 1
        return False

    def __call__(self, fn):
        import functools

        @functools.wraps(fn)
        def wrapped(*a, **k):
            with inference_kernels():
                return fn(*a, **k)

        return wrapped


def _inference_launch() -> bool:
    return getattr(_region, "depth", 0) > 0 and not torch.is_grad_enabled()


def launch(specs: Sequence[GemmSpec], force_bn: int = 0) -> None:
    """Run one or two problems in a single persistent launch. Without a forced tile shape, launches made while autograd
    is off inside an :class:`inference_kernels` region may use K-splitting clusters for problems of a few hundred rows (a
    different, still deterministic, order of the sum over K); launches of a training step never do."""
    if force_bn == 0 and _inference_launch():
        force_bn = INFERENCE_AUTO
    _ext.get().gemm_grouped([s.as_tuple() for s in specs], int(force_bn))


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn=False, b_mn=False, out: Optional[torch.Tensor] = None,
         bias=None, residual=None, flags: int = 0, force_bn: int = 0) -> torch.Tensor:
    """Single dense problem; allocates the output when none is given."""
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        width = N // 2 if (flags & ACT_SWIGLU) else N
        out = torch.empty((M, width), device=a.device,
                          dtype=torch.float32 if (flags & OUT_FP32) else torch.bfloat16)
    launch([GemmSpec(a, b, out, a_mn=a_mn, b_mn=b_mn, bias=bias, residual=residual, flags=flags)], force_bn)
    return out


def check_status(device: Optional[torch.device] = None) -> None:
    """Raise if a kernel gave up on one of its bounded waits since the last check (synchronises)."""
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    st = _ext.get().read_status(idx)
    if st != 0:
        raise RuntimeError(f"wallx_b200: a device-side wait timed out (status {st}); results are invalid")


_CALIBRATED = set()


def calibrate_tile_rates(device: Optional[torch.device] = None, force: bool = False):
    """Measure, once per process and device, the rate of each tile shape of the GEMM core (128 x 256 / 128 x 128 /
    128 x 64 single-CTA tiles, 256 x 256 CTA pairs) on a problem that fills the device, and hand the four numbers to the
    tile cost model (which otherwise uses the figures of one B200). Takes a few milliseconds; call it outside any
    stream capture. Returns the rates in TFLOP/s."""
    C = _ext.get()
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    if idx in _CALIBRATED and not force:
        return C.gemm_tile_rates([])
    dev = torch.device("cuda", idx)
    M, N, K = 8192, 4096, 4096
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    b = torch.randn(N, K, device=dev).to(torch.bfloat16)
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    spec = GemmSpec(a, b, out)
    rates = []
    for bn in (256, 128, 64, 512):
        try:
            for _ in range(2):
                launch([spec], bn)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(3):
                launch([spec], bn)
            e1.record()
            torch.cuda.synchronize(dev)
            rates.append(3 * 2.0 * M * N * K / (e0.elapsed_time(e1) * 1e-3) / 1e12)
        except RuntimeError:  # CTA pairs cannot be scheduled on this device: keep the start-up value out of the race
            rates.append(1e-3 if bn == 512 else 0.0)
    _CALIBRATED.add(idx)
    return C.gemm_tile_rates([float(r) for r in rates])
