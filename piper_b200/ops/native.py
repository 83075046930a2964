"""Loading of the native sm_100a library and the per-device status word.

``lib()`` returns ``torch.ops.piper_c`` after loading
``piper_b200/lib/libpiper_b200.so``.  On a machine with a GPU a missing
library is an error (the CUDA path must never silently fall back); on a
CPU-only machine the ops in this package use their PyTorch reference bodies
and ``lib()`` is never reached.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libpiper_b200.so"
_loaded = False
_status: dict[int, torch.Tensor] = {}
_status_detail: dict[int, torch.Tensor] = {}
_cdll = None

STATUS_MESSAGES = {
    0: "ok",
    1: "an mbarrier wait inside a kernel ran out of polls",
    2: "a wait on a peer GPU's flag ran out of polls",
    3: "a kernel rejected an argument (index out of range)",
}


class PiperKernelError(RuntimeError):
    """A kernel recorded a non-zero status word (bounded wait expired, bad index)."""


class PiperCommTimeout(PiperKernelError):
    """A fused collective kernel gave up waiting for a peer."""


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def lib():
    """Load the native library once and return the ``torch.ops.piper_c`` namespace."""
    global _loaded
    if not _loaded:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"native library {_LIB_PATH} is missing; build it with `python -m piper_b200.build` "
                "(CUDA tensors are never routed to a PyTorch fallback)"
            )
        torch.ops.load_library(str(_LIB_PATH))
        _loaded = True
    return torch.ops.piper_c


def cdll() -> ctypes.CDLL:
    """The same library through ctypes, for its exported ``extern \"C\"`` entry points."""
    global _cdll
    if _cdll is None:
        lib()
        _cdll = ctypes.CDLL(str(_LIB_PATH), mode=os.RTLD_GLOBAL if hasattr(os, "RTLD_GLOBAL") else 0)
    return _cdll


def status_tensor(device: torch.device | None = None) -> torch.Tensor:
    """One int32 status word per device, shared by all kernels launched from this process."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        # word 0 is the status; a peer wait that runs out leaves (tag, flag index, wanted value) in words 1..3
        _status_detail[idx] = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
        t = _status[idx] = _status_detail[idx][:1]
        lib().set_status_word(t)          # kernels whose bindings take no status argument report into it too
    return t


def status_detail(device: torch.device | None = None) -> list:
    """(tag of the wait that gave up, index of the flag it waited for, value it wanted); synchronises."""
    status_tensor(device)
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    return [int(v) for v in _status_detail[idx][1:].tolist()]


def check_status(device: torch.device | None = None, *, reset: bool = True) -> None:
    """Synchronising read of the status word; raises if a kernel recorded a failure."""
    if not torch.cuda.is_available():
        return
    t = status_tensor(device)
    code = int(t.item())
    if code != 0:
        detail = f" (tag of the check or wait and two values describing it: {status_detail(device)})"
        if reset:
            t.zero_()
        raise_for_status(code, detail)


def raise_for_status(code: int, detail: str = "") -> None:
    """Raise the error that status word ``code`` stands for (nothing for 0)."""
    if code == 0:
        return
    msg = STATUS_MESSAGES.get(code, f"unknown status {code}")
    raise (PiperCommTimeout if code == 2 else PiperKernelError)(f"kernel status {code}: {msg}{detail}")


class StatusMonitor:
    """Reads the status word once per training step without stalling the host.

    ``post()`` enqueues a copy of the word into pinned host memory behind the step's work and records an
    event; ``poll()`` (called at the start of the next step) looks at that copy once its event has completed
    and raises ``PiperCommTimeout`` / ``PiperKernelError`` if a kernel of the earlier step gave up: a fused
    collective that timed out has skipped its update, so training must not continue on stale replicas.
    ``source`` defaults to the device's status word; tests pass their own tensor.
    """

    def __init__(self, device: torch.device, source: torch.Tensor | None = None) -> None:
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.source = source if source is not None else (status_tensor(self.device) if self.cuda else None)
        self.host = torch.zeros(1, dtype=torch.int32)
        if self.cuda:
            self.host = self.host.pin_memory()
        self.event = None
        self.pending = False

    def post(self) -> None:
        if self.source is None or self.pending:
            return
        self.host.copy_(self.source, non_blocking=True)
        if self.cuda:
            self.event = torch.cuda.Event()
            self.event.record(torch.cuda.current_stream(self.device))
        self.pending = True

    def poll(self, wait: bool = False) -> None:
        if not self.pending:
            return
        if self.event is not None:
            if wait:
                self.event.synchronize()
            elif not self.event.query():
                return
        self.pending = False
        code = int(self.host[0])
        if code != 0:
            detail = ""
            if self.source is not None:
                if self.cuda:
                    detail = f" (tag of the check or wait and two values describing it: {status_detail(self.device)})"
                self.source.zero_()
            raise_for_status(code, detail)
