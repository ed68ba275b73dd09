"""ctypes binding of the in-tree native libraries.

``cuda_lib()`` returns the sm_100a kernel library (``_native/liblbann_b200.so``) and
fails loudly when it is missing, so a GPU run never falls back to PyTorch kernels
silently.  ``host_lib()`` returns the C++ host runtime (checkpoint container, I/O
thread pool, graph utilities), which also works on CPU-only machines.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_NATIVE = os.path.join(os.path.dirname(_HERE), "_native")
_lock = threading.Lock()
_cuda = None
_host = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float

DT_F16, DT_BF16, DT_F32 = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_LEAKY, ACT_GELU, ACT_TANH, ACT_SIGMOID = 0, 1, 2, 3, 4, 5

STATUS_TEXT = {
    0: "ok",
    1: "timeout waiting for a TMA stage",
    2: "timeout waiting for a free pipeline stage",
    3: "timeout waiting for an accumulator",
    4: "timeout waiting for the epilogue to drain an accumulator",
    5: "timeout waiting for a flag from another rank",
    6: "bad argument seen on the device",
}


class NativeError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float16:
        return DT_F16
    if dt == torch.bfloat16:
        return DT_BF16
    if dt == torch.float32:
        return DT_F32
    raise NativeError(f"unsupported dtype {dt}")


def _load(name: str):
    path = os.path.join(_NATIVE, name)
    if not os.path.exists(path):
        # Build on demand (needs nvcc / g++); a GPU box normally receives the built files.
        from .. import _build
        _build.build_native()
    if not os.path.exists(path):
        raise NativeError(f"native library {path} is missing; run `python -m lbann_b200._build`")
    return ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)


def cuda_lib():
    global _cuda
    if _cuda is None:
        with _lock:
            if _cuda is None:
                lib = _load("liblbann_b200.so")
                lib.lb_consume_status.restype = c_int
                lib.lb_consume_status.argtypes = [c_void_p]
                lib.lb_status_ptr.restype = c_void_p
                lib.lb_sm_count.restype = c_int
                _cuda = lib
    return _cuda


def host_lib():
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                _host = _load("liblbann_b200_host.so")
    return _host


def have_cuda_lib() -> bool:
    return os.path.exists(os.path.join(_NATIVE, "liblbann_b200.so"))


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr() -> int:
    """The current CUDA stream's handle (the raw getter avoids building a Stream object on
    every kernel launch: ~17 us -> <1 us)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what} failed with code {rc}")


_status_listeners = []


def on_status(fn) -> None:
    """``fn(code)`` is called whenever ``consume_status`` finds a non-zero device status."""
    _status_listeners.append(fn)


def set_wait_budget_ns(ns: int) -> None:
    """Budget of the device-side waits on other ranks (0 restores the built-in 2 s)."""
    lib = cuda_lib()
    lib.lb_set_wait_budget_ns.restype = c_int
    lib.lb_set_wait_budget_ns.argtypes = [ctypes.c_ulonglong]
    check(lib.lb_set_wait_budget_ns(int(ns)), "lb_set_wait_budget_ns")


def consume_status(raise_on_error: bool = True) -> int:
    """Synchronise the current stream and return (and clear) the device status word."""
    code = cuda_lib().lb_consume_status(stream_ptr())
    if code:
        for fn in list(_status_listeners):
            fn(code)
    if code and raise_on_error:
        raise NativeError(f"device reported: {STATUS_TEXT.get(code, code)}")
    return code


_launch_count = 0


def count_launch(n: int = 1) -> None:
    """Bookkeeping for benchmarks: number of this library's kernels launched."""
    global _launch_count
    _launch_count += n


def launches() -> int:
    return _launch_count


# --------------------------------------------------------------------------- split-K scratch
_splitk_sms: dict = {}      # device index -> SM count
splitk_offers = 0           # how many launches were lent scratch (tests read it)


def offer_splitk(rows: int, cols: int, device) -> "torch.Tensor | None":
    """Lends scratch memory to the GEMM / convolution launch that the calling thread makes
    NEXT, so that a product with few output tiles and a long reduction can be cut along the
    reduction (``csrc/tc_pipeline.cuh``).  Offered only where that can pay: an output of at
    most half a wave of 128 x 256 tiles.  Returns the workspace tensor; the caller holds it
    until the launch is enqueued."""
    global splitk_offers
    if rows * cols > 74 * 128 * 256 or os.environ.get("LBANN_DISABLE_SPLITK", "") not in ("", "0"):
        return None
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    lib = cuda_lib()
    sms = _splitk_sms.get(idx)
    if sms is None:
        lib.lb_splitk_offer.restype = c_int
        lib.lb_splitk_offer.argtypes = [c_void_p, ctypes.c_longlong]
        sms = _splitk_sms[idx] = int(lib.lb_sm_count())
    bn = 256 if cols > 128 else 128
    ws = torch.empty(sms * 128 * bn, dtype=torch.float32, device=device)
    check(lib.lb_splitk_offer(ws.data_ptr(), ws.numel() * 4), "lb_splitk_offer")
    splitk_offers += 1
    return ws
