"""ctypes binding of libes_b200.so (the C ABI declared in include/es_b200.h).

The library is the only compute path: if it is missing it is built in-tree with nvcc, and if that is impossible
the import fails loudly — there is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p, POINTER, c_uint32
from pathlib import Path

_LIB = None

OK = 0
BF16, FP16 = 0, 1


class EsB200Error(RuntimeError):
    """Raised when a C-ABI call returns a non-zero status (the analogue of the reference's TORCH_CHECK failures)."""


def _declare(lib):
    lib.es_b200_version.restype = c_char_p
    lib.es_b200_strerror.restype = c_char_p
    lib.es_b200_strerror.argtypes = [c_int]
    lib.es_b200_last_error.restype = c_char_p
    lib.es_b200_mxfp8_grouped_quant.restype = c_int
    lib.es_b200_mxfp8_grouped_quant.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                c_int, c_int64, c_int, c_void_p]
    lib.es_b200_mxfp8_silu_mul_grouped_quant.restype = c_int
    lib.es_b200_mxfp8_silu_mul_grouped_quant.argtypes = lib.es_b200_mxfp8_grouped_quant.argtypes
    lib.es_b200_grouped_mm_scratch_bytes.restype = c_size_t
    lib.es_b200_grouped_mm_scratch_bytes.argtypes = [c_int, c_int64, c_int, c_int]
    lib.es_b200_mxfp8_grouped_mm.restype = c_int
    lib.es_b200_mxfp8_grouped_mm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                             c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int64, c_void_p,
                                             c_size_t, c_void_p]
    lib.es_b200_mxfp8_grouped_mm_scatter.restype = c_int
    lib.es_b200_mxfp8_grouped_mm_scatter.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                     c_void_p, c_int, c_int64, c_int, c_int, c_int64, c_void_p,
                                                     POINTER(c_void_p), c_int, c_int64, c_void_p, c_size_t, c_void_p]
    lib.es_b200_fp8_blockwise_grouped_mm.restype = c_int
    lib.es_b200_fp8_blockwise_grouped_mm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                     c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_void_p,
                                                     c_size_t, c_void_p]
    lib.es_b200_ep_dispatch_quant_push.restype = c_int
    lib.es_b200_ep_dispatch_quant_push.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, POINTER(c_void_p),
                                                   POINTER(c_void_p), c_int, c_int, c_int, c_int, c_int, c_int64,
                                                   c_void_p, c_int, c_void_p]
    lib.es_b200_ep_side_record_bytes.restype = c_int
    lib.es_b200_ep_side_record_bytes.argtypes = [c_int]
    lib.es_b200_ep_unpack_side.restype = c_int
    lib.es_b200_ep_unpack_side.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p]
    lib.es_b200_ep_combine_push.restype = c_int
    lib.es_b200_ep_combine_push.argtypes = [c_void_p, c_void_p, c_void_p, POINTER(c_void_p), c_int, c_int64, c_int64,
                                            c_int, c_int, c_void_p]
    lib.es_b200_ep_topk_weighted_sum.restype = c_int
    lib.es_b200_ep_topk_weighted_sum.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.es_b200_ep_barrier.restype = c_int
    lib.es_b200_ep_barrier.argtypes = [POINTER(c_void_p), c_int, c_int, c_void_p]
    lib.es_b200_ep_barrier_limit.restype = c_int
    lib.es_b200_ep_barrier_limit.argtypes = [POINTER(c_void_p), c_int, c_int, c_int64, c_void_p]
    lib.es_b200_ep_route_count.restype = c_int
    lib.es_b200_ep_route_count.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, POINTER(c_void_p), c_int,
                                           c_int, c_void_p]
    lib.es_b200_ep_route_count_static.restype = c_int
    lib.es_b200_ep_route_count_static.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, POINTER(c_void_p), c_int,
                                                  c_int, c_void_p]
    lib.es_b200_ep_route_tables.restype = c_int
    lib.es_b200_ep_route_tables.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_int64, c_void_p]
    lib.es_b200_error_epoch.restype = ctypes.c_uint64
    lib.es_b200_error_epoch.argtypes = []
    lib.es_b200_set_tunable.restype = c_int
    lib.es_b200_set_tunable.argtypes = [c_char_p, c_int]
    lib.es_b200_check_status.restype = c_int
    lib.es_b200_check_status.argtypes = [c_void_p, POINTER(c_uint32)]


def library_path() -> Path:
    return Path(__file__).resolve().parent / "lib" / "libes_b200.so"


def load():
    """Load (building first if needed) libes_b200.so and return the ctypes handle."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not path.exists():
        from . import build as _build
        _build.build()
    if not path.exists():
        raise ImportError(f"{path} is missing and could not be built; es_b200 has no fallback path")
    lib = ctypes.CDLL(str(path))
    _declare(lib)
    _LIB = lib
    return lib


_TORCH_OPS = None


def torch_ops():
    """The operators as registered with the torch dispatcher (namespace es_b200; schemas of the reference's
    expert_specialization.cpp:56-66): loads — building first if needed — libes_b200_torch.so, which forwards to the C
    ABI after the reference's argument checks."""
    global _TORCH_OPS
    if _TORCH_OPS is not None:
        return _TORCH_OPS
    import torch
    from . import build as _build
    load()                                     # libes_b200.so first: the registration library links against it
    path = _build.TORCH_LIB
    if not path.exists():
        _build.build_torch_ops()
    if not path.exists():
        raise ImportError(f"{path} is missing and could not be built; es_b200 has no fallback path")
    torch.ops.load_library(str(path))
    _TORCH_OPS = torch.ops.es_b200
    return _TORCH_OPS


def check(status: int):
    if status != OK:
        lib = load()
        msg = lib.es_b200_last_error().decode() or lib.es_b200_strerror(status).decode()
        raise EsB200Error(msg)


_SCRATCH = {}


def grouped_mm_scratch(device, stream_ptr: int):
    """Work-counter scratch of the grouped GEMMs for calls on (device, stream): zeroed once when it is created, left
    zeroed by every call, so one buffer per stream serves every call on that stream (graph replays included)."""
    import torch
    key = (device.index, stream_ptr)
    lib = load()
    epoch = int(lib.es_b200_error_epoch())
    entry = _SCRATCH.get(key)
    if entry is None or entry[1] != epoch:
        # first use, or a device-side error was reported since the buffer was last zeroed: (re-)zero it on the stream
        with torch.cuda.stream(torch.cuda.ExternalStream(stream_ptr, device=device) if stream_ptr else
                               torch.cuda.default_stream(device)):
            if entry is None:
                nbytes = int(lib.es_b200_grouped_mm_scratch_bytes(0, 0, 0, 0))
                buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
            else:
                buf = entry[0]
                buf.zero_()
        entry = (buf, epoch)
        _SCRATCH[key] = entry
    return entry[0]


def set_tunable(name: str, value: int):
    check(load().es_b200_set_tunable(name.encode(), int(value)))
