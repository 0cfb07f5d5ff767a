"""ctypes binding to the in-tree CUDA kernel library (``velogb10_b200/_C.so``).

The library is built by ``velogb10_b200.ops.build``. Loading fails loudly when the binary is
missing or was built from different sources than the ones on disk, so a GPU run can never fall
back silently to a non-native path.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build as _build

_lib: Optional[ctypes.CDLL] = None

c_int, c_float, c_void_p, c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """Load (building first if needed and possible) and return the kernel library."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    if not _build.is_fresh():
        try:
            _build.build()
        except Exception as e:  # no nvcc on this machine, or a compile error
            if not os.path.exists(path):
                raise KernelError(f"kernel library missing and could not be built: {e}") from e
            raise KernelError(f"kernel library is stale and could not be rebuilt: {e}") from e
    L = ctypes.CDLL(path)
    L.vg_build_id.restype = ctypes.c_char_p
    L.vg_attn_scratch_floats.restype = c_ll
    L.vg_gdn_chunk_work_bytes.restype = c_ll
    bid = L.vg_build_id().decode()
    if bid != _build.source_hash():
        raise KernelError(f"kernel library build id {bid} does not match sources {_build.source_hash()}")
    _lib = L
    return L


def ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0) if t is None else c_void_p(t.data_ptr())


def stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


launches = 0        # kernels enqueued through this module since import (each wrapper reports its count)


def check(rc: int, what: str, kernels: int = 1):
    global launches
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")
    launches += kernels


def count_launches(fn) -> int:
    """Number of kernels ``fn()`` enqueues through this library."""
    before = launches
    fn()
    return launches - before


_err_words = {}


def err_word(device=None) -> torch.Tensor:
    """Per-device int32 status word the kernels write bounded-wait failures into."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = _err_words.get(dev)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=dev)
        _err_words[dev] = w
    return w


def check_err_word(device=None):
    w = err_word(device)
    v = int(w.item())
    if v != 0:
        w.zero_()
        names = {1: "TMA stage wait", 2: "free-stage wait", 3: "accumulator wait", 4: "peer flag wait",
                 5: "bad argument", 6: "dequant stage wait", 7: "wait for the other CTAs of the grid"}
        raise KernelError(f"a kernel reported a bounded-wait failure: {names.get(v, v)}")
