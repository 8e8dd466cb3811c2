"""ctypes access to the CPU emulator (libb200ipc_emu.so) for the tests."""
import ctypes

import numpy as np

from gpu_ipc_example_b200._ext import emulator_path

OPS = {"parallel": 0, "sequential": 1, "ring": 2, "bisect": 3, "oneshot": 4, "ag_ring": 5, "ag_direct": 6, "reduce_scatter": 7}
PROTOS = {"LL8": 0, "LL16": 1, "LL128": 2, "LL512": 3}

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(emulator_path()))
        _lib.b200emu_heap_bytes.restype = ctypes.c_uint64
        _lib.b200emu_layout.restype = ctypes.c_uint64
        _lib.b200emu_layout.argtypes = [ctypes.c_int, ctypes.c_uint64]
        _lib.b200emu_seq_advance.restype = ctypes.c_uint32
        _lib.b200emu_seq_advance.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_uint64]
        _lib.b200emu_to_float.restype = ctypes.c_float
        _lib.b200emu_to_float.argtypes = [ctypes.c_int, ctypes.c_uint16]
        _lib.b200emu_from_float.restype = ctypes.c_uint16
        _lib.b200emu_from_float.argtypes = [ctypes.c_int, ctypes.c_float]
        _lib.b200emu_run_rank.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                          ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int, ctypes.c_uint32,
                                          ctypes.c_uint32, ctypes.c_uint64, ctypes.c_void_p]
        _lib.b200emu_peek.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_void_p]
    return _lib


def run_threads(world, op, proto, ins, outs, nelems, nwires, seq=1, flags=0, timeout_ms=2000, mute=-1, skip=-1, dtype=0,
                heaps=None):
    """ins/outs: lists of numpy uint16/float16 arrays.  Returns (rc, status rows)."""
    L = lib()
    P = ctypes.c_void_p * world
    ip = P(*[a.ctypes.data for a in ins])
    op_ = P(*[a.ctypes.data for a in outs])
    st = (ctypes.c_uint32 * (8 * world))()
    rc = L.b200emu_run_threads(world, OPS[op], PROTOS[proto], dtype, ip, op_, ctypes.c_uint64(nelems), nwires,
                               ctypes.c_uint32(seq), ctypes.c_uint32(flags), ctypes.c_uint64(timeout_ms), mute, skip, st, heaps)
    rows = [list(st[8 * r:8 * r + 8]) for r in range(world)]
    return rc, rows


def wire_image(proto, payload, flag):
    L = lib()
    payload = np.ascontiguousarray(payload, dtype=np.uint32)
    img = np.zeros(128, dtype=np.uint32)
    n = L.b200emu_wire_image(PROTOS[proto], payload.ctypes.data_as(ctypes.c_void_p), len(payload), ctypes.c_uint32(flag),
                             img.ctypes.data_as(ctypes.c_void_p))
    return img[:n]
