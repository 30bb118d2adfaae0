"""ctypes loader for libdarkforest_ring.so (include/darkforest_ring.h): the sequence-parallel ring
attention whose hop loop, NCCL exchange and schedule live in C++ behind the C ABI.

`Ring` wraps one handle for torch CUDA tensors; the tests and the benchmark use it. The unique id that
every rank needs is produced on rank 0 (`unique_id()`) and distributed by the caller (the benchmark
broadcasts it with torch.distributed, the tests pass it through a file).

torch must be imported before this library is loaded: the process then uses the NCCL that torch
brought along instead of loading a second copy.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
RING_LIB_PATH = os.path.join(_HERE, "lib", "libdarkforest_ring.so")
RING_HEADER_PATH = os.path.join(_HERE, "..", "include", "darkforest_ring.h")

LAYOUT_CONTIGUOUS, LAYOUT_ZIGZAG, LAYOUT_BALANCED = 0, 1, 2
LAYOUTS = {"contiguous": LAYOUT_CONTIGUOUS, "zigzag": LAYOUT_ZIGZAG, "balanced": LAYOUT_BALANCED}
UNIQUE_ID_BYTES = 128
DF_ERR_RING_TIMEOUT, DF_ERR_NCCL = 7, 8

_P = ctypes.c_void_p
_U32 = ctypes.c_uint32
_U64 = ctypes.c_uint64
_I = ctypes.c_int

RING_PROTOTYPES = {
    "df_ring_unique_id": (_I, [_P]),
    "df_ring_create": (_I, [ctypes.POINTER(_P), _P, _I, _I, _I, _U32, _U32, _U32, _I, ctypes.c_float, _I, _U32]),
    "df_ring_workspace_bytes": (_U64, [_P]),
    "df_ring_forward": (_I, [_P, _P, _P, _P, _P, _P, _P, _U64, _P]),
    "df_ring_backward": (_I, [_P] * 10 + [_P, _U64, _P]),
    "df_ring_wait": (_I, [_P, _P, _U32]),
    "df_ring_last_nccl_result": (_I, [_P]),
    "df_ring_destroy": (_I, [_P]),
    "df_ring_hop_blocks": (_I, [_I, _I, _I, _I, _I, _P]),
}

_lib = None


def ring_lib() -> ctypes.CDLL:
    """The loaded ring library. Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(RING_LIB_PATH):
            raise RuntimeError(f"{RING_LIB_PATH} is missing: build it with `make -C {_HERE}`")
        import torch  # noqa: F401  (brings its NCCL into the process first)
        L = ctypes.CDLL(RING_LIB_PATH)
        for name, (res, args) in RING_PROTOTYPES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


class RingError(RuntimeError):
    def __init__(self, status, what):
        super().__init__(f"{what} failed with status {status}")
        self.status = status


def unique_id() -> bytes:
    buf = ctypes.create_string_buffer(UNIQUE_ID_BYTES)
    st = ring_lib().df_ring_unique_id(ctypes.cast(buf, _P))
    if st != 0:
        raise RingError(st, "df_ring_unique_id")
    return buf.raw


def hop_blocks(rank: int, world: int, layout: str, causal: bool, hop: int):
    """[(q_slot, k_slot, k_chunks, diagonal)] of one hop, from the library's own schedule (host only)."""
    out = (ctypes.c_int * 12)()
    n = ring_lib().df_ring_hop_blocks(rank, world, LAYOUTS[layout], int(causal), hop, ctypes.cast(out, _P))
    if n < 0:
        raise ValueError("bad schedule arguments")
    return [tuple(out[4 * i + j] for j in range(4)) for i in range(n)]


class Ring:
    """One rank's ring handle plus its workspace (a torch byte tensor allocated once, here)."""

    def __init__(self, uid: bytes, rank: int, world: int, layout: str, n_heads: int, local_len: int, d_head: int,
                 bf16: bool, scale: float, causal: bool = True, timeout_ms: int = 30000, device=None):
        import torch
        self._h = _P()
        self._lib = ring_lib()
        idbuf = ctypes.create_string_buffer(uid, UNIQUE_ID_BYTES)
        st = self._lib.df_ring_create(ctypes.byref(self._h), ctypes.cast(idbuf, _P), rank, world, LAYOUTS[layout], n_heads,
                                      local_len, d_head, int(bf16), float(scale), int(causal), timeout_ms)
        if st != 0:
            self._h = _P()
            raise RingError(st, "df_ring_create")
        self.H, self.L, self.D, self.bf16 = n_heads, local_len, d_head, bf16
        self.ws_bytes = int(self._lib.df_ring_workspace_bytes(self._h))
        self.workspace = torch.empty(self.ws_bytes + 256, dtype=torch.uint8, device=device or "cuda")
        self._ws_ptr = (self.workspace.data_ptr() + 255) // 256 * 256

    @staticmethod
    def _stream(stream):
        import torch
        s = torch.cuda.current_stream() if stream is None else stream
        return _P(s.cuda_stream)

    def forward(self, q, k, v, out, lse, stream=None):
        st = self._lib.df_ring_forward(self._h, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                       self._ws_ptr, self.ws_bytes, self._stream(stream))
        if st != 0:
            raise RingError(st, "df_ring_forward")
        return out, lse

    def backward(self, q, k, v, out, d_out, lse, d_q, d_k, d_v, stream=None):
        st = self._lib.df_ring_backward(self._h, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), d_out.data_ptr(),
                                        lse.data_ptr(), d_q.data_ptr(), d_k.data_ptr(), d_v.data_ptr(), self._ws_ptr,
                                        self.ws_bytes, self._stream(stream))
        if st != 0:
            raise RingError(st, "df_ring_backward")
        return d_q, d_k, d_v

    def wait(self, stream=None, timeout_ms: int = 0) -> int:
        return self._lib.df_ring_wait(self._h, self._stream(stream), timeout_ms)

    def close(self):
        if self._h:
            self._lib.df_ring_destroy(self._h)
            self._h = _P()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
