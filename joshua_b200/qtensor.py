"""Host-side mirror of the reference's quantized operator objects.

`QTensor` plays the part of the reference's borrowed block tensors
(`MmapBlocks<T>`, `MmapBlocksIq2Xxs`, `MmapBlocksMxfp4`, src/mmap_tensor.rs:54-513)
and exposes the same `QuantizedType` surface — `matmul_t`, `matmul_t_f16`,
`embedding`, `dequantize`, `dtype`, `storage_size_in_bytes`, `block_size`,
`from_float` (which refuses) — with the same argument meaning and the same
failures, each a thin call into the C ABI.  `QMatMul` is the `Module` the
loaders hold (`QMatMul::from_qtensor(..).forward(xs)`,
src/quantized_qwen3_moe.rs:185,220-226).  Nothing here computes: without the
CUDA library these classes cannot be constructed.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _lib
from ._lib import JoshuaB200Error, check
from .synth import BLOCK, NAMES


class Context:
    """One CUDA device (`jq_init`).  One per process is the intended use."""

    def __init__(self, device: int = 0):
        self._h = ctypes.c_void_p()
        check(_lib.lib().jq_init(device, ctypes.byref(self._h)))
        self.device = device

    def close(self) -> None:
        if self._h:
            _lib.lib().jq_free(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_default_ctx: dict[int, Context] = {}


def default_context(device: int = 0) -> Context:
    if device not in _default_ctx:
        _default_ctx[device] = Context(device)
    return _default_ctx[device]


def _np_ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


class QTensor:
    """Raw GGUF blocks resident on the device."""

    def __init__(self, handle: ctypes.c_void_p, ctx: Context, keepalive=None):
        self._h = handle
        self.ctx = ctx
        self._keep = keepalive

    # ── construction ────────────────────────────────────────────────────
    @classmethod
    def from_bytes(cls, type_id: int, raw, ctx: Context | None = None) -> "QTensor":
        """Upload a tensor's raw GGUF bytes (the counterpart of borrowing them from the mapping)."""
        ctx = ctx or default_context()
        raw = np.frombuffer(raw, dtype=np.uint8) if isinstance(raw, (bytes, bytearray, memoryview)) else \
            np.ascontiguousarray(raw, dtype=np.uint8)
        h = ctypes.c_void_p()
        check(_lib.lib().jq_weight_upload(ctx._h, type_id, _np_ptr(raw), raw.size, ctypes.byref(h)))
        return cls(h, ctx)

    @classmethod
    def from_device(cls, type_id: int, tensor, ctx: Context | None = None) -> "QTensor":
        """Adopt a flat torch.uint8 CUDA tensor holding raw blocks (kept alive by this object)."""
        ctx = ctx or default_context(tensor.device.index or 0)
        h = ctypes.c_void_p()
        check(_lib.lib().jq_weight_from_device(ctx._h, type_id, tensor.data_ptr(), tensor.numel(), ctypes.byref(h)))
        return cls(h, ctx, keepalive=tensor)

    def slice_blocks(self, block0: int, n_blocks: int) -> "QTensor":
        """Blocks [block0, block0+n_blocks) sharing this tensor's memory (per-expert slicing)."""
        h = ctypes.c_void_p()
        check(_lib.lib().jq_weight_slice(self._h, block0, n_blocks, ctypes.byref(h)))
        return QTensor(h, self.ctx, keepalive=self)

    def __del__(self):
        try:
            if self._h:
                _lib.lib().jq_weight_free(self._h)
                self._h = ctypes.c_void_p()
        except Exception:
            pass

    # ── QuantizedType surface ───────────────────────────────────────────
    def dtype(self) -> int:
        return _lib.lib().jq_weight_type(self._h)

    def storage_size_in_bytes(self) -> int:
        return _lib.lib().jq_weight_storage_size(self._h)

    size = storage_size_in_bytes

    def block_size(self) -> int:
        return _lib.lib().jq_weight_block_elems(self._h)

    def as_ptr(self) -> int:
        return _lib.lib().jq_weight_device_ptr(self._h) or 0

    def matmul_t(self, mkn, lhs, dst=None, *, lhs_len=None, dst_len=None) -> np.ndarray:
        """dst[m, n] = lhs[m, k] . W[n, k]^T with HOST buffers (f32 numpy arrays)."""
        m, k, n = mkn
        lhs = np.ascontiguousarray(lhs, dtype=np.float32).reshape(-1)
        if dst is None:
            dst = np.empty(m * n if dst_len is None else max(dst_len, m * n), dtype=np.float32)
        flat = dst.reshape(-1)
        check(_lib.lib().jq_matmul_t(self._h, m, k, n, _np_ptr(lhs), lhs.size if lhs_len is None else lhs_len,
                                     _np_ptr(flat), m * n if dst_len is None else dst_len))
        return dst if dst.ndim == 2 else flat[: m * n].reshape(m, n)

    def matmul_t_f16(self, mkn, lhs) -> np.ndarray:
        m, k, n = mkn
        lhs = np.ascontiguousarray(lhs, dtype=np.float16).reshape(-1)
        dst = np.empty(m * n, dtype=np.float16)
        check(_lib.lib().jq_matmul_t_f16(self._h, m, k, n, _np_ptr(lhs), lhs.size, _np_ptr(dst), dst.size))
        return dst.reshape(m, n)

    def dequantize(self, elem_count: int, two_step: bool = True) -> np.ndarray:
        out = np.empty(elem_count, dtype=np.float32)
        check(_lib.lib().jq_dequantize(self._h, _np_ptr(out), elem_count, int(two_step)))
        return out

    def embedding(self, ids, rows: int, hidden: int) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        out = np.empty((ids.size, hidden), dtype=np.float32)
        check(_lib.lib().jq_embedding(self._h, _np_ptr(ids), ids.size, rows, hidden, _np_ptr(out)))
        return out

    def from_float(self, xs) -> None:
        xs = np.ascontiguousarray(xs, dtype=np.float32)
        check(_lib.lib().jq_weight_from_float(self._h, _np_ptr(xs), xs.size))

    # ── device-resident product ─────────────────────────────────────────
    def matmul_t_dev(self, mkn, lhs, dst, stream=None) -> None:
        """Same product on torch CUDA tensors (f32, contiguous), on torch's current stream."""
        import torch

        m, k, n = mkn
        s = torch.cuda.current_stream(lhs.device).cuda_stream if stream is None else stream
        check(_lib.lib().jq_matmul_t_dev(self._h, m, k, n, lhs.data_ptr(), dst.data_ptr(), s))

    def dequantize_dev(self, out, two_step: bool = True, stream=None) -> None:
        import torch

        s = torch.cuda.current_stream(out.device).cuda_stream if stream is None else stream
        check(_lib.lib().jq_dequantize_dev(self._h, out.data_ptr(), out.numel(), int(two_step), s))


class QMatMul:
    """`QMatMul::from_qtensor(w).forward(xs)`: xs [..., k] f32 on the device -> [..., n]."""

    def __init__(self, qtensor: QTensor, n: int, k: int):
        elems, nbytes = BLOCK[qtensor.dtype()]
        if k % elems or qtensor.storage_size_in_bytes() != n * (k // elems) * nbytes:
            raise JoshuaB200Error(_lib.E_INVALID,
                                  f"{NAMES[qtensor.dtype()]}: {qtensor.storage_size_in_bytes()} bytes do not hold "
                                  f"a [{n}, {k}] tensor")
        self.w, self.n, self.k = qtensor, n, k

    @classmethod
    def from_qtensor(cls, qtensor: QTensor, shape) -> "QMatMul":
        return cls(qtensor, shape[0], shape[1])

    def forward(self, xs):
        import torch

        if xs.dtype != torch.float32 or not xs.is_cuda:
            raise JoshuaB200Error(_lib.E_INVALID, "QMatMul.forward expects an f32 CUDA tensor")
        x2 = xs.reshape(-1, self.k).contiguous()
        out = torch.empty((x2.shape[0], self.n), dtype=torch.float32, device=xs.device)
        self.w.matmul_t_dev((x2.shape[0], self.k, self.n), x2, out)
        return out.reshape(*xs.shape[:-1], self.n)
