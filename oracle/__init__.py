"""ctypes front end of the CPU oracle (`joshua_oracle.cpp`).

TEST INFRASTRUCTURE, NOT PRODUCT CODE: only the tests, the smoke check and the
CPU-baseline legs of the benchmark import this package.  See the header of
`joshua_oracle.cpp` for what it restates and which parts of it are pinned by
golden vectors.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libjoshua_oracle.so"

Q8_0, Q2_K, Q4_K, IQ2_XXS, MXFP4 = 8, 10, 12, 16, 39

GATE_SOFTMAX, GATE_SIGMOID, GATE_SQRT_SOFTPLUS = 0, 1, 2
OOB_ERROR, OOB_SKIP = 0, 1
RENORM_CLAMP, RENORM_PLUS_EPS = 0, 1


class OracleError(RuntimeError):
    """Raised where the reference returns `Err` (bad shapes, partial blocks ...)."""


def build(force: bool = False) -> Path:
    """Compile the oracle with the Makefile beside it (gcc, a second or two)."""
    src = _HERE / "joshua_oracle.cpp"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "libjoshua_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


class _MoeCfg(ctypes.Structure):
    _fields_ = [
        ("gating", ctypes.c_int32),
        ("n_expert", ctypes.c_int32),
        ("n_used", ctypes.c_int32),
        ("hidden", ctypes.c_int32),
        ("inter", ctypes.c_int32),
        ("n_group", ctypes.c_int32),
        ("topk_group", ctypes.c_int32),
        ("norm", ctypes.c_int32),
        ("renorm_mode", ctypes.c_int32),
        ("oob_policy", ctypes.c_int32),
        ("decode_path", ctypes.c_int32),
        ("scale", ctypes.c_float),
        ("clamp", ctypes.c_float),
    ]


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(_LIB_PATH))
        _lib.jo_last_error.restype = ctypes.c_char_p
        _lib.jo_f16_to_f32.restype = ctypes.c_float
        _lib.jo_f16_to_f32.argtypes = [ctypes.c_uint16]
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise OracleError(lib().jo_last_error().decode())


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    if isinstance(a, (bytes, bytearray, memoryview)):
        return np.frombuffer(a, dtype=np.uint8)
    return np.ascontiguousarray(a, dtype=np.uint8)


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def threads() -> int:
    return lib().jo_threads()


def block_size(type_id: int) -> tuple[int, int]:
    """(elements, bytes) of one block of a GGUF type."""
    e, b = ctypes.c_uint64(), ctypes.c_uint64()
    _check(lib().jo_block_size(type_id, ctypes.byref(e), ctypes.byref(b)))
    return e.value, b.value


def e8m0_to_f32(e: int):
    """2^(e-127) as float32, or None for the reserved code 0xFF (src/mxfp4.rs:67-75)."""
    out = ctypes.c_float()
    ok = lib().jo_e8m0_to_f32(ctypes.c_uint8(e), ctypes.byref(out))
    return np.float32(out.value) if ok else None


def f16_to_f32(h: int) -> np.float32:
    return np.float32(lib().jo_f16_to_f32(h))


def dequantize(type_id: int, raw, two_step: bool = False) -> np.ndarray:
    """Decode whole blocks.  `two_step` picks the separately rounded k-quant form."""
    raw = _u8(raw)
    elems, nbytes = block_size(type_id)
    n_out = raw.size // nbytes * elems if raw.size % nbytes == 0 else 0
    out = np.empty(n_out, dtype=np.float32)
    _check(lib().jo_dequantize(type_id, _p(raw), ctypes.c_uint64(raw.size), _p(out), ctypes.c_uint64(n_out),
                               int(two_step)))
    return out


def matmul_t(type_id: int, mkn, lhs, raw, *, threads: int = 0, scalar: bool = False, dst=None,
             lhs_len=None, dst_len=None) -> np.ndarray:
    """dst[m, n] = lhs[m, k] . W[n, k]^T over raw blocks, the reference's way.

    threads=0 uses every core (the reference's default), 1 is the serial row
    loop.  `scalar` forces the block-at-a-time scalar loop.  `dst`, when
    given, is written in place (to show that the product is assigned, never
    accumulated).  `lhs_len` / `dst_len` override the lengths announced to the
    validator, to exercise its error paths.
    """
    m, k, n = mkn
    lhs = _f32(lhs).reshape(-1)
    raw = _u8(raw)
    if dst is None:
        dst = np.zeros(m * n if dst_len is None else max(dst_len, m * n), dtype=np.float32)
    flat = dst.reshape(-1)
    _check(lib().jo_matmul_t(type_id, ctypes.c_uint64(m), ctypes.c_uint64(k), ctypes.c_uint64(n), _p(lhs),
                             ctypes.c_uint64(lhs.size if lhs_len is None else lhs_len), _p(raw),
                             ctypes.c_uint64(raw.size), _p(flat),
                             ctypes.c_uint64(m * n if dst_len is None else dst_len), int(threads), int(scalar)))
    return dst if dst.ndim == 2 else flat[: m * n].reshape(m, n)


def moe_cfg(*, gating, n_expert, n_used, hidden, inter, n_group=1, topk_group=1, norm=True,
            renorm_mode=RENORM_CLAMP, oob_policy=OOB_ERROR, decode_path=True, scale=1.0, clamp=0.0) -> _MoeCfg:
    return _MoeCfg(gating, n_expert, n_used, hidden, inter, n_group, topk_group, int(norm), renorm_mode,
                   oob_policy, int(decode_path), scale, clamp)


def moe_logits(x, router) -> np.ndarray:
    x, router = _f32(x), _f32(router)
    T, h = x.shape
    E = router.shape[0]
    out = np.empty((T, E), dtype=np.float32)
    _check(lib().jo_moe_logits(_p(x), ctypes.c_uint64(T), ctypes.c_uint64(h), _p(router), ctypes.c_uint64(E),
                               _p(out)))
    return out


def moe_route(cfg: _MoeCfg, logits, bias=None, forced_ids=None):
    logits = _f32(logits)
    T = logits.shape[0]
    ids = np.empty((T, cfg.n_used), dtype=np.uint32)
    wts = np.empty((T, cfg.n_used), dtype=np.float32)
    b = _f32(bias) if bias is not None else None
    f = np.ascontiguousarray(forced_ids, dtype=np.uint32) if forced_ids is not None else None
    _check(lib().jo_moe_route(ctypes.byref(cfg), _p(logits), ctypes.c_uint64(T), _p(b) if b is not None else None,
                              _p(f) if f is not None else None, _p(ids), _p(wts)))
    return ids, wts


def moe_dispatch(cfg: _MoeCfg, x, ids, wts, types, banks, shared_types=None, shared=None, threads: int = 0):
    """Routed experts (+ optional shared expert) for tokens x [T, h].

    `banks` = (gate, up, down) raw byte arrays, each a contiguous
    [n_expert, out, in] tensor; `types` their three GGUF type ids.
    """
    x = _f32(x)
    T = x.shape[0]
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    wts = _f32(wts)
    banks = [_u8(b) for b in banks]
    tarr = (ctypes.c_int32 * 3)(*types)
    barr = (ctypes.c_void_p * 3)(*[b.ctypes.data for b in banks])
    if shared is not None:
        shared = [_u8(b) for b in shared]
        starr = (ctypes.c_int32 * 3)(*shared_types)
        sbarr = (ctypes.c_void_p * 3)(*[b.ctypes.data for b in shared])
    else:
        starr, sbarr = None, None
    y = np.empty((T, cfg.hidden), dtype=np.float32)
    _check(lib().jo_moe_dispatch(ctypes.byref(cfg), _p(x), ctypes.c_uint64(T), _p(ids), _p(wts), tarr, barr, starr,
                                 sbarr, _p(y), int(threads)))
    return y
