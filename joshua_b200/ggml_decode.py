"""Host-side numpy decoders for GGUF block types: raw bytes -> float32.

Used where the reference decodes a tensor once at load time on the CPU: router matrices, biases and norm
weights that happen to be stored quantized (`ffn_gate_inp` is "dequantised to f32 and transposed once",
src/quantized_qwen3_moe.rs:654-657), and the streamed loader's `decode_raw_to_f32` (src/quant_matmul.rs:36-103).
The hot path never comes through here: matmuls run on the device over the raw blocks.

Every decoder restates the published ggml block layout of its type (the reference takes the k-quant and legacy
decoders from candle's `k_quants::*::to_float`, a port of ggml's `dequantize_row_*`; that crate is not part of
the reference tree, so for these types the decode is anchored on the format definition).  Arithmetic is float32
with the roundings of the scalar ggml loops: `fl(fl(d * sc) * q) - fl(dmin * m)` for the k-quants with minima,
`fl(fl(d * sc) * q)` for Q6_K / Q3_K, `fl(q * d) (+ m)` for the 32-value legacy blocks.
"""
from __future__ import annotations

import numpy as np

F = np.float32


def _blocks(raw, nbytes):
    b = np.ascontiguousarray(np.asarray(raw, dtype=np.uint8).reshape(-1))
    if b.size % nbytes:
        raise ValueError(f"{b.size} bytes is not a whole number of {nbytes}-byte blocks")
    return b.reshape(-1, nbytes)


def _f16(cols):
    return np.ascontiguousarray(cols).view(np.float16).astype(F).reshape(-1)


def _mul(a, b):
    return (a.astype(F) * b.astype(F)).astype(F)


def q4_0(raw):
    b = _blocks(raw, 18)
    d = _f16(b[:, 0:2])[:, None]
    qs = b[:, 2:]
    q = np.concatenate([(qs & 0xF).astype(np.int16) - 8, (qs >> 4).astype(np.int16) - 8], axis=1)  # values j and j + 16
    return _mul(q, d).reshape(-1)


def q4_1(raw):
    b = _blocks(raw, 20)
    d, m = _f16(b[:, 0:2])[:, None], _f16(b[:, 2:4])[:, None]
    qs = b[:, 4:]
    q = np.concatenate([qs & 0xF, qs >> 4], axis=1)
    return (_mul(q, d) + m).astype(F).reshape(-1)


def _q5_codes(qh_bytes, qs):
    qh = np.ascontiguousarray(qh_bytes).view(np.uint32).reshape(-1, 1)
    j = np.arange(16, dtype=np.uint32)[None, :]
    lo = (qs & 0xF) | (((qh >> j) << 4) & 0x10).astype(np.uint8)
    hi = (qs >> 4) | ((qh >> (j + 12)) & 0x10).astype(np.uint8)
    return np.concatenate([lo, hi], axis=1)


def q5_0(raw):
    b = _blocks(raw, 22)
    d = _f16(b[:, 0:2])[:, None]
    q = _q5_codes(b[:, 2:6], b[:, 6:]).astype(np.int16) - 16
    return _mul(q, d).reshape(-1)


def q5_1(raw):
    b = _blocks(raw, 24)
    d, m = _f16(b[:, 0:2])[:, None], _f16(b[:, 2:4])[:, None]
    q = _q5_codes(b[:, 4:8], b[:, 8:])
    return (_mul(q, d) + m).astype(F).reshape(-1)


def q8_0(raw):
    b = _blocks(raw, 34)
    return _mul(b[:, 2:].view(np.int8), _f16(b[:, 0:2])[:, None]).reshape(-1)


def q8_1(raw):
    b = _blocks(raw, 36)   # f16 d, f16 s (d * sum of codes, unused by the decode), 32 int8
    return _mul(b[:, 4:].view(np.int8), _f16(b[:, 0:2])[:, None]).reshape(-1)


def _k4_scales(s):
    """[nb, 12] packed bytes -> six-bit (scales [nb, 8], minima [nb, 8]) (`get_scale_min_k4`)."""
    sc = np.empty((s.shape[0], 8), dtype=np.uint8)
    mn = np.empty_like(sc)
    for j in range(8):
        if j < 4:
            sc[:, j] = s[:, j] & 63
            mn[:, j] = s[:, j + 4] & 63
        else:
            sc[:, j] = (s[:, j + 4] & 0xF) | ((s[:, j - 4] >> 6) << 4)
            mn[:, j] = (s[:, j + 4] >> 4) | ((s[:, j] >> 6) << 4)
    return sc, mn


def q2_k(raw):
    b = _blocks(raw, 84)
    nb = b.shape[0]
    scales, qs = b[:, 0:16], b[:, 16:80].reshape(nb, 2, 32)
    d, dmin = _f16(b[:, 80:82]), _f16(b[:, 82:84])
    # value sg*128 + 32*i + byte <- (qs[sg, byte] >> 2i) & 3; 16-value group = scale byte index in value order
    q = np.stack([(qs >> (2 * i)) & 3 for i in range(4)], axis=2).reshape(nb, 16, 16)
    d1 = _mul(d[:, None], scales & 0xF)
    m1 = _mul(dmin[:, None], scales >> 4)
    return (_mul(d1[:, :, None], q) - m1[:, :, None]).astype(F).reshape(-1)


def q3_k(raw):
    b = _blocks(raw, 110)
    nb = b.shape[0]
    hmask, qs, sb = b[:, 0:32], b[:, 32:96].reshape(nb, 2, 32), b[:, 96:108]
    d = _f16(b[:, 108:110])
    aux = np.ascontiguousarray(sb).view(np.uint32).reshape(nb, 3)
    k1, k2 = np.uint32(0x03030303), np.uint32(0x0F0F0F0F)
    tmp = aux[:, 2]
    a0 = (aux[:, 0] & k2) | (((tmp >> 0) & k1) << 4)
    a1 = (aux[:, 1] & k2) | (((tmp >> 2) & k1) << 4)
    a2 = ((aux[:, 0] >> 4) & k2) | (((tmp >> 4) & k1) << 4)
    a3 = ((aux[:, 1] >> 4) & k2) | (((tmp >> 6) & k1) << 4)
    sc = np.stack([a0, a1, a2, a3], axis=1).astype(np.uint32).view(np.uint8).reshape(nb, 16).view(np.int8).astype(np.int16) - 32
    out = np.empty((nb, 256), dtype=F)
    for half in range(2):
        for j in range(4):           # shift 2j, mask bit 4*half + j
            bit = np.uint8(1 << (4 * half + j))
            two = ((qs[:, half, :] >> (2 * j)) & 3).astype(np.int16)
            q = two - np.where(hmask & bit, 0, 4).astype(np.int16)     # [nb, 32]
            for part in range(2):    # 16 values each, consecutive scales
                dl = _mul(d, sc[:, 8 * half + 2 * j + part])
                o = 128 * half + 32 * j + 16 * part
                out[:, o:o + 16] = _mul(dl[:, None], q[:, 16 * part:16 * part + 16])
    return out.reshape(-1)


def q4_k(raw):
    b = _blocks(raw, 144)
    nb = b.shape[0]
    d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
    sc, mn = _k4_scales(b[:, 4:16])
    qs = b[:, 16:].reshape(nb, 4, 32)
    q = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(nb, 8, 32)
    d1, m1 = _mul(d[:, None], sc), _mul(dmin[:, None], mn)
    return (_mul(d1[:, :, None], q) - m1[:, :, None]).astype(F).reshape(-1)


def q5_k(raw):
    b = _blocks(raw, 176)
    nb = b.shape[0]
    d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
    sc, mn = _k4_scales(b[:, 4:16])
    qh, qs = b[:, 16:48], b[:, 48:].reshape(nb, 4, 32)
    groups = []
    for j in range(4):
        groups.append((qs[:, j] & 0xF) + np.where(qh & np.uint8(1 << (2 * j)), 16, 0).astype(np.uint8))
        groups.append((qs[:, j] >> 4) + np.where(qh & np.uint8(2 << (2 * j)), 16, 0).astype(np.uint8))
    q = np.stack(groups, axis=1)     # [nb, 8, 32]
    d1, m1 = _mul(d[:, None], sc), _mul(dmin[:, None], mn)
    return (_mul(d1[:, :, None], q) - m1[:, :, None]).astype(F).reshape(-1)


def q6_k(raw):
    b = _blocks(raw, 210)
    nb = b.shape[0]
    ql, qh = b[:, 0:128].reshape(nb, 2, 64), b[:, 128:192].reshape(nb, 2, 32)
    sc = b[:, 192:208].view(np.int8).reshape(nb, 2, 8)
    d = _f16(b[:, 208:210])
    out = np.empty((nb, 2, 4, 32), dtype=F)
    for half in range(2):
        lo, hi, h = ql[:, half, :32], ql[:, half, 32:], qh[:, half]
        codes = [(lo & 0xF) | ((h & 3) << 4), (hi & 0xF) | (((h >> 2) & 3) << 4),
                 (lo >> 4) | (((h >> 4) & 3) << 4), (hi >> 4) | (((h >> 6) & 3) << 4)]
        for part, c in enumerate(codes):
            q = c.astype(np.int16) - 32                                   # [nb, 32]
            s = sc[:, half, 2 * part:2 * part + 2]                        # scales of values 0..15 and 16..31
            ds = _mul(d[:, None], s)                                      # fl(d * sc)
            out[:, half, part] = _mul(np.repeat(ds, 16, axis=1), q)
    return out.reshape(-1)


def q8_k(raw):
    b = _blocks(raw, 292)
    d = np.ascontiguousarray(b[:, 0:4]).view(np.float32).reshape(-1, 1)
    return _mul(b[:, 4:260].view(np.int8), d).reshape(-1)


def iq2_xxs(raw):
    from ._iq2xxs_grid import grid_bytes

    b = _blocks(raw, 66)
    nb = b.shape[0]
    d = _f16(b[:, 0:2])
    words = np.ascontiguousarray(b[:, 2:]).view(np.uint32).reshape(nb, 8, 2)
    lo, hi = words[:, :, 0], words[:, :, 1]
    db = _mul(_mul(d[:, None], (F(0.5) + (hi >> 28).astype(F)).astype(F)), F(0.25))     # [nb, 8]
    grid = grid_bytes()                                                                # [256, 8] uint8
    out = np.empty((nb, 8, 4, 8), dtype=F)
    bits = np.arange(8, dtype=np.uint32)
    for l in range(4):
        code = (lo >> (8 * l)) & 0xFF
        idx = (hi >> (7 * l)) & 127
        par = np.zeros_like(idx)
        for i in range(7):
            par ^= (idx >> i) & 1
        signs = idx | (par << 7)
        sgn = np.where((signs[:, :, None] >> bits) & 1, F(-1), F(1))
        out[:, :, l, :] = _mul(_mul(db[:, :, None], grid[code]), sgn)
    return out.reshape(-1)


_E2M1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=F)


def mxfp4(raw):
    b = _blocks(raw, 17)
    e = b[:, 0].astype(np.uint32)
    scale = np.where(e == 0, np.uint32(0x00400000), e << 23).astype(np.uint32).view(F)
    qs = b[:, 1:]
    codes = np.concatenate([qs & 0xF, qs >> 4], axis=1)
    out = _mul(scale[:, None], _E2M1[codes])
    out[e == 255] = 0
    return out.reshape(-1)


def f16(raw):
    return np.ascontiguousarray(np.asarray(raw, dtype=np.uint8)).view(np.float16).astype(F)


DECODERS = {1: f16, 2: q4_0, 3: q4_1, 6: q5_0, 7: q5_1, 8: q8_0, 9: q8_1, 10: q2_k, 11: q3_k, 12: q4_k, 13: q5_k,
            14: q6_k, 15: q8_k, 16: iq2_xxs, 39: mxfp4}


def dequantize(type_id: int, raw) -> np.ndarray:
    """All blocks of `raw` as float32 (`decode_raw_to_f32`; type 0 and unknown ids have no decoder here)."""
    if type_id not in DECODERS:
        raise ValueError(f"no decoder for GGUF type id {type_id}")
    return DECODERS[type_id](raw)
