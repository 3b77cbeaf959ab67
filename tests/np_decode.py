"""Vectorised numpy decoders for the five block formats.

A second, independently written statement of the block layouts (the first is
the C++ oracle), used by the CPU tests to cross-check the oracle and by nothing
else.  All arithmetic is float32 with separate roundings; the k-quants are
decoded in the separately rounded form fl(fl(d*sc)*q) - fl(dmin*m)).
Layouts: src/kquant_dot.rs:22-33,53-118, src/iq2xxs.rs:44-71, src/mxfp4.rs:45-94.
"""
import numpy as np

GOLDEN = __import__("pathlib").Path(__file__).resolve().parent / "golden"


def _f16(raw2):
    return np.ascontiguousarray(raw2).view(np.float16).astype(np.float32).reshape(-1)


def q8_0(raw):
    b = np.asarray(raw, dtype=np.uint8).reshape(-1, 34)
    d = _f16(b[:, 0:2])
    q = b[:, 2:].view(np.int8).astype(np.float32)
    return (q * d[:, None]).astype(np.float32).reshape(-1)


def q4k_scales(sbytes):
    """[nb, 12] packed bytes -> (sc [nb, 8], mn [nb, 8])."""
    s = sbytes.astype(np.uint8)
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


def q4k(raw):
    b = np.asarray(raw, dtype=np.uint8).reshape(-1, 144)
    nb = b.shape[0]
    d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
    sc, mn = q4k_scales(b[:, 4:16])
    qs = b[:, 16:].reshape(nb, 4, 32)
    q = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(nb, 8, 32).astype(np.float32)  # pair = 2c + r
    d1 = (d[:, None] * sc.astype(np.float32)).astype(np.float32)
    m1 = (dmin[:, None] * mn.astype(np.float32)).astype(np.float32)
    w = (d1[:, :, None] * q).astype(np.float32) - m1[:, :, None]
    return w.astype(np.float32).reshape(-1)


def q2k(raw):
    b = np.asarray(raw, dtype=np.uint8).reshape(-1, 84)
    nb = b.shape[0]
    scales = b[:, 0:16]
    qs = b[:, 16:80].reshape(nb, 2, 32)
    d, dmin = _f16(b[:, 80:82]), _f16(b[:, 82:84])
    # value sg*128 + 32*i + byte  <- (qs[sg, byte] >> 2i) & 3
    q = np.stack([(qs >> (2 * i)) & 3 for i in range(4)], axis=2).reshape(nb, 16, 16).astype(np.float32)
    d1 = (d[:, None] * (scales & 0xF).astype(np.float32)).astype(np.float32)
    m1 = (dmin[:, None] * (scales >> 4).astype(np.float32)).astype(np.float32)
    w = (d1[:, :, None] * q).astype(np.float32) - m1[:, :, None]
    return w.astype(np.float32).reshape(-1)


def iq2xxs_tables():
    import re

    hdr = (GOLDEN.parent.parent / "joshua_b200" / "csrc" / "iq2xxs_grid_packed.h").read_text()
    body = hdr.split("{", 1)[1].split("}", 1)[0]
    packed = [int(x) for x in re.findall(r"\d+", body)]
    level = np.array([8, 25, 43], dtype=np.float32)
    grid = np.empty((256, 8), dtype=np.float32)
    for i, c in enumerate(packed):
        for j in range(8):
            grid[i, j] = level[c % 3]
            c //= 3
    signs = np.empty((128, 8), dtype=np.float32)
    for i in range(128):
        byte = i | ((bin(i).count("1") & 1) << 7)
        for j in range(8):
            signs[i, j] = -1.0 if (byte >> j) & 1 else 1.0
    return grid, signs


def iq2xxs(raw):
    grid, signs = iq2xxs_tables()
    b = np.asarray(raw, dtype=np.uint8).reshape(-1, 66)
    nb = b.shape[0]
    d = _f16(b[:, 0:2])
    words = np.ascontiguousarray(b[:, 2:]).view("<u4").reshape(nb, 8, 2)
    lo, hi = words[:, :, 0], words[:, :, 1]
    db = ((d[:, None] * (np.float32(0.5) + (hi >> 28).astype(np.float32))).astype(np.float32) * np.float32(0.25))
    out = np.empty((nb, 8, 4, 8), dtype=np.float32)
    for l in range(4):
        g = grid[(lo >> (8 * l)) & 0xFF]
        s = signs[(hi >> (7 * l)) & 127]
        out[:, :, l, :] = ((db[:, :, None] * g).astype(np.float32) * s).astype(np.float32)
    return out.reshape(-1)


E2M1 = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)


def mxfp4(raw):
    b = np.asarray(raw, dtype=np.uint8).reshape(-1, 17)
    e = b[:, 0].astype(np.uint32)
    bits = np.where(e == 0, np.uint32(0x00400000), e << 23).astype(np.uint32)
    scale = bits.view(np.float32)
    lo = E2M1[b[:, 1:] & 0xF]
    hi = E2M1[b[:, 1:] >> 4]
    with np.errstate(over="ignore", invalid="ignore"):
        w = np.concatenate([lo, hi], axis=1) * scale[:, None]
    w[e == 0xFF] = 0.0
    return w.astype(np.float32).reshape(-1)


DECODERS = {8: q8_0, 10: q2k, 12: q4k, 16: iq2xxs, 39: mxfp4}
