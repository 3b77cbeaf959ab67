"""Seeded synthetic GGUF block data.

Weights are generated directly as raw block bytes, never through a quantiser:
every byte pattern is a valid block for all five formats (the reference relies
on the same fact, src/kquant_dot.rs:225-228, src/iq2xxs.rs:431-433), so uniform
random bytes give uniform codes, and only the fp16 / E8M0 scale fields need
shaping to keep decoded weights in a sane range.

Two generators with the same distributions: numpy (host arrays, for parity
tests against the CPU oracle) and torch (device-resident, for benchmark banks
of several GB that would be slow to draw on the host).
"""
from __future__ import annotations

import numpy as np

Q8_0, Q2_K, Q4_K, IQ2_XXS, MXFP4 = 8, 10, 12, 16, 39
# the block types of the reference's generic (decode a row, then dot) path
Q4_0, Q4_1, Q5_0, Q5_1, Q8_1, Q3_K, Q5_K, Q6_K, Q8_K = 2, 3, 6, 7, 9, 11, 13, 14, 15
GENERIC_TYPES = (Q4_0, Q4_1, Q5_0, Q5_1, Q8_1, Q3_K, Q5_K, Q6_K, Q8_K)

# type id -> (elements per block, bytes per block)
BLOCK = {Q8_0: (32, 34), Q2_K: (256, 84), Q4_K: (256, 144), IQ2_XXS: (256, 66), MXFP4: (32, 17),
         Q4_0: (32, 18), Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24), Q8_1: (32, 36), Q3_K: (256, 110),
         Q5_K: (256, 176), Q6_K: (256, 210), Q8_K: (256, 292)}
NAMES = {Q8_0: "q8_0", Q2_K: "q2_k", Q4_K: "q4_k", IQ2_XXS: "iq2_xxs", MXFP4: "mxfp4", Q4_0: "q4_0", Q4_1: "q4_1",
         Q5_0: "q5_0", Q5_1: "q5_1", Q8_1: "q8_1", Q3_K: "q3_k", Q5_K: "q5_k", Q6_K: "q6_k", Q8_K: "q8_k"}

# byte offsets of the fp16 scale fields inside a block (Q8_K carries one f32 scale at offset 0 instead)
_F16_FIELDS = {Q8_0: (0,), Q2_K: (80, 82), Q4_K: (0, 2), IQ2_XXS: (0,), MXFP4: (), Q4_0: (0,), Q4_1: (0, 2),
               Q5_0: (0,), Q5_1: (0, 2), Q8_1: (0, 2), Q3_K: (108,), Q5_K: (0, 2), Q6_K: (208,), Q8_K: ()}
_SCALE_LO, _SCALE_HI = 1e-3, 1e-2
_E8M0_LO, _E8M0_HI = 118, 130  # inclusive


def tensor_bytes(type_id: int, rows: int, cols: int) -> int:
    elems, nbytes = BLOCK[type_id]
    if cols % elems:
        raise ValueError(f"{NAMES[type_id]}: {cols} columns is not a multiple of {elems}")
    return rows * (cols // elems) * nbytes


def random_blocks(type_id: int, n_blocks: int, rng: np.random.Generator) -> np.ndarray:
    """`n_blocks` raw blocks as a uint8 array [n_blocks, block_bytes]."""
    _, nbytes = BLOCK[type_id]
    raw = rng.integers(0, 256, size=(n_blocks, nbytes), dtype=np.uint8)
    for off in _F16_FIELDS[type_id]:
        scale = rng.uniform(_SCALE_LO, _SCALE_HI, size=n_blocks).astype(np.float16)
        raw[:, off : off + 2] = scale.view(np.uint8).reshape(n_blocks, 2)
    if type_id == Q8_0:
        # int8 values uniform in [-127, 127]: -128 is folded onto -127
        q = raw[:, 2:].view(np.int8)
        q[q == -128] = -127
    if type_id == MXFP4:
        raw[:, 0] = rng.integers(_E8M0_LO, _E8M0_HI + 1, size=n_blocks, dtype=np.uint8)
    if type_id == Q8_K:
        scale = rng.uniform(_SCALE_LO, _SCALE_HI, size=n_blocks).astype(np.float32)
        raw[:, 0:4] = scale.view(np.uint8).reshape(n_blocks, 4)
    return raw


def random_weight(type_id: int, rows: int, cols: int, seed: int) -> np.ndarray:
    """A [rows, cols] weight matrix as flat raw bytes in GGUF row-major block order."""
    elems, _ = BLOCK[type_id]
    rng = np.random.default_rng(seed)
    return random_blocks(type_id, rows * (cols // elems), rng).reshape(-1)


def random_activations(m: int, k: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((m, k), dtype=np.float32)


def random_weight_torch(type_id: int, rows: int, cols: int, seed: int, device):
    """Device-resident counterpart of `random_weight` (a flat torch.uint8 tensor)."""
    import torch

    elems, nbytes = BLOCK[type_id]
    n_blocks = rows * (cols // elems)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    raw = torch.randint(0, 256, (n_blocks, nbytes), dtype=torch.uint8, device=device, generator=gen)
    for off in _F16_FIELDS[type_id]:
        scale = torch.empty(n_blocks, device=device, dtype=torch.float32).uniform_(_SCALE_LO, _SCALE_HI, generator=gen)
        raw[:, off : off + 2] = scale.to(torch.float16).view(torch.uint8).reshape(n_blocks, 2)
    if type_id == Q8_0:
        q = raw[:, 2:]
        q[q == 128] = 129  # int8 -128 -> -127
    if type_id == MXFP4:
        raw[:, 0] = torch.randint(_E8M0_LO, _E8M0_HI + 1, (n_blocks,), dtype=torch.uint8, device=device, generator=gen)
    return raw.reshape(-1)
