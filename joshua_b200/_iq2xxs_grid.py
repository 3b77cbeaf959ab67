"""The IQ2_XXS codebook as a numpy array, expanded from the packed table the CUDA library is built from
(`csrc/iq2xxs_grid_packed.h`: 256 base-3 words, digit j of word i selects byte j of entry i from 8 / 25 / 43;
the table restated in the reference at src/iq2xxs.rs:453-710)."""
from __future__ import annotations

import re
from functools import lru_cache
from pathlib import Path

import numpy as np


@lru_cache(maxsize=1)
def grid_bytes() -> np.ndarray:
    text = (Path(__file__).resolve().parent / "csrc" / "iq2xxs_grid_packed.h").read_text()
    body = text.split("JQ_IQ2XXS_GRID_PACKED[256] = {", 1)[1].split("};", 1)[0]
    words = [int(w) for w in re.findall(r"\d+", body)]
    assert len(words) == 256
    levels = np.array([8, 25, 43], dtype=np.uint8)
    out = np.empty((256, 8), dtype=np.uint8)
    for i, c in enumerate(words):
        for j in range(8):
            out[i, j] = levels[c % 3]
            c //= 3
    return out
