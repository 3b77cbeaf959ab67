"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import re

import pytest

from joshua_b200 import _lib
from tests.conftest import ROOT


def declared_symbols():
    text = (ROOT / "include" / "joshua_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(jq_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    assert "jq_matmul_t" in names and "jq_weight_upload" in names and len(names) >= 15


def test_library_exports_every_declared_symbol():
    from joshua_b200 import build

    build.build()
    handle = ctypes.CDLL(str(_lib.LIB_PATH))
    missing = [n for n in declared_symbols() if not hasattr(handle, n)]
    assert not missing, missing


def test_python_binding_covers_every_declared_symbol():
    assert sorted(_lib._SIGNATURES) == declared_symbols()


def test_block_sizes_without_a_device():
    e, b = ctypes.c_uint64(), ctypes.c_uint64()
    from joshua_b200 import gguf, synth

    for t, want in synth.BLOCK.items():       # every block type with a decoder, sizes as src/gguf_ext.rs:483-512
        assert _lib.lib().jq_block_size(t, ctypes.byref(e), ctypes.byref(b)) == 0
        assert (e.value, b.value) == want == gguf.TYPE_SIZES[t]
    for t in (0, 1, 17, 26, 30, 40):          # float / integer / unknown ids are not block types of this library
        assert _lib.lib().jq_block_size(t, ctypes.byref(e), ctypes.byref(b)) == _lib.E_TYPE


def test_product_fails_loudly_without_a_device():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from joshua_b200 import qtensor

    with pytest.raises(_lib.JoshuaB200Error, match="no CPU path"):
        qtensor.Context(0)
