"""Host-side mirror of the reference's MoE layer (`Moe::forward`).

`Moe` holds what the loaders' `Moe` structs hold (router, optional selection
bias, expert banks, optional shared expert, routing rule;
src/quantized_qwen3_moe.rs:404-410, src/quantized_deepseek2.rs:508-519,
src/quantized_deepseek4.rs:1340-1351) and forwards to the C ABI.  All
arithmetic runs in the CUDA library.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import check
from .qtensor import Context, QTensor, default_context

GATE_SOFTMAX, GATE_SIGMOID, GATE_SQRT_SOFTPLUS = 0, 1, 2
OOB_ERROR, OOB_SKIP = 0, 1


class MoeConfigC(ctypes.Structure):
    _fields_ = [
        ("gating", ctypes.c_int32), ("n_expert", ctypes.c_uint32), ("n_used", ctypes.c_uint32),
        ("hidden", ctypes.c_uint32), ("inter", ctypes.c_uint32), ("n_group", ctypes.c_uint32),
        ("topk_group", ctypes.c_uint32), ("norm", ctypes.c_int32), ("renorm_plus_eps", ctypes.c_int32),
        ("oob_policy", ctypes.c_int32), ("scale", ctypes.c_float), ("clamp", ctypes.c_float),
    ]


@dataclass
class MoeConfig:
    gating: int
    n_expert: int
    n_used: int
    hidden: int
    inter: int
    n_group: int = 1
    topk_group: int = 1
    norm: bool = True
    renorm_plus_eps: bool = False
    oob_policy: int = OOB_ERROR
    scale: float = 1.0
    clamp: float = 0.0

    def to_c(self) -> MoeConfigC:
        return MoeConfigC(self.gating, self.n_expert, self.n_used, self.hidden, self.inter, self.n_group,
                          self.topk_group, int(self.norm), int(self.renorm_plus_eps), self.oob_policy, self.scale,
                          self.clamp)


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


class Moe:
    def __init__(self, cfg: MoeConfig, router, gate: QTensor | None, up: QTensor | None, down: QTensor | None,
                 bias=None, shared=None,
                 ctx: Context | None = None):
        self.cfg, self.ctx = cfg, ctx or default_context()
        router = np.ascontiguousarray(router, dtype=np.float32)
        bias = np.ascontiguousarray(bias, dtype=np.float32) if bias is not None else None
        self._keep = (gate, up, down, shared)
        sh = [w._h for w in shared] if shared else [None, None, None]
        gh, uh, dh = (gate._h, up._h, down._h) if gate is not None else (None, None, None)
        self._h = ctypes.c_void_p()
        c = cfg.to_c()
        check(_lib.lib().jq_moe_create(self.ctx._h, ctypes.byref(c), _ptr(router), _ptr(bias), gh, uh, dh, sh[0],
                                       sh[1], sh[2], ctypes.byref(self._h)))

    def __del__(self):
        try:
            if self._h:
                _lib.lib().jq_moe_free(self._h)
                self._h = ctypes.c_void_p()
        except Exception:
            pass

    def forward(self, xs, forced_ids=None) -> np.ndarray:
        """xs: host f32 [..., hidden] -> same shape (Moe::forward reshapes [b, seq, h] to [b*seq, h])."""
        x = np.ascontiguousarray(xs, dtype=np.float32)
        x2 = x.reshape(-1, self.cfg.hidden)
        f = np.ascontiguousarray(forced_ids, dtype=np.uint32) if forced_ids is not None else None
        y = np.empty_like(x2)
        check(_lib.lib().jq_moe_forward(self._h, _ptr(x2), x2.shape[0], _ptr(f), _ptr(y)))
        return y.reshape(x.shape)

    def last_routing(self, n_tokens: int):
        ids = np.empty((n_tokens, self.cfg.n_used), dtype=np.uint32)
        wts = np.empty((n_tokens, self.cfg.n_used), dtype=np.float32)
        check(_lib.lib().jq_moe_last_routing(self._h, n_tokens, _ptr(ids), _ptr(wts)))
        return ids, wts

    # ── device-resident entries (torch CUDA tensors) ────────────────────
    def reserve(self, n_tokens: int, n_rows: int = 0) -> None:
        check(_lib.lib().jq_moe_reserve(self._h, n_tokens, n_rows))

    @staticmethod
    def _stream(t, stream):
        import torch

        return torch.cuda.current_stream(t.device).cuda_stream if stream is None else stream

    def forward_dev(self, x, y, forced_ids=None, stream=None) -> None:
        T = x.numel() // self.cfg.hidden
        check(_lib.lib().jq_moe_forward_dev(self._h, x.data_ptr(), T,
                                            forced_ids.data_ptr() if forced_ids is not None else None,
                                            y.data_ptr(), self._stream(x, stream)))

    def route_dev(self, x, ids, wts, forced_ids=None, stream=None) -> None:
        T = x.numel() // self.cfg.hidden
        check(_lib.lib().jq_moe_route_dev(self._h, x.data_ptr(), T,
                                          forced_ids.data_ptr() if forced_ids is not None else None,
                                          ids.data_ptr(), wts.data_ptr(), self._stream(x, stream)))

    def experts_dev(self, x_rows, expert_ids, out_rows, stream=None) -> None:
        R = x_rows.numel() // self.cfg.hidden
        check(_lib.lib().jq_moe_experts_dev(self._h, x_rows.data_ptr(), R, expert_ids.data_ptr(),
                                            out_rows.data_ptr(), self._stream(x_rows, stream)))

    def experts_replay_dev(self, x, stream=None) -> None:
        """The expert matmuls alone over the job list of the last decode-sized call (a measurement aid)."""
        check(_lib.lib().jq_moe_experts_replay_dev(self._h, x.data_ptr(), self._stream(x, stream)))

    def status(self) -> None:
        check(_lib.lib().jq_moe_status(self._h))
