"""Host side of the Higgs-style speech model's delay pattern over the C ABI (include/omni_b200_ops.h).

Names follow crates/omni-higgs-audio/src/delay.rs: ``Delay.forced_from``, ``Delay.advance``, ``undelay``; ``BOC`` and
``EOC`` are the last two codes of every codebook.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib as L

CODEBOOKS, BOC, EOC = 8, 1024, 1025


class Delay:
    """Which codebooks of the next step are not drawn, and when generation ends (delay.rs:19-46)."""

    def __init__(self):
        self._d = L.HiggsDelay(0, 0, 0)
        self._lib = L.load()

    def forced_from(self) -> int:
        return self._lib.omni_higgs_delay_forced_from(C.byref(self._d))

    def advance(self, first: int) -> bool:
        return bool(self._lib.omni_higgs_delay_advance(C.byref(self._d), int(first)))

    def force_row(self, draw_all: bool = False):
        """The `force` row of the next step: -1 for the codebooks that draw, BOC from `forced_from` on."""
        f = self.forced_from()
        return [-1 if b < f else BOC for b in range(CODEBOOKS)]


def undelay(rows) -> np.ndarray:
    """Frames inside delayed rows: frame t takes codebook c from row t + c (delay.rs:50-54)."""
    rows = np.ascontiguousarray(np.asarray(rows, dtype=np.int32).reshape(-1, CODEBOOKS))
    frames = np.zeros((max(len(rows) - CODEBOOKS + 1, 0), CODEBOOKS), dtype=np.int32)
    i32p = C.POINTER(C.c_int32)
    n = L.load().omni_higgs_undelay(rows.ctypes.data_as(i32p), len(rows), frames.ctypes.data_as(i32p))
    assert n == len(frames)
    return frames
