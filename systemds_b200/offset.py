"""Delta-coded sorted row lists, as ``runtime/compress/colgroup/offset`` holds them.

``OffsetFactory.createOffset`` (OffsetFactory.java:105-149) picks Empty / Single / Two /
Byte / Char; the byte form stores gaps as u8 with ``0`` meaning "+255 and continue"
(OffsetByte.java:201-213), the char form does the same with u16 and 65535
(OffsetChar.java:172-180). The encoders here are vectorised restatements of
``createByte`` (:238-283) and ``createChar`` (:296-338): a gap ``g`` becomes
``g // maxV`` continuation zeros and ``g % maxV``, except that a multiple of ``maxV``
is written as one fewer zero followed by ``maxV`` itself.
"""
from __future__ import annotations

import numpy as np

OFF_EMPTY, OFF_SINGLE, OFF_TWO, OFF_BYTE, OFF_CHAR = range(5)
OFF_NAMES = ["EMPTY", "SINGLE", "TWO", "BYTE", "CHAR"]
BYTE_MAXV = 255
CHAR_MAXV = 65535


def _byte_array_cost(n: int) -> float:  # utils/MemoryEstimates.java:68-84
    size = 8 + 20
    if n <= 4:
        return size + 4
    size += n
    diff = (n - 4) % 8
    return size + (8 - diff if diff > 0 else 0)


def _char_array_cost(n: int) -> float:  # utils/MemoryEstimates.java:92-105
    size = 8 + 20
    if n <= 2:
        return size + 4
    size += 2 * n
    diff = (2 * n - 4) % 8
    return size + (8 - diff if diff > 0 else 0)


class AOffset:
    def __init__(self, otype: int, first: int, last: int, size: int, data=None, no_zero=False, no_over_half=False):
        self.type = int(otype)
        self.first = int(first)  # offsetToFirst
        self.last = int(last)  # offsetToLast
        self.size = int(size)  # number of rows listed
        self.data = data  # uint8 / uint16 deltas (None for Empty/Single/Two)
        self.no_zero = bool(no_zero)  # OffsetByteNZ / OffsetChar noZero flavour
        self.no_over_half = bool(no_over_half)  # OffsetByteUNZ flavour

    def getOffsetToFirst(self):
        return self.first

    def getOffsetToLast(self):
        return self.last

    def getSize(self):
        return self.size

    def decode(self) -> np.ndarray:
        """All listed rows, in order (what walking the reference iterator yields)."""
        if self.type == OFF_EMPTY:
            return np.zeros(0, np.int32)
        if self.type == OFF_SINGLE:
            return np.array([self.first], np.int32)
        if self.type == OFF_TWO:
            return np.array([self.first, self.last], np.int32)
        maxv = BYTE_MAXV if self.type == OFF_BYTE else CHAR_MAXV
        d = self.data.astype(np.int64)
        inc = np.where(d == 0, maxv, d)
        pos = self.first + np.cumsum(inc)
        rows = pos[d != 0]
        return np.concatenate([[self.first], rows]).astype(np.int32)

    def nbytes(self) -> int:
        return 0 if self.data is None else self.data.nbytes

    def __repr__(self):
        return f"Offset{OFF_NAMES[self.type]}(first={self.first}, last={self.last}, size={self.size})"


class OffsetFactory:
    @staticmethod
    def _encode(gaps: np.ndarray, maxv: int, dtype):
        div = gaps // maxv
        mod = gaps % maxv
        lens = np.where(mod == 0, div, div + 1)
        end = np.cumsum(lens)
        out = np.zeros(int(end[-1]) if end.size else 0, dtype)
        out[end - 1] = np.where(mod == 0, maxv, mod).astype(dtype)
        return out

    @staticmethod
    def createOffset(indexes) -> AOffset:
        idx = np.asarray(indexes, dtype=np.int64)
        n = int(idx.shape[0])
        if n == 0:
            return AOffset(OFF_EMPTY, 0, 0, 0)
        if idx[0] < 0:
            raise ValueError("Invalid negative offset")
        first, last = int(idx[0]), int(idx[-1])
        if n == 1:
            return AOffset(OFF_SINGLE, first, last, 1)
        if n == 2:
            return AOffset(OFF_TWO, first, last, 2)
        gaps = np.diff(idx)
        if np.any(gaps <= 0):
            raise ValueError("Invalid input to create offset, all values should be continuously increasing")
        end_length = n - 1
        rng = last - first
        corr_b = max(rng - end_length * 256, 0) // 256  # OffsetFactory.java:228-234
        corr_c = max(rng - end_length * 65535, 0) // 65535
        byte_size = int(16 + 4 + 4 + 4 + 8 + _byte_array_cost(end_length + corr_b))  # OffsetByte.java:100-104
        char_size = int(16 + 4 + 4 + 8 + _char_array_cost(end_length + corr_c))  # OffsetChar.java:88-92
        if byte_size < char_size:
            data = OffsetFactory._encode(gaps, BYTE_MAXV, np.uint8)
            no_zero = data.shape[0] == end_length
            no_over_half = bool(np.all(data.view(np.int8) >= 1))
            return AOffset(OFF_BYTE, first, last, n, data, no_zero, no_over_half)
        data = OffsetFactory._encode(gaps, CHAR_MAXV, np.uint16)
        return AOffset(OFF_CHAR, first, last, n, data, data.shape[0] == end_length)
