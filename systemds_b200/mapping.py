"""Index maps (row -> dictionary id) in the reference's in-memory representations.

Mirrors ``runtime/compress/colgroup/mapping``: ``AMapToData`` and its seven storage
classes, plus ``MapToFactory.create`` (MapToFactory.java:102-117). Arrays are kept
exactly as the JVM holds them (native-endian), which is what crosses the JNI boundary:

* MapToBit      ``long[ceil(size/64)]``, bit ``r & 63`` of word ``r >> 6`` (MapToBit.java:100-103)
* MapToUByte    ``byte[size]`` with ids 0..127, no mask (MapToUByte.java:51-53)
* MapToByte     ``byte[size]``, id = ``b & 0xFF`` (MapToByte.java:67-69)
* MapToChar     ``char[size]`` (u16) (MapToChar.java:68-70)
* MapToCharPByte ``char[size]`` + ``byte[size]``, id = ``c + (b << 16)`` (MapToCharPByte.java:67-69)
* MapToInt      ``int[size]`` (MapToInt.java:63-65)
* MapToZero     size only (MapToZero.java:48)
"""
from __future__ import annotations

import numpy as np

MAP_ZERO, MAP_BIT, MAP_UBYTE, MAP_BYTE, MAP_CHAR, MAP_CHAR_BYTE, MAP_INT = range(7)
MAP_NAMES = ["ZERO", "BIT", "UBYTE", "BYTE", "CHAR", "CHAR_BYTE", "INT"]


class AMapToData:
    """A map of ``size`` cells holding ids below ``unique``."""

    def __init__(self, mtype: int, size: int, unique: int, data=None, data2=None):
        self.type = int(mtype)
        self.size = int(size)
        self.unique = int(unique)
        self.data = data  # primary array (None for MapToZero)
        self.data2 = data2  # the byte plane of MapToCharPByte

    # --- reference API ---------------------------------------------------------------------
    def getIndex(self, r: int) -> int:
        t = self.type
        if t == MAP_ZERO:
            return 0
        if t == MAP_BIT:
            return int((int(self.data[r >> 6]) >> (r & 63)) & 1)
        if t == MAP_CHAR_BYTE:
            return int(self.data[r]) + (int(self.data2[r]) << 16)
        return int(self.data[r])

    def getUnique(self) -> int:
        return self.unique

    def decode(self) -> np.ndarray:
        """All ids as int32 (host-side helper; the device has its own decode kernels)."""
        t = self.type
        if t == MAP_ZERO:
            return np.zeros(self.size, np.int32)
        if t == MAP_BIT:
            b = np.unpackbits(self.data.view(np.uint8), bitorder="little")[: self.size]
            return b.astype(np.int32)
        if t == MAP_CHAR_BYTE:
            return self.data.astype(np.int32) + (self.data2.astype(np.int32) << 16)
        return self.data.astype(np.int32)

    def getCounts(self) -> np.ndarray:
        """Histogram of ids (MapToByte.java:168-188, MapToBit.java:195-201, MapToChar.java:242)."""
        return np.bincount(self.decode(), minlength=max(self.unique, 1)).astype(np.int64)

    def slice(self, rl: int, ru: int) -> "AMapToData":
        """Cells [rl, ru) as a map of the same type (AMapToData.slice)."""
        ids = self.decode()[rl:ru]
        return MapToFactory.create_from(ids, self.unique, force_type=self.type)

    def nbytes(self) -> int:
        n = 0 if self.data is None else self.data.nbytes
        return n + (0 if self.data2 is None else self.data2.nbytes)

    def __repr__(self):
        return f"MapTo{MAP_NAMES[self.type]}(size={self.size}, unique={self.unique})"


class DeviceMap(AMapToData):
    """A map whose cells already live in device memory, in the same storage layout (MapToBit words, bytes, u16 or
    i32). ``dptr`` is the device address, ``owner`` whatever keeps that memory alive (a tensor). Registered with
    ``cla_add_group_ddc_dev``; the native library copies it device to device when the block is finalized."""

    def __init__(self, mtype: int, size: int, unique: int, dptr: int, nbytes: int, owner=None):
        super().__init__(mtype, size, unique)
        if mtype not in (MAP_BIT, MAP_UBYTE, MAP_BYTE, MAP_CHAR, MAP_INT):
            raise ValueError("device-resident maps: MapToBit, MapToUByte, MapToByte, MapToChar or MapToInt")
        self.dptr = int(dptr)
        self._nbytes = int(nbytes)
        self.owner = owner

    def decode(self):
        raise RuntimeError("a device-resident map has no host copy; decode it through cla_group_decode")

    def nbytes(self) -> int:
        return self._nbytes


class MapToFactory:
    @staticmethod
    def type_for(size: int, unique: int) -> int:
        """MapToFactory.create's thresholds (MapToFactory.java:102-117)."""
        if unique <= 1:
            return MAP_ZERO
        if unique == 2 and size > 32:
            return MAP_BIT
        if unique <= 128:
            return MAP_UBYTE
        if unique <= 256:
            return MAP_BYTE
        if unique <= 65536:
            return MAP_CHAR
        if unique <= 8388608:
            return MAP_CHAR_BYTE
        return MAP_INT

    @staticmethod
    def create_from(ids, unique: int, force_type: int | None = None) -> AMapToData:
        """Build the map the factory would pick for ``unique`` ids and fill it from ``ids``."""
        ids = np.asarray(ids)
        size = int(ids.shape[0])
        t = MapToFactory.type_for(size, unique) if force_type is None else int(force_type)
        if t == MAP_ZERO:
            return AMapToData(t, size, unique)
        if t == MAP_BIT:
            packed = np.packbits(ids.astype(np.uint8), bitorder="little")
            words = np.zeros((size + 63) // 64 * 8, np.uint8)
            words[: packed.shape[0]] = packed
            return AMapToData(t, size, unique, words.view(np.uint64))
        if t in (MAP_UBYTE, MAP_BYTE):
            return AMapToData(t, size, unique, np.ascontiguousarray(ids.astype(np.uint8)))
        if t == MAP_CHAR:
            return AMapToData(t, size, unique, np.ascontiguousarray(ids.astype(np.uint16)))
        if t == MAP_CHAR_BYTE:
            i32 = ids.astype(np.int32)
            return AMapToData(t, size, unique, np.ascontiguousarray((i32 & 0xFFFF).astype(np.uint16)),
                              np.ascontiguousarray((i32 >> 16).astype(np.uint8)))
        return AMapToData(t, size, unique, np.ascontiguousarray(ids.astype(np.int32)))

    @staticmethod
    def wrap(mtype: int, size: int, unique: int, data, data2=None) -> AMapToData:
        """Adopt arrays that already are in the reference representation (no copy)."""
        return AMapToData(mtype, size, unique, data, data2)
