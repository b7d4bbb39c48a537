"""Column groups of a CompressedMatrixBlock, as immutable host records.

Mirrors ``runtime/compress/colgroup``: the classes keep the reference's names and field
meaning (``_colIndexes``, ``_dict``, ``_data``, ``_indexes``, ``_defaultTuple``, ``_ptr``)
and hold the arrays in the layout the JVM holds them, which is what the native boundary
receives. Nothing here computes products; that happens on the device.

* ColGroupDDC            ColGroupDDC.java:79-89     one map cell per row
* ColGroupSDC            ColGroupSDC.java:67-99     offsets of non-default rows + map over them + default tuple
* ColGroupSDCZeros       ColGroupSDCZeros.java:75-92  same with an all-zero default
* ColGroupSDCSingle      ColGroupSDCSingle.java:83-105  offsets only, one non-default tuple, default tuple
* ColGroupSDCSingleZeros ColGroupSDCSingleZeros.java:82-93
* ColGroupRLE / OLE      AColGroupOffset.java:39-55  ``_ptr[nVals+1]`` into u16 ``_data``
* ColGroupUncompressed   ColGroupUncompressed.java:84  dense block [nRows x gCols]
* ColGroupConst / Empty  ColGroupConst.java, ColGroupEmpty.java
"""
from __future__ import annotations

import numpy as np

from .mapping import AMapToData, MapToFactory
from .offset import AOffset, OffsetFactory

BITMAP_BLOCK_SZ = 65535  # CompressionSettings.java:46
CM = 65535


def _cols(colIndexes) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(colIndexes, dtype=np.int32).reshape(-1))


def _dict(values, nCols: int) -> np.ndarray:
    d = np.ascontiguousarray(np.asarray(values, dtype=np.float64)).reshape(-1, nCols)
    return d


class AColGroup:
    def __init__(self, colIndexes):
        self._colIndexes = _cols(colIndexes)

    def getNumCols(self) -> int:
        return int(self._colIndexes.shape[0])

    def getColIndices(self) -> np.ndarray:
        return self._colIndexes

    def getNumValues(self) -> int:
        return 0

    def getCompType(self) -> str:
        return type(self).__name__.replace("ColGroup", "")

    def index_bytes(self) -> int:
        """Bytes of index structure + dictionary (what one pass over the group must read)."""
        return 0


class ADictBasedColGroup(AColGroup):
    def __init__(self, colIndexes, dict_):
        super().__init__(colIndexes)
        self._dict = _dict(dict_, self.getNumCols())  # [nVals x gCols] row-major (Dictionary.java:94-97)

    def getNumValues(self) -> int:
        return int(self._dict.shape[0])


class ColGroupDDC(ADictBasedColGroup):
    def __init__(self, colIndexes, dict_, data: AMapToData):
        super().__init__(colIndexes, dict_)
        self._data = data
        if data.unique > max(self.getNumValues(), 1):
            # ColGroupDDC.java:90-103 (debug invariant)
            raise ValueError("Invalid construction of DDC group: map has more unique values than the dictionary")

    def row_ids(self, nRows: int) -> np.ndarray:
        return self._data.decode()

    def index_bytes(self) -> int:
        return self._data.nbytes() + self._dict.nbytes


class ColGroupDDCFOR(ColGroupDDC):
    """Frame-of-reference DDC: value = dict[id] + reference (ColGroupDDCFOR.java:62-75). For the products it is
    ``ColGroupDDC(dict) + 1 * reference^T``: ``extractCommon`` (:385-389) moves the reference into constV."""

    def __init__(self, colIndexes, dict_, reference, data: AMapToData):
        super().__init__(colIndexes, dict_, data)
        self._reference = np.ascontiguousarray(np.asarray(reference, dtype=np.float64).reshape(-1))
        if self._reference.shape[0] != self.getNumCols():
            raise ValueError("reference tuple must have one value per column")


class ASDC(ADictBasedColGroup):
    """Common state of the four SDC variants (ASDC.java:42-52, ASDCZero.java)."""

    def __init__(self, colIndexes, numRows: int, dict_, indexes: AOffset, data: AMapToData | None,
                 defaultTuple=None):
        super().__init__(colIndexes, dict_)
        self._numRows = int(numRows)
        self._indexes = indexes
        self._data = data  # None for the Single variants
        self._defaultTuple = None if defaultTuple is None else np.ascontiguousarray(
            np.asarray(defaultTuple, dtype=np.float64).reshape(-1))
        if data is not None and data.size != indexes.size:
            raise ValueError("Invalid SDC group: map size differs from the number of offsets")

    def row_ids(self, nRows: int) -> np.ndarray:
        ids = np.full(nRows, -1, np.int32)
        rows = self._indexes.decode()
        ids[rows] = 0 if self._data is None else self._data.decode()
        return ids

    def index_bytes(self) -> int:
        n = self._indexes.nbytes() + self._dict.nbytes
        return n + (0 if self._data is None else self._data.nbytes())


class ColGroupSDC(ASDC):
    def __init__(self, colIndexes, numRows, dict_, defaultTuple, indexes, data):
        super().__init__(colIndexes, numRows, dict_, indexes, data, defaultTuple)

    @staticmethod
    def create(colIndexes, numRows, dict_, defaultTuple, indexes, data):
        """Routes an all-zero default to ColGroupSDCZeros (ColGroupSDC.java:101-117)."""
        dt = np.asarray(defaultTuple, dtype=np.float64)
        if not np.any(dt != 0):
            return ColGroupSDCZeros(colIndexes, numRows, dict_, indexes, data)
        return ColGroupSDC(colIndexes, numRows, dict_, dt, indexes, data)


class ColGroupSDCFOR(ASDC):
    """Frame-of-reference SDC: listed rows hold dict[id] + reference, all other rows the reference
    (ColGroupSDCFOR.java:80-87,162-163); = ``ColGroupSDCZeros(dict) + 1 * reference^T`` for the products."""

    def __init__(self, colIndexes, numRows, dict_, indexes, data, reference):
        super().__init__(colIndexes, numRows, dict_, indexes, data, None)
        self._reference = np.ascontiguousarray(np.asarray(reference, dtype=np.float64).reshape(-1))


class ColGroupSDCZeros(ASDC):
    def __init__(self, colIndexes, numRows, dict_, indexes, data):
        super().__init__(colIndexes, numRows, dict_, indexes, data, None)


class ColGroupSDCSingle(ASDC):
    def __init__(self, colIndexes, numRows, dict_, defaultTuple, indexes):
        super().__init__(colIndexes, numRows, dict_, indexes, None, defaultTuple)


class ColGroupSDCSingleZeros(ASDC):
    def __init__(self, colIndexes, numRows, dict_, indexes):
        super().__init__(colIndexes, numRows, dict_, indexes, None, None)


class AColGroupOffset(ADictBasedColGroup):
    def __init__(self, colIndexes, numRows, zeros, dict_, data, ptr):
        super().__init__(colIndexes, dict_)
        self._numRows = int(numRows)
        self._zeros = bool(zeros)
        self._data = np.ascontiguousarray(np.asarray(data, dtype=np.uint16))
        self._ptr = np.ascontiguousarray(np.asarray(ptr, dtype=np.int32))
        if self._ptr.shape[0] != self.getNumValues() + 1:
            raise ValueError("Invalid offset group: _ptr must have nVals + 1 entries")

    def index_bytes(self) -> int:
        return self._data.nbytes + self._ptr.nbytes + self._dict.nbytes


class ColGroupRLE(AColGroupOffset):
    @staticmethod
    def genRLEBitmap(offsets) -> np.ndarray:
        """``(gap, len)`` u16 pairs of one value's sorted row list (ColGroupRLE.java:1073-1157).

        A gap above 65535 is written as ``(65535, 0)`` filler pairs; a run is closed once it
        holds 65535 rows and continues as a new run with gap 0.
        """
        off = np.asarray(offsets, dtype=np.int64)
        if off.size == 0:
            return np.zeros(0, np.uint16)
        brk = np.flatnonzero(np.diff(off) != 1) + 1
        starts = off[np.concatenate([[0], brk])]
        ends = off[np.concatenate([brk - 1, [off.size - 1]])] + 1
        lens = ends - starts
        # split runs longer than 65535 into full pieces and a tail
        pieces = (lens + CM - 1) // CM
        rep = np.repeat(np.arange(starts.size), pieces)
        within = np.arange(rep.size) - np.repeat(np.cumsum(pieces) - pieces, pieces)
        s2 = starts[rep] + within * CM
        l2 = np.minimum(lens[rep] - within * CM, CM)
        prev_end = np.concatenate([[0], (s2 + l2)[:-1]])
        gaps = s2 - prev_end
        fill = np.maximum(gaps - 1, 0) // CM  # number of (65535, 0) pairs before the run
        total = int(np.sum(fill) + s2.size)
        out = np.zeros((total, 2), np.uint16)
        out[:, 0] = CM  # fillers by default
        pos = np.cumsum(fill + 1) - 1  # slot of each real run
        out[pos, 0] = (gaps - fill * CM).astype(np.uint16)
        out[pos, 1] = l2.astype(np.uint16)
        return out.reshape(-1)

    @staticmethod
    def from_runs(colIndexes, dict_, starts, lens, vals, numRows) -> "ColGroupRLE":
        """Encode runs given as (first row, length, tuple id), sorted by first row and not overlapping, without
        materialising one id per row: per value, ``(gap, len)`` pairs under the encoder's rules
        (ColGroupRLE.java:1073-1157: gaps above 65535 become ``(65535, 0)`` fillers, runs are cut at 65535 rows)."""
        starts = np.asarray(starts, dtype=np.int64)
        lens = np.asarray(lens, dtype=np.int64)
        vals = np.asarray(vals, dtype=np.int64)
        nVals = _dict(dict_, len(_cols(colIndexes))).shape[0]
        chunks, ptr = [], [0]
        covered = int(lens.sum())
        for k in range(nVals):
            sel = np.flatnonzero((vals == k) & (lens > 0))
            st, ln = starts[sel], lens[sel]
            if st.size:
                # merge runs of this value that touch (the per-row encoder would see them as one run)
                touch = np.concatenate([[False], st[1:] == (st + ln)[:-1]])
                first = np.flatnonzero(~touch)
                ends = np.concatenate([(st + ln)[first[1:] - 1], [(st + ln)[-1]]])
                st, ln = st[first], ends - st[first]
                pieces = (ln + CM - 1) // CM
                rep = np.repeat(np.arange(st.size), pieces)
                within = np.arange(rep.size) - np.repeat(np.cumsum(pieces) - pieces, pieces)
                s2 = st[rep] + within * CM
                l2 = np.minimum(ln[rep] - within * CM, CM)
                prev_end = np.concatenate([[0], (s2 + l2)[:-1]])
                gaps = s2 - prev_end
                fill = np.maximum(gaps - 1, 0) // CM
                enc = np.zeros((int(np.sum(fill) + s2.size), 2), np.uint16)
                enc[:, 0] = CM
                pos = np.cumsum(fill + 1) - 1
                enc[pos, 0] = (gaps - fill * CM).astype(np.uint16)
                enc[pos, 1] = l2.astype(np.uint16)
                enc = enc.reshape(-1)
            else:
                enc = np.zeros(0, np.uint16)
            chunks.append(enc)
            ptr.append(ptr[-1] + enc.shape[0])
        data = np.concatenate(chunks) if chunks else np.zeros(0, np.uint16)
        return ColGroupRLE(colIndexes, int(numRows), covered < int(numRows), dict_, data, ptr)

    @staticmethod
    def from_row_ids(colIndexes, dict_, ids, numRows=None) -> "ColGroupRLE":
        """Encode per-row ids (-1 = no tuple, i.e. zero row) into the RLE group."""
        ids = np.asarray(ids)
        nRows = ids.shape[0] if numRows is None else numRows
        nVals = _dict(dict_, len(_cols(colIndexes))).shape[0]
        order = np.argsort(ids, kind="stable")
        sorted_ids = ids[order]
        bounds = np.searchsorted(sorted_ids, np.arange(nVals + 1))
        chunks, ptr = [], [0]
        for k in range(nVals):
            enc = ColGroupRLE.genRLEBitmap(order[bounds[k]:bounds[k + 1]])
            chunks.append(enc)
            ptr.append(ptr[-1] + enc.shape[0])
        data = np.concatenate(chunks) if chunks else np.zeros(0, np.uint16)
        zeros = bool(np.any(ids < 0))
        return ColGroupRLE(colIndexes, nRows, zeros, dict_, data, ptr)

    def row_ids(self, nRows: int) -> np.ndarray:
        ids = np.full(nRows, -1, np.int32)
        for k in range(self.getNumValues()):
            d = self._data[self._ptr[k]:self._ptr[k + 1]].astype(np.int64).reshape(-1, 2)
            ends = np.cumsum(d.sum(axis=1))
            starts = ends - d[:, 1]
            for s, e in zip(starts[d[:, 1] > 0], ends[d[:, 1] > 0]):
                ids[s:e] = k
        return ids


class ColGroupOLE(AColGroupOffset):
    @staticmethod
    def genOffsetBitmap(offsets) -> np.ndarray:
        """Segments ``[n, o_1..o_n]`` per 65535-row window (ColGroupOLE.java:558-599)."""
        off = np.asarray(offsets, dtype=np.int64)
        if off.size == 0:
            return np.zeros(0, np.uint16)
        seg = off // BITMAP_BLOCK_SZ
        nblk = int(seg[-1]) + 1
        cnt = np.bincount(seg, minlength=nblk)
        out = np.zeros(nblk + off.size, np.uint16)
        hdr = np.arange(nblk) + np.concatenate([[0], np.cumsum(cnt)[:-1]])
        out[hdr] = cnt.astype(np.uint16)
        out[np.arange(off.size) + seg + 1] = (off % BITMAP_BLOCK_SZ).astype(np.uint16)
        return out

    @staticmethod
    def from_row_ids(colIndexes, dict_, ids, numRows=None) -> "ColGroupOLE":
        ids = np.asarray(ids)
        nRows = ids.shape[0] if numRows is None else numRows
        nVals = _dict(dict_, len(_cols(colIndexes))).shape[0]
        order = np.argsort(ids, kind="stable")
        sorted_ids = ids[order]
        bounds = np.searchsorted(sorted_ids, np.arange(nVals + 1))
        chunks, ptr = [], [0]
        for k in range(nVals):
            enc = ColGroupOLE.genOffsetBitmap(order[bounds[k]:bounds[k + 1]])
            chunks.append(enc)
            ptr.append(ptr[-1] + enc.shape[0])
        data = np.concatenate(chunks) if chunks else np.zeros(0, np.uint16)
        return ColGroupOLE(colIndexes, nRows, bool(np.any(ids < 0)), dict_, data, ptr)

    def row_ids(self, nRows: int) -> np.ndarray:
        ids = np.full(nRows, -1, np.int32)
        for k in range(self.getNumValues()):
            d = self._data[self._ptr[k]:self._ptr[k + 1]].astype(np.int64)
            bix, seg = 0, 0
            while bix < d.shape[0]:
                n = int(d[bix])
                ids[seg * BITMAP_BLOCK_SZ + d[bix + 1:bix + 1 + n]] = k
                bix += n + 1
                seg += 1
        return ids


class ColGroupUncompressed(AColGroup):
    def __init__(self, colIndexes, data):
        super().__init__(colIndexes)
        self._data = np.ascontiguousarray(np.asarray(data, dtype=np.float64)).reshape(-1, self.getNumCols())

    def index_bytes(self) -> int:
        return self._data.nbytes


class ColGroupUncompressedDev(AColGroup):
    """An uncompressed group whose dense ``[nRows x gCols]`` block already lives in device memory (``dptr``; ``owner``
    keeps it alive). Registered with ``cla_add_group_uncompressed_dev``."""

    def __init__(self, colIndexes, numRows: int, dptr: int, owner=None):
        super().__init__(colIndexes)
        self._numRows = int(numRows)
        self.dptr = int(dptr)
        self.owner = owner

    def index_bytes(self) -> int:
        return self._numRows * self.getNumCols() * 8


class ColGroupConst(ADictBasedColGroup):
    def __init__(self, colIndexes, values):
        super().__init__(colIndexes, values)
        if self._dict.shape[0] != 1:
            raise ValueError("ColGroupConst holds exactly one tuple")


class ColGroupEmpty(AColGroup):
    pass


def sdc_from_row_ids(colIndexes, dict_, ids, defaultTuple=None):
    """Build the SDC variant the reference factories would (ids < 0 = default rows)."""
    ids = np.asarray(ids)
    nRows = ids.shape[0]
    rows = np.flatnonzero(ids >= 0)
    off = OffsetFactory.createOffset(rows)
    d = _dict(dict_, len(_cols(colIndexes)))
    zero_default = defaultTuple is None or not np.any(np.asarray(defaultTuple) != 0)
    if d.shape[0] == 1:
        if zero_default:
            return ColGroupSDCSingleZeros(colIndexes, nRows, d, off)
        return ColGroupSDCSingle(colIndexes, nRows, d, defaultTuple, off)
    m = MapToFactory.create_from(ids[rows], d.shape[0])
    if zero_default:
        return ColGroupSDCZeros(colIndexes, nRows, d, off, m)
    return ColGroupSDC(colIndexes, nRows, d, defaultTuple, off, m)
