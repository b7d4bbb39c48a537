"""Serialized form of a ``CompressedMatrixBlock`` (the reference's ``write(DataOutput)`` / ``read(DataInput)``).

Big-endian ``DataOutput`` layout, field by field as the reference writes it:

* block  (runtime/compress/CompressedMatrixBlock.java:470-519): ``int rlen, int clen, long nonZeros,
  boolean overlapping``, then ``int nGroups`` and the groups (colgroup/ColGroupIO.java:48-139).
* group  (colgroup/AColGroup.java:207-212): ``byte ColGroupType.ordinal()`` (enum order AColGroup.java:89-92), the
  column index, then per class: dictionary groups add the dictionary (ADictBasedColGroup.java:225-228); DDC the map
  (ColGroupDDC.java:794-797); SDC offsets, map, default tuple (ColGroupSDC.java:446-452); SDCZeros offsets, map
  (ColGroupSDCZeros.java:645-649); SDCSingle offsets, default tuple (ColGroupSDCSingle.java:412-417);
  SDCSingleZeros offsets (ColGroupSDCSingleZeros.java:644-647); RLE / OLE ``int len, int[] ptr, int len, char[]
  data, boolean zeros`` (AColGroupOffset.java:115-127); DDCFOR / SDCFOR their reference tuple last
  (ColGroupDDCFOR.java:222-227, ColGroupSDCFOR.java:229-235); Uncompressed a ``MatrixBlock``
  (ColGroupUncompressed.java:657-660); Const only its dictionary; Empty nothing more.
* column index (colgroup/indexes/*.java, type byte = IColIndex.ColIndexType ordinal): SINGLE ``int``; TWO ``int,
  int``; ARRAY ``int n, int[n]``; RANGE ``int l, int u``; TWORANGE ``int l1, int n1, int l2, int n2``;
  COMBINED two nested indexes.
* dictionary (colgroup/dictionary/DictionaryFactory.java:54-77): FP64_DICT ``int n, double[n]``
  (Dictionary.java:361-376); MATRIX_BLOCK_DICT a ``MatrixBlock`` (MatrixBlockDictionary.java:1910-1919); IDENTITY
  ``int n`` (IdentityDictionary.java:382-389). The quantised, placeholder, identity-slice and delta dictionaries are
  not supported.
* map (colgroup/mapping/Map*.java ``write``; type byte = MAP_TYPE ordinal): ZERO ``int size``; BIT ``int size, int
  words, long[words]``; UBYTE / BYTE ``int unique, int n, byte[n]``; CHAR ``int unique, int n, char[n]``; CHAR_BYTE
  ``int unique, int n, char[n], byte[n]``; INT ``int unique, int n, int[n]``.
* offsets (colgroup/offset/Offset*.java ``write``; type byte = OFF_TYPE_SPECIALIZATIONS ordinal, OffsetFactory.java:
  46-52): BYTE ``int first, int n, int last, int size, byte[n]``; BYTENZ / BYTEUNZ ``int first, int n, int last,
  byte[n]``; CHAR ``int first, int n, int last, char[n]``; SINGLE ``int``; TWO ``int, int``; EMPTY nothing.
* ``MatrixBlock`` (runtime/matrix/data/MatrixBlock.java:2111-2165,2335-2370): ``int rlen, int clen, byte
  BlockType`` then EMPTY nothing; DENSE ``double[rlen*clen]``; SPARSE ``nnz`` (long if rlen*clen > Integer.MAX_VALUE
  else int) and per row ``int n, (int col, double v)[n]``; ULTRA_SPARSE ``int nnz`` and ``(int row, int col, double
  v)`` triples, or ``(int row, double v)`` pairs when clen == 1. The de-duplicated dense block is not supported.

No byte stream written by a JVM exists on this machine, so this module is checked by round trips, by streams
assembled by hand from the layout above, and by the reference's exact-size formulas (``getExactSizeOnDisk``).
"""
from __future__ import annotations

import struct

import numpy as np

from . import colgroup as cg
from .mapping import (AMapToData, MAP_BIT, MAP_BYTE, MAP_CHAR, MAP_CHAR_BYTE, MAP_INT, MAP_UBYTE, MAP_ZERO)
from .offset import AOffset, OFF_BYTE, OFF_CHAR, OFF_EMPTY, OFF_SINGLE, OFF_TWO

# ColGroupType ordinals (colgroup/AColGroup.java:89-92)
(GT_UNCOMPRESSED, GT_RLE, GT_OLE, GT_DDC, GT_CONST, GT_EMPTY, GT_SDC, GT_SDC_SINGLE, GT_SDC_SINGLE_ZEROS, GT_SDC_ZEROS,
 GT_SDCFOR, GT_DDCFOR, GT_DDCLZW, GT_DELTA_DDC, GT_LINEAR_FUNCTIONAL) = range(15)
# IColIndex.ColIndexType ordinals (colgroup/indexes/IColIndex.java:33-35)
IX_SINGLE, IX_TWO, IX_ARRAY, IX_RANGE, IX_TWORANGE, IX_COMBINED = range(6)
# DictionaryFactory.Type ordinals
(DT_FP64, DT_MATRIX_BLOCK, DT_INT8, DT_IDENTITY, DT_IDENTITY_SLICE, DT_PLACE_HOLDER, DT_DELTA) = range(7)
# OFF_TYPE_SPECIALIZATIONS ordinals
(OS_BYTE, OS_CHAR, OS_SINGLE, OS_TWO, OS_EMPTY, OS_BYTEUNZ, OS_BYTENZ) = range(7)
# Types.BlockType ordinals (common/Types.java:440-446)
(BT_EMPTY, BT_ULTRA_SPARSE, BT_SPARSE, BT_DENSE, BT_DEDUP) = range(5)
INT_MAX = 2147483647


class WireFormatError(ValueError):
    """The stream is truncated, holds an unknown type ordinal, or uses a class outside this library's scope."""


# ---------------------------------------------------------------------------------------------------------
# reading
# ---------------------------------------------------------------------------------------------------------
class _In:
    def __init__(self, buf):
        self.b = memoryview(buf).cast("B")
        self.p = 0

    def _take(self, n):
        if self.p + n > len(self.b):
            raise WireFormatError("stream ends inside a field (offset %d, need %d bytes)" % (self.p, n))
        v = self.b[self.p:self.p + n]
        self.p += n
        return v

    def byte(self):
        return self._take(1)[0]

    def boolean(self):
        return self._take(1)[0] != 0

    def int(self):
        return struct.unpack(">i", self._take(4))[0]

    def long(self):
        return struct.unpack(">q", self._take(8))[0]

    def array(self, dtype, n):
        if n < 0:
            raise WireFormatError("negative array length")
        dt = np.dtype(dtype)
        raw = self._take(n * dt.itemsize)
        return np.frombuffer(raw, dtype=dt.newbyteorder(">"), count=n).astype(dt.newbyteorder("="))


def _ordinal(v, n, what):
    if v >= n:
        raise WireFormatError("unknown %s ordinal %d" % (what, v))
    return v


def _read_col_index(s: _In) -> np.ndarray:
    t = _ordinal(s.byte(), 6, "column index type")
    if t == IX_SINGLE:
        return np.array([s.int()], np.int32)
    if t == IX_TWO:
        return np.array([s.int(), s.int()], np.int32)
    if t == IX_ARRAY:
        return s.array(np.int32, s.int())
    if t == IX_RANGE:
        lo, hi = s.int(), s.int()
        return np.arange(lo, hi, dtype=np.int32)
    if t == IX_TWORANGE:
        l1, n1, l2, n2 = s.int(), s.int(), s.int(), s.int()
        return np.concatenate([np.arange(l1, l1 + n1), np.arange(l2, l2 + n2)]).astype(np.int32)
    return np.concatenate([_read_col_index(s), _read_col_index(s)]).astype(np.int32)  # COMBINED: left then right


def read_matrix_block(s: _In) -> np.ndarray:
    """A ``MatrixBlock`` as a dense ``[rlen x clen]`` array (MatrixBlock.java:2111-2165)."""
    rlen, clen = s.int(), s.int()
    fmt = _ordinal(s.byte(), 5, "block format")
    # an empty block needs no bytes at all, every other format at least an eighth of a byte per cell would be odd:
    # refuse dimensions the rest of the stream cannot account for (a corrupted length must not allocate without bound)
    limit = (1 << 28) if fmt == BT_EMPTY else 64 * (len(s.b) - s.p) + 1024
    if rlen < 0 or clen < 0 or rlen * clen > limit:
        raise WireFormatError("block of %d x %d cells cannot come from the %d bytes left" % (rlen, clen, len(s.b) - s.p))
    out = np.zeros((rlen, clen), np.float64)
    if fmt == BT_EMPTY:
        return out
    if fmt == BT_DENSE:
        return s.array(np.float64, rlen * clen).reshape(rlen, clen)
    if fmt == BT_SPARSE:
        s.long() if rlen * clen > INT_MAX else s.int()  # nnz; the rows carry their own counts
        for r in range(rlen):
            n = s.int()
            if n:
                rec = np.frombuffer(s._take(12 * n), dtype=np.dtype([("c", ">i4"), ("v", ">f8")]), count=n)
                out[r, rec["c"].astype(np.int64)] = rec["v"]
        return out
    if fmt == BT_ULTRA_SPARSE:
        nnz = s.int()
        if clen > 1:
            rec = np.frombuffer(s._take(16 * nnz), dtype=np.dtype([("r", ">i4"), ("c", ">i4"), ("v", ">f8")]), count=nnz)
            out[rec["r"].astype(np.int64), rec["c"].astype(np.int64)] = rec["v"]
        else:
            rec = np.frombuffer(s._take(12 * nnz), dtype=np.dtype([("r", ">i4"), ("v", ">f8")]), count=nnz)
            out[rec["r"].astype(np.int64), 0] = rec["v"]
        return out
    raise WireFormatError("de-duplicated dense blocks are not supported")


def _read_dictionary(s: _In, gCols: int) -> np.ndarray:
    t = _ordinal(s.byte(), 7, "dictionary type")
    if t == DT_FP64:
        n = s.int()
        if n % gCols:
            raise WireFormatError("dictionary of %d values does not divide into %d columns" % (n, gCols))
        return s.array(np.float64, n).reshape(-1, gCols)
    if t == DT_MATRIX_BLOCK:
        m = read_matrix_block(s)
        if m.shape[1] != gCols:
            raise WireFormatError("matrix-block dictionary has %d columns, the group %d" % (m.shape[1], gCols))
        return m
    if t == DT_IDENTITY:
        n = s.int()
        if n != gCols:
            raise WireFormatError("identity dictionary of %d columns on a group of %d" % (n, gCols))
        return np.eye(n)
    raise WireFormatError("dictionary type ordinal %d is not supported" % t)


def _read_map(s: _In) -> AMapToData:
    t = _ordinal(s.byte(), 7, "map type")
    if t == MAP_ZERO:
        return AMapToData(MAP_ZERO, s.int(), 1)
    if t == MAP_BIT:
        size, words = s.int(), s.int()
        return AMapToData(MAP_BIT, size, 2, s.array(np.uint64, words))
    unique, n = s.int(), s.int()
    if t in (MAP_UBYTE, MAP_BYTE):
        return AMapToData(t, n, unique, s.array(np.uint8, n))
    if t == MAP_CHAR:
        return AMapToData(t, n, unique, s.array(np.uint16, n))
    if t == MAP_CHAR_BYTE:
        c = s.array(np.uint16, n)
        return AMapToData(t, n, unique, c, s.array(np.uint8, n))
    return AMapToData(MAP_INT, n, unique, s.array(np.int32, n))


def _read_offsets(s: _In) -> AOffset:
    t = _ordinal(s.byte(), 7, "offset type")
    if t == OS_EMPTY:
        return AOffset(OFF_EMPTY, 0, 0, 0)
    if t == OS_SINGLE:
        v = s.int()
        return AOffset(OFF_SINGLE, v, v, 1)
    if t == OS_TWO:
        a, b = s.int(), s.int()
        return AOffset(OFF_TWO, a, b, 2)
    first, n, last = s.int(), s.int(), s.int()
    if t == OS_BYTE:
        size = s.int()
        return AOffset(OFF_BYTE, first, last, size, s.array(np.uint8, n))
    if t in (OS_BYTENZ, OS_BYTEUNZ):
        return AOffset(OFF_BYTE, first, last, n + 1, s.array(np.uint8, n), no_zero=True, no_over_half=(t == OS_BYTEUNZ))
    d = s.array(np.uint16, n)
    nz = int(np.count_nonzero(d))
    return AOffset(OFF_CHAR, first, last, nz + 1, d, no_zero=(nz == n))


def _read_group(s: _In, nRows: int) -> cg.AColGroup:
    t = _ordinal(s.byte(), 15, "column group type")
    cols = _read_col_index(s)
    gc = len(cols)
    if t == GT_EMPTY:
        return cg.ColGroupEmpty(cols)
    if t == GT_UNCOMPRESSED:
        m = read_matrix_block(s)
        if m.shape != (nRows, gc):
            raise WireFormatError("uncompressed group of shape %s in a block of %d rows, %d columns" % (m.shape, nRows, gc))
        return cg.ColGroupUncompressed(cols, m)
    if t in (GT_DDCLZW, GT_DELTA_DDC, GT_LINEAR_FUNCTIONAL):
        raise WireFormatError("column group type ordinal %d is not supported" % t)
    d = _read_dictionary(s, gc)
    if t == GT_CONST:
        return cg.ColGroupConst(cols, d)
    if t == GT_DDC:
        return cg.ColGroupDDC(cols, d, _read_map(s))
    if t == GT_DDCFOR:
        m = _read_map(s)
        return cg.ColGroupDDCFOR(cols, d, s.array(np.float64, gc), m)
    if t in (GT_RLE, GT_OLE):
        ptr = s.array(np.int32, s.int())
        data = s.array(np.uint16, s.int())
        zeros = s.boolean()
        return (cg.ColGroupRLE if t == GT_RLE else cg.ColGroupOLE)(cols, nRows, zeros, d, data, ptr)
    off = _read_offsets(s)
    if t == GT_SDC:
        m = _read_map(s)
        return cg.ColGroupSDC(cols, nRows, d, s.array(np.float64, gc), off, m)
    if t == GT_SDC_ZEROS:
        return cg.ColGroupSDCZeros(cols, nRows, d, off, _read_map(s))
    if t == GT_SDC_SINGLE:
        return cg.ColGroupSDCSingle(cols, nRows, d, s.array(np.float64, gc), off)
    if t == GT_SDC_SINGLE_ZEROS:
        return cg.ColGroupSDCSingleZeros(cols, nRows, d, off)
    m = _read_map(s)  # SDCFOR
    return cg.ColGroupSDCFOR(cols, nRows, d, off, m, s.array(np.float64, gc))


def read_compressed_matrix_block(buf):
    """``CompressedMatrixBlock.read(DataInput)``: returns ``(block, nonZeros, bytesConsumed)``."""
    from .cmb import CompressedMatrixBlock
    s = _In(buf)
    rlen, clen, nnz, overlapping = s.int(), s.int(), s.long(), s.boolean()
    n = s.int()
    if rlen < 0 or clen < 0 or n < 0:
        raise WireFormatError("negative dimension in the block header")
    groups = [_read_group(s, rlen) for _ in range(n)]
    return CompressedMatrixBlock(rlen, clen, groups, overlapping), nnz, s.p


# ---------------------------------------------------------------------------------------------------------
# writing
# ---------------------------------------------------------------------------------------------------------
class _Out:
    def __init__(self):
        self.parts = []

    def byte(self, v):
        self.parts.append(struct.pack(">B", v & 0xFF))

    def boolean(self, v):
        self.parts.append(b"\x01" if v else b"\x00")

    def int(self, v):
        self.parts.append(struct.pack(">i", int(v)))

    def long(self, v):
        self.parts.append(struct.pack(">q", int(v)))

    def array(self, a, dtype):
        self.parts.append(np.ascontiguousarray(a).astype(np.dtype(dtype).newbyteorder(">")).tobytes())

    def bytes(self):
        return b"".join(self.parts)


def _write_col_index(o: _Out, cols: np.ndarray):
    """The index class ``ColIndexFactory.create(int[])`` picks (ColIndexFactory.java:62-73)."""
    n = len(cols)
    if n == 1:
        o.byte(IX_SINGLE), o.int(cols[0])
    elif n == 2:
        o.byte(IX_TWO), o.int(cols[0]), o.int(cols[1])
    elif np.array_equal(cols, np.arange(cols[0], cols[0] + n)):
        o.byte(IX_RANGE), o.int(cols[0]), o.int(cols[0] + n)
    else:
        o.byte(IX_ARRAY), o.int(n), o.array(cols, np.int32)


def write_matrix_block(o: _Out, m: np.ndarray):
    """``MatrixBlock.write`` of a block held dense in memory (MatrixBlock.java:2335-2370): the on-disk format
    follows ``evalSparseFormatOnDisk`` (:1362-1372) and ``isUltraSparseSerialize`` (:1209-1211)."""
    rlen, clen = m.shape
    o.int(rlen), o.int(clen)
    nnz = int(np.count_nonzero(m))
    if nnz == 0:
        o.byte(BT_EMPTY)
        return
    header = 9
    size_dense = header + rlen * clen * 8
    size_sparse = header + (8 if rlen * clen > INT_MAX else 4) + rlen * 4 + nnz * 12
    size_ultra = header + 4 + nnz * 16
    sparse_dst = (nnz / rlen / clen < 0.4) and (size_sparse < size_dense or size_ultra < size_dense)
    if sparse_dst and nnz < rlen:
        o.byte(BT_ULTRA_SPARSE), o.int(nnz)
        r, c = np.nonzero(m)
        if clen > 1:
            rec = np.empty(nnz, dtype=np.dtype([("r", ">i4"), ("c", ">i4"), ("v", ">f8")]))
            rec["r"], rec["c"], rec["v"] = r, c, m[r, c]
        else:
            rec = np.empty(nnz, dtype=np.dtype([("r", ">i4"), ("v", ">f8")]))
            rec["r"], rec["v"] = r, m[r, 0]
        o.parts.append(rec.tobytes())
    elif sparse_dst:
        o.byte(BT_SPARSE)
        o.long(nnz) if rlen * clen > INT_MAX else o.int(nnz)
        for r in range(rlen):
            c = np.nonzero(m[r])[0]
            o.int(len(c))
            if len(c):
                rec = np.empty(len(c), dtype=np.dtype([("c", ">i4"), ("v", ">f8")]))
                rec["c"], rec["v"] = c, m[r, c]
                o.parts.append(rec.tobytes())
    else:
        o.byte(BT_DENSE), o.array(m.reshape(-1), np.float64)


def _write_dictionary(o: _Out, d: np.ndarray):
    o.byte(DT_FP64), o.int(d.size), o.array(d.reshape(-1), np.float64)


def _write_map(o: _Out, m: AMapToData):
    o.byte(m.type)
    if m.type == MAP_ZERO:
        o.int(m.size)
    elif m.type == MAP_BIT:
        o.int(m.size), o.int(len(m.data)), o.array(m.data, np.uint64)
    else:
        o.int(m.unique), o.int(len(m.data))
        o.array(m.data, {MAP_UBYTE: np.uint8, MAP_BYTE: np.uint8, MAP_CHAR: np.uint16, MAP_CHAR_BYTE: np.uint16,
                         MAP_INT: np.int32}[m.type])
        if m.type == MAP_CHAR_BYTE:
            o.array(m.data2, np.uint8)


def _write_offsets(o: _Out, f: AOffset):
    if f.type == OFF_EMPTY:
        o.byte(OS_EMPTY)
    elif f.type == OFF_SINGLE:
        o.byte(OS_SINGLE), o.int(f.first)
    elif f.type == OFF_TWO:
        o.byte(OS_TWO), o.int(f.first), o.int(f.last)
    elif f.type == OFF_BYTE:
        t = OS_BYTEUNZ if f.no_over_half else (OS_BYTENZ if f.no_zero else OS_BYTE)
        o.byte(t), o.int(f.first), o.int(len(f.data)), o.int(f.last)
        if t == OS_BYTE:
            o.int(f.size)
        o.array(f.data, np.uint8)
    else:
        o.byte(OS_CHAR), o.int(f.first), o.int(len(f.data)), o.int(f.last), o.array(f.data, np.uint16)


def _write_group(o: _Out, g: cg.AColGroup):
    def head(t):
        o.byte(t)
        _write_col_index(o, g.getColIndices())

    if isinstance(g, cg.ColGroupEmpty):
        head(GT_EMPTY)
    elif isinstance(g, cg.ColGroupUncompressed):
        head(GT_UNCOMPRESSED)
        write_matrix_block(o, g._data)
    elif isinstance(g, cg.ColGroupConst):
        head(GT_CONST), _write_dictionary(o, g._dict)
    elif isinstance(g, cg.ColGroupDDCFOR):
        head(GT_DDCFOR), _write_dictionary(o, g._dict), _write_map(o, g._data), o.array(g._reference, np.float64)
    elif isinstance(g, cg.ColGroupDDC):
        head(GT_DDC), _write_dictionary(o, g._dict), _write_map(o, g._data)
    elif isinstance(g, cg.AColGroupOffset):
        head(GT_RLE if isinstance(g, cg.ColGroupRLE) else GT_OLE)
        _write_dictionary(o, g._dict)
        o.int(len(g._ptr)), o.array(g._ptr, np.int32), o.int(len(g._data)), o.array(g._data, np.uint16)
        o.boolean(g._zeros)
    elif isinstance(g, cg.ColGroupSDCFOR):
        head(GT_SDCFOR), _write_dictionary(o, g._dict), _write_offsets(o, g._indexes), _write_map(o, g._data)
        o.array(g._reference, np.float64)
    elif isinstance(g, cg.ColGroupSDC):
        head(GT_SDC), _write_dictionary(o, g._dict), _write_offsets(o, g._indexes), _write_map(o, g._data)
        o.array(g._defaultTuple, np.float64)
    elif isinstance(g, cg.ColGroupSDCZeros):
        head(GT_SDC_ZEROS), _write_dictionary(o, g._dict), _write_offsets(o, g._indexes), _write_map(o, g._data)
    elif isinstance(g, cg.ColGroupSDCSingle):
        head(GT_SDC_SINGLE), _write_dictionary(o, g._dict), _write_offsets(o, g._indexes)
        o.array(g._defaultTuple, np.float64)
    elif isinstance(g, cg.ColGroupSDCSingleZeros):
        head(GT_SDC_SINGLE_ZEROS), _write_dictionary(o, g._dict), _write_offsets(o, g._indexes)
    else:
        raise WireFormatError("cannot serialize a group of class %s" % type(g).__name__)


def write_compressed_matrix_block(cmb, nonZeros: int = -1) -> bytes:
    """``CompressedMatrixBlock.write(DataOutput)`` without its "smaller when uncompressed" rewrite (:497-516),
    which changes the groups rather than the format."""
    o = _Out()
    o.int(cmb.getNumRows()), o.int(cmb.getNumColumns()), o.long(nonZeros), o.boolean(cmb.isOverlapping())
    groups = cmb.getColGroups()
    o.int(len(groups))
    for g in groups:
        _write_group(o, g)
    return o.bytes()
