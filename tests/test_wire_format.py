"""The serialized CompressedMatrixBlock format (systemds_b200/wire.py): round trips, streams assembled by hand from
the reference's write() methods, and the reference's exact-size formulas. No stream written by a JVM exists here,
so parity of this reader is unpinned beyond those three."""
import struct

import numpy as np
import pytest

from systemds_b200 import colgroup as cg
from systemds_b200 import datagen
from systemds_b200.wire import (WireFormatError, read_compressed_matrix_block, write_compressed_matrix_block)
from tests.util import dense_of, rel_err

ALL = datagen.KINDS + ("ddcfor", "sdcfor")


def same_group(a, b, nRows):
    assert type(a) is type(b)
    assert np.array_equal(a.getColIndices(), b.getColIndices())
    if isinstance(a, cg.ADictBasedColGroup):
        assert np.array_equal(a._dict, b._dict)
    if hasattr(a, "row_ids"):
        assert np.array_equal(a.row_ids(nRows), b.row_ids(nRows))
    for name in ("_defaultTuple", "_reference", "_ptr"):
        if getattr(a, name, None) is not None:
            assert np.array_equal(getattr(a, name), getattr(b, name))
    if isinstance(a, cg.ColGroupUncompressed):
        assert np.array_equal(a._data, b._data)
    if isinstance(a, cg.ASDC):
        assert (a._indexes.type, a._indexes.first, a._indexes.last, a._indexes.size) == \
               (b._indexes.type, b._indexes.first, b._indexes.last, b._indexes.size)
        if a._indexes.data is not None:
            assert np.array_equal(a._indexes.data, b._indexes.data)
    if getattr(a, "_data", None) is not None and hasattr(a._data, "type"):
        assert (a._data.type, a._data.size, a._data.unique) == (b._data.type, b._data.size, b._data.unique)


@pytest.mark.parametrize("nRows", [1, 40, 1000, 70001])
@pytest.mark.parametrize("overlap", [False, True])
def test_round_trip_every_group_class(nRows, overlap):
    cmb = datagen.random_cmb(900 + nRows, nRows, ALL, overlap)
    buf = write_compressed_matrix_block(cmb, nonZeros=123)
    back, nnz, used = read_compressed_matrix_block(buf + b"trailing")
    assert used == len(buf) and nnz == 123
    assert (back.rlen, back.clen, back.isOverlapping()) == (cmb.rlen, cmb.clen, cmb.isOverlapping())
    assert len(back.getColGroups()) == len(cmb.getColGroups())
    for a, b in zip(cmb.getColGroups(), back.getColGroups()):
        same_group(a, b, nRows)
    assert np.array_equal(dense_of(back), dense_of(cmb))
    assert write_compressed_matrix_block(back, 123) == buf


def be(fmt, *v):
    return struct.pack(">" + fmt, *v)


def test_hand_assembled_stream():
    """Every byte below is placed by the layout of the reference's write() methods, not by this library's writer."""
    n = 6
    s = be("iiq?", n, 7, 17, False) + be("i", 6)
    # DDC on column 0: SINGLE index, FP64 dictionary {1.5, -2}, MapToUByte
    s += be("b", 3) + be("bi", 0, 0) + be("bi2d", 0, 2, 1.5, -2.0) + be("bii6B", 2, 2, n, 0, 1, 1, 0, 1, 0)
    # SDCZeros on columns 1,2: TWO index, dictionary as a dense MatrixBlock [2 x 2], OffsetByte {1, 4}, MapToBit-free
    # map of two cells (MapToUByte, unique 2)
    s += be("b", 9) + be("bii", 1, 1, 2) + be("b", 1) + be("iib4d", 2, 2, 3, 1.0, 2.0, 3.0, 4.0)
    s += be("biiiiB", 0, 1, 1, 4, 2, 3) + be("bii2B", 2, 2, 2, 1, 0)
    # RLE on column 3: value 7.0 on rows [2, 5): ptr {0, 2}, data {2, 3}, zeros = true
    s += be("b", 1) + be("bi", 0, 3) + be("bid", 0, 1, 7.0) + be("iii", 2, 0, 2) + be("iHH", 2, 2, 3) + be("?", True)
    # Const on column 4 (value 0.25) and Empty on column 5
    s += be("b", 4) + be("bi", 0, 4) + be("bid", 0, 1, 0.25)
    s += be("b", 5) + be("bi", 0, 5)
    # Uncompressed on column 6: ultra-sparse MatrixBlock [6 x 1] with one non-zero, (row 3, 9.0)
    s += be("b", 0) + be("bi", 0, 6) + be("iib", n, 1, 1) + be("i", 1) + be("id", 3, 9.0)
    cmb, nnz, used = read_compressed_matrix_block(s)
    assert used == len(s) and nnz == 17
    want = np.zeros((n, 7))
    want[:, 0] = [1.5, -2, -2, 1.5, -2, 1.5]
    want[1, 1:3] = [3.0, 4.0]
    want[4, 1:3] = [1.0, 2.0]
    want[2:5, 3] = 7.0
    want[:, 4] = 0.25
    want[3, 6] = 9.0
    assert np.array_equal(dense_of(cmb), want)


def test_index_and_block_variants():
    n = 3
    # one DDC group over columns given as COMBINED(RANGE[4,6), TWORANGE(0,2 | 8,1)), MapToZero, sparse dictionary block
    idx = be("b", 5) + be("bii", 3, 4, 6) + be("biiii", 4, 0, 2, 8, 1)
    dict_sparse = be("b", 1) + be("iib", 1, 5, 2) + be("i", 2) + be("i", 2) + be("id", 1, 5.0) + be("id", 4, -1.0)
    s = be("iiq?", n, 9, -1, False) + be("i", 1) + be("b", 3) + idx + dict_sparse + be("bi", 0, n)
    cmb, _, used = read_compressed_matrix_block(s)
    assert used == len(s)
    g = cmb.getColGroups()[0]
    assert list(g.getColIndices()) == [4, 5, 0, 1, 8]
    want = np.zeros((n, 9))
    want[:, 5] = 5.0
    want[:, 8] = -1.0
    assert np.array_equal(dense_of(cmb), want)
    # ARRAY index with an uncompressed sparse block
    s = be("iiq?", 2, 4, -1, False) + be("i", 1) + be("b", 0) + be("bi3i", 2, 3, 0, 2, 3)
    s += be("iib", 2, 3, 2) + be("i", 2) + be("i", 1) + be("id", 2, 8.0) + be("i", 1) + be("id", 0, 6.0)
    cmb, _, _ = read_compressed_matrix_block(s)
    assert np.array_equal(dense_of(cmb), np.array([[0, 0, 0, 8.0], [6.0, 0, 0, 0]]))


def exact_size_on_disk(g, nRows):
    """getExactSizeOnDisk of each class, restated from the reference (AColGroup.java:214-221 = 1 + index;
    Dictionary.java:379-381; Map*.getExactSizeOnDisk; Offset*.getExactSizeOnDisk; AColGroupOffset.java:129-137)."""
    c = g.getNumCols()
    cols = g.getColIndices()
    idx = 5 if c == 1 else 9 if (c == 2 or np.array_equal(cols, np.arange(cols[0], cols[0] + c))) else 5 + 4 * c
    size = 1 + idx
    if isinstance(g, cg.ColGroupEmpty):
        return size
    if isinstance(g, cg.ColGroupUncompressed):
        return None  # depends on the block format chosen; covered by the round trip
    size += 1 + 4 + 8 * g._dict.size

    def map_size(m):
        return {0: 1 + 4, 1: 1 + 4 + 4 + 8 * (0 if m.data is None else len(m.data))}.get(
            m.type, 1 + 4 + 4 + m.size * {2: 1, 3: 1, 4: 2, 5: 3, 6: 4}.get(m.type, 0))

    def off_size(f):
        if f.type == 0:
            return 1
        if f.type == 1:
            return 1 + 4
        if f.type == 2:
            return 1 + 8
        if f.type == 3:
            return 1 + 12 + len(f.data) + (0 if (f.no_zero or f.no_over_half) else 4)
        return 1 + 12 + 2 * len(f.data)

    if isinstance(g, cg.ColGroupDDC):
        size += map_size(g._data) + (8 * c if isinstance(g, cg.ColGroupDDCFOR) else 0)
    elif isinstance(g, cg.AColGroupOffset):
        size += 4 + 4 * len(g._ptr) + 4 + 2 * len(g._data) + 1
    elif isinstance(g, cg.ASDC):
        size += off_size(g._indexes)
        if g._data is not None:
            size += map_size(g._data)
        if g._defaultTuple is not None or isinstance(g, cg.ColGroupSDCFOR):
            size += 8 * c
    return size


def test_sizes_match_reference_formulas():
    nRows = 5000
    cmb = datagen.random_cmb(77, nRows, tuple(k for k in ALL if k != "unc"))
    total = 4 + 4 + 8 + 1 + 4
    for g in cmb.getColGroups():
        total += exact_size_on_disk(g, nRows)
    assert len(write_compressed_matrix_block(cmb)) == total


def test_errors():
    cmb = datagen.random_cmb(5, 100, ("ddc", "sdc", "rle"))
    buf = write_compressed_matrix_block(cmb)
    for cut in (3, 20, len(buf) - 1):
        with pytest.raises(WireFormatError):
            read_compressed_matrix_block(buf[:cut])
    bad = bytearray(buf)
    bad[21] = 12  # group type DDCLZW: outside the supported classes
    with pytest.raises(WireFormatError):
        read_compressed_matrix_block(bytes(bad))
    bad[21] = 99
    with pytest.raises(WireFormatError):
        read_compressed_matrix_block(bytes(bad))


def test_corrupted_streams_are_refused_not_crashed_on():
    """Mutated streams (flipped bytes, truncations, overwritten length fields): both readers either accept the
    stream or refuse it with their error type; neither crashes, hangs or allocates without bound."""
    from systemds_b200 import native
    from systemds_b200.native import ptr
    L = native.lib()
    rng = np.random.default_rng(0)
    for it in range(400):
        cmb = datagen.random_cmb(it % 37, int(rng.choice([1, 5, 40, 300])), tuple(rng.choice(ALL, size=int(rng.integers(1, 6)))))
        b = bytearray(cmb.write())
        if it % 3 == 0:
            for _ in range(int(rng.integers(1, 4))):
                b[int(rng.integers(0, len(b)))] = int(rng.integers(0, 256))
        elif it % 3 == 1:
            b = b[:int(rng.integers(0, len(b)))]
        else:
            i = int(rng.integers(0, max(1, len(b) - 4)))
            b[i:i + 4] = int(rng.integers(0, 2 ** 32)).to_bytes(4, "big")
        raw = np.frombuffer(bytes(b) + b"\0", dtype=np.uint8)
        h = L.cla_read_block(ptr(raw), len(b), None, None)
        assert h > 0 or h in (-2, -3, -4, -7)  # bad argument / unsupported / shape / no memory
        if h > 0:
            assert L.cla_destroy(h) == 0
        try:
            read_compressed_matrix_block(bytes(b))
        except ValueError:  # WireFormatError, or a group constructor's own check
            pass


def test_native_reader_parses_without_a_gpu():
    """cla_read_block registers the groups of a stream (no device work before cla_finalize)."""
    import ctypes as C
    from systemds_b200 import native
    from systemds_b200.native import ptr
    L = native.lib()
    cmb = datagen.random_cmb(3, 1000, ALL)
    buf = np.frombuffer(cmb.write(55) + b"xyz", dtype=np.uint8)
    nnz, used = C.c_int64(), C.c_int64()
    h = L.cla_read_block(ptr(buf), len(buf), C.byref(nnz), C.byref(used))
    assert h > 0 and nnz.value == 55 and used.value == len(buf) - 3
    st = native.cla_stats()
    assert L.cla_stats_get(h, C.byref(st)) == 0
    n_for = sum(isinstance(g, (cg.ColGroupDDCFOR, cg.ColGroupSDCFOR)) for g in cmb.getColGroups())
    assert (st.n_rows, st.n_cols, st.n_groups) == (1000, cmb.clen, len(cmb.getColGroups()) + n_for)
    assert L.cla_destroy(h) == 0
    assert L.cla_read_block(ptr(buf), 40, None, None) == -2        # truncated: CLA_ERR_BAD_ARG
    bad = buf.copy()
    bad[21] = 13                                                     # DeltaDDC
    assert L.cla_read_block(ptr(bad), len(bad), None, None) == -3  # CLA_ERR_UNSUPPORTED
    assert L.cla_read_block(None, 10, None, None) == -2


@pytest.mark.gpu
@pytest.mark.parametrize("nRows", [40, 5000, 70001])
def test_native_reader_products_on_gpu(nRows):
    """A block ingested from its byte stream by the native reader gives the same bits as the same block
    registered group by group."""
    from systemds_b200 import CompressedMatrixBlock
    from systemds_b200.cmb import CLALibDecompress, CLALibLeftMultBy, CLALibRightMultBy
    cmb = datagen.random_cmb(40 + nRows, nRows, ALL)
    fromBytes = CompressedMatrixBlock.read_to_device(cmb.write())
    assert fromBytes.getColGroups() == [] and (fromBytes.rlen, fromBytes.clen) == (cmb.rlen, cmb.clen)
    cmb.to_device()
    assert np.array_equal(CLALibDecompress.decompress(fromBytes), CLALibDecompress.decompress(cmb))
    assert rel_err(CLALibDecompress.decompress(fromBytes), dense_of(cmb)) < 1e-14  # default + (dict - default) rounds once
    rng = np.random.default_rng(nRows)
    V = rng.standard_normal((cmb.clen, 9))
    assert np.array_equal(CLALibRightMultBy.rightMultByMatrix(fromBytes, V), CLALibRightMultBy.rightMultByMatrix(cmb, V))
    y = rng.standard_normal((1, nRows))
    a, b = CLALibLeftMultBy.leftMultByMatrix(fromBytes, y), CLALibLeftMultBy.leftMultByMatrix(cmb, y)
    assert np.allclose(a, b, rtol=1e-12, atol=1e-12 * np.abs(y).sum())
    for gi in range(len(cmb.getColGroups())):
        assert np.array_equal(fromBytes.group_row_ids(cmb._reg_index[gi]), cmb.group_row_ids(gi))
    fromBytes.free()
    cmb.free()
