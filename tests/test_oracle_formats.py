"""Pins the CPU oracle's index-structure formats against the reference's own golden vectors."""
import numpy as np
import pytest

from systemds_b200 import mapping, offset
from systemds_b200.colgroup import ColGroupOLE, ColGroupRLE


def test_ole_golden(oracle, golden):
    for case in golden["ole_gen_offset_bitmap"]["cases"]:
        got = oracle.ole_gen_offset_bitmap(case["offsets"])
        if case["expected"] is None:
            assert got is None
        else:
            assert got.tolist() == case["expected"]
            assert ColGroupOLE.genOffsetBitmap(case["offsets"]).tolist() == case["expected"]


def test_rle_boundaries(oracle, golden):
    for case in golden["rle_boundaries"]["cases"]:
        rows = np.arange(case["start"], case["start"] + case["len"])
        assert oracle.rle_gen_bitmap(rows).tolist() == case["expected"]
        assert ColGroupRLE.genRLEBitmap(rows).tolist() == case["expected"]


def test_offset_round_trip_golden(oracle, golden):
    for lst in golden["offset_round_trip"]["lists"]:
        t, first, last, data, flags = oracle.offset_create(lst)
        rows = oracle.offset_decode(t, first, last, data)
        assert rows.tolist() == lst
        if lst:
            assert last == lst[-1] and first == lst[0]
        # the host-side encoder must produce the identical stream
        o = offset.OffsetFactory.createOffset(lst)
        assert o.type == t and o.first == first and o.last == last and o.size == len(lst)
        if data is None:
            assert o.data is None
        else:
            assert o.data.dtype == data.dtype and o.data.tolist() == data.tolist()
            assert o.no_zero == bool(flags & 1)
        assert o.decode().tolist() == lst


def test_offset_byte_edge_encodings(oracle):
    # gap of exactly 255 is one byte 0xFF; 256 = one continuation zero then 1; 510 = zero then 0xFF
    head = list(range(30))  # enough small gaps that the byte form is the smaller one
    for gap, enc in [(255, [255]), (256, [0, 1]), (510, [0, 255]), (511, [0, 0, 1]), (765, [0, 0, 255])]:
        lst = head + [29 + gap, 29 + gap + 45]
        exp = [1] * 29 + enc + [45]
        t, first, last, data, _ = oracle.offset_create(lst)
        assert t == offset.OFF_BYTE and data.tolist() == exp
        assert offset.OffsetFactory.createOffset(lst).data.tolist() == exp
        assert oracle.offset_decode(t, first, last, data).tolist() == lst


def test_offset_slice_golden(oracle, golden):
    g = golden["offset_slice"]
    t, first, last, data, _ = oracle.offset_create(g["list"])
    rows = oracle.offset_decode(t, first, last, data)
    sl = rows[(rows >= g["lo"]) & (rows < g["hi"])] - g["lo"]
    assert sl.tolist() == g["expected"]


def test_offset_random_round_trip(oracle):
    rng = np.random.default_rng(5)
    for n, span in [(50, 300), (400, 100000), (3000, 4000), (2000, 70_000_000), (10, 2_000_000)]:
        lst = np.sort(rng.choice(span, size=n, replace=False))
        t, first, last, data, _ = oracle.offset_create(lst)
        assert oracle.offset_decode(t, first, last, data).tolist() == lst.tolist()
        o = offset.OffsetFactory.createOffset(lst)
        assert o.type == t and (o.data is None) == (data is None)
        if data is not None:
            assert np.array_equal(o.data, data)
        assert np.array_equal(o.decode(), lst)


def test_binary_map_golden(oracle, golden):
    data = np.array(golden["binary_map"]["data"])
    m = mapping.MapToFactory.create_from(data, 2)
    assert m.type == mapping.MAP_BIT  # 142 cells > 32
    assert oracle.map_decode(m.type, m.data, None, m.size).tolist() == data.tolist()
    assert m.decode().tolist() == data.tolist()
    assert [m.getIndex(i) for i in range(m.size)] == data.tolist()
    assert m.getCounts().tolist() == [int((data == 0).sum()), int((data == 1).sum())]


def test_map_type_thresholds(oracle, golden):
    for size, unique, expected in golden["map_type_thresholds"]["cases"]:
        assert oracle.map_type_for(size, unique) == expected
        assert mapping.MapToFactory.type_for(size, unique) == expected


@pytest.mark.parametrize("unique", [1, 2, 3, 128, 129, 256, 257, 70000])
def test_map_decode_all_types(oracle, unique):
    rng = np.random.default_rng(unique)
    ids = rng.integers(0, unique, size=1000)
    m = mapping.MapToFactory.create_from(ids, unique)
    assert oracle.map_decode(m.type, m.data, m.data2, m.size).tolist() == ids.tolist()
    assert m.decode().tolist() == ids.tolist()
    # every wider map type must reproduce the narrow one (MappingTestUtil.getAllHigherVersions)
    for t in range(m.type + 1, 7):
        if t == mapping.MAP_BIT and unique > 2:
            continue
        if t == mapping.MAP_UBYTE and unique > 128:
            continue
        w = mapping.MapToFactory.create_from(ids, unique, force_type=t)
        assert oracle.map_decode(w.type, w.data, w.data2, w.size).tolist() == ids.tolist()


def test_offset_preagg_golden(oracle, golden):
    """OffsetPreAggTests: pre-aggregation over a zero map equals the sum of the listed left cells."""
    from systemds_b200.cmb import CompressedMatrixBlock
    from systemds_b200.colgroup import ColGroupSDCZeros
    for case in golden["offset_preagg"]["cases"]:
        offs = case["offsets"]
        for t in [mapping.MAP_BIT, mapping.MAP_UBYTE, mapping.MAP_BYTE, mapping.MAP_CHAR, mapping.MAP_CHAR_BYTE,
                  mapping.MAP_INT]:
            m = mapping.MapToFactory.create_from(np.zeros(len(offs), np.int64), 2, force_type=t)
            g = ColGroupSDCZeros([0], 5, np.array([[1.0], [100.0]]), offset.OffsetFactory.createOffset(offs), m)
            om = oracle.OracleMatrix(CompressedMatrixBlock(5, 1, [g]), threads=1)
            assert om.lmm(np.array(case["left"], float).reshape(1, -1))[0, 0] == case["expected"]
