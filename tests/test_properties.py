"""Property tests (hypothesis) of the index-structure encoders: the host-side factories and the oracle's C
restatement must produce the same arrays for any sorted row list, and decoding must give the list back. The gap
distributions are chosen to reach the continuation codes (255 / 65535), the byte-versus-char choice and the
65535-row segment boundaries of OLE / run-length limits of RLE."""
import numpy as np
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from systemds_b200 import offset
from systemds_b200.colgroup import ColGroupOLE, ColGroupRLE

SET = dict(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture, HealthCheck.too_slow])

gaps = st.one_of(st.integers(1, 3), st.integers(1, 300), st.sampled_from([254, 255, 256, 509, 510, 511, 65534, 65535, 65536,
                                                                           131070, 131071]), st.integers(1, 200000))


@st.composite
def sorted_rows(draw, min_size=1, max_size=400):
    first = draw(st.integers(0, 70000))
    g = draw(st.lists(gaps, min_size=min_size - 1 if min_size > 0 else 0, max_size=max_size))
    return np.cumsum([first] + g).astype(np.int64)


@given(rows=sorted_rows())
@settings(**SET)
def test_offsets_host_equals_oracle_and_round_trip(oracle, rows):
    t, first, last, data, _ = oracle.offset_create(rows)
    assert oracle.offset_decode(t, first, last, data).tolist() == rows.tolist()
    o = offset.OffsetFactory.createOffset(rows)
    assert (o.type, o.first, o.last) == (t, first, last)
    assert (o.data is None) == (data is None)
    if data is not None:
        assert np.array_equal(o.data, data)
    assert np.array_equal(o.decode(), rows)
    assert o.size == len(rows)


@st.composite
def runs_rows(draw):
    """Rows of one value: a few runs (some longer than 65535, some after gaps longer than 65535)."""
    pos, out = draw(st.integers(0, 70000)), []
    for _ in range(draw(st.integers(1, 6))):
        length = draw(st.one_of(st.integers(1, 40), st.sampled_from([65534, 65535, 65536, 70000])))
        out.append(np.arange(pos, pos + length))
        pos += length + draw(st.one_of(st.integers(1, 50), st.sampled_from([65535, 65536, 140000])))
    return np.concatenate(out).astype(np.int64)


@given(rows=runs_rows())
@settings(**SET)
def test_rle_host_equals_oracle_and_decodes(oracle, rows):
    enc = ColGroupRLE.genRLEBitmap(rows)
    assert np.array_equal(enc, oracle.rle_gen_bitmap(rows))
    assert len(enc) % 2 == 0
    pos, got = 0, []
    for gap, length in zip(enc[0::2].astype(np.int64), enc[1::2].astype(np.int64)):  # ColGroupRLE.java:114-117
        pos += gap
        got.append(np.arange(pos, pos + length))
        pos += length
    assert np.array_equal(np.concatenate(got), rows)


@given(rows=sorted_rows(max_size=200))
@settings(**SET)
def test_ole_host_equals_oracle_and_decodes(oracle, rows):
    enc = ColGroupOLE.genOffsetBitmap(rows)
    assert np.array_equal(enc, oracle.ole_gen_offset_bitmap(rows))
    seg, i, got = 0, 0, []
    while i < len(enc):  # [n, o_1 .. o_n] per 65535-row segment (ColGroupOLE.java:558-599)
        n = int(enc[i])
        got.extend(seg * 65535 + enc[i + 1:i + 1 + n].astype(np.int64))
        i += n + 1
        seg += 1
    assert got == rows.tolist()
