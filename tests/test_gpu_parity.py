"""GPU parity: every product and every decoded index structure through the C ABI against the CPU oracle."""
import numpy as np
import pytest

from systemds_b200 import CLAError, CompressedMatrixBlock, datagen
from systemds_b200 import colgroup as cg
from systemds_b200.cmb import (CHAIN_XtwXv, CLALibDecompress, CLALibLeftMultBy, CLALibMatrixMult, CLALibMMChain, CLALibRightMultBy,
                               CLALibTSMM)
from systemds_b200.mapping import MapToFactory
from tests.util import TOL, abs_dense_of, dense_of, rel_err

pytestmark = pytest.mark.gpu

CASES = [
    ("all", datagen.KINDS, False),
    ("for", ("ddcfor", "sdcfor", "ddc", "sdcfor", "rle", "ddcfor"), False),
    ("ddc_only", ("ddc", "ddc", "ddc2", "ddc_bit", "ddc_char"), False),
    ("ddc_u8", ("ddc", "ddc", "ddc2", "ddc_bit", "const"), False),
    ("sparse", ("sdc", "sdcz", "sdcs", "sdcsz", "const", "empty"), False),
    ("runs", ("rle", "rle", "ole", "ddc"), False),
    ("overlap", ("ddc", "sdc", "rle", "ddc2", "const", "sdcz"), True),
]


def seed_of(name, n):
    return sum(map(ord, name)) + n


@pytest.mark.parametrize("name,kinds,overlap", CASES)
@pytest.mark.parametrize("nRows", [1, 37, 1024, 5000, 70001])
def test_decode_bit_exact(oracle, name, kinds, overlap, nRows):
    """Decoded maps, offsets, run boundaries and counts are bit-exact (device decode kernels vs oracle vs host)."""
    cmb = datagen.random_cmb(seed_of(name, nRows), nRows, kinds, overlap).to_device()
    om = oracle.OracleMatrix(cmb)
    for gi, g in enumerate(cmb.getColGroups()):
        want = om.group_row_ids(gi)
        got = cmb.group_row_ids(gi)
        assert np.array_equal(got, want), f"group {gi} ({type(g).__name__}) decodes differently"
        if hasattr(g, "row_ids"):
            assert np.array_equal(got, g.row_ids(nRows))
        if g.getNumValues() and not isinstance(g, cg.ColGroupConst):
            assert np.array_equal(cmb.group_counts(gi), om.group_counts(gi))
    cmb.free()


@pytest.mark.parametrize("name,kinds,overlap", CASES)
@pytest.mark.parametrize("nRows", [1, 37, 1024, 5000, 70001])
def test_products_vs_oracle(oracle, name, kinds, overlap, nRows):
    cmb = datagen.random_cmb(seed_of(name, nRows), nRows, kinds, overlap).to_device()
    X = dense_of(cmb)
    aX = np.abs(X)
    om = oracle.OracleMatrix(cmb)
    rng = np.random.default_rng(nRows)
    assert rel_err(CLALibDecompress.decompress(cmb), om.decompress()) < 1e-14
    for vc in (1, 5, 13, 64, 70):
        V = rng.standard_normal((cmb.clen, vc))
        got = CLALibRightMultBy.rightMultByMatrix(cmb, V)
        assert got.shape == (nRows, vc)
        assert rel_err(got, om.rmm(V), aX @ np.abs(V) + 1e-300) < TOL
        assert got.nnz == int(np.count_nonzero(got))
    for q in (1, 6):
        Yt = rng.standard_normal((q, nRows))
        got = CLALibLeftMultBy.leftMultByMatrix(cmb, Yt)
        assert rel_err(got, om.lmm(Yt), np.abs(Yt) @ aX + 1e-300) < TOL
    got = CLALibTSMM.leftMultByTransposeSelf(cmb)
    if not overlap:
        sc = aX.T @ aX + 1e-300
        # within TOL of the exact product; the reference's own row-by-row summation (and so the oracle's)
        # drifts by up to n * eps / 2 on columns with a constant part, hence the looser oracle bound
        assert rel_err(got, oracle.dense_tsmm_ld(X), sc) < TOL
        assert rel_err(got, om.tsmm(), sc) < TOL + nRows * 1.2e-16
    else:
        # overlapping block (lib/CLALibTSMM.java:130-133 runs it single-threaded on the decompressed sum): a cell is a
        # sum over groups, so the error is measured against the magnitude of the summed parts
        aP = abs_dense_of(cmb)
        assert rel_err(got, oracle.dense_tsmm_ld(X), aP.T @ aP + 1e-300) < TOL
    assert np.array_equal(got, got.T)
    v = rng.standard_normal(cmb.clen)
    w = rng.standard_normal(nRows)
    s = aX.T @ (aX @ np.abs(v)) + 1e-300
    assert rel_err(CLALibMMChain.mmChain(cmb, v).ravel(), om.mmchain(v).ravel(), s) < 10 * TOL
    sw = aX.T @ (np.abs(w) * (aX @ np.abs(v))) + 1e-300
    assert rel_err(CLALibMMChain.mmChain(cmb, v, w, CHAIN_XtwXv).ravel(), om.mmchain(v, w, 1).ravel(), sw) < 10 * TOL
    cmb.free()


def _ddc_matrix(nRows, cards, seed, const_col=False, pair=False):
    rng = np.random.default_rng(seed)
    groups, c = [], 0
    for k in cards:
        w = 2 if (pair and c % 3 == 0) else 1
        groups.append(cg.ColGroupDDC(list(range(c, c + w)), rng.standard_normal((k, w)),
                                     MapToFactory.create_from(rng.integers(0, k, nRows), k)))
        c += w
    if const_col:
        groups.append(cg.ColGroupConst([c], [[0.75]]))
        c += 1
    return CompressedMatrixBlock(nRows, c, groups)


@pytest.mark.parametrize("nRows", [4096, 70001, 262144 + 17])
@pytest.mark.parametrize("shape", ["card16", "card256", "mixed", "mixed_const_pairs"])
def test_fast_vector_paths(oracle, nRows, shape):
    """The specialised DDC kernels (X v, t(y) X, t(X)(X v)) on the shapes of the headline workloads."""
    rng = np.random.default_rng(nRows)
    if shape == "card16":
        cmb = _ddc_matrix(nRows, [16] * 100, 1)
    elif shape == "card256":
        cmb = _ddc_matrix(nRows, [256] * 200, 2)
    elif shape == "mixed":
        cmb = _ddc_matrix(nRows, list(rng.integers(2, 256, 150)) + [2, 2, 255, 129], 3)
    else:
        cmb = _ddc_matrix(nRows, list(rng.integers(2, 256, 70)), 4, const_col=True, pair=True)
    cmb.to_device()
    om = oracle.OracleMatrix(cmb)
    X = dense_of(cmb)
    aX = np.abs(X)
    v = rng.standard_normal(cmb.clen)
    y = rng.standard_normal((1, nRows))
    assert rel_err(CLALibRightMultBy.rightMultByMatrix(cmb, v), om.rmm(v), aX @ np.abs(v).reshape(-1, 1) + 1e-300) < TOL
    assert rel_err(CLALibLeftMultBy.leftMultByMatrix(cmb, y), om.lmm(y), np.abs(y) @ aX + 1e-300) < TOL
    s = aX.T @ (aX @ np.abs(v)) + 1e-300
    assert rel_err(CLALibMMChain.mmChain(cmb, v).ravel(), om.mmchain(v).ravel(), s) < 10 * TOL
    # a few vectors at once: served by the same kernels; left rows go four, two and one at a time (7 = 4 + 2 + 1)
    V = rng.standard_normal((cmb.clen, 4))
    Y = rng.standard_normal((7, nRows))
    assert rel_err(CLALibRightMultBy.rightMultByMatrix(cmb, V), om.rmm(V), aX @ np.abs(V) + 1e-300) < TOL
    assert rel_err(CLALibLeftMultBy.leftMultByMatrix(cmb, Y), om.lmm(Y), np.abs(Y) @ aX + 1e-300) < TOL
    st = cmb.stats()
    assert st["kernel_launches"] > 0 and st["calls_rmm"] >= 2 and st["calls_lmm"] >= 2
    # decompress straight from the column-per-lane layout (every column a slot) or by the tile kernel (const column):
    # a cell is one dictionary value (plus the column constant), so both are exact (lib/CLALibDecompress.java:427-434)
    assert np.array_equal(np.array(CLALibDecompress.decompress(cmb)), X)
    cmb.free()


def test_products_repeat_bit_identical():
    """The vector kernels (specialised and general) and the tensor-core RMM form every output row's sum in a fixed
    order: a second call returns the same bits. (TSMM, the general left product and the constant-column row sum
    combine partial sums with atomics, as the reference's parallel paths do with tasks, and are checked to
    tolerance only.)"""
    cmb = _ddc_matrix(300001, [16] * 40 + [200] * 30, 9).to_device()
    rng = np.random.default_rng(3)
    v = rng.standard_normal(cmb.clen)
    V = rng.standard_normal((cmb.clen, 64))
    y = rng.standard_normal((1, 300001))
    for f in (lambda: CLALibRightMultBy.rightMultByMatrix(cmb, v), lambda: CLALibRightMultBy.rightMultByMatrix(cmb, V),
              lambda: CLALibLeftMultBy.leftMultByMatrix(cmb, y), lambda: CLALibMMChain.mmChain(cmb, v)):
        a = np.array(f())
        assert np.array_equal(a, np.array(f()))
    cmb.free()


@pytest.mark.parametrize("nRows", [50000, 70001])
def test_right_products_repeat_bit_identical_mixed_groups(nRows):
    """X %*% v and X %*% V on a block with SDC, RLE, uncompressed, constant and wide-map groups: the sparse groups'
    terms reach every output row in list order (staged per group in the vector kernel, queues sorted by table row
    in the tensor-core kernel), so repeated calls agree bit for bit, also when another handle's kernels share the
    GPU."""
    import threading
    cmb = datagen.random_cmb(99 + nRows, nRows, ("ddc", "sdc", "rle", "unc", "const", "ddc_char", "sdc", "rle")).to_device()
    other = _ddc_matrix(200001, [16] * 30 + [250] * 10, 21).to_device()
    rng = np.random.default_rng(5)
    v = rng.standard_normal(cmb.clen)
    V3 = rng.standard_normal((cmb.clen, 3))
    V16 = rng.standard_normal((cmb.clen, 16))
    vo = rng.standard_normal(other.clen)
    want = [np.array(CLALibRightMultBy.rightMultByMatrix(cmb, x)) for x in (v, V3, V16)]
    stop = []

    def noise():
        while not stop:
            CLALibMMChain.mmChain(other, vo)

    t = threading.Thread(target=noise)
    t.start()
    try:
        for _ in range(5):
            for x, w in zip((v, V3, V16), want):
                got = np.array(CLALibRightMultBy.rightMultByMatrix(cmb, x))
                dev = float(np.max(np.abs(got - w)) / (np.max(np.abs(w)) + 1e-300))
                assert np.array_equal(got, w), f"repeat differs, max deviation {dev:.3e} of the largest entry"
    finally:
        stop.append(1)
        t.join()
    cmb.free()
    other.free()


def test_tsmm_integer_exact(oracle):
    """Integer-valued dictionaries: the self product is exact (CLALibMMChainTest.java:159-171 asks for 0 ULP)."""
    cmb = datagen.random_cmb(11, 3000, ("ddc", "ddc2", "sdcz", "rle", "ddc_bit"), integer=True).to_device()
    X = dense_of(cmb)
    assert np.array_equal(CLALibTSMM.leftMultByTransposeSelf(cmb), X.T @ X)
    cmb.free()


@pytest.mark.parametrize("kinds", [("ddc",) * 9, ("ddc", "ddc2", "ddcfor", "ddc2", "ddc"), ("ddc_char", "ddc_char", "ddc_char")])
def test_tsmm_compact_records(oracle, kinds):
    """t(X) X on blocks of dense-map groups of one map width: the kernel's compact column records (single-column
    groups; co-coded groups and constant parts; 16-bit maps)."""
    for nRows in (33, 70001):
        cmb = datagen.random_cmb(321 + nRows, nRows, kinds).to_device()
        X = dense_of(cmb)
        got = CLALibTSMM.leftMultByTransposeSelf(cmb)
        assert rel_err(got, oracle.dense_tsmm_ld(X), np.abs(X).T @ np.abs(X) + 1e-300) < TOL
        assert np.array_equal(got, got.T)
        cmb.free()


def test_tsmm_wide(oracle):
    """More than one 64-column block, ragged edge."""
    cmb = _ddc_matrix(9000, [7] * 150, 5).to_device()
    X = dense_of(cmb)
    got = CLALibTSMM.leftMultByTransposeSelf(cmb)
    assert rel_err(got, oracle.dense_tsmm_ld(X), np.abs(X).T @ np.abs(X)) < TOL
    cmb.free()


def test_empty_and_errors():
    e = datagen.random_cmb(1, 0, ("ddc", "sdcz")).to_device()
    assert CLALibRightMultBy.rightMultByMatrix(e, np.ones((2, 3))).shape == (0, 3)
    assert np.array_equal(CLALibLeftMultBy.leftMultByMatrix(e, np.zeros((2, 0))), np.zeros((2, 2)))
    assert np.array_equal(CLALibTSMM.leftMultByTransposeSelf(e), np.zeros((2, 2)))
    e.free()
    cmb = datagen.random_cmb(2, 100, ("ddc", "sdcz")).to_device()
    with pytest.raises(CLAError) as ex:
        CLALibRightMultBy.rightMultByMatrix(cmb, np.ones((3, 1)))
    assert ex.value.code == -4
    with pytest.raises(CLAError):
        CLALibLeftMultBy.leftMultByMatrix(cmb, np.ones((1, 99)))
    cmb.free()
    with pytest.raises(RuntimeError):
        cmb.handle()


def test_full_size_checksum_config2(oracle):
    """Full-size t(y) %*% X (10M x 200): with y = 1 the product equals counts . dictionary, a checksum built
    from the bit-exact device histograms; linearity ties a random y to it."""
    cmb, y = datagen.config2(nRows=10_000_000, nCols=200)
    cmb.to_device()
    ones = np.ones((1, cmb.rlen))
    got = CLALibLeftMultBy.leftMultByMatrix(cmb, ones).ravel()
    want = np.array([float(cmb.group_counts(g).astype(np.float64) @ cmb.getColGroups()[g]._dict[:, 0]) for g in range(200)])
    scale = np.array([float(cmb.group_counts(g).astype(np.float64) @ np.abs(cmb.getColGroups()[g]._dict[:, 0])) for g in range(200)])
    assert rel_err(got, want, scale) < TOL
    a = CLALibLeftMultBy.leftMultByMatrix(cmb, y).ravel()
    b = CLALibLeftMultBy.leftMultByMatrix(cmb, 2.0 * y + ones).ravel()
    assert rel_err(b, 2.0 * a + got, 2 * np.sqrt(cmb.rlen) + scale) < 1e-11
    # sampled rows of X %*% v against the host records
    v = np.random.default_rng(0).standard_normal(200)
    u = CLALibRightMultBy.rightMultByMatrix(cmb, v).ravel()
    rows = np.random.default_rng(1).integers(0, cmb.rlen, 50)
    for r in rows:
        ref = sum(g._dict[g._data.getIndex(int(r)), 0] * v[c] for c, g in enumerate(cmb.getColGroups()))
        assert abs(u[r] - ref) <= 1e-12 * 200 * 4
    cmb.free()


def test_pageable_operands_through_the_pinned_ring():
    """Host operands in ordinary (pageable) memory, as a JVM heap array is, are moved through the handle's pinned
    ring by host threads; pinned operands take plain asynchronous copies. Both must give the same bits: t(y) %*% X
    (upload of y in slices, the product of a row range starting when its last slice is queued), X %*% v (download of
    the result) and decompress (a download of many ring rounds)."""
    import torch
    nRows = (1 << 20) + 777
    cmb = _ddc_matrix(nRows, [256] * 24, 11)
    cmb.to_device()
    rng = np.random.default_rng(5)
    y = rng.standard_normal((1, nRows))                       # pageable
    y_pin = torch.from_numpy(y.copy()).pin_memory().numpy()   # pinned
    a = np.array(CLALibLeftMultBy.leftMultByMatrix(cmb, y))
    b = np.array(CLALibLeftMultBy.leftMultByMatrix(cmb, y_pin))
    assert np.array_equal(a, b)
    X = dense_of(cmb)
    assert rel_err(a, y @ X, np.abs(y) @ np.abs(X) + 1e-300) < TOL
    v = rng.standard_normal(cmb.clen)
    u = np.array(CLALibRightMultBy.rightMultByMatrix(cmb, v)).ravel()    # 8 MB result into a pageable array
    assert rel_err(u, X @ v, np.abs(X) @ np.abs(v) + 1e-300) < TOL
    assert np.array_equal(np.array(CLALibRightMultBy.rightMultByMatrix(cmb, v)).ravel(), u)
    assert np.array_equal(np.array(CLALibDecompress.decompress(cmb)), X)  # 200 MB: the ring is reused many times
    cmb.free()


def test_benchmark_shapes_against_oracle(oracle):
    """The five benchmark configurations at sizes the oracle finishes in seconds, each through its own operation."""
    # configs[0] at full size: X %*% v, 1M x 100, 16 values per column
    cmb, v = datagen.config1()
    om = oracle.OracleMatrix(cmb.to_device())
    got, want = CLALibRightMultBy.rightMultByMatrix(cmb, v), om.rmm(v)
    assert rel_err(got, want, np.abs(want) + np.sqrt(100.0)) < TOL
    cmb.free()
    # configs[1] at 300k rows: t(y) %*% X, 256 values per column; variant b holds two-column dictionaries
    for variant in ("a", "b"):
        cmb, y = datagen.config2(nRows=300_000, variant=variant)
        om = oracle.OracleMatrix(cmb.to_device())
        y = y.reshape(1, -1)
        got, want = CLALibLeftMultBy.leftMultByMatrix(cmb, y), om.lmm(y)
        assert rel_err(got, want, np.abs(want) + np.sqrt(cmb.rlen)) < TOL
        cmb.free()
    # configs[2] at 60k rows: X %*% V with DDC / SDCZeros / RLE / uncompressed groups, V 500 x 64
    cmb, V = datagen.config3(nRows=60_000)
    om = oracle.OracleMatrix(cmb.to_device())
    got, want = CLALibRightMultBy.rightMultByMatrix(cmb, V), om.rmm(V)
    assert rel_err(got, want, np.abs(want) + np.sqrt(500.0)) < TOL
    cmb.free()
    # configs[3] at 200k rows: t(X) %*% X, 1000 values per column, Zipf ids, MapToChar
    cmb = datagen.config4(nRows=200_000).to_device()
    X = dense_of(cmb)
    got = CLALibTSMM.leftMultByTransposeSelf(cmb)
    assert rel_err(got, oracle.dense_tsmm_ld(X), np.abs(X).T @ np.abs(X)) < TOL
    assert np.array_equal(got, got.T)
    cmb.free()
    # configs[4] at 30k rows x 1000 columns: one lmCG step t(X)(Xv) with bit / ubyte / byte maps
    cmb, v = datagen.config5(nRows=30_000)
    om = oracle.OracleMatrix(cmb.to_device())
    aX = np.abs(dense_of(cmb))
    got, want = CLALibMMChain.mmChain(cmb, v).ravel(), om.mmchain(v).ravel()
    assert rel_err(got, want, aX.T @ (aX @ np.abs(v).ravel())) < 10 * TOL
    cmb.free()


@pytest.mark.parametrize("force", ["CHAR_BYTE", "INT", "BYTE", "CHAR"])
def test_wide_map_types(oracle, force):
    """MapToCharPByte / MapToInt (and forced wider storage of small ids, MappingTestUtil.getAllHigherVersions)."""
    from systemds_b200 import mapping
    rng = np.random.default_rng(9)
    nRows, card = 30000, {"CHAR_BYTE": 70000, "INT": 70000, "BYTE": 100, "CHAR": 100}[force]
    ids = rng.integers(0, card, nRows)
    ids[:3] = [0, card - 1, card // 2]
    m = mapping.MapToFactory.create_from(ids, card, force_type=getattr(mapping, "MAP_" + force))
    off_rows = np.sort(rng.choice(nRows, 2000, replace=False))
    from systemds_b200.offset import OffsetFactory
    ms = mapping.MapToFactory.create_from(rng.integers(0, card, 2000), card, force_type=getattr(mapping, "MAP_" + force))
    groups = [cg.ColGroupDDC([0], rng.standard_normal((card, 1)), m),
              cg.ColGroupSDCZeros([1], nRows, rng.standard_normal((card, 1)), OffsetFactory.createOffset(off_rows), ms)]
    cmb = CompressedMatrixBlock(nRows, 2, groups).to_device()
    om = oracle.OracleMatrix(cmb)
    for gi in range(2):
        assert np.array_equal(cmb.group_row_ids(gi), om.group_row_ids(gi))
        assert np.array_equal(cmb.group_counts(gi), om.group_counts(gi))
    X = dense_of(cmb)
    V = rng.standard_normal((2, 3))
    y = rng.standard_normal((2, nRows))
    assert rel_err(CLALibRightMultBy.rightMultByMatrix(cmb, V), om.rmm(V), np.abs(X) @ np.abs(V) + 1e-300) < TOL
    assert rel_err(CLALibLeftMultBy.leftMultByMatrix(cmb, y), om.lmm(y), np.abs(y) @ np.abs(X) + 1e-300) < TOL
    cmb.free()


def test_matrix_multiply_transposes(oracle):
    """CLALibMatrixMult.matrixMultiply: the four transpose combinations against numpy on the decompressed matrix."""
    from systemds_b200 import CLALibMatrixMult
    cmb = datagen.random_cmb(4, 3000, ("ddc", "sdc", "rle", "unc")).to_device()
    X = dense_of(cmb)
    rng = np.random.default_rng(2)
    A = rng.standard_normal((3, 3000))
    B = rng.standard_normal((cmb.clen, 4))
    assert rel_err(CLALibMatrixMult.matrixMultiply(cmb, B), X @ B, np.abs(X) @ np.abs(B)) < TOL
    assert rel_err(CLALibMatrixMult.matrixMultiply(cmb, B.T.copy(), False, True), X @ B, np.abs(X) @ np.abs(B)) < TOL
    assert rel_err(CLALibMatrixMult.matrixMultiply(A, cmb), A @ X, np.abs(A) @ np.abs(X)) < TOL
    assert rel_err(CLALibMatrixMult.matrixMultiply(A.T.copy(), cmb, True, False), A @ X, np.abs(A) @ np.abs(X)) < TOL
    assert rel_err(CLALibMatrixMult.matrixMultiply(cmb, A.T.copy(), True, False), X.T @ A.T, np.abs(X).T @ np.abs(A).T) < TOL
    assert rel_err(cmb.aggregateBinaryOperations(A, cmb), A @ X, np.abs(A) @ np.abs(X)) < TOL
    cmb.free()


def test_sharded_partials_add_up(oracle):
    """Two row shards as two handles on one GPU: partial t(Y)X, t(X)X and mmchain results sum to the full product."""
    from systemds_b200 import shard
    cmb = datagen.random_cmb(33, 20000, ("ddc", "ddc2", "sdc", "rle", "ole", "unc", "const", "sdcsz"))
    X = dense_of(cmb)
    aX = np.abs(X)
    rng = np.random.default_rng(1)
    y = rng.standard_normal((2, cmb.rlen))
    v = rng.standard_normal(cmb.clen)
    lmm = np.zeros((2, cmb.clen))
    tsmm = np.zeros((cmb.clen, cmb.clen))
    chain = np.zeros((cmb.clen, 1))
    for (a, b), s in zip(shard.shard_bounds(cmb.rlen, 2), shard.shard(cmb, 2)):
        s.to_device()
        lmm += CLALibLeftMultBy.leftMultByMatrix(s, y[:, a:b])
        tsmm += CLALibTSMM.leftMultByTransposeSelf(s)
        chain += CLALibMMChain.mmChain(s, v)
        s.free()
    assert rel_err(lmm, oracle.dense_lmm_ld(X, y), np.abs(y) @ aX) < TOL
    assert rel_err(tsmm, oracle.dense_tsmm_ld(X), aX.T @ aX) < TOL
    assert rel_err(chain.ravel(), X.T @ (X @ v), aX.T @ (aX @ np.abs(v))) < 10 * TOL


@pytest.mark.parametrize("nRows", [5000, 70001])
def test_mixed_fast_and_general(oracle, nRows):
    """Vector products on a mixed matrix: the specialised kernels take the byte-map DDC groups, the general
    kernels add the SDC / RLE / uncompressed / wide-map groups and the constant part exactly once."""
    kinds = ("ddc",) * 14 + ("ddc2",) * 3 + ("ddc_bit", "sdc", "sdcz", "rle", "ole", "unc", "const", "ddc_char", "sdcs")
    cmb = datagen.random_cmb(77 + nRows, nRows, kinds).to_device()
    om = oracle.OracleMatrix(cmb)
    X = dense_of(cmb)
    aX = np.abs(X)
    rng = np.random.default_rng(nRows)
    v = rng.standard_normal(cmb.clen)
    y = rng.standard_normal((1, nRows))
    w = rng.standard_normal(nRows)
    assert rel_err(CLALibRightMultBy.rightMultByMatrix(cmb, v), om.rmm(v), aX @ np.abs(v).reshape(-1, 1) + 1e-300) < TOL
    assert rel_err(CLALibLeftMultBy.leftMultByMatrix(cmb, y), om.lmm(y), np.abs(y) @ aX + 1e-300) < TOL
    s = aX.T @ (np.abs(w) * (aX @ np.abs(v))) + 1e-300
    assert rel_err(CLALibMMChain.mmChain(cmb, v, w, CHAIN_XtwXv).ravel(), om.mmchain(v, w, 1).ravel(), s) < 10 * TOL
    # multi-column operands still take the general kernels for every group
    V = rng.standard_normal((cmb.clen, 3))
    assert rel_err(CLALibRightMultBy.rightMultByMatrix(cmb, V), om.rmm(V), aX @ np.abs(V) + 1e-300) < TOL
    cmb.free()


def test_offset_and_run_edge_cases(oracle):
    """Listed-row counts 0 / 1 / 2 (OffsetEmpty / Single / Two), byte and char delta streams with continuation
    zeros, and RLE / OLE runs and gaps across the 65535 boundaries: decode bit-exact, products within tolerance."""
    from systemds_b200.offset import OFF_BYTE, OFF_CHAR, OFF_EMPTY, OFF_SINGLE, OFF_TWO
    nRows = 300_000
    rng = np.random.default_rng(3)
    d1 = np.array([[1.5], [-2.0]])
    cases = {
        "empty": np.array([], int), "single": np.array([123_456]), "two": np.array([5, 299_999]),
        "byte_cont": np.sort(np.concatenate([np.arange(0, 200_000, 7), [200_000 + 255, 200_000 + 255 * 2, 200_000 + 255 * 5 + 1]])),
        "char": np.sort(rng.choice(nRows, 300, replace=False)),
        "char_cont": np.array([0, 10, 65_545, 65_545 + 65_535 * 2, 299_000]),
    }
    want_type = {"empty": OFF_EMPTY, "single": OFF_SINGLE, "two": OFF_TWO, "byte_cont": OFF_BYTE, "char": OFF_CHAR,
                 "char_cont": OFF_CHAR}
    groups, c = [], 0
    for name, rows in cases.items():
        ids = np.full(nRows, -1, np.int32)
        ids[rows] = rng.integers(0, 2, rows.shape[0])
        g = cg.sdc_from_row_ids([c], d1, ids, None if c % 2 else [0.25])
        assert g._indexes.type == want_type[name], name
        groups.append(g)
        c += 1
    # runs: one run of 150000 rows (split at 65535), a gap above 2 * 65535, single-row runs around the boundaries
    ids = np.full(nRows, -1, np.int32)
    ids[100:150_100] = 0
    ids[290_000:290_001] = 1
    ids[65_534:65_537] = 1
    for cls in (cg.ColGroupRLE, cg.ColGroupOLE):
        groups.append(cls.from_row_ids([c], np.array([[0.5], [3.0]]), ids))
        c += 1
    cmb = CompressedMatrixBlock(nRows, c, groups).to_device()
    om = oracle.OracleMatrix(cmb)
    for gi, g in enumerate(groups):
        assert np.array_equal(cmb.group_row_ids(gi), g.row_ids(nRows)), f"group {gi}"
        assert np.array_equal(cmb.group_row_ids(gi), om.group_row_ids(gi))
        assert np.array_equal(cmb.group_counts(gi), om.group_counts(gi))
    X = dense_of(cmb)
    V = rng.standard_normal((c, 9))
    y = rng.standard_normal((2, nRows))
    assert rel_err(CLALibRightMultBy.rightMultByMatrix(cmb, V), om.rmm(V), np.abs(X) @ np.abs(V) + 1e-300) < TOL
    assert rel_err(CLALibRightMultBy.rightMultByMatrix(cmb, V[:, 0]), om.rmm(V[:, 0]), np.abs(X) @ np.abs(V[:, :1]) + 1e-300) < TOL
    assert rel_err(CLALibLeftMultBy.leftMultByMatrix(cmb, y), om.lmm(y), np.abs(y) @ np.abs(X) + 1e-300) < TOL
    assert rel_err(CLALibTSMM.leftMultByTransposeSelf(cmb), oracle.dense_tsmm_ld(X), np.abs(X).T @ np.abs(X) + 1e-300) < TOL
    assert rel_err(CLALibDecompress.decompress(cmb), X) < 1e-14
    cmb.free()


TMM_CASES = [
    (("ddc", "sdc", "rle", "const"), ("ddc2", "sdcz", "ole", "unc")),
    (("unc", "ddc", "sdcs"), ("unc", "rle", "ddc_char", "sdc", "empty")),
    (("ddc",) * 70, ("ddc",) * 3),
    (("ddcfor", "sdcfor", "ddc_bit"), ("sdcsz", "ddc", "ddc")),
    # mixed left sides against a right side of byte-map dense-map groups only
    (("ddc", "sdc", "rle", "unc", "ddc2", "sdcz", "const"), ("ddc",) * 5),
    (("sdc", "ddc_char", "rle"), ("ddc", "ddc2", "ddc_bit", "ddc")),
]


@pytest.mark.parametrize("case", range(len(TMM_CASES)))
@pytest.mark.parametrize("nRows", [1, 1000, 70001])
def test_compressed_times_compressed(oracle, case, nRows):
    """t(A) %*% B with both sides compressed (leftMultByMatrixTransposed on two blocks, and the transpose
    cases of CLALibMatrixMult.matrixMultiply for two compressed operands)."""
    ka, kb = TMM_CASES[case]
    A = datagen.random_cmb(500 + case, nRows, ka).to_device()
    B = datagen.random_cmb(600 + case, nRows, kb).to_device()
    XA, XB = dense_of(A), dense_of(B)
    scale = np.abs(XA).T @ np.abs(XB) + 1e-300
    want = oracle.OracleMatrix(A).tmm(oracle.OracleMatrix(B))
    got = CLALibLeftMultBy.leftMultByMatrixTransposed(B, A)
    assert got.shape == (A.clen, B.clen)
    assert rel_err(got, want, scale) < TOL
    assert rel_err(got, XA.T @ XB, scale) < TOL
    assert got.nnz == int(np.count_nonzero(got))
    assert rel_err(CLALibMatrixMult.matrixMultiply(A, B, True, False), want, scale) < TOL
    # same block on both sides equals TSMM
    if not any(k == "unc" for k in ka):
        both = CLALibLeftMultBy.leftMultByMatrixTransposed(A, A)
        assert rel_err(both, XA.T @ XA, np.abs(XA).T @ np.abs(XA) + 1e-300) < TOL
    with pytest.raises(CLAError):
        CLALibMatrixMult.matrixMultiply(A, B, False, True)
    A.free()
    B.free()


PAIR_CASES = [
    (("ddc2", "ddc2", "ddc2"), ("ddc2", "ddc2"), False),
    (("ddc2", "ddcfor", "ddc2", "const"), ("ddc2", "ddc_bit", "ddc2", "ddcfor"), False),
    (("ddc2", "ole", "ddc2"), ("ddc2", "ddc2", "empty"), False),
    (("ddc2", "ddc2", "ddc2", "const"), ("ddc2", "ddc2", "ddc2"), True),
]


@pytest.mark.parametrize("case", range(len(PAIR_CASES)))
@pytest.mark.parametrize("nRows", [1, 1000, 70001])
def test_products_on_the_dictionaries(oracle, case, nRows):
    """t(A) %*% B and t(X) %*% X when every group is a dense-map group and there are few co-coded groups: the joint
    count tables of the group pairs (integer histograms) times the dictionaries, instead of decompressing
    (APreAgg.leftMultByAColGroup, AColGroupCompressed.tsmm, APreAgg.tsmmAColGroup). Checked against the oracle's pair
    pre-aggregation and the dense product; the self-product is bit-symmetric; the integer case is exact."""
    ka, kb, overlap = PAIR_CASES[case]
    A = datagen.random_cmb(700 + case, nRows, ka, overlap).to_device()
    B = datagen.random_cmb(800 + case, nRows, kb, overlap).to_device()
    XA, XB = dense_of(A), dense_of(B)
    aA, aB = abs_dense_of(A), abs_dense_of(B)
    scale = aA.T @ aB + 1e-300
    k0 = A.stats()["kernel_launches"]
    got = CLALibLeftMultBy.leftMultByMatrixTransposed(B, A)
    # the pair path launches a handful of kernels, never one decompress + GEMM per row chunk
    assert A.stats()["kernel_launches"] - k0 <= 9
    assert rel_err(got, XA.T @ XB, scale) < TOL
    if not overlap:
        assert rel_err(got, oracle.OracleMatrix(A).tmm(oracle.OracleMatrix(B)), scale) < TOL
    self_ = CLALibTSMM.leftMultByTransposeSelf(A)
    assert rel_err(self_, oracle.dense_tsmm_ld(XA), aA.T @ aA + 1e-300) < TOL
    assert np.array_equal(self_, self_.T)
    A.free()
    B.free()
    # integer dictionaries: exact (lib/CLALibMMChainTest's 0-ULP bar for the self-product)
    if not overlap and not any("for" in k for k in ka):  # the generator draws frame-of-reference tuples as reals
        Ai = datagen.random_cmb(900 + case, nRows, ka, integer=True).to_device()
        Xi = dense_of(Ai)
        assert np.array_equal(np.array(CLALibTSMM.leftMultByTransposeSelf(Ai)), Xi.T @ Xi)
        Ai.free()


@pytest.mark.parametrize("name,kinds,overlap", CASES)
@pytest.mark.parametrize("nRows", [1, 37, 5000, 70001])
def test_min_max_aggregates(oracle, name, kinds, overlap, nRows):
    """uacmin / uacmax / uarmin / uarmax / uamin / uamax. Row-wise and overlapping cases are true extrema of the
    decompressed rows (one rounding for default + (dict - default)); column-wise and full extrema of
    non-overlapping blocks follow the reference's dictionary-based definition."""
    from systemds_b200.cmb import CLALibCompAgg
    cmb = datagen.random_cmb(seed_of(name, nRows) + 5, nRows, kinds, overlap).to_device()
    X = dense_of(cmb)
    sc = np.abs(X).max() + 1.0
    assert np.abs(CLALibCompAgg.rowMins(cmb).ravel() - X.min(axis=1)).max() < 1e-14 * sc
    assert np.abs(CLALibCompAgg.rowMaxs(cmb).ravel() - X.max(axis=1)).max() < 1e-14 * sc
    has_for = any(isinstance(g, (cg.ColGroupDDCFOR, cg.ColGroupSDCFOR)) for g in cmb.getColGroups())
    if overlap or has_for:
        lo, hi = X.min(axis=0), X.max(axis=0)
    else:
        lo, hi = oracle.col_minmax(cmb)
        assert np.all(lo <= X.min(axis=0) + 1e-14 * sc) and np.all(hi >= X.max(axis=0) - 1e-14 * sc)
    tol = 1e-14 * sc if (overlap or has_for) else 0.0
    assert np.abs(CLALibCompAgg.colMins(cmb).ravel() - lo).max() <= tol
    assert np.abs(CLALibCompAgg.colMaxs(cmb).ravel() - hi).max() <= tol
    assert abs(CLALibCompAgg.min(cmb) - lo.min()) <= tol and abs(CLALibCompAgg.max(cmb) - hi.max()) <= tol
    cmb.free()


@pytest.mark.parametrize("single", [False, True])
def test_decompress_keeps_registered_values_under_a_large_default(single):
    """A listed row of an SDC group decompresses to its registered dictionary value, bit for bit, also when the
    default tuple is many orders of magnitude larger (lib/CLALibDecompress.java:310-357 writes the value itself;
    the products work on dict - default and fold the default into the constants, colgroup/ColGroupSDC.java:483-489)."""
    rng = np.random.default_rng(11)
    nRows = 5000
    groups = []
    for c in range(3):
        card = 1 if single else 6
        ids = np.full(nRows, -1, np.int32)
        mask = rng.random(nRows) < 0.1
        ids[mask] = rng.integers(0, card, int(mask.sum()))
        groups.append(cg.sdc_from_row_ids([c], rng.standard_normal((card, 1)) * 1e-3, ids, np.array([1e6 + c])))
    cmb = CompressedMatrixBlock(nRows, 3, groups).to_device()
    assert np.array_equal(np.array(CLALibDecompress.decompress(cmb)), dense_of(cmb))
    # the products see the same cells as (d - default) + default, like the reference after extractCommon: their
    # error is relative to those two terms, not to the small cell
    v = rng.standard_normal(3)
    X = dense_of(cmb)
    defs = np.array([1e6, 1e6 + 1, 1e6 + 2])
    assert rel_err(CLALibRightMultBy.rightMultByMatrix(cmb, v).ravel(), X @ v, (np.abs(X - defs) + np.abs(defs)) @ np.abs(v)) < TOL
    cmb.free()


def test_concurrent_handles_and_shared_handle():
    """Calls on different handles may run concurrently (one stream per handle); calls on one handle are serialised
    by its mutex. Both must give the single-threaded bits."""
    import threading
    a = _ddc_matrix(200001, [16] * 30 + [250] * 10, 21).to_device()
    b = datagen.random_cmb(99, 50000, ("ddc", "sdc", "rle", "unc", "const", "ddc_char")).to_device()
    rng = np.random.default_rng(5)
    va, vb = rng.standard_normal(a.clen), rng.standard_normal(b.clen)
    Vb = rng.standard_normal((b.clen, 16))
    want = [np.array(CLALibRightMultBy.rightMultByMatrix(a, va)), np.array(CLALibMMChain.mmChain(a, va)),
            np.array(CLALibRightMultBy.rightMultByMatrix(b, vb)), np.array(CLALibRightMultBy.rightMultByMatrix(b, Vb))]
    bad = []

    def work(which):
        for _ in range(10):
            if which == 0:
                got = [CLALibRightMultBy.rightMultByMatrix(a, va), CLALibMMChain.mmChain(a, va)]
                ref = want[:2]
            else:
                got = [CLALibRightMultBy.rightMultByMatrix(b, vb), CLALibRightMultBy.rightMultByMatrix(b, Vb)]
                ref = want[2:]
            for g, w in zip(got, ref):
                g = np.array(g)
                if not np.array_equal(g, w):
                    # a reordered sum shows up as ~1e-16 of the largest entry, a race as something much larger
                    bad.append((which, float(np.max(np.abs(g - w)) / (np.max(np.abs(w)) + 1e-300))))

    threads = [threading.Thread(target=work, args=(i % 2,)) for i in range(4)]  # two threads per handle
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not bad, f"(handle, max deviation relative to the largest entry): {sorted(set(bad))[:8]}"
    a.free()
    b.free()


@pytest.mark.parametrize("seed", range(24))
def test_random_blocks_every_product(oracle, seed):
    """Randomly drawn blocks (group kinds, row counts around the 256 / 1024 / 65535 boundaries of the index
    structures, operand widths) through every product, against the oracle."""
    rng = np.random.default_rng(9000 + seed)
    nRows = int(rng.choice([1, 2, 31, 32, 33, 255, 256, 257, 1023, 1024, 1025, 2049, 4097, 65535, 65536, 65537, 70001,
                            131073]))
    pool = datagen.KINDS + ("ddcfor", "sdcfor", "ddc", "ddc", "ddc")
    kinds = tuple(rng.choice(pool, size=int(rng.integers(1, 14))))
    overlap = bool(rng.integers(0, 4) == 0)
    cmb = datagen.random_cmb(9100 + seed, nRows, kinds, overlap)
    if seed % 2:  # columns on very different scales: errors must stay relative to each row's own terms
        for g in cmb.getColGroups():
            f = 10.0 ** int(rng.integers(-4, 5))
            for name in ("_dict", "_defaultTuple", "_reference", "_data"):
                a = getattr(g, name, None)
                if isinstance(a, np.ndarray) and a.dtype == np.float64:
                    a *= f
    cmb.to_device()
    om = oracle.OracleMatrix(cmb)
    X = dense_of(cmb)
    aX = np.abs(X)
    vc = int(rng.choice([1, 2, 3, 7, 8, 13, 64, 65]))
    V = rng.standard_normal((cmb.clen, vc))
    got = CLALibRightMultBy.rightMultByMatrix(cmb, V)
    assert rel_err(got, om.rmm(V), aX @ np.abs(V) + 1e-300) < TOL, (kinds, nRows, vc)
    q = int(rng.choice([1, 2, 5]))
    Yt = rng.standard_normal((q, nRows))
    assert rel_err(CLALibLeftMultBy.leftMultByMatrix(cmb, Yt), om.lmm(Yt), np.abs(Yt) @ aX + 1e-300) < TOL, (kinds, nRows, q)
    # a cell of a plain block is one dictionary value (rounded once where a default tuple is folded in); cells of
    # overlapping or frame-of-reference blocks are sums whose terms may cancel
    summed = overlap or any(k in ("ddcfor", "sdcfor") for k in kinds)
    assert rel_err(CLALibDecompress.decompress(cmb), X) < (TOL if summed else 1e-14), (kinds, nRows)
    got = CLALibTSMM.leftMultByTransposeSelf(cmb)
    aP = abs_dense_of(cmb) if summed else aX
    assert rel_err(got, oracle.dense_tsmm_ld(X), aP.T @ aP + 1e-300) < TOL, (kinds, nRows)
    v = rng.standard_normal(cmb.clen)
    w = rng.standard_normal(nRows)
    sw = aX.T @ (np.abs(w) * (aX @ np.abs(v))) + 1e-300
    assert rel_err(CLALibMMChain.mmChain(cmb, v, w, CHAIN_XtwXv).ravel(), om.mmchain(v, w, 1).ravel(), sw) < 10 * TOL
    cmb.free()


def test_rows_without_open_runs_are_exact_zeros(oracle):
    """X v on RLE groups whose runs leave rows uncovered: those rows are exactly zero (the kernel turns runs into
    +P / -P boundaries and prefix sums, whose rounding residue must not leak into rows where no run is open),
    and the returned non-zero count matches."""
    rng = np.random.default_rng(12)
    groups = []
    for c in range(7):
        ids = np.full(3 * 1024 + 1, -1)
        pos = int(rng.integers(0, 40))
        while pos < ids.shape[0]:
            ln = int(rng.integers(1, 300))
            ids[pos:pos + ln] = int(rng.integers(0, 5))
            pos += ln + int(rng.integers(1, 200))
        groups.append(cg.ColGroupRLE.from_row_ids([c], rng.standard_normal((5, 1)) * 10.0 ** rng.integers(-3, 4), ids))
    cmb = CompressedMatrixBlock(3 * 1024 + 1, 7, groups).to_device()
    X = dense_of(cmb)
    v = rng.standard_normal(7)
    got = CLALibRightMultBy.rightMultByMatrix(cmb, v)
    zero_rows = np.flatnonzero(np.abs(X).sum(axis=1) == 0)
    assert zero_rows.size > 0 and np.all(np.asarray(got)[zero_rows] == 0.0)
    assert rel_err(got, oracle.OracleMatrix(cmb).rmm(v), np.abs(X) @ np.abs(v).reshape(-1, 1) + 1e-300) < TOL
    assert got.nnz == int(np.count_nonzero(X @ v))
    cmb.free()


def test_many_sparse_groups_wide_rhs(oracle):
    """More than 256 SDC / RLE groups: the tensor-core RMM falls back to its first-generation kernel (one lane per
    group covers 256 of each)."""
    kinds = ("sdcz",) * 150 + ("sdc",) * 120 + ("rle",) * 270 + ("ddc",) * 5
    cmb = datagen.random_cmb(4242, 3001, kinds).to_device()
    om = oracle.OracleMatrix(cmb)
    aX = np.abs(dense_of(cmb))
    rng = np.random.default_rng(8)
    V = rng.standard_normal((cmb.clen, 17))
    assert rel_err(CLALibRightMultBy.rightMultByMatrix(cmb, V), om.rmm(V), aX @ np.abs(V) + 1e-300) < TOL
    v = rng.standard_normal(cmb.clen)
    assert rel_err(CLALibRightMultBy.rightMultByMatrix(cmb, v), om.rmm(v), aX @ np.abs(v).reshape(-1, 1) + 1e-300) < TOL
    y = rng.standard_normal((1, cmb.rlen))
    assert rel_err(CLALibLeftMultBy.leftMultByMatrix(cmb, y), om.lmm(y), np.abs(y) @ aX + 1e-300) < TOL
    cmb.free()


def test_double_compressed_transpose_rules():
    """The remaining flag combinations for two compressed operands (CLALibMatrixMult.java:96-124)."""
    m1 = datagen.random_cmb(801, 40, ("ddc", "sdc", "rle", "const")).to_device()       # [40 x c1]
    m2 = datagen.random_cmb(802, 6, ("ddc",) * 37 + ("sdcz", "unc")).to_device()       # [6 x 40]
    X1, X2 = dense_of(m1), dense_of(m2)
    if X2.shape[1] == 40:
        r = CLALibMatrixMult.matrixMultiply(m2, m1)                                    # plain: right side decompressed
        assert rel_err(r, X2 @ X1, np.abs(X2) @ np.abs(X1) + 1e-300) < TOL
        r = CLALibMatrixMult.matrixMultiply(m1, m2, True, True)                        # t(m1) t(m2) = t(m2 m1)
        assert r.shape == (X1.shape[1], 6)
        assert rel_err(r, X1.T @ X2.T, np.abs(X1).T @ np.abs(X2).T + 1e-300) < TOL
    else:
        pytest.fail("generator produced %d columns" % X2.shape[1])
    m1.free()
    m2.free()


def test_sum_aggregates():
    from systemds_b200.cmb import CLALibCompAgg
    cmb = datagen.random_cmb(8, 20000, datagen.KINDS).to_device()
    X = dense_of(cmb)
    assert rel_err(CLALibCompAgg.colSums(cmb), X.sum(axis=0, keepdims=True), np.abs(X).sum(axis=0, keepdims=True) + 1e-300) < TOL
    assert rel_err(CLALibCompAgg.rowSums(cmb), X.sum(axis=1, keepdims=True), np.abs(X).sum(axis=1, keepdims=True) + 1e-300) < TOL
    assert abs(CLALibCompAgg.sum(cmb) - X.sum()) <= TOL * np.abs(X).sum()
    cmb.free()


def test_groups_registered_from_device_memory(oracle):
    """cla_add_group_ddc_dev / cla_add_group_uncompressed_dev: a block whose maps and dense values are handed over as
    device buffers gives the same bits as the same block registered from host arrays, for every map class the call
    takes; an id outside the dictionary is refused when the block is finalized."""
    import torch
    from systemds_b200.mapping import DeviceMap, MAP_BIT, MAP_BYTE, MAP_CHAR, MAP_INT, MAP_UBYTE
    rng = np.random.default_rng(77)
    nRows = 70001
    dev = torch.device("cuda", 0)
    host_groups, dev_groups, keep = [], [], []
    specs = [(2, MAP_BIT), (100, MAP_UBYTE), (250, MAP_BYTE), (900, MAP_CHAR), (70000, MAP_INT)]
    for c, (card, mt) in enumerate(specs):
        ids = rng.integers(0, card, nRows)
        d = rng.standard_normal((card, 1))
        m = MapToFactory.create_from(ids, card, force_type=mt)
        host_groups.append(cg.ColGroupDDC([c], d, m))
        t = torch.from_numpy(m.data.view(np.uint8).copy()).to(dev)
        keep.append(t)
        dev_groups.append(cg.ColGroupDDC([c], d, DeviceMap(mt, nRows, card, t.data_ptr(), t.numel(), owner=t)))
    dense = rng.standard_normal((nRows, 3))
    td = torch.from_numpy(dense).to(dev)
    nc = len(specs)
    host_groups.append(cg.ColGroupUncompressed([nc, nc + 1, nc + 2], dense))
    dev_groups.append(cg.ColGroupUncompressedDev([nc, nc + 1, nc + 2], nRows, td.data_ptr(), owner=td))
    a = CompressedMatrixBlock(nRows, nc + 3, host_groups).to_device()
    b = CompressedMatrixBlock(nRows, nc + 3, dev_groups).to_device()
    v = rng.standard_normal(nc + 3)
    V = rng.standard_normal((nc + 3, 16))
    y = rng.standard_normal((1, nRows))
    for f in (lambda m: CLALibRightMultBy.rightMultByMatrix(m, v), lambda m: CLALibRightMultBy.rightMultByMatrix(m, V),
              lambda m: CLALibDecompress.decompress(m)):
        assert np.array_equal(np.array(f(a)), np.array(f(b)))
    X = dense_of(a)
    assert rel_err(CLALibLeftMultBy.leftMultByMatrix(b, y), y @ X, np.abs(y) @ np.abs(X)) < TOL
    assert rel_err(CLALibTSMM.leftMultByTransposeSelf(b), oracle.dense_tsmm_ld(X), np.abs(X).T @ np.abs(X)) < TOL
    for gi in range(nc):
        assert np.array_equal(b.group_row_ids(gi), a.group_row_ids(gi))
    a.free()
    b.free()
    bad = torch.full((nRows,), 7, dtype=torch.uint8, device=dev)
    g = cg.ColGroupDDC([0], rng.standard_normal((5, 1)), DeviceMap(MAP_UBYTE, nRows, 5, bad.data_ptr(), nRows, owner=bad))
    with pytest.raises(CLAError):
        CompressedMatrixBlock(nRows, 1, [g]).to_device()


@pytest.mark.parametrize("kinds,overlap", [(("ddc", "ddc2", "sdc", "rle", "unc", "const", "ole"), False),
                                           (("ddc2", "ddc2", "ddc_bit"), False), (("ddc", "sdc", "rle", "ddc2"), True)])
@pytest.mark.parametrize("nRows", [1, 1000, 70001])
def test_right_product_kept_compressed(oracle, kinds, overlap, nRows):
    """rightMultByMatrix(..., allowOverlap=True) (RMMOverlapping, lib/CLALibRightMultBy.java:157-201): the result is an
    overlapping block on the device that shares the operand's index structures. Its decompressed form equals the dense
    product, it takes further products, it survives its parent, and t(X) %*% (X %*% v) through it equals mmChain."""
    rng = np.random.default_rng(nRows)
    X_ = datagen.random_cmb(1200 + nRows, nRows, kinds, overlap).to_device()
    X = dense_of(X_)
    aX = abs_dense_of(X_)
    for vc in (1, 5):
        V = rng.standard_normal((X_.clen, vc))
        R = CLALibRightMultBy.rightMultByMatrix(X_, V, allowOverlap=True)
        assert isinstance(R, CompressedMatrixBlock) and R.isOverlapping() and (R.rlen, R.clen) == (nRows, vc)
        sc = aX @ np.abs(V) + 1e-300
        assert rel_err(CLALibDecompress.decompress(R), X @ V, sc) < TOL
        assert rel_err(CLALibDecompress.decompress(R), CLALibRightMultBy.rightMultByMatrix(X_, V), sc) < TOL
        W = rng.standard_normal((vc, 3))
        assert rel_err(CLALibRightMultBy.rightMultByMatrix(R, W), (X @ V) @ W, sc @ np.abs(W) + 1e-300) < TOL
        y = rng.standard_normal((2, nRows))
        assert rel_err(CLALibLeftMultBy.leftMultByMatrix(R, y), y @ (X @ V), np.abs(y) @ sc + 1e-300) < TOL
        # t(X) %*% (X %*% V): two compressed blocks
        got = CLALibLeftMultBy.leftMultByMatrixTransposed(R, X_)
        assert rel_err(got, X.T @ (X @ V), aX.T @ sc + 1e-300) < 10 * TOL
        R.free()
    v = rng.standard_normal(X_.clen)
    s = aX.T @ (aX @ np.abs(v)) + 1e-300
    assert rel_err(CLALibMMChain.mmChain(X_, v, allowOverlap=True).ravel(), CLALibMMChain.mmChain(X_, v).ravel(), s) < 10 * TOL
    # the result outlives the block it came from
    R = CLALibRightMultBy.rightMultByMatrix(X_, v, allowOverlap=True)
    X_.free()
    assert rel_err(CLALibDecompress.decompress(R).ravel(), X @ v, aX @ np.abs(v) + 1e-300) < TOL
    R.free()
