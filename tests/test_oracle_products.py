"""The oracle's products against a long-double dense evaluation of the decompressed matrix.

This is the reference's own notion of correctness (compressed op == uncompressed op on the
decompressed block, CompressedTestBase.java:465-880), applied to the restatement.
"""
import numpy as np
import pytest

from systemds_b200 import datagen
from tests.util import TOL, dense_of, rel_err

CASES = [
    ("all", datagen.KINDS, False),
    ("for", ("ddcfor", "sdcfor", "ddc", "sdcfor", "rle", "ddcfor"), False),
    ("ddc_only", ("ddc", "ddc", "ddc2", "ddc_bit", "ddc_char"), False),
    ("sparse", ("sdc", "sdcz", "sdcs", "sdcsz", "const", "empty"), False),
    ("runs", ("rle", "rle", "ole", "ddc"), False),
    ("overlap", ("ddc", "sdc", "rle", "ddc2", "const", "sdcz"), True),
]


@pytest.mark.parametrize("name,kinds,overlap", CASES)
@pytest.mark.parametrize("nRows", [1, 37, 1024, 5000])
def test_oracle_vs_dense(oracle, name, kinds, overlap, nRows):
    cmb = datagen.random_cmb(sum(map(ord, name)) + nRows, nRows, kinds, overlap)
    X = dense_of(cmb)
    om = oracle.OracleMatrix(cmb, threads=3)
    assert rel_err(om.decompress(), X) < 1e-14  # default + (dict - default) rounds once
    rng = np.random.default_rng(nRows)
    for vc in (1, 5):
        V = rng.standard_normal((cmb.clen, vc))
        assert rel_err(om.rmm(V), oracle.dense_rmm_ld(X, V), np.abs(X) @ np.abs(V) + 1e-300) < TOL
    for q in (1, 6):
        Yt = rng.standard_normal((q, nRows))
        assert rel_err(om.lmm(Yt), oracle.dense_lmm_ld(X, Yt), np.abs(Yt) @ np.abs(X) + 1e-300) < TOL
    if not overlap:
        ref = oracle.dense_tsmm_ld(X)
        for fb in (True, False):
            if not fb and "unc" in kinds:
                continue
            assert rel_err(om.tsmm(allow_fallback=fb), ref, np.abs(X).T @ np.abs(X) + 1e-300) < TOL
    v = rng.standard_normal(cmb.clen)
    w = rng.standard_normal(nRows)
    ref_u = X @ v
    s = np.abs(X).T @ (np.abs(X) @ np.abs(v)) + 1e-300
    assert rel_err(om.mmchain(v).ravel(), X.T @ ref_u, s) < 1e-11
    assert rel_err(om.mmchain(v, w, 1).ravel(), X.T @ (w * ref_u), np.abs(X).T @ (np.abs(w) * (np.abs(X) @ np.abs(v))) + 1e-300) < 1e-11


@pytest.mark.parametrize("nRows", [1, 37, 5000])
def test_oracle_compressed_times_compressed(oracle, nRows):
    """t(A) %*% B on two compressed blocks against the dense product (and against itself with one thread)."""
    pairs = [(("ddc", "sdc", "rle", "const"), ("ddc2", "sdcz", "ole", "unc")),
             (("unc", "ddc", "sdcs", "sdcfor"), ("unc", "rle", "ddc_char", "sdc", "empty")),
             (datagen.KINDS, datagen.KINDS)]
    for i, (ka, kb) in enumerate(pairs):
        A = datagen.random_cmb(31 + i + nRows, nRows, ka)
        B = datagen.random_cmb(41 + i + nRows, nRows, kb)
        XA, XB = dense_of(A), dense_of(B)
        sc = np.abs(XA).T @ np.abs(XB) + 1e-300
        got = oracle.OracleMatrix(A, threads=3).tmm(oracle.OracleMatrix(B, threads=3))
        assert got.shape == (A.clen, B.clen)
        assert rel_err(got, XA.T @ XB, sc) < TOL
        assert rel_err(got, oracle.OracleMatrix(A, threads=1).tmm(oracle.OracleMatrix(B, threads=1)), sc) < TOL


def test_tsmm_integer_exact(oracle):
    """CLALibMMChainTest.java:159-171: integer-valued dictionaries give a 0-ULP self product."""
    cmb = datagen.random_cmb(11, 3000, ("ddc", "ddc2", "sdcz", "rle", "ddc_bit"), integer=True)
    X = dense_of(cmb)
    om = oracle.OracleMatrix(cmb, threads=2)
    assert np.array_equal(om.tsmm(allow_fallback=False), X.T @ X)
    assert np.array_equal(om.tsmm(allow_fallback=True), X.T @ X)


def test_counts_and_row_ids(oracle):
    cmb = datagen.random_cmb(3, 4000, datagen.KINDS)
    om = oracle.OracleMatrix(cmb)
    for gi, g in enumerate(cmb.getColGroups()):
        if hasattr(g, "row_ids"):
            ids = g.row_ids(cmb.rlen)
            assert np.array_equal(om.group_row_ids(gi), ids)
            if g.getNumValues():
                assert np.array_equal(om.group_counts(gi), np.bincount(ids[ids >= 0], minlength=g.getNumValues()))


def test_empty_operands(oracle):
    cmb = datagen.random_cmb(1, 0, ("ddc", "sdcz"))
    om = oracle.OracleMatrix(cmb)
    assert om.rmm(np.ones((2, 3))).shape == (0, 3)
    assert np.array_equal(om.lmm(np.zeros((2, 0))), np.zeros((2, 2)))
    assert np.array_equal(om.tsmm(), np.zeros((2, 2)))
