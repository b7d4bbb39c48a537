"""Shared helpers of the parity tests."""
import numpy as np

from systemds_b200 import colgroup as cg


def dense_of(cmb) -> np.ndarray:
    """Decompress on the host with numpy, straight from the group records (independent of oracle and GPU)."""
    X = np.zeros((cmb.rlen, cmb.clen))
    for g in cmb.getColGroups():
        cols = g.getColIndices()
        if isinstance(g, cg.ColGroupUncompressed):
            X[:, cols] += g._data
        elif isinstance(g, cg.ColGroupConst):
            X[:, cols] += g._dict[0]
        elif isinstance(g, cg.ColGroupEmpty):
            pass
        else:
            ids = g.row_ids(cmb.rlen)
            d = g._dict
            default = getattr(g, "_defaultTuple", None)
            if default is None:
                default = np.zeros(len(cols))
            vals = np.where((ids >= 0)[:, None], d[np.maximum(ids, 0)], default[None, :])
            X[:, cols] += vals
            if hasattr(g, "_reference"):
                X[:, cols] += g._reference
    return X


def abs_dense_of(cmb) -> np.ndarray:
    """Sum over the groups of the absolute values each contributes to a cell: the magnitude of the terms behind a
    cell of an overlapping or frame-of-reference block (equals |X| for a plain block)."""
    A = np.zeros((cmb.rlen, cmb.clen))
    for g in cmb.getColGroups():
        one = type(cmb)(cmb.rlen, cmb.clen, [g], False)
        ref = getattr(g, "_reference", None)
        if ref is not None:  # a frame-of-reference cell is dictionary value + reference: two terms
            cols = g.getColIndices()
            X = dense_of(one)
            X[:, cols] -= ref
            A += np.abs(X)
            A[:, cols] += np.abs(ref)
        else:
            A += np.abs(dense_of(one))
    return A


def rel_err(got, ref, scale=None) -> float:
    """max |got - ref| relative to the magnitude of the terms that were summed (norm-wise relative error)."""
    got, ref = np.asarray(got, float), np.asarray(ref, float)
    if ref.size == 0:
        return 0.0
    s = np.maximum(np.abs(ref), np.max(np.abs(ref)) * 1e-3 if scale is None else scale)
    s = np.where(s == 0, 1.0, s)
    return float(np.max(np.abs(got - ref) / s))


TOL = 1e-12  # relative tolerance for FP64 products (reordered summation)
