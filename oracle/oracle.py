"""ctypes binding of the CPU oracle (``oracle/libcla_oracle.so``) -- TEST INFRASTRUCTURE ONLY.

Only tests, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may import this module.
It feeds the same host-side column-group records that the product uploads to the GPU into the
CPU restatement of the reference algorithms (see cla_oracle.cpp for the file:line citations).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcla_oracle.so")
_P, _I32, _I64 = C.c_void_p, C.c_int32, C.c_int64
_lib = None


def build(force: bool = False) -> str:
    src = [os.path.join(HERE, f) for f in ("cla_oracle.cpp", "cla_oracle.h", "Makefile")]
    stale = force or not os.path.exists(LIB_PATH) or any(os.path.getmtime(s) > os.path.getmtime(LIB_PATH) for s in src)
    if stale:
        r = subprocess.run(["make", "-C", HERE] + (["-B"] if force else []), capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("oracle build failed:\n" + r.stdout + r.stderr)
    return LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        l = C.CDLL(LIB_PATH)
        sig = {
            "ocl_map_type_for": ([_I64, _I64], C.c_int),
            "ocl_ole_gen_offset_bitmap": ([_P, _I64, _P, _I64], _I64),
            "ocl_rle_gen_bitmap": ([_P, _I64, _P, _I64], _I64),
            "ocl_offset_create": ([_P, _I64, _P, _P, _P, _P, _I64, _P], _I64),
            "ocl_offset_decode": ([_I32, _I32, _I32, _P, _I64, _P, _I64], _I64),
            "ocl_map_decode": ([_I32, _P, _P, _I64, _P], None),
            "ocl_create": ([_I32, _I32], _P),
            "ocl_destroy": ([_P], None),
            "ocl_add_ddc": ([_P, _P, _I32, _P, _I32, _I32, _P, _P, _I64], C.c_int),
            "ocl_add_sdc": ([_P, _P, _I32, _P, _I32, _P, _I32, _I32, _I32, _P, _I64, _I32, _P, _P, _I64], C.c_int),
            "ocl_add_rle": ([_P, _P, _I32, _P, _I32, _P, _P, _I64], C.c_int),
            "ocl_add_ole": ([_P, _P, _I32, _P, _I32, _P, _P, _I64], C.c_int),
            "ocl_add_uncompressed": ([_P, _P, _I32, _P], C.c_int),
            "ocl_add_const": ([_P, _P, _I32, _P], C.c_int),
            "ocl_add_empty": ([_P, _P, _I32], C.c_int),
            "ocl_num_groups": ([_P], _I32),
            "ocl_compressed_bytes": ([_P], _I64),
            "ocl_group_row_ids": ([_P, _I32, _P], None),
            "ocl_group_counts": ([_P, _I32, _P], None),
            "ocl_decompress": ([_P, _P, C.c_int], None),
            "ocl_rmm": ([_P, _P, _I32, _P, C.c_int], None),
            "ocl_lmm": ([_P, _P, _I32, _P, C.c_int], None),
            "ocl_tsmm": ([_P, _P, C.c_int, C.c_int], None),
            "ocl_mmchain": ([_P, _P, _P, C.c_int, _P, C.c_int], None),
            "ocl_tmm": ([_P, _P, _P, C.c_int], None),
            "ocl_dense_rmm_ld": ([_P, _I64, _I32, _P, _I32, _P], None),
            "ocl_dense_lmm_ld": ([_P, _I64, _I32, _P, _I32, _P], None),
            "ocl_dense_tsmm_ld": ([_P, _I64, _I32, _P], None),
            "ocl_max_threads": ([], C.c_int),
        }
        for n, (a, r) in sig.items():
            f = getattr(l, n)
            f.argtypes = a
            f.restype = r
        _lib = l
    return _lib


def _p(a):
    return C.c_void_p(0) if a is None else C.c_void_p(a.ctypes.data)


def _f64(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.float64))


# ---- format level ------------------------------------------------------------------------------
def map_type_for(size, unique):
    return int(lib().ocl_map_type_for(size, unique))


def ole_gen_offset_bitmap(offsets):
    off = np.ascontiguousarray(np.asarray(offsets, dtype=np.int32))
    n = lib().ocl_ole_gen_offset_bitmap(_p(off), off.shape[0], None, 0)
    if n < 0:
        return None
    out = np.zeros(n, np.uint16)
    lib().ocl_ole_gen_offset_bitmap(_p(off), off.shape[0], _p(out), n)
    return out


def rle_gen_bitmap(offsets):
    off = np.ascontiguousarray(np.asarray(offsets, dtype=np.int32))
    n = lib().ocl_rle_gen_bitmap(_p(off), off.shape[0], None, 0)
    if n < 0:
        return None
    out = np.zeros(n, np.uint16)
    lib().ocl_rle_gen_bitmap(_p(off), off.shape[0], _p(out), n)
    return out


def offset_create(indexes):
    """-> (type, first, last, data array or None, flags)"""
    idx = np.ascontiguousarray(np.asarray(indexes, dtype=np.int32))
    t, f, la, fl = C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32()
    n = lib().ocl_offset_create(_p(idx), idx.shape[0], C.byref(t), C.byref(f), C.byref(la), None, 0, C.byref(fl))
    buf = np.zeros(max(int(n), 1) * 2, np.uint8)
    n = lib().ocl_offset_create(_p(idx), idx.shape[0], C.byref(t), C.byref(f), C.byref(la), _p(buf), n, C.byref(fl))
    data = None
    if t.value == 3:
        data = buf[:n].copy()
    elif t.value == 4:
        data = buf[: 2 * n].view(np.uint16).copy()
    return t.value, f.value, la.value, data, fl.value


def offset_decode(otype, first, last, data):
    n = lib().ocl_offset_decode(otype, first, last, _p(data), 0 if data is None else data.shape[0], None, 0)
    rows = np.zeros(max(int(n), 1), np.int32)
    lib().ocl_offset_decode(otype, first, last, _p(data), 0 if data is None else data.shape[0], _p(rows), n)
    return rows[:n]


def map_decode(mtype, data, data2, size):
    ids = np.zeros(size, np.int32)
    lib().ocl_map_decode(mtype, _p(data), _p(data2), size, _p(ids))
    return ids


# ---- matrix level ------------------------------------------------------------------------------
class OracleMatrix:
    """The oracle's copy of a CompressedMatrixBlock (host records from systemds_b200.colgroup)."""

    def __init__(self, cmb, threads: int | None = None):
        from systemds_b200 import colgroup as cg  # the host records are shared vocabulary, not compute
        L = lib()
        self.nRows, self.nCols = cmb.rlen, cmb.clen
        self.k = int(threads) if threads else int(L.ocl_max_threads())
        self.h = L.ocl_create(cmb.rlen, cmb.clen)
        self.nvals = []
        self.reg_index = []
        n_native = 0
        for g in cmb.getColGroups():
            cols, gc = _p(g._colIndexes), g.getNumCols()
            self.nvals.append(g.getNumValues())
            self.reg_index.append(n_native)
            n_native += 1
            if hasattr(g, "_reference"):  # frame-of-reference group: extractCommon -> plain group + constant tuple
                L.ocl_add_const(self.h, cols, gc, _p(g._reference))
                n_native += 1
                self.reg_index[-1] = n_native - 1
            if isinstance(g, cg.ColGroupDDC):
                m = g._data
                L.ocl_add_ddc(self.h, cols, gc, _p(g._dict), g.getNumValues(), m.type, _p(m.data), _p(m.data2), m.size)
            elif isinstance(g, cg.ASDC):
                o, m = g._indexes, g._data
                dummy = np.zeros(1, np.int64)
                mp = None if m is None else (_p(dummy) if m.data is None else _p(m.data))
                L.ocl_add_sdc(self.h, cols, gc, _p(g._dict), g.getNumValues(), _p(g._defaultTuple), o.type, o.first,
                              o.last, _p(o.data), 0 if o.data is None else o.data.shape[0],
                              0 if m is None else m.type, mp, None if m is None else _p(m.data2), o.size)
            elif isinstance(g, cg.ColGroupRLE):
                L.ocl_add_rle(self.h, cols, gc, _p(g._dict), g.getNumValues(), _p(g._ptr), _p(g._data), g._data.shape[0])
            elif isinstance(g, cg.ColGroupOLE):
                L.ocl_add_ole(self.h, cols, gc, _p(g._dict), g.getNumValues(), _p(g._ptr), _p(g._data), g._data.shape[0])
            elif isinstance(g, cg.ColGroupUncompressed):
                L.ocl_add_uncompressed(self.h, cols, gc, _p(g._data))
            elif isinstance(g, cg.ColGroupConst):
                L.ocl_add_const(self.h, cols, gc, _p(g._dict))
            elif isinstance(g, cg.ColGroupEmpty):
                L.ocl_add_empty(self.h, cols, gc)
            else:
                raise TypeError(type(g).__name__)

    def __del__(self):
        try:
            lib().ocl_destroy(self.h)
        except Exception:
            pass

    def group_row_ids(self, g):
        ids = np.zeros(self.nRows, np.int32)
        lib().ocl_group_row_ids(self.h, self.reg_index[g], _p(ids))
        return ids

    def group_counts(self, g):
        c = np.zeros(max(self.nvals[g], 1), np.int64)
        lib().ocl_group_counts(self.h, self.reg_index[g], _p(c))
        return c[: self.nvals[g]]

    def decompress(self):
        out = np.zeros((self.nRows, self.nCols))
        lib().ocl_decompress(self.h, _p(out), self.k)
        return out

    def rmm(self, V):
        V = _f64(V)
        if V.ndim == 1:
            V = V.reshape(-1, 1)
        out = np.zeros((self.nRows, V.shape[1]))
        lib().ocl_rmm(self.h, _p(V), V.shape[1], _p(out), self.k)
        return out

    def lmm(self, Yt):
        Yt = _f64(Yt)
        if Yt.ndim == 1:
            Yt = Yt.reshape(1, -1)
        out = np.zeros((Yt.shape[0], self.nCols))
        lib().ocl_lmm(self.h, _p(Yt), Yt.shape[0], _p(out), self.k)
        return out

    def tsmm(self, allow_fallback=True):
        out = np.zeros((self.nCols, self.nCols))
        lib().ocl_tsmm(self.h, _p(out), self.k, int(allow_fallback))
        return out

    def tmm(self, right):
        """t(self) %*% right for another OracleMatrix with the same number of rows."""
        out = np.zeros((self.nCols, right.nCols))
        lib().ocl_tmm(self.h, right.h, _p(out), self.k)
        return out

    def mmchain(self, v, w=None, ctype=0):
        v = _f64(v).reshape(-1)
        wv = None if w is None else _f64(w).reshape(-1)
        out = np.zeros((self.nCols, 1))
        lib().ocl_mmchain(self.h, _p(v), _p(wv), int(ctype), _p(out), self.k)
        return out


def dense_rmm_ld(X, V):
    X, V = _f64(X), _f64(V)
    if V.ndim == 1:
        V = V.reshape(-1, 1)
    out = np.zeros((X.shape[0], V.shape[1]))
    lib().ocl_dense_rmm_ld(_p(X), X.shape[0], X.shape[1], _p(V), V.shape[1], _p(out))
    return out


def dense_lmm_ld(X, Yt):
    X, Yt = _f64(X), _f64(Yt)
    if Yt.ndim == 1:
        Yt = Yt.reshape(1, -1)
    out = np.zeros((Yt.shape[0], X.shape[1]))
    lib().ocl_dense_lmm_ld(_p(X), X.shape[0], X.shape[1], _p(Yt), Yt.shape[0], _p(out))
    return out


def dense_tsmm_ld(X):
    X = _f64(X)
    out = np.zeros((X.shape[1], X.shape[1]))
    lib().ocl_dense_tsmm_ld(_p(X), X.shape[0], X.shape[1], _p(out))
    return out


def col_minmax(cmb):
    """Column minima and maxima of a non-overlapping block as the reference computes them: per group from the
    dictionary, every entry counting whether used or not (AColGroupCompressed.computeColMxx): DDC / Const
    ``_dict.aggregateCols`` (ColGroupDDC.java:831-833, ColGroupConst.java:370-372); SDC / SDCSingle dictionary and
    default tuple (ColGroupSDC.java:182-186); SDCZeros / SDCSingleZeros dictionary and 0 (ColGroupSDCZeros.java:
    807-812); RLE / OLE dictionary and 0 when ``_zeros`` (ColGroupRLE.java:730-735); FOR groups dictionary +
    reference (and the reference itself for SDCFOR's unlisted rows); Empty 0; Uncompressed from its data."""
    from systemds_b200 import colgroup as cg
    lo = np.full(cmb.getNumColumns(), np.inf)
    hi = np.full(cmb.getNumColumns(), -np.inf)

    def add(cols, vals):
        vals = np.atleast_2d(np.asarray(vals, dtype=np.float64))
        lo[cols] = np.minimum(lo[cols], vals.min(axis=0))
        hi[cols] = np.maximum(hi[cols], vals.max(axis=0))

    n = cmb.getNumRows()
    for g in cmb.getColGroups():
        cols = g.getColIndices()
        if isinstance(g, cg.ColGroupEmpty):
            add(cols, np.zeros(len(cols)))
        elif isinstance(g, cg.ColGroupUncompressed):
            add(cols, g._data)
        elif isinstance(g, cg.ColGroupDDCFOR):
            add(cols, g._dict + g._reference)
        elif isinstance(g, cg.ColGroupSDCFOR):
            add(cols, g._dict + g._reference)
            add(cols, g._reference)
        elif isinstance(g, (cg.ColGroupDDC, cg.ColGroupConst)):
            add(cols, g._dict)
        elif isinstance(g, cg.ASDC):
            add(cols, g._dict)
            add(cols, np.zeros(len(cols)) if g._defaultTuple is None else g._defaultTuple)
        elif isinstance(g, cg.AColGroupOffset):
            add(cols, g._dict)
            if int((g.row_ids(n) >= 0).sum()) < n:
                add(cols, np.zeros(len(cols)))
    return lo, hi
