"""CompressedMatrixBlock and the four CLA matrix-multiply entry points, backed by the native library.

Mirrors the reference's operator API for this path:

* ``CompressedMatrixBlock``  runtime/compress/CompressedMatrixBlock.java:108-132 (fields), :587-627 (products)
* ``CLALibRightMultBy.rightMultByMatrix``  runtime/compress/lib/CLALibRightMultBy.java:57
* ``CLALibLeftMultBy.leftMultByMatrix``    runtime/compress/lib/CLALibLeftMultBy.java:126
* ``CLALibTSMM.leftMultByTransposeSelf``   runtime/compress/lib/CLALibTSMM.java:59
* ``CLALibMMChain.mmChain``                runtime/compress/lib/CLALibMMChain.java:92
* ``CLALibDecompress.decompress``          runtime/compress/lib/CLALibDecompress.java:56

The column groups live on the device after ``to_device``; each product is one C-ABI call. Failures
raise ``CLAError`` (the reference wraps its failures in DMLCompressionException / RuntimeException).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import native
from .colgroup import (AColGroup, ASDC, AColGroupOffset, ColGroupConst, ColGroupDDC, ColGroupDDCFOR, ColGroupEmpty,
                       ColGroupOLE, ColGroupRLE, ColGroupSDCFOR, ColGroupUncompressed, ColGroupUncompressedDev)
from .mapping import DeviceMap
from .native import check, ptr

CHAIN_XtXv, CHAIN_XtwXv = 0, 1


def _f64(a, shape=None) -> np.ndarray:
    a = np.ascontiguousarray(np.asarray(a, dtype=np.float64))
    return a if shape is None else a.reshape(shape)


class CompressedMatrixBlock:
    def __init__(self, rlen: int, clen: int, colGroups=None, overlapping: bool = False):
        self.rlen = int(rlen)
        self.clen = int(clen)
        self._colGroups: list[AColGroup] = list(colGroups or [])
        self.overlappingColGroups = bool(overlapping)
        self._handle = 0
        self.device = None

    # --- reference accessors -------------------------------------------------------------------
    def getNumRows(self):
        return self.rlen

    def getNumColumns(self):
        return self.clen

    def getColGroups(self):
        return self._colGroups

    def allocateColGroup(self, g: AColGroup):
        if self._handle:
            raise RuntimeError("block is already on the device")
        self._colGroups.append(g)

    def isOverlapping(self):
        return self.overlappingColGroups

    def isEmpty(self):
        return self.rlen == 0 or self.clen == 0 or len(self._colGroups) == 0

    def index_bytes(self) -> int:
        return sum(g.index_bytes() for g in self._colGroups)

    # --- serialized form (CompressedMatrixBlock.java:470-519) -----------------------------------
    def write(self, nonZeros: int = -1) -> bytes:
        """The byte stream of ``write(DataOutput)``."""
        from . import wire
        return wire.write_compressed_matrix_block(self, nonZeros)

    @staticmethod
    def read(buf) -> "CompressedMatrixBlock":
        """``CompressedMatrixBlock.read(DataInput)``: host-side groups, not yet on the device."""
        from . import wire
        return wire.read_compressed_matrix_block(buf)[0]

    @staticmethod
    def read_to_device(buf, device: int = 0) -> "CompressedMatrixBlock":
        """Hands the byte stream to the native library's own reader (``cla_read_block``) and uploads: no host-side
        group objects are built, ``getColGroups()`` stays empty."""
        L = native.lib()
        raw = np.frombuffer(bytes(buf), dtype=np.uint8)
        used = C.c_int64(0)
        h = check(L.cla_read_block(ptr(raw), raw.shape[0], None, C.byref(used)))
        st = native.cla_stats()
        try:
            check(L.cla_stats_get(h, C.byref(st)))
            check(L.cla_finalize(h, int(device)))
        except Exception:
            L.cla_destroy(h)
            raise
        cmb = CompressedMatrixBlock(st.n_rows, st.n_cols)
        cmb._handle, cmb.device, cmb._reg_index = h, int(device), list(range(st.n_groups))
        return cmb

    # --- device residency ----------------------------------------------------------------------
    def to_device(self, device: int = 0) -> "CompressedMatrixBlock":
        """Register every group with the native library and upload (cla_create .. cla_finalize)."""
        if self._handle:
            return self
        L = native.lib()
        h = check(L.cla_create(self.rlen, self.clen, int(self.overlappingColGroups)))
        try:
            self._reg_index = []  # native group index of every column group (FOR groups register a second, constant one)
            n_native = 0
            for g in self._colGroups:
                self._reg_index.append(n_native)
                self._add(L, h, g)
                n_native += 1
                if isinstance(g, (ColGroupDDCFOR, ColGroupSDCFOR)):
                    # IFrameOfReferenceGroup.extractCommon (CLALibUtils.java:196-197): the reference becomes constV
                    check(L.cla_add_group_const(h, ptr(g._colIndexes), g.getNumCols(), ptr(g._reference)))
                    n_native += 1
            check(L.cla_finalize(h, int(device)))
        except Exception:
            L.cla_destroy(h)
            raise
        self._handle = h
        self.device = int(device)
        return self

    def _add(self, L, h, g: AColGroup):
        cols, gc = ptr(g._colIndexes), g.getNumCols()
        if isinstance(g, ColGroupDDC) and isinstance(g._data, DeviceMap):
            m = g._data
            check(L.cla_add_group_ddc_dev(h, cols, gc, ptr(g._dict), g.getNumValues(), m.type, C.c_void_p(m.dptr), m.size))
        elif isinstance(g, ColGroupUncompressedDev):
            if g._numRows != self.rlen:
                raise ValueError("uncompressed group must have one row per matrix row")
            check(L.cla_add_group_uncompressed_dev(h, cols, gc, C.c_void_p(g.dptr)))
        elif isinstance(g, ColGroupDDC):
            m = g._data
            check(L.cla_add_group_ddc(h, cols, gc, ptr(g._dict), g.getNumValues(), m.type, ptr(m.data), ptr(m.data2),
                                      m.size))
        elif isinstance(g, ASDC):
            o, m = g._indexes, g._data
            check(L.cla_add_group_sdc(h, cols, gc, ptr(g._dict), g.getNumValues(), ptr(g._defaultTuple), o.type,
                                      o.first, o.last, ptr(o.data), 0 if o.data is None else o.data.shape[0], o.size,
                                      0 if m is None else m.type, None if m is None else self._map_ptr(m),
                                      None if m is None else ptr(m.data2)))
        elif isinstance(g, ColGroupRLE):
            check(L.cla_add_group_rle(h, cols, gc, ptr(g._dict), g.getNumValues(), ptr(g._ptr), ptr(g._data),
                                      g._data.shape[0]))
        elif isinstance(g, ColGroupOLE):
            check(L.cla_add_group_ole(h, cols, gc, ptr(g._dict), g.getNumValues(), ptr(g._ptr), ptr(g._data),
                                      g._data.shape[0]))
        elif isinstance(g, ColGroupUncompressed):
            if g._data.shape[0] != self.rlen:
                raise ValueError("uncompressed group must have one row per matrix row")
            check(L.cla_add_group_uncompressed(h, cols, gc, ptr(g._data)))
        elif isinstance(g, ColGroupConst):
            check(L.cla_add_group_const(h, cols, gc, ptr(g._dict)))
        elif isinstance(g, ColGroupEmpty):
            check(L.cla_add_group_empty(h, cols, gc))
        else:
            raise native.CLAError(-3, f"unsupported column group {type(g).__name__}")

    @staticmethod
    def _map_ptr(m):
        # a MapToZero over the listed rows still marks "has a map": pass a non-null dummy
        if m.data is None:
            return C.c_void_p(C.addressof(_DUMMY))
        return ptr(m.data)

    def handle(self) -> int:
        if not self._handle:
            raise RuntimeError("CompressedMatrixBlock is not on the device; call to_device() first")
        return self._handle

    def free(self):
        if self._handle:
            native.lib().cla_destroy(self._handle)
            self._handle = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def stats(self) -> dict:
        st = native.cla_stats()
        check(native.lib().cla_stats_get(self.handle(), C.byref(st)))
        return {n: getattr(st, n) for n, _ in st._fields_}

    # --- the MatrixBlock operator API of the reference (CompressedMatrixBlock.java:587-627) -----
    def aggregateBinaryOperations(self, m1, m2, transposeLeft: bool = False, transposeRight: bool = False):
        """``m1 %*% m2`` where one side is this block (CLALibMatrixMult.matrixMultiply picks right / left)."""
        if m1 is not self and m2 is not self:
            raise ValueError("one operand must be this CompressedMatrixBlock")
        return CLALibMatrixMult.matrixMultiply(m1, m2, transposeLeft, transposeRight)

    def transposeSelfMatrixMultOperations(self):
        return CLALibTSMM.leftMultByTransposeSelf(self)

    def chainMatrixMultOperations(self, v, w=None, ctype=CHAIN_XtXv):
        return CLALibMMChain.mmChain(self, v, w, ctype)

    def decompress(self):
        return CLALibDecompress.decompress(self)

    # --- decoded index structures --------------------------------------------------------------
    def group_row_ids(self, g: int) -> np.ndarray:
        ids = np.empty(self.rlen, np.int32)
        check(native.lib().cla_group_decode(self.handle(), self._reg_index[g], ptr(ids)))
        return ids

    def group_counts(self, g: int) -> np.ndarray:
        counts = np.zeros(max(self._colGroups[g].getNumValues(), 1), np.int64)
        check(native.lib().cla_group_counts(self.handle(), self._reg_index[g], ptr(counts)))
        return counts[: self._colGroups[g].getNumValues()]


_DUMMY = C.c_int64(0)


class _Result(np.ndarray):
    """Dense result with the non-zero count the native call returned (MatrixBlock.getNonZeros)."""
    nnz = -1


def _wrap(a: np.ndarray, nnz: int) -> np.ndarray:
    r = a.view(_Result)
    r.nnz = nnz
    return r


class CLALibMatrixMult:
    """``CLALibMatrixMult.matrixMultiply`` (runtime/compress/lib/CLALibMatrixMult.java:42-94): resolves the
    transpose flags so that the compressed side is multiplied as it is stored, then picks right or left."""

    @staticmethod
    def matrixMultiply(m1, m2, transposeLeft: bool = False, transposeRight: bool = False) -> np.ndarray:
        c1, c2 = isinstance(m1, CompressedMatrixBlock), isinstance(m2, CompressedMatrixBlock)
        if c1 and c2:
            return CLALibMatrixMult._doubleCompressedMatrixMultiply(m1, m2, transposeLeft, transposeRight)
        if not c1 and not c2:
            raise native.CLAError(-3, "matrixMultiply: at least one operand must be compressed")
        if (c1 and transposeLeft) or (c2 and transposeRight):
            # t(X) %*% B = t(t(B) %*% X) and A %*% t(X) = t(X %*% t(A)): swap sides (:50-59), transpose the result
            r = CLALibMatrixMult.matrixMultiply(m2, m1, not transposeRight, not transposeLeft)
            return _wrap(np.ascontiguousarray(np.asarray(r).T), r.nnz)
        if c1:
            B = _f64(m2)
            B = B.reshape(-1, 1) if B.ndim == 1 else B
            return CLALibRightMultBy.rightMultByMatrix(m1, np.ascontiguousarray(B.T) if transposeRight else B)
        A = _f64(m1)
        A = A.reshape(1, -1) if A.ndim == 1 else A
        return CLALibLeftMultBy.leftMultByMatrix(m2, np.ascontiguousarray(A.T) if transposeLeft else A)


    @staticmethod
    def _doubleCompressedMatrixMultiply(m1, m2, transposeLeft: bool, transposeRight: bool) -> np.ndarray:
        """Both operands compressed (CLALibMatrixMult.java:96-124): ``m1 %*% m2`` decompresses the right side,
        ``t(m1) %*% m2`` stays compressed on both sides, ``m1 %*% t(m2)`` is not implemented by the reference
        either, and ``t(m1) %*% t(m2)`` is ``t(m2 %*% m1)``."""
        if not transposeLeft and not transposeRight:
            return CLALibRightMultBy.rightMultByMatrix(m1, np.asarray(CLALibDecompress.decompress(m2)))
        if transposeLeft and not transposeRight:
            return CLALibLeftMultBy.leftMultByMatrixTransposed(m2, m1)
        if not transposeLeft and transposeRight:
            raise native.CLAError(-3, "Not Implemented compressed Matrix Mult to produce larger matrix")
        r = CLALibMatrixMult.matrixMultiply(m2, m1)
        return _wrap(np.ascontiguousarray(np.asarray(r).T), r.nnz)


class CLALibRightMultBy:
    @staticmethod
    def rightMultByMatrix(m1: CompressedMatrixBlock, m2, allowOverlap: bool = False):
        """``m1 %*% m2``. With ``allowOverlap`` the result stays compressed (CLALibRightMultBy.java:51,157-201): an
        overlapping ``CompressedMatrixBlock`` on the device that shares ``m1``'s index structures."""
        V = _f64(m2)
        if V.ndim == 1:
            V = V.reshape(-1, 1)
        if V.shape[0] != m1.clen:
            raise native.CLAError(-4, "rightMultByMatrix: inner dimensions do not match")
        if allowOverlap:
            h = check(native.lib().cla_rmm_overlapping(m1.handle(), ptr(V), V.shape[0], V.shape[1]))
            st = native.cla_stats()
            check(native.lib().cla_stats_get(h, C.byref(st)))
            ret = CompressedMatrixBlock(m1.rlen, V.shape[1], overlapping=True)
            ret._handle, ret.device, ret._reg_index = h, m1.device, list(range(st.n_groups))
            return ret
        out = np.empty((m1.rlen, V.shape[1]), np.float64)
        nnz = check(native.lib().cla_rmm(m1.handle(), ptr(V), V.shape[0], V.shape[1], ptr(out)))
        return _wrap(out, nnz)


class CLALibLeftMultBy:
    @staticmethod
    def leftMultByMatrix(right: CompressedMatrixBlock, left) -> np.ndarray:
        """``left %*% right`` with ``left`` dense ``[q x nRows]``."""
        Yt = _f64(left)
        if Yt.ndim == 1:
            Yt = Yt.reshape(1, -1)
        if Yt.shape[1] != right.rlen:
            raise native.CLAError(-4, "leftMultByMatrix: inner dimensions do not match")
        out = np.empty((Yt.shape[0], right.clen), np.float64)
        nnz = check(native.lib().cla_lmm(right.handle(), ptr(Yt), Yt.shape[0], ptr(out)))
        return _wrap(out, nnz)

    @staticmethod
    def leftMultByMatrixTransposed(right: CompressedMatrixBlock, left) -> np.ndarray:
        """``t(left) %*% right`` with ``left`` dense ``[nRows x q]`` (CLALibLeftMultBy.java:73-83) or a second
        compressed block over the same rows (:100-112)."""
        if isinstance(left, CompressedMatrixBlock):
            if left.rlen != right.rlen:
                raise native.CLAError(-4, "leftMultByMatrixTransposed: inner dimensions do not match")
            out = np.empty((left.clen, right.clen), np.float64)
            nnz = check(native.lib().cla_tmm(left.handle(), right.handle(), ptr(out)))
            return _wrap(out, nnz)
        L = _f64(left)
        if L.ndim == 1:
            L = L.reshape(-1, 1)
        return CLALibLeftMultBy.leftMultByMatrix(right, np.ascontiguousarray(L.T))


class CLALibTSMM:
    @staticmethod
    def leftMultByTransposeSelf(cmb: CompressedMatrixBlock) -> np.ndarray:
        out = np.empty((cmb.clen, cmb.clen), np.float64)
        nnz = check(native.lib().cla_tsmm(cmb.handle(), ptr(out)))
        return _wrap(out, nnz)


class CLALibMMChain:
    @staticmethod
    def mmChain(x: CompressedMatrixBlock, v, w=None, ctype: int = CHAIN_XtXv, allowOverlap: bool = False) -> np.ndarray:
        """``t(x) %*% (w * (x %*% v))``. ``allowOverlap`` (XtXv only) keeps the intermediate ``x %*% v`` compressed and
        multiplies the two compressed blocks (CLALibMMChain.java:109-122,128-131)."""
        v = _f64(v).reshape(-1)
        if v.shape[0] != x.clen:
            raise native.CLAError(-4, "mmChain: v must have nCols entries")
        if allowOverlap and ctype == CHAIN_XtXv:
            tmp = CLALibRightMultBy.rightMultByMatrix(x, v, allowOverlap=True)
            try:
                return CLALibLeftMultBy.leftMultByMatrixTransposed(tmp, x)
            finally:
                tmp.free()
        wv = None
        if ctype == CHAIN_XtwXv:
            if w is None:
                raise native.CLAError(-2, "mmChain: XtwXv needs w")
            wv = _f64(w).reshape(-1)
            if wv.shape[0] != x.rlen:
                raise native.CLAError(-4, "mmChain: w must have nRows entries")
        out = np.empty((x.clen, 1), np.float64)
        nnz = check(native.lib().cla_mmchain(x.handle(), ptr(v), ptr(wv), int(ctype), ptr(out)))
        return _wrap(out, nnz)


class CLALibCompAgg:
    """Sum and min / max aggregates of ``CLALibCompAgg.aggregateUnary`` (runtime/compress/lib/CLALibCompAgg.java):
    uack+, uark+, uak+, uacmin/max, uarmin/max, uamin/max."""

    @staticmethod
    def colSums(cmb: CompressedMatrixBlock) -> np.ndarray:
        out = np.empty((1, cmb.clen), np.float64)
        check(native.lib().cla_unary_agg(cmb.handle(), 0, ptr(out)))
        return out

    @staticmethod
    def rowSums(cmb: CompressedMatrixBlock) -> np.ndarray:
        out = np.empty((cmb.rlen, 1), np.float64)
        check(native.lib().cla_unary_agg(cmb.handle(), 1, ptr(out)))
        return out

    @staticmethod
    def sum(cmb: CompressedMatrixBlock) -> float:
        out = np.empty(1, np.float64)
        check(native.lib().cla_unary_agg(cmb.handle(), 2, ptr(out)))
        return float(out[0])


    @staticmethod
    def _agg(cmb, op, shape):
        out = np.empty(shape, np.float64)
        check(native.lib().cla_unary_agg(cmb.handle(), op, ptr(out)))
        return out

    @staticmethod
    def colMins(cmb: CompressedMatrixBlock) -> np.ndarray:
        return CLALibCompAgg._agg(cmb, 3, (1, cmb.clen))

    @staticmethod
    def colMaxs(cmb: CompressedMatrixBlock) -> np.ndarray:
        return CLALibCompAgg._agg(cmb, 4, (1, cmb.clen))

    @staticmethod
    def rowMins(cmb: CompressedMatrixBlock) -> np.ndarray:
        return CLALibCompAgg._agg(cmb, 5, (cmb.rlen, 1))

    @staticmethod
    def rowMaxs(cmb: CompressedMatrixBlock) -> np.ndarray:
        return CLALibCompAgg._agg(cmb, 6, (cmb.rlen, 1))

    @staticmethod
    def min(cmb: CompressedMatrixBlock) -> float:
        return float(CLALibCompAgg._agg(cmb, 7, (1,))[0])

    @staticmethod
    def max(cmb: CompressedMatrixBlock) -> float:
        return float(CLALibCompAgg._agg(cmb, 8, (1,))[0])


class CLALibDecompress:
    @staticmethod
    def decompress(cmb: CompressedMatrixBlock) -> np.ndarray:
        out = np.empty((cmb.rlen, cmb.clen), np.float64)
        nnz = check(native.lib().cla_decompress(cmb.handle(), ptr(out)))
        return _wrap(out, nnz)
