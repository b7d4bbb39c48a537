"""Row sharding of a CompressedMatrixBlock (one shard per GPU).

Every index structure is per row (DDC map) or a sorted row list (SDC offsets, RLE / OLE runs), and dictionaries
are small, so a matrix splits by rows with the dictionaries replicated. The semantics follow the reference's row
slicing where it has one -- ``AMapToData.slice``, ``AOffset.slice`` with the first offset re-based to the slice
start (colgroup/offset/AOffset.java:578, ColGroupSDCZeros.java:820-830) -- and extend it to RLE and OLE, whose
``sliceRows`` the reference does not implement (ColGroupRLE.java:974-976): runs and segments are cut at the
shard boundary and re-encoded from the shard's first row.

Each shard's products are the exact products of its rows (constant columns included), so the partial results of
``t(Y) %*% X``, ``t(X) %*% X`` and the mmchain over all shards add up to the full result.
"""
from __future__ import annotations

import numpy as np

from . import colgroup as cg
from .cmb import CompressedMatrixBlock
from .mapping import MapToFactory
from .offset import OffsetFactory


def shard_bounds(nRows: int, nShards: int, align: int = 128):
    """Contiguous row ranges, one per shard, starting on multiples of ``align`` (64 keeps bit maps word aligned)."""
    per = -(-nRows // nShards)
    per = -(-per // align) * align
    return [(min(nRows, i * per), min(nRows, (i + 1) * per)) for i in range(nShards)]


def slice_group(g, rl: int, ru: int, nRows: int):
    n = ru - rl
    cols = g.getColIndices()
    if isinstance(g, cg.ColGroupDDC):
        ids = g._data.decode()[rl:ru]
        m = MapToFactory.create_from(ids, g._data.unique, force_type=g._data.type)
        if isinstance(g, cg.ColGroupDDCFOR):
            return cg.ColGroupDDCFOR(cols, g._dict, g._reference, m)
        return cg.ColGroupDDC(cols, g._dict, m)
    if isinstance(g, cg.ASDC):
        rows = g._indexes.decode()
        sel = (rows >= rl) & (rows < ru)
        off = OffsetFactory.createOffset(rows[sel] - rl)
        if isinstance(g, cg.ColGroupSDCFOR):
            m = MapToFactory.create_from(g._data.decode()[sel], g._data.unique, force_type=g._data.type)
            return cg.ColGroupSDCFOR(cols, n, g._dict, off, m, g._reference)
        if g._data is None:
            if g._defaultTuple is None:
                return cg.ColGroupSDCSingleZeros(cols, n, g._dict, off)
            return cg.ColGroupSDCSingle(cols, n, g._dict, g._defaultTuple, off)
        m = MapToFactory.create_from(g._data.decode()[sel], g._data.unique, force_type=g._data.type)
        if g._defaultTuple is None:
            return cg.ColGroupSDCZeros(cols, n, g._dict, off, m)
        return cg.ColGroupSDC(cols, n, g._dict, g._defaultTuple, off, m)
    if isinstance(g, cg.ColGroupRLE):
        return cg.ColGroupRLE.from_row_ids(cols, g._dict, g.row_ids(nRows)[rl:ru])
    if isinstance(g, cg.ColGroupOLE):
        return cg.ColGroupOLE.from_row_ids(cols, g._dict, g.row_ids(nRows)[rl:ru])
    if isinstance(g, cg.ColGroupUncompressed):
        return cg.ColGroupUncompressed(cols, g._data[rl:ru])
    if isinstance(g, (cg.ColGroupConst, cg.ColGroupEmpty)):
        return g
    raise TypeError(type(g).__name__)


def slice_rows(cmb: CompressedMatrixBlock, rl: int, ru: int) -> CompressedMatrixBlock:
    """Rows [rl, ru) of ``cmb`` as a new (host-side) block."""
    if not (0 <= rl <= ru <= cmb.rlen):
        raise ValueError("row range outside the matrix")
    groups = [slice_group(g, rl, ru, cmb.rlen) for g in cmb.getColGroups()]
    return CompressedMatrixBlock(ru - rl, cmb.clen, groups, cmb.isOverlapping())


def shard(cmb: CompressedMatrixBlock, nShards: int):
    return [slice_rows(cmb, a, b) for a, b in shard_bounds(cmb.rlen, nShards)]
