"""Seeded synthetic compressed matrices, generated directly as column groups.

The five workloads follow the benchmark configurations of this path (shapes, cardinalities and
value distributions); ``random_cmb`` builds small mixed matrices covering every group type for
the parity tests. Random streams are counter based (Philox keyed by seed, counter = (group, row
block)), so any row range that starts on a ``BLOCK`` boundary can be generated on its own --
that is how row shards are produced without materialising the whole matrix.
"""
from __future__ import annotations

import numpy as np

from .colgroup import (ColGroupConst, ColGroupDDC, ColGroupDDCFOR, ColGroupEmpty, ColGroupOLE, ColGroupRLE, ColGroupSDC,
                       ColGroupSDCFOR, ColGroupUncompressed, sdc_from_row_ids)
from .cmb import CompressedMatrixBlock
from .mapping import MapToFactory

BLOCK = 1 << 20  # rows per random block


def _rng(seed: int, group: int, block: int = 0, stream: int = 0) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=int(seed), counter=[int(group), int(block), int(stream), 0]))


def _blocks(row0: int, n: int):
    if row0 % BLOCK:
        raise ValueError("row ranges must start on a BLOCK boundary")
    b = row0 // BLOCK
    done = 0
    while done < n:
        m = min(BLOCK, n - done)
        yield b, done, m
        done += m
        b += 1


def uniform_ids(seed, group, row0, n, card, dtype=None) -> np.ndarray:
    dt = dtype or (np.uint8 if card <= 256 else (np.uint16 if card <= 65536 else np.int32))
    out = np.empty(n, dt)
    for b, o, m in _blocks(row0, n):
        out[o:o + m] = _rng(seed, group, b).integers(0, card, size=BLOCK, dtype=dt)[:m]
    return out


def zipf_ids(seed, group, row0, n, card, s=1.1) -> np.ndarray:
    """Ids distributed Zipf(s) over ranks 0..card-1 (rank = dictionary id), by inverse CDF."""
    w = 1.0 / np.power(np.arange(1, card + 1, dtype=np.float64), s)
    cdf = np.cumsum(w / w.sum())
    dt = np.uint8 if card <= 256 else (np.uint16 if card <= 65536 else np.int32)
    out = np.empty(n, dt)
    for b, o, m in _blocks(row0, n):
        u = _rng(seed, group, b).random(BLOCK)[:m]
        out[o:o + m] = np.minimum(np.searchsorted(cdf, u), card - 1).astype(dt)
    return out


def normal(seed, group, shape, stream=7) -> np.ndarray:
    return _rng(seed, group, 0, stream).standard_normal(shape)


def _ddc(col, dict_, ids, card):
    return ColGroupDDC([col] if np.isscalar(col) else col, dict_, MapToFactory.create_from(ids, card))


# ---- the five workloads ----------------------------------------------------------------------------
def config1(nRows=1_000_000, nCols=100, seed=1001, row0=0):
    """X %*% v: single-column DDC groups, 16 values N(0,1) each, uniform ids (MapToUByte). v ~ N(0,1)."""
    groups = [_ddc(c, normal(seed, c, (16, 1)), uniform_ids(seed, c, row0, nRows, 16), 16) for c in range(nCols)]
    v = normal(seed, 1 << 20, (nCols, 1))
    return CompressedMatrixBlock(nRows, nCols, groups), v


def config2(nRows=10_000_000, nCols=200, seed=1002, variant="a", row0=0):
    """t(y) %*% X: cardinality 256 per column (MapToByte). Variants: a = single columns, b = pairs whose
    second column is a fixed permutation of the first (joint cardinality 256), c = independent pairs
    co-coded with 65536 tuples (MapToChar). y ~ N(0,1), generated for the same row range."""
    groups = []
    if variant == "a":
        for c in range(nCols):
            groups.append(_ddc(c, normal(seed, c, (256, 1)), uniform_ids(seed, c, row0, nRows, 256), 256))
    elif variant == "b":
        for p in range(nCols // 2):
            d0 = normal(seed, 2 * p, (256, 1))
            d1 = normal(seed, 2 * p + 1, (256, 1))
            perm = _rng(seed, 2 * p + 1, 0, 3).permutation(256)
            groups.append(_ddc([2 * p, 2 * p + 1], np.hstack([d0, d1[perm]]), uniform_ids(seed, 2 * p, row0, nRows, 256), 256))
    elif variant == "c":
        for p in range(nCols // 2):
            d0 = normal(seed, 2 * p, (256, 1)).reshape(-1)
            d1 = normal(seed, 2 * p + 1, (256, 1)).reshape(-1)
            dict_ = np.stack([np.repeat(d0, 256), np.tile(d1, 256)], axis=1)
            ids = uniform_ids(seed, 2 * p, row0, nRows, 256).astype(np.uint16) * 256 + uniform_ids(seed, 2 * p + 1, row0, nRows, 256)
            groups.append(_ddc([2 * p, 2 * p + 1], dict_, ids, 65536))
    else:
        raise ValueError(variant)
    y = np.empty(nRows)
    for b, o, m in _blocks(row0, nRows):
        y[o:o + m] = _rng(seed, 1 << 20, b).standard_normal(BLOCK)[:m]
    return CompressedMatrixBlock(nRows, nCols, groups), y.reshape(1, -1)


def _geometric_runs(seed, group, nRows, nVals, mean_len):
    """Consecutive runs with geometric lengths; the value of a run is uniform and differs from the previous one."""
    rng = _rng(seed, group, 0, 1)
    n_est = int(nRows / mean_len * 1.2) + 16
    lens = rng.geometric(1.0 / mean_len, size=n_est)
    while lens.sum() < nRows:
        lens = np.concatenate([lens, rng.geometric(1.0 / mean_len, size=n_est)])
    ends = np.cumsum(lens)
    nruns = int(np.searchsorted(ends, nRows)) + 1
    lens = lens[:nruns].copy()
    lens[-1] -= ends[nruns - 1] - nRows
    step = rng.integers(1, nVals, size=nruns) if nVals > 1 else np.zeros(nruns, np.int64)
    vals = np.cumsum(step) % nVals
    return np.repeat(vals, lens).astype(np.int32)


def config3(nRows=10_000_000, nCols=500, vCols=64, seed=1003):
    """X %*% V on mixed groups: 40% DDC (4 values), 30% SDCZeros (5% non-default rows, 8 values),
    20% RLE (32 values, geometric runs of mean 1000), 10% one dense uncompressed group. V ~ N(0,1)."""
    n_ddc, n_sdc, n_rle = int(nCols * 0.4), int(nCols * 0.3), int(nCols * 0.2)
    n_unc = nCols - n_ddc - n_sdc - n_rle
    groups, c = [], 0
    for _ in range(n_ddc):
        groups.append(_ddc(c, normal(seed, c, (4, 1)), uniform_ids(seed, c, 0, nRows, 4), 4))
        c += 1
    for _ in range(n_sdc):
        rng = _rng(seed, c, 0, 2)
        mask = rng.random(nRows) < 0.05
        ids = np.full(nRows, -1, np.int32)
        ids[mask] = rng.integers(0, 8, size=int(mask.sum()))
        groups.append(sdc_from_row_ids([c], normal(seed, c, (8, 1)), ids))
        c += 1
    for _ in range(n_rle):
        groups.append(ColGroupRLE.from_row_ids([c], normal(seed, c, (32, 1)), _geometric_runs(seed, c, nRows, 32, 1000)))
        c += 1
    if n_unc:
        groups.append(ColGroupUncompressed(list(range(c, c + n_unc)), _rng(seed, c, 0, 4).standard_normal((nRows, n_unc))))
    V = normal(seed, 1 << 20, (nCols, vCols))
    return CompressedMatrixBlock(nRows, nCols, groups), V


def config4(nRows=20_000_000, nCols=100, card=1000, seed=1004, row0=0):
    """t(X) %*% X: single-column DDC, 1000 values U(-1,1), Zipf(1.1) ids (MapToChar)."""
    groups = []
    for c in range(nCols):
        d = _rng(seed, c, 0, 7).uniform(-1.0, 1.0, size=(card, 1))
        groups.append(_ddc(c, d, zipf_ids(seed, c, row0, nRows, card), card))
    return CompressedMatrixBlock(nRows, nCols, groups)


def config5(nRows=12_500_000, nCols=1000, seed=1005, row0=0):
    """lmCG inner step w = t(X) (X v) + 1e-3 v: single-column DDC, per-column cardinality uniform in [2, 255]
    (MapToBit / MapToUByte / MapToByte by cardinality). Rows [row0, row0 + nRows) of the full matrix."""
    cards = _rng(seed, 1 << 21, 0, 5).integers(2, 256, size=nCols)
    groups = []
    for c in range(nCols):
        k = int(cards[c])
        groups.append(_ddc(c, normal(seed, c, (k, 1)), uniform_ids(seed, c, row0, nRows, k), k))
    v = normal(seed, 1 << 20, (nCols, 1))
    return CompressedMatrixBlock(nRows, nCols, groups), v


# ---- small mixed matrices for parity tests ---------------------------------------------------------
KINDS = ("ddc", "ddc2", "ddc_bit", "ddc_char", "sdc", "sdcz", "sdcs", "sdcsz", "rle", "ole", "unc", "const", "empty")


def random_group(kind, cols, nRows, rng, integer=False):
    gc = len(cols)

    def dict_(n):
        d = rng.integers(-3, 4, size=(n, gc)).astype(np.float64) if integer else rng.standard_normal((n, gc))
        return d

    if kind in ("ddc", "ddc2"):
        card = int(rng.integers(3, 60))
        return ColGroupDDC(cols, dict_(card), MapToFactory.create_from(rng.integers(0, card, nRows), card))
    if kind == "ddcfor":
        card = int(rng.integers(3, 40))
        return ColGroupDDCFOR(cols, dict_(card), rng.standard_normal(gc), MapToFactory.create_from(rng.integers(0, card, nRows), card))
    if kind == "sdcfor":
        base = random_group("sdcz", cols, nRows, rng, integer)
        if base._data is None:  # one tuple only: give it a map so the FOR class (which always has one) applies
            base = random_group("ddcfor", cols, nRows, rng, integer)
            return base
        return ColGroupSDCFOR(cols, nRows, base._dict, base._indexes, base._data, rng.standard_normal(gc))
    if kind == "ddc_bit":
        return ColGroupDDC(cols, dict_(2), MapToFactory.create_from(rng.integers(0, 2, nRows), 2))
    if kind == "ddc_char":
        card = int(rng.integers(300, 900))
        return ColGroupDDC(cols, dict_(card), MapToFactory.create_from(rng.integers(0, card, nRows), card))
    if kind in ("sdc", "sdcz", "sdcs", "sdcsz"):
        card = 1 if kind in ("sdcs", "sdcsz") else int(rng.integers(2, 12))
        dens = float(rng.choice([0.002, 0.05, 0.3]))
        ids = np.full(nRows, -1, np.int32)
        mask = rng.random(nRows) < dens
        ids[mask] = rng.integers(0, card, int(mask.sum()))
        default = None if kind in ("sdcz", "sdcsz") else (rng.integers(1, 4, gc).astype(np.float64) if integer else rng.standard_normal(gc))
        return sdc_from_row_ids(cols, dict_(card), ids, default)
    if kind in ("rle", "ole"):
        card = int(rng.integers(2, 9))
        mean = float(rng.choice([3, 40, 900]))
        lens = rng.geometric(1.0 / mean, size=int(nRows / mean * 2) + 8)
        vals = rng.integers(-1, card, size=lens.shape[0])  # -1 = rows without a tuple
        ids = np.repeat(vals, lens)[:nRows].astype(np.int32)
        if ids.shape[0] < nRows:
            ids = np.concatenate([ids, np.full(nRows - ids.shape[0], -1, np.int32)])
        cls = ColGroupRLE if kind == "rle" else ColGroupOLE
        return cls.from_row_ids(cols, dict_(card), ids)
    if kind == "unc":
        return ColGroupUncompressed(cols, rng.integers(-3, 4, size=(nRows, gc)).astype(np.float64) if integer else rng.standard_normal((nRows, gc)))
    if kind == "const":
        return ColGroupConst(cols, dict_(1))
    if kind == "empty":
        return ColGroupEmpty(cols)
    raise ValueError(kind)


def random_cmb(seed, nRows, kinds=KINDS, overlapping=False, integer=False):
    """One group per entry of ``kinds``; 'ddc2' and 'unc' span two columns. With ``overlapping`` every
    group draws its columns from the full range, so columns are covered by several groups."""
    rng = np.random.default_rng(seed)
    widths = [2 if k in ("ddc2", "unc") else 1 for k in kinds]
    nCols = sum(widths)
    groups, c = [], 0
    for k, w in zip(kinds, widths):
        cols = sorted(rng.choice(nCols, size=w, replace=False).tolist()) if overlapping else list(range(c, c + w))
        groups.append(random_group(k, cols, nRows, rng, integer))
        c += w
    return CompressedMatrixBlock(nRows, nCols, groups, overlapping)
