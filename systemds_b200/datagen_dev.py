"""The five benchmark workloads generated on the GPU at their full sizes.

``datagen.py`` draws every map on the host (numpy Philox streams; that is what the parity tests use, because the CPU
oracle needs the same arrays). At the benchmark sizes that costs minutes per rank (12.5 G cells for one shard of the
lmCG workload), so the functions here draw the large index maps and the dense block with torch on the device, in the
reference's storage layouts, and register them through ``cla_add_group_ddc_dev`` / ``cla_add_group_uncompressed_dev``.
The small index structures (SDC offset lists, RLE runs) are still built on the host, directly from geometric gaps and
run lengths instead of one id per row. Same shapes, cardinalities and distributions as ``datagen.config1..5``; the
streams differ (torch's Philox, seeded by ``seed`` and the shard's first row).

torch is used for device memory and random numbers only.
"""
from __future__ import annotations

import numpy as np

from .cmb import CompressedMatrixBlock
from .colgroup import ColGroupDDC, ColGroupRLE, ColGroupSDCZeros, ColGroupUncompressedDev
from .datagen import _rng, normal
from .mapping import MAP_BIT, DeviceMap, MapToFactory
from .offset import OffsetFactory


def _gen(seed: int, row0: int, device):
    import torch
    g = torch.Generator(device=device)
    g.manual_seed((int(seed) << 20) ^ (int(row0) // 1024))
    return g


def _uniform_map(n: int, card: int, gen, device) -> DeviceMap:
    """Uniform ids in [0, card) in the map class ``MapToFactory`` picks (MapToFactory.java:102-117)."""
    import torch
    t = MapToFactory.type_for(n, card)
    if t == MAP_BIT:  # long[] words, bit r & 63 of word r >> 6, LSB first (MapToBit.java:100-103)
        nb = (n + 63) // 64 * 8
        bits = torch.randint(0, 2, (nb * 8,), dtype=torch.uint8, device=device, generator=gen)
        if nb * 8 > n:
            bits[n:] = 0
        w = (bits.view(-1, 8) * (2 ** torch.arange(8, device=device, dtype=torch.uint8))).sum(dim=1, dtype=torch.uint8)
        return DeviceMap(t, n, card, w.data_ptr(), w.numel(), owner=w)
    if card <= 256:
        ids = torch.randint(0, card, (n,), dtype=torch.uint8, device=device, generator=gen)
        return DeviceMap(t, n, card, ids.data_ptr(), n, owner=ids)
    ids = torch.randint(0, card, (n,), dtype=torch.int16 if card <= 32768 else torch.int32, device=device, generator=gen)
    if ids.dtype == torch.int32:
        ids = (ids & 0xFFFF).to(torch.int16)  # u16 bit pattern (MapToChar holds char[])
    return DeviceMap(t, n, card, ids.data_ptr(), n * 2, owner=ids)


def config1(nRows=1_000_000, nCols=100, seed=1001, row0=0, device=0):
    """X %*% v: single-column DDC, 16 values N(0,1), uniform ids (MapToUByte)."""
    import torch
    dev = torch.device("cuda", device)
    gen = _gen(seed, row0, dev)
    groups = [ColGroupDDC([c], normal(seed, c, (16, 1)), _uniform_map(nRows, 16, gen, dev)) for c in range(nCols)]
    return CompressedMatrixBlock(nRows, nCols, groups), normal(seed, 1 << 20, (nCols, 1))


def config2(nRows=10_000_000, nCols=200, seed=1002, row0=0, device=0):
    """t(y) %*% X: single-column DDC, 256 values N(0,1), uniform ids (MapToByte); y ~ N(0,1) as a device tensor."""
    import torch
    dev = torch.device("cuda", device)
    gen = _gen(seed, row0, dev)
    groups = [ColGroupDDC([c], normal(seed, c, (256, 1)), _uniform_map(nRows, 256, gen, dev)) for c in range(nCols)]
    y = torch.randn(nRows, dtype=torch.float64, device=dev, generator=gen)
    return CompressedMatrixBlock(nRows, nCols, groups), y


def config3(nRows=10_000_000, nCols=500, vCols=64, seed=1003, row0=0, device=0):
    """X %*% V on mixed groups: 40% DDC (4 values), 30% SDCZeros (5% listed rows, 8 values), 20% RLE (32 values,
    geometric runs of mean 1000, a run's value differs from the previous one), 10% one dense uncompressed group."""
    import torch
    dev = torch.device("cuda", device)
    gen = _gen(seed, row0, dev)
    n_ddc, n_sdc, n_rle = int(nCols * 0.4), int(nCols * 0.3), int(nCols * 0.2)
    n_unc = nCols - n_ddc - n_sdc - n_rle
    blk = row0 // 1024
    groups, c = [], 0
    for _ in range(n_ddc):
        groups.append(ColGroupDDC([c], normal(seed, c, (4, 1)), _uniform_map(nRows, 4, gen, dev)))
        c += 1
    for _ in range(n_sdc):  # Bernoulli(0.05) rows = geometric gaps
        rng = _rng(seed, c, blk, 2)
        gaps = rng.geometric(0.05, size=int(nRows * 0.05 * 1.1) + 64)
        rows = np.cumsum(gaps) - 1
        while rows[-1] < nRows:
            more = rng.geometric(0.05, size=gaps.shape[0])
            rows = np.concatenate([rows, rows[-1] + np.cumsum(more)])
        rows = rows[rows < nRows]
        ids = rng.integers(0, 8, size=rows.shape[0])
        groups.append(ColGroupSDCZeros([c], nRows, normal(seed, c, (8, 1)), OffsetFactory.createOffset(rows),
                                       MapToFactory.create_from(ids, 8)))
        c += 1
    for _ in range(n_rle):
        rng = _rng(seed, c, blk, 1)
        lens = rng.geometric(1.0 / 1000, size=int(nRows / 1000 * 1.2) + 16)
        while lens.sum() < nRows:
            lens = np.concatenate([lens, rng.geometric(1.0 / 1000, size=lens.shape[0])])
        ends = np.cumsum(lens)
        k = int(np.searchsorted(ends, nRows)) + 1
        lens = lens[:k].copy()
        lens[-1] -= ends[k - 1] - nRows
        vals = np.cumsum(rng.integers(1, 32, size=k)) % 32
        groups.append(ColGroupRLE.from_runs([c], normal(seed, c, (32, 1)), np.cumsum(lens) - lens, lens, vals, nRows))
        c += 1
    if n_unc:
        dense = torch.randn((nRows, n_unc), dtype=torch.float64, device=dev, generator=gen)
        groups.append(ColGroupUncompressedDev(list(range(c, c + n_unc)), nRows, dense.data_ptr(), owner=dense))
    return CompressedMatrixBlock(nRows, nCols, groups), normal(seed, 1 << 20, (nCols, vCols))


def config4(nRows=20_000_000, nCols=100, card=1000, seed=1004, row0=0, device=0, s=1.1):
    """t(X) %*% X: single-column DDC, 1000 values U(-1,1), ids Zipf(1.1) over ranks 0..999 by inverse CDF (MapToChar)."""
    import torch
    dev = torch.device("cuda", device)
    gen = _gen(seed, row0, dev)
    w = 1.0 / np.power(np.arange(1, card + 1, dtype=np.float64), s)
    cdf = torch.from_numpy(np.cumsum(w / w.sum())).to(dev)
    groups = []
    for c in range(nCols):
        u = torch.rand(nRows, dtype=torch.float64, device=dev, generator=gen)
        ids = torch.searchsorted(cdf, u).clamp_(max=card - 1).to(torch.int16)
        d = _rng(seed, c, 0, 7).uniform(-1.0, 1.0, size=(card, 1))
        groups.append(ColGroupDDC([c], d, DeviceMap(MapToFactory.type_for(nRows, card), nRows, card, ids.data_ptr(),
                                                    nRows * 2, owner=ids)))
    return CompressedMatrixBlock(nRows, nCols, groups)


def config5(nRows=12_500_000, nCols=1000, seed=1005, row0=0, device=0):
    """lmCG inner step: single-column DDC, per-column cardinality uniform in [2, 255] (MapToBit / MapToUByte /
    MapToByte by cardinality), N(0,1) dictionaries, uniform ids. The cardinalities and dictionaries are the same
    for every shard; the ids depend on ``row0``."""
    import torch
    dev = torch.device("cuda", device)
    gen = _gen(seed, row0, dev)
    cards = _rng(seed, 1 << 21, 0, 5).integers(2, 256, size=nCols)
    groups = []
    for c in range(nCols):
        k = int(cards[c])
        groups.append(ColGroupDDC([c], normal(seed, c, (k, 1)), _uniform_map(nRows, k, gen, dev)))
    return CompressedMatrixBlock(nRows, nCols, groups), normal(seed, 1 << 20, (nCols, 1))


def release_sources(cmb: CompressedMatrixBlock) -> None:
    """Drop the generator's device tensors once the block is on the device (the native library holds its own copy)."""
    for g in cmb.getColGroups():
        d = getattr(g, "_data", None)
        if isinstance(d, DeviceMap):
            d.owner = None
        if isinstance(g, ColGroupUncompressedDev):
            g.owner = None
