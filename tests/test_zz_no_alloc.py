"""The allocation-free left vector product against the regular entry point.

Some hosts cannot allocate device memory at call time (their own pool owns the GPU, or cudaMalloc's device
synchronisation is not acceptable on their hot path); `cla_lmm_vec_noalloc_dev` keeps its scratch in a fixed array
inside the library instead. This file is collected last on purpose: if it fails, every other test has already run.
"""
import ctypes as C

import numpy as np
import pytest

from systemds_b200 import CompressedMatrixBlock, datagen, native
from systemds_b200 import colgroup as cg
from systemds_b200.mapping import MapToFactory
from systemds_b200.native import CLAError, check

pytestmark = pytest.mark.gpu


def _matrix(nRows, seed):
    rng = np.random.default_rng(seed)
    groups = []
    cards = [256] * 40 + list(rng.integers(2, 256, 30)) + [2, 2]
    for c, k in enumerate(cards):
        groups.append(cg.ColGroupDDC([c], rng.standard_normal((int(k), 1)),
                                     MapToFactory.create_from(rng.integers(0, k, nRows), int(k))))
    groups.append(cg.ColGroupConst([len(cards)], [[-1.5]]))  # exercises the row-sum slot of the fixed scratch
    return CompressedMatrixBlock(nRows, len(cards) + 1, groups)


def test_noalloc_matches_regular_entry_point_twice():
    import torch
    L = native.lib()
    dev = torch.device("cuda", 0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for nRows, seed in [(70001, 1), (262144, 2)]:  # two calls in a row share the fixed scratch
        cmb = _matrix(nRows, seed).to_device(0)
        y = torch.from_numpy(np.random.default_rng(seed).standard_normal(nRows)).to(dev)
        want = torch.zeros(cmb.clen, dtype=torch.float64, device=dev)
        got = torch.full((cmb.clen,), 7.0, dtype=torch.float64, device=dev)
        check(L.cla_lmm_dev(cmb.handle(), C.c_void_p(y.data_ptr()), 1, C.c_void_p(want.data_ptr()), stream))
        for _ in range(2):
            got.fill_(7.0)
            check(L.cla_lmm_vec_noalloc_dev(cmb.handle(), C.c_void_p(y.data_ptr()), C.c_void_p(got.data_ptr()), stream))
            torch.cuda.synchronize()
            w, g = want.cpu().numpy(), got.cpu().numpy()
            scale = np.maximum(np.abs(w), 1e-3 * np.abs(w).max())
            assert np.max(np.abs(g - w) / scale) < 1e-12
        cmb.free()


def test_noalloc_rejects_what_it_cannot_run():
    import torch
    L = native.lib()
    cmb = datagen.random_cmb(5, 8192, ("ddc", "sdcz", "rle")).to_device(0)  # not all dense-map groups
    y = torch.zeros(8192, dtype=torch.float64, device="cuda:0")
    out = torch.zeros(cmb.clen, dtype=torch.float64, device="cuda:0")
    with pytest.raises(CLAError) as e:
        check(L.cla_lmm_vec_noalloc_dev(cmb.handle(), C.c_void_p(y.data_ptr()), C.c_void_p(out.data_ptr()), None))
    assert e.value.code == -3
    cmb.free()
