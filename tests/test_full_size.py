"""The benchmark workloads at their full sizes, generated on the device (systemds_b200.datagen_dev), checked through
size-independent properties: sums of a product against products of sums, the quadratic form against the squared
norm, symmetry. (At these sizes the CPU oracle would run for minutes; the same kernels are compared with it on the
same shapes at smaller sizes in test_gpu_parity.py.)"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _P(t):
    return C.c_void_p(t.data_ptr())


def _setup():
    import torch
    from systemds_b200 import native
    return torch, native.lib(), native.check, torch.device("cuda", 0), C.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_mixed_groups_wide_right_product_full_size():
    """configs[2], 10,000,000 x 500 mixed groups, V 500 x 64: colSums(X %*% V) == colSums(X) %*% V, and rows drawn at
    random equal the same rows of a second call (fixed summation order)."""
    torch, L, check, dev, s = _setup()
    from systemds_b200 import datagen_dev
    n = 10_000_000
    cmb, V = datagen_dev.config3(nRows=n)
    cmb.to_device(0)
    datagen_dev.release_sources(cmb)
    h = cmb.handle()
    Vd = torch.from_numpy(np.ascontiguousarray(V)).to(dev)
    out = torch.empty((n, 64), dtype=torch.float64, device=dev)
    check(L.cla_rmm_dev(h, _P(Vd), 500, 64, _P(out), s))
    lhs = out.sum(dim=0).cpu().numpy()
    sample = out[::1_000_003].clone()
    ones = torch.ones(n, dtype=torch.float64, device=dev)
    cs = torch.empty(500, dtype=torch.float64, device=dev)
    check(L.cla_lmm_dev(h, _P(ones), 1, _P(cs), s))
    torch.cuda.synchronize()
    rhs = cs.cpu().numpy() @ V
    lo, hi = np.empty(1), np.empty(1)
    check(L.cla_unary_agg(h, 7, C.c_void_p(lo.ctypes.data)))  # uamin
    check(L.cla_unary_agg(h, 8, C.c_void_p(hi.ctypes.data)))  # uamax
    bound = n * max(abs(lo[0]), abs(hi[0])) * np.abs(V).sum(axis=0)  # upper bound of the summed magnitudes
    assert np.max(np.abs(lhs - rhs) / bound) < 1e-12
    check(L.cla_rmm_dev(h, _P(Vd), 500, 64, _P(out), s))
    torch.cuda.synchronize()
    assert torch.equal(out[::1_000_003], sample)
    cmb.free()


def test_self_product_full_size():
    """configs[3], 20,000,000 x 100, 1000 values per column, Zipf ids: 1' (X'X) 1 == |X 1|^2 and the result is
    bit-symmetric."""
    torch, L, check, dev, s = _setup()
    from systemds_b200 import datagen_dev
    n = 20_000_000
    cmb = datagen_dev.config4(nRows=n)
    cmb.to_device(0)
    datagen_dev.release_sources(cmb)
    h = cmb.handle()
    Cd = torch.empty((100, 100), dtype=torch.float64, device=dev)
    check(L.cla_tsmm_dev(h, _P(Cd), s))
    ones = torch.ones(100, dtype=torch.float64, device=dev)
    u = torch.empty(n, dtype=torch.float64, device=dev)
    check(L.cla_rmm_dev(h, _P(ones), 100, 1, _P(u), s))
    torch.cuda.synchronize()
    Cm = Cd.cpu().numpy()
    assert np.array_equal(Cm, Cm.T)
    quad, norm2 = float(Cm.sum()), float((u * u).sum())
    # |X|' |X| summed is the magnitude behind the quadratic form; the diagonal alone (all squares) bounds it from below
    assert abs(quad - norm2) <= 1e-12 * float(np.abs(Cm).sum())
    assert np.all(np.diag(Cm) > 0)
    cmb.free()


def test_lmcg_step_full_size():
    """configs[4], one 12,500,000 x 1000 shard: v' (X'(X v)) == |X v|^2, and the step is reproducible bit for bit."""
    torch, L, check, dev, s = _setup()
    from systemds_b200 import datagen_dev
    n = 12_500_000
    cmb, v = datagen_dev.config5(nRows=n)
    cmb.to_device(0)
    datagen_dev.release_sources(cmb)
    h = cmb.handle()
    vd = torch.from_numpy(np.ascontiguousarray(v.reshape(-1))).to(dev)
    w = torch.empty(1000, dtype=torch.float64, device=dev)
    u = torch.empty(n, dtype=torch.float64, device=dev)
    check(L.cla_mmchain_dev(h, _P(vd), None, 0, _P(w), _P(u), s))
    torch.cuda.synchronize()
    quad, norm2 = float(vd @ w), float(u @ u)
    assert abs(quad - norm2) <= 1e-12 * norm2
    w2 = torch.empty_like(w)
    check(L.cla_mmchain_dev(h, _P(vd), None, 0, _P(w2), _P(u), s))
    torch.cuda.synchronize()
    assert torch.equal(w, w2)
    cmb.free()
