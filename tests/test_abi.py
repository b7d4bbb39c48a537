"""The C-ABI library: loads, exports every symbol the header declares, validates arguments on the host."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from systemds_b200 import native
from systemds_b200.native import CLAError, check, ptr

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    txt = open(os.path.join(ROOT, "include", "systemds_cla.h")).read()
    txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
    return sorted(set(re.findall(r"\b(cla_[a-z0-9_]+)\s*\(", txt)))


def test_exports_every_declared_symbol():
    lib = C.CDLL(native.LIB_PATH)
    names = header_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in systemds_cla.h but not exported"
    assert set(names) == set(native.SIGNATURES), "ctypes signatures out of sync with the header"


def test_host_side_validation():
    L = native.lib()
    with pytest.raises(CLAError) as e:
        check(L.cla_create(-1, 2, 0))
    assert e.value.code == -2
    h = check(L.cla_create(10, 2, 0))
    cols = np.array([0], np.int32)
    d = np.array([1.0, 2.0])
    good = np.array([0, 1] * 5, np.uint8)
    with pytest.raises(CLAError) as e:  # map shorter than the matrix
        check(L.cla_add_group_ddc(h, ptr(cols), 1, ptr(d), 2, 3, ptr(good), None, 9))
    assert e.value.code == -4
    with pytest.raises(CLAError) as e:  # id beyond the dictionary
        check(L.cla_add_group_ddc(h, ptr(cols), 1, ptr(d), 2, 3, ptr(np.full(10, 2, np.uint8)), None, 10))
    assert e.value.code == -2 and "id" in str(e.value)
    with pytest.raises(CLAError) as e:  # column outside the matrix
        check(L.cla_add_group_ddc(h, ptr(np.array([2], np.int32)), 1, ptr(d), 2, 3, ptr(good), None, 10))
    assert e.value.code == -4
    assert check(L.cla_add_group_ddc(h, ptr(cols), 1, ptr(d), 2, 3, ptr(good), None, 10)) == 0
    with pytest.raises(CLAError) as e:  # RLE _ptr must span _data
        check(L.cla_add_group_rle(h, ptr(cols), 1, ptr(d), 2, ptr(np.array([0, 2, 3], np.int32)),
                                  ptr(np.array([0, 3, 1, 1], np.uint16)), 4))
    assert e.value.code == -2
    with pytest.raises(CLAError) as e:  # products need finalize first
        check(L.cla_tsmm(h, ptr(np.zeros(4))))
    assert e.value.code == -6
    with pytest.raises(CLAError) as e:
        check(L.cla_rmm(12345678, None, 0, 0, None))
    assert e.value.code == -1
    check(L.cla_destroy(h))
    with pytest.raises(CLAError):
        check(L.cla_destroy(h))


def test_no_cpu_fallback():
    """Without a CUDA device finalize must fail loudly (there is no CPU path in the product)."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    L = native.lib()
    h = check(L.cla_create(4, 1, 0))
    with pytest.raises(CLAError) as e:
        check(L.cla_finalize(h, 0))
    assert e.value.code == -5
    L.cla_destroy(h)
