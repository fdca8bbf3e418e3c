"""tlb_argmax_into - the argmax entry point that allocates nothing - against tlb_argmax, through the
C ABI.  The file name sorts last on purpose: the check must hold after every other GPU test has used
the library, as well as when this file runs alone."""
import ctypes as C

import numpy as np
import pytest

import tl_b200 as tl
from tl_b200 import lib

pytestmark = pytest.mark.gpu
T = tl.Tensor.from_numpy
MAX_ELEMS = 1024 * 4096     # limit stated in include/tlb200.h


def pool_in_use():
    used, reserved = C.c_uint64(), C.c_uint64()
    tl.check(lib().tlb_mem_stats(C.byref(used), C.byref(reserved)))
    return used.value


def test_matches_argmax_on_two_calls_in_a_row():
    tl.init()
    rng = np.random.default_rng(11)
    out = tl.Tensor.zeros((1,))
    inputs = []
    # a vocabulary-sized vector with planted ties, then a short one right after it: the second call
    # must not see anything the first left in the shared scratch
    a = rng.standard_normal(128256).astype(np.float32)
    a[[17, 4095, 4096, 90001, 128255]] = 9.0
    inputs.append(a)
    inputs.append(rng.standard_normal(33).astype(np.float32))
    inputs.append(rng.standard_normal(MAX_ELEMS).astype(np.float32))     # exactly the limit
    for tie in (tl.TIE_LAST, tl.TIE_FIRST):
        for a in inputs:
            x = T(a)
            want = x.argmax(tie).item_i64()
            before = pool_in_use()
            got1 = int(x.argmax_into(out, tie).numpy()[0])
            got2 = int(x.argmax_into(out, tie).numpy()[0])
            assert pool_in_use() == before, "tlb_argmax_into must not take memory from the pool"
            assert got1 == want and got2 == want
            ref = np.flatnonzero(a == a.max())
            assert want == (ref[0] if tie == tl.TIE_FIRST else ref[-1])


def test_rejects_what_it_cannot_hold():
    tl.init()
    out = tl.Tensor.zeros((1,))
    too_big = tl.Tensor.zeros((MAX_ELEMS + 1,))
    with pytest.raises(tl.TlbError, match="exceed the fixed scratch"):
        too_big.argmax_into(out)
    assert too_big.argmax().item_i64() == MAX_ELEMS      # the allocating entry point has no such limit (all zeros, last index)
    with pytest.raises(tl.TlbError):
        tl.Tensor.zeros((0,)).argmax_into(out)
    with pytest.raises(tl.TlbError):
        T(np.zeros(4, np.float32)).argmax_into(tl.Tensor.zeros((0,)))
    assert lib().tlb_argmax_into(None, None, 0) != 0
    # the library still works after the refusals
    assert int(T(np.array([1, 5, 2], np.float32)).argmax_into(out).numpy()[0]) == 1
