"""
The bounded-wait path on a GPU, without faulting or hanging it: a wait that nothing will satisfy runs out after the limit
the test passes (1 ms), the kernel stores its code in the status word and returns, the host turns the word into an
exception, and the context keeps working afterwards.
"""

import ctypes as C
import time

import pytest
import torch

from nunchaku_rocm_b200 import _lib as L

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_sets_the_status_word_and_returns(cuda_dev):
    lib = L.lib()
    word = torch.zeros(1, dtype=torch.int32, device=cuda_dev)
    t0 = time.perf_counter()
    with torch.cuda.device(cuda_dev):
        L.check(lib.nb_debug_expire_wait(L.ptr(word), 1000, L.stream_of(word)), "nb_debug_expire_wait")
    torch.cuda.synchronize(cuda_dev)
    assert time.perf_counter() - t0 < 1.0, "the wait did not stop at its limit"
    assert int(word.item()) == 0x7E1
    # limits outside 1 us .. 1 s are refused before anything is launched
    assert lib.nb_debug_expire_wait(L.ptr(word), 0, None) == L.NB_ERR_INVALID
    assert lib.nb_debug_expire_wait(L.ptr(word), 2_000_000, None) == L.NB_ERR_INVALID


def test_the_host_surfaces_an_expired_wait_as_an_error_and_recovers(cuda_dev):
    from nunchaku_rocm_b200.ops.triton.gemm_w4a4 import gemm_w4a4

    lib = L.lib()
    L.check_device_status(cuda_dev)  # clean before
    w = L.status_word(cuda_dev)
    with torch.cuda.device(cuda_dev):
        L.check(lib.nb_debug_expire_wait(L.ptr(w), 1000, L.stream_of(w)), "nb_debug_expire_wait")
    with pytest.raises(L.KernelWaitExpired, match="0x7e1"):
        L.check_device_status(cuda_dev)
    assert L.device_status(cuda_dev) == 0  # cleared by the check, like the reference's last-error read
    # the context is intact: a GEMM right after gives the exact unit-scale result
    M = N = 128
    K = 128
    act = torch.full((M, K // 2), 0x11, dtype=torch.uint8, device=cuda_dev)  # every value 1
    wgt = torch.full((N, K // 2), 0x22, dtype=torch.uint8, device=cuda_dev)  # every value 2
    ones_a = torch.ones(K // 64, M, dtype=torch.bfloat16, device=cuda_dev)
    ones_w = torch.ones(K // 64, N, dtype=torch.bfloat16, device=cuda_dev)
    out = gemm_w4a4(act, wgt, None, ones_a, ones_w)
    torch.cuda.synchronize(cuda_dev)
    assert bool((out.float() == 2.0 * K).all())
    L.check_device_status(cuda_dev)
