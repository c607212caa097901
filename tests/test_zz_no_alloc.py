"""
nb_gemm_w4a4_noalloc: the W4A4 GEMM with its scratch block in a fixed device array of the library (no allocation by the
library or, for scratch, by the caller).  Checked against nb_gemm_w4a4 with caller-provided scratch on the same inputs:
the two run the same kernels, so the outputs must be bit-equal.  This file sorts last on purpose: the entry point has
to work on a device context that has already run every other kernel, and alone.
"""

import ctypes as C

import pytest
import torch

from oracle import w4a4 as ow

pytestmark = pytest.mark.gpu


def _problem(M, N, K, R, dev, seed):
    g = torch.Generator().manual_seed(seed)
    act = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g)
    wgt = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    asc = (torch.rand(K // 64, M, generator=g) * 0.2 + 0.01).to(torch.bfloat16)
    wsc = (torch.rand(K // 64, N, generator=g) * 0.02 + 0.005).to(torch.bfloat16)
    bias = torch.randn(N, generator=g).to(torch.bfloat16)
    la = torch.randn(M, R, generator=g) * 0.5
    lu = (torch.randn(N, R, generator=g) * 0.05).to(torch.bfloat16)
    cpu = dict(act=act, wgt=wgt, asc=asc, wsc=wsc, bias=bias, la=la, lu=lu)
    return cpu, {k: v.to(dev) for k, v in cpu.items()}


def _args(d, out):
    from nunchaku_rocm_b200 import _lib as L
    from nunchaku_rocm_b200.ops.triton.gemm_w4a4 import _gemm_args

    return _gemm_args(d["act"], d["wgt"], out, d["asc"], d["wsc"], d["bias"], d["la"], d["lu"], None, False, False, False,
                      None, torch.bfloat16, L.IMPL_AUTO)


def _run_both(M, N, K, R, dev, seed):
    from nunchaku_rocm_b200 import _lib as L

    lib = L.lib()
    cpu, d = _problem(M, N, K, R, dev, seed)
    stream = L.stream_of(d["act"])

    # existing entry point, scratch from the caller
    out_ref = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    a = _args(d, out_ref)
    need = lib.nb_gemm_w4a4_scratch_bytes(C.byref(a), None, L.EPI_STORE)
    assert 0 < need <= L.NOALLOC_SCRATCH_BYTES
    scratch = torch.empty(need, dtype=torch.uint8, device=dev)
    a.scratch, a.scratch_bytes = L.ptr(scratch), need
    L.check(lib.nb_gemm_w4a4(C.byref(a), None, L.EPI_STORE, stream), "nb_gemm_w4a4")

    # new entry point: no scratch in the argument block at all
    out_new = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    b = _args(d, out_new)
    assert not b.scratch and b.scratch_bytes == 0
    L.check(lib.nb_gemm_w4a4_noalloc(C.byref(b), None, L.EPI_STORE, stream), "nb_gemm_w4a4_noalloc")
    torch.cuda.synchronize(dev)
    assert L.device_status(dev) == 0
    return cpu, out_ref, out_new


def test_noalloc_matches_existing_entry_point_twice_in_a_row(cuda_dev):
    # two calls in a row of different shapes: the second reuses the array the first left dirty
    for (M, N, K, R, seed) in [(256, 384, 512, 32, 1), (200, 264, 256, 16, 2)]:
        cpu, out_ref, out_new = _run_both(M, N, K, R, cuda_dev, seed)
        assert torch.equal(out_ref, out_new), f"{M}x{N}x{K}: outputs differ between the two entry points"
        want = ow.gemm_w4a4(cpu["act"], cpu["wgt"], cpu["asc"], cpu["wsc"], bias=cpu["bias"], lora_act=cpu["la"],
                            lora_up=cpu["lu"])
        assert ow.rel_fro(out_new.float().cpu(), want.float()) <= 1e-2  # the stated bf16 tolerance of the path


def _both_entries(a_ref, a_new, epi, kind, dev):
    """Run the caller-scratch entry on `a_ref` and the fixed-array entry on `a_new` (same inputs, separate outputs)."""
    from nunchaku_rocm_b200 import _lib as L

    lib = L.lib()
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    need = lib.nb_gemm_w4a4_scratch_bytes(C.byref(a_ref), epi, kind)
    assert 0 < need <= L.NOALLOC_SCRATCH_BYTES
    scratch = torch.empty(need, dtype=torch.uint8, device=dev)
    a_ref.scratch, a_ref.scratch_bytes = L.ptr(scratch), need
    L.check(lib.nb_gemm_w4a4(C.byref(a_ref), epi, kind, stream), "nb_gemm_w4a4")
    L.check(lib.nb_gemm_w4a4_noalloc(C.byref(a_new), epi, kind, stream), "nb_gemm_w4a4_noalloc")
    torch.cuda.synchronize(dev)
    assert L.device_status(dev) == 0


def test_noalloc_qk_epilogue_on_the_tensor_core_kernel(cuda_dev):
    # the fused Q/K RMSNorm + RoPE epilogue reads its operands from the same fixed array
    from nunchaku_rocm_b200 import _lib as L

    M, N, K, R = 200, 768, 256, 16
    _, d = _problem(M, N, K, R, cuda_dev, 3)
    g = torch.Generator().manual_seed(4)
    nq = (1 + 0.05 * torch.randn(128, generator=g)).to(torch.bfloat16).to(cuda_dev)
    nk = (1 + 0.05 * torch.randn(128, generator=g)).to(torch.bfloat16).to(cuda_dev)
    th = torch.rand(M, 64, generator=g) * 6.28
    rot = torch.stack([torch.sin(th), torch.cos(th)], -1).reshape(M, 128).float().contiguous().to(cuda_dev)
    qk = L.QKArgs(L.ptr(nq), L.ptr(nk), L.ptr(rot), rot.stride(0), M, 1e-6)
    outs = [torch.zeros(M, N, dtype=torch.bfloat16, device=cuda_dev) for _ in range(2)]
    a_ref, a_new = _args(d, outs[0]), _args(d, outs[1])
    assert L.lib().nb_gemm_w4a4_uses_tcgen05(C.byref(a_ref), C.byref(qk), L.EPI_QK) == 1
    _both_entries(a_ref, a_new, C.byref(qk), L.EPI_QK, cuda_dev)
    assert torch.equal(outs[0], outs[1])
    assert bool(outs[1].float().abs().sum() > 0)


def test_noalloc_generic_kernel_with_gelu_requant(cuda_dev):
    # the CUDA-core kernel keeps the fp32 tile (M * N * 4 bytes) of its row epilogue in the array
    from nunchaku_rocm_b200 import _lib as L

    M, N, K, R = 136, 256, 256, 16
    _, d = _problem(M, N, K, R, cuda_dev, 5)
    g = torch.Generator().manual_seed(6)
    smooth = (torch.rand(N, generator=g) + 0.5).to(torch.bfloat16).to(cuda_dev)
    ld = (torch.randn(N, 16, generator=g) * 0.05).to(torch.bfloat16).to(cuda_dev)
    res = []
    for _ in range(2):
        qout = torch.zeros(M, N // 2, dtype=torch.uint8, device=cuda_dev)
        osc = torch.zeros(N // 64, M, dtype=torch.bfloat16, device=cuda_dev)
        lao = torch.zeros(M, 16, dtype=torch.float32, device=cuda_dev)
        q = L.RequantArgs()
        q.qout, q.oscales, q.smooth, q.lora_down, q.lora_act_out = L.ptr(qout), L.ptr(osc), L.ptr(smooth), L.ptr(ld), L.ptr(lao)
        q.R2, q.shift = 16, 0.171875
        q.stride_qm, q.stride_osg, q.stride_ld, q.stride_lom = qout.stride(0), osc.stride(0), ld.stride(0), lao.stride(0)
        res.append((qout, osc, lao, q))
    a_ref, a_new = _args(d, None), _args(d, None)
    a_ref.impl = a_new.impl = L.IMPL_GENERIC
    lib = L.lib()
    stream = C.c_void_p(torch.cuda.current_stream(cuda_dev).cuda_stream)
    need = lib.nb_gemm_w4a4_scratch_bytes(C.byref(a_ref), C.byref(res[0][3]), L.EPI_GELU_QUANT)
    assert need == M * N * 4
    scratch = torch.empty(need, dtype=torch.uint8, device=cuda_dev)
    a_ref.scratch, a_ref.scratch_bytes = L.ptr(scratch), need
    L.check(lib.nb_gemm_w4a4(C.byref(a_ref), C.byref(res[0][3]), L.EPI_GELU_QUANT, stream), "nb_gemm_w4a4")
    L.check(lib.nb_gemm_w4a4_noalloc(C.byref(a_new), C.byref(res[1][3]), L.EPI_GELU_QUANT, stream), "noalloc")
    torch.cuda.synchronize(cuda_dev)
    for x, y in zip(res[0][:3], res[1][:3]):
        assert torch.equal(x, y)
    assert bool(res[1][0].any())


def test_noalloc_nvfp4_block_scaled_kernel(cuda_dev):
    # NVFP4 keeps its scale chunks and the rounded lora_act in the array
    from nunchaku_rocm_b200 import _lib as L
    from nunchaku_rocm_b200.ops.triton.gemm_w4a4 import _gemm_args

    M, N, K, R = 256, 256, 512, 16
    g = torch.Generator().manual_seed(7)
    act = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g).to(cuda_dev)
    wgt = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g).to(cuda_dev)
    asc = (torch.rand(K // 16, M, generator=g) * 0.5 + 0.05).to(torch.float8_e4m3fn).to(cuda_dev)
    wsc = (torch.rand(K // 16, N, generator=g) * 0.05 + 0.01).to(torch.float8_e4m3fn).to(cuda_dev)
    bias = torch.randn(N, generator=g).to(torch.bfloat16).to(cuda_dev)
    la = (torch.randn(M, R, generator=g) * 0.5).to(cuda_dev)
    lu = (torch.randn(N, R, generator=g) * 0.05).to(torch.bfloat16).to(cuda_dev)
    wcs = (torch.rand(N, generator=g) + 0.5).to(torch.bfloat16).to(cuda_dev)
    outs = [torch.zeros(M, N, dtype=torch.bfloat16, device=cuda_dev) for _ in range(2)]
    mk = lambda o: _gemm_args(act, wgt, o, asc, wsc, bias, la, lu, wcs, False, False, True, 0.75, torch.bfloat16, L.IMPL_AUTO)
    a_ref, a_new = mk(outs[0]), mk(outs[1])
    assert L.lib().nb_gemm_w4a4_uses_tcgen05(C.byref(a_ref), None, L.EPI_STORE) == 1
    _both_entries(a_ref, a_new, None, L.EPI_STORE, cuda_dev)
    assert torch.equal(outs[0], outs[1])
    assert bool(outs[1].float().abs().sum() > 0)


def test_noalloc_rejects_sizes_beyond_its_capacity(cuda_dev):
    from nunchaku_rocm_b200 import _lib as L

    lib = L.lib()
    M, N, K = 4096, 4096, 4096  # needs ~ (M + N) * K = 32 MiB of widened operands: beyond the 16 MiB array
    act = torch.zeros(M, K // 2, dtype=torch.uint8, device=cuda_dev)
    wgt = torch.zeros(N, K // 2, dtype=torch.uint8, device=cuda_dev)
    d = dict(act=act, wgt=wgt, asc=torch.ones(K // 64, M, dtype=torch.bfloat16, device=cuda_dev),
             wsc=torch.ones(K // 64, N, dtype=torch.bfloat16, device=cuda_dev), bias=None, la=None, lu=None)
    out = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=cuda_dev)
    a = _args(d, out)
    assert lib.nb_gemm_w4a4_scratch_bytes(C.byref(a), None, L.EPI_STORE) > L.NOALLOC_SCRATCH_BYTES
    rc = lib.nb_gemm_w4a4_noalloc(C.byref(a), None, L.EPI_STORE, L.stream_of(act))
    assert rc == L.NB_ERR_TOO_LARGE
    assert b"capacity" in lib.nb_strerror(rc)
    torch.cuda.synchronize(cuda_dev)
    assert bool((out == 7.0).all()), "a refused call must not launch anything"
