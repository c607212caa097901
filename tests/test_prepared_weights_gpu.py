"""
Load-time weight preparation of the int4 tensor-core GEMM (`nb_gemm_w4a4_prepare_weights`): a call that is handed the
prepared buffer must give bit-identical results to one that widens the weights in its own pre-pass, and the operator
layer's cache must notice in-place weight updates.
"""

import ctypes as C

import pytest
import torch

from nunchaku_rocm_b200 import _lib as L
from nunchaku_rocm_b200.ops.triton import gemm_w4a4 as G

pytestmark = pytest.mark.gpu
T = torch.bfloat16


def _inputs(dev, M=300, N=384, K=512, R=32, seed=0):
    g = torch.Generator().manual_seed(seed)
    p = dict(
        act=torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g),
        wgt=torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g),
        ascales=(torch.rand(K // 64, M, generator=g) * 0.05 + 0.01).to(T),
        wscales=(torch.rand(K // 64, N, generator=g) * 0.02 + 0.005).to(T),
        bias=(torch.randn(N, generator=g) * 0.1).to(T),
        lora_act=torch.randn(M, R, generator=g) * 0.1,
        lora_up=(torch.randn(N, R, generator=g) * 0.05).to(T),
    )
    return {k: v.to(dev) for k, v in p.items()}


def _call(p, monkeypatch=None, disabled=False):
    if disabled:
        monkeypatch.setenv("NUNCHAKU_B200_PREPARED_WEIGHTS_MB", "0")
    elif monkeypatch is not None:
        monkeypatch.delenv("NUNCHAKU_B200_PREPARED_WEIGHTS_MB", raising=False)
    out = torch.empty(p["act"].shape[0], p["wgt"].shape[0], dtype=T, device=p["act"].device)
    G.gemm_w4a4(p["act"], p["wgt"], out, p["ascales"], p["wscales"], p["bias"], p["lora_act"], p["lora_up"])
    return out


def test_prepared_and_unprepared_calls_agree_bit_for_bit(cuda_dev, monkeypatch):
    p = _inputs(cuda_dev)
    G.clear_prepared_weights()
    ref = _call(p, monkeypatch, disabled=True)
    assert not G._PREPARED
    first = _call(p, monkeypatch)   # prepares
    assert len(G._PREPARED) == 1
    second = _call(p, monkeypatch)  # reuses
    assert len(G._PREPARED) == 1
    assert torch.equal(ref, first) and torch.equal(ref, second)
    assert L.device_status(cuda_dev) == 0


def test_in_place_weight_update_invalidates_the_entry(cuda_dev, monkeypatch):
    p = _inputs(cuda_dev, seed=1)
    G.clear_prepared_weights()
    before = _call(p, monkeypatch)
    g = torch.Generator().manual_seed(2)
    p["wgt"].copy_(torch.randint(0, 256, p["wgt"].shape, dtype=torch.uint8, generator=g).to(cuda_dev))
    after = _call(p, monkeypatch)
    assert not torch.equal(before, after)
    assert torch.equal(after, _call(p, monkeypatch, disabled=True))
    # scales too
    p["wscales"].mul_(2)
    assert torch.equal(_call(p, monkeypatch), _call(p, monkeypatch, disabled=True))
    # a view of the same memory (the int8 parameter seen as uint8) shares the entry
    n = len(G._PREPARED)
    q = dict(p, wgt=p["wgt"].view(torch.int8).view(torch.uint8))
    assert torch.equal(_call(q, monkeypatch), _call(p, monkeypatch)) and len(G._PREPARED) == n
    G.clear_prepared_weights()
    assert not G._PREPARED


def test_buffers_used_inside_a_graph_capture_outlive_the_cache(cuda_dev, monkeypatch):
    # a captured call bakes the prepared buffer's address into the graph: clearing or evicting the cache must not free it
    p = _inputs(cuda_dev, seed=3)
    G.clear_prepared_weights(release_pinned=True)
    want = _call(p, monkeypatch)  # prepares the entry outside the capture
    out = torch.zeros_like(want)
    side = torch.cuda.Stream(cuda_dev)
    side.wait_stream(torch.cuda.current_stream(cuda_dev))
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            G.gemm_w4a4(p["act"], p["wgt"], out, p["ascales"], p["wscales"], p["bias"], p["lora_act"], p["lora_up"])
    torch.cuda.current_stream(cuda_dev).wait_stream(side)
    (entry,) = G._PREPARED.values()
    assert entry[G._E_PINNED]
    monkeypatch.setenv("NUNCHAKU_B200_PREPARED_WEIGHTS_MB", "1")  # a budget that evicts everything evictable
    q = _inputs(cuda_dev, M=128, N=256, K=256, seed=4)
    _call(q)
    assert entry in G._PREPARED.values(), "a pinned entry was evicted"
    G.clear_prepared_weights()
    assert not G._PREPARED and len(G._PINNED_BUFFERS) == 1
    filler = [torch.full((entry[G._E_BUF].numel(),), 0xAB, dtype=torch.uint8, device=cuda_dev) for _ in range(4)]
    graph.replay()
    torch.cuda.synchronize(cuda_dev)
    assert torch.equal(out, want), "the replay read a buffer that had been released"
    del filler, graph
    G.clear_prepared_weights(release_pinned=True)
    assert not G._PINNED_BUFFERS


def test_c_abi_prepared_bytes_and_scratch(cuda_dev):
    p = _inputs(cuda_dev, M=256, N=256, K=256)
    out = torch.empty(256, 256, dtype=T, device=cuda_dev)
    a = G._gemm_args(p["act"], p["wgt"], out, p["ascales"], p["wscales"], p["bias"], p["lora_act"], p["lora_up"], None,
                     False, False, False, 1.0, T, L.IMPL_AUTO)
    lib = L.lib()
    nbytes = lib.nb_gemm_w4a4_prepared_bytes(C.byref(a))
    assert nbytes >= 256 * 256 + (256 // 64) * 256 * 2
    need_plain = lib.nb_gemm_w4a4_scratch_bytes(C.byref(a), None, L.EPI_STORE)
    buf = torch.empty(nbytes, dtype=torch.uint8, device=cuda_dev)
    assert lib.nb_gemm_w4a4_prepare_weights(C.byref(a), L.ptr(buf), nbytes - 1, None) != 0  # too small
    assert lib.nb_gemm_w4a4_prepare_weights(C.byref(a), L.ptr(buf), nbytes, L.stream_of(out)) == 0
    a.wgt_prepared, a.wgt_prepared_bytes = L.ptr(buf), nbytes
    need_prepared = lib.nb_gemm_w4a4_scratch_bytes(C.byref(a), None, L.EPI_STORE)
    # the call no longer keeps the weight side in scratch (the buffer holds the scale order of both tensor-core kernels,
    # a call needs one of them)
    assert 256 * 256 <= need_plain - need_prepared <= nbytes
    # an NVFP4 weight's prepared form is its block scales in the MMA's chunk layout: 512 bytes per 128 rows and 64 k
    a.fp4 = 1
    assert lib.nb_gemm_w4a4_prepared_bytes(C.byref(a)) == (256 // 128) * (256 // 64) * 512
    a.K = 96
    assert lib.nb_gemm_w4a4_prepared_bytes(C.byref(a)) == 0


@pytest.mark.parametrize("M,N,K", [(300, 384, 512), (256, 768, 320)])
def test_nvfp4_prepared_scales_agree_bit_for_bit(cuda_dev, monkeypatch, M, N, K):
    g = torch.Generator().manual_seed(M + N)
    dv = lambda t: t.to(cuda_dev)
    act = dv(torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g))
    wgt = dv(torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g))
    asc = dv((torch.rand(K // 16, M, generator=g) * 0.05 + 0.01).to(torch.float8_e4m3fn))
    wsc = dv((torch.rand(K // 16, N, generator=g) * 0.05 + 0.01).to(torch.float8_e4m3fn))
    wcs = dv((torch.rand(N, generator=g) * 0.5 + 0.5).to(T))

    def call(disabled):
        if disabled:
            monkeypatch.setenv("NUNCHAKU_B200_PREPARED_WEIGHTS_MB", "0")
        else:
            monkeypatch.delenv("NUNCHAKU_B200_PREPARED_WEIGHTS_MB", raising=False)
        return G.gemm_w4a4(act, wgt, None, asc, wsc, wcscales=wcs, alpha=0.75, fp4=True, out_dtype=T)

    G.clear_prepared_weights()
    ref = call(True)
    assert not G._PREPARED
    first, second = call(False), call(False)
    assert len(G._PREPARED) == 1
    assert torch.equal(ref, first) and torch.equal(ref, second)
    assert L.device_status(cuda_dev) == 0
    G.clear_prepared_weights()
