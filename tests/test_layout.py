"""The checkpoint-layout converter against fixtures produced by the reference's packer and its inverse
(tests/golden/make_golden.py; reference tests: tests/triton/test_layout.py:20-66)."""

import pytest
import torch

from nunchaku_rocm_b200.ops.triton import layout
from tests.conftest import load_golden


def test_weight_layout_matches_reference_packer():
    g = load_golden("layout")
    n, k = g["codes"].shape
    assert torch.equal(layout.unpack_weight(g["packed_w"], n, k), g["unpacked_w"])
    assert torch.equal(layout.unpack_weight(g["packed_w"], n, k), g["codes"] & 0xF)
    assert torch.equal(layout.pack_weight(g["codes"]), g["packed_w"])
    nat = layout.unpack_weight_packed_nibbles(g["packed_w"], n, k)
    assert nat.dtype == torch.uint8 and nat.shape == (n, k // 2)
    assert torch.equal((nat & 0xF).to(torch.int32), (g["codes"] & 0xF)[:, 0::2])
    assert torch.equal((nat >> 4).to(torch.int32), (g["codes"] & 0xF)[:, 1::2])


def _eq(a, b):
    return a.shape == b.shape and torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))


def test_scale_layouts_match_reference_packer():
    g = load_golden("layout")
    n = g["scale"].shape[0]
    assert _eq(layout.unpack_scale(g["packed_s"], n, 64), g["unpacked_s"])
    assert _eq(layout.unpack_scale(g["packed_s"], n, 64), g["scale"].t().contiguous())
    assert _eq(layout.pack_scale(g["scale"].t().contiguous(), 64), g["packed_s"])
    assert _eq(layout.unpack_scale(g["packed_c"].reshape(1, -1), n, -1), g["unpacked_c"])
    assert _eq(layout.unpack_scale(g["packed_c"].reshape(1, -1), n, -1), g["chan"])
    assert _eq(layout.pack_scale(g["chan"], -1), g["packed_c"])
    assert _eq(layout.unpack_scale(g["packed_m"], n, 16), g["unpacked_m"])
    assert _eq(layout.pack_scale(g["micro"].t().contiguous(), 16), g["packed_m"])


def test_lowrank_layouts_match_reference_packer():
    g = load_golden("layout")
    assert _eq(layout.unpack_lowrank_weight(g["packed_up"], down=False), g["up"])
    assert _eq(layout.unpack_lowrank_weight(g["packed_down"], down=True), g["down_t"])
    assert _eq(layout.pack_lowrank_weight(g["up"], down=False), g["packed_up"])
    assert _eq(layout.pack_lowrank_weight(g["down_t"], down=True), g["packed_down"])


def test_convert_linear_round_trip():
    from nunchaku_rocm_b200.models.linear import SVDQW4A4Linear

    torch.manual_seed(0)
    n, k, r = 256, 384, 32
    for precision in ("int4", "nvfp4"):
        G = 16 if precision == "nvfp4" else 64
        lin = SVDQW4A4Linear(k, n, rank=r, precision=precision)
        codes = torch.randint(0, 16, (n, k), dtype=torch.int32)
        ws = torch.rand(k // G, n) * 0.02 + 0.01
        ws = ws.to(torch.float8_e4m3fn) if precision == "nvfp4" else ws.to(torch.bfloat16)
        bias, smooth = torch.randn(n).bfloat16(), (torch.rand(k) + 0.5).bfloat16()
        down, up = torch.randn(k, r).bfloat16(), torch.randn(n, r).bfloat16()
        lin.qweight.data = layout.pack_weight(codes)
        lin.wscales.data = layout.pack_scale(ws.float().bfloat16() if precision == "nvfp4" else ws, G).view(k // G, n)
        lin.bias.data = layout.pack_scale(bias, -1)
        lin.smooth_factor.data = layout.pack_scale(smooth, -1)
        lin.proj_down.data = layout.pack_lowrank_weight(down.t().contiguous(), down=True)
        lin.proj_up.data = layout.pack_lowrank_weight(up, down=False)
        if precision == "nvfp4":
            wcs = (torch.rand(n) + 0.5).bfloat16()
            lin.wcscales.data = layout.pack_scale(wcs, -1)
        layout.convert_svdq_linear_to_natural_layout(lin)
        assert torch.equal((lin.qweight.view(torch.uint8) & 0xF).int(), codes[:, 0::2])
        assert torch.equal((lin.qweight.view(torch.uint8) >> 4).int(), codes[:, 1::2])
        assert _eq(lin.wscales.data, ws) and _eq(lin.bias.data, bias) and _eq(lin.smooth_factor.data, smooth)
        assert _eq(lin.proj_down.data, down) and _eq(lin.proj_up.data, up)
        if precision == "nvfp4":
            assert _eq(lin.wcscales.data, wcs)


@pytest.mark.gpu
@pytest.mark.parametrize("n,k", [(128, 128), (384, 256), (3072, 3072)])
def test_weight_layout_kernel_matches_index_formula(n, k):
    """The device kernel (one word permutation per 128 x 64 block) against the index formula run by torch on the host."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    g = torch.Generator().manual_seed(n + k)
    stored = torch.randint(-128, 128, (n, k // 2), dtype=torch.int8, generator=g)
    want = layout.unpack_weight_packed_nibbles(stored, n, k)  # host: gather by formula
    got = layout.unpack_weight_packed_nibbles(stored.cuda(), n, k)
    assert got.is_cuda and got.dtype == torch.uint8 and got.shape == (n, k // 2)
    assert torch.equal(got.cpu(), want)
    # and it inverts the forward direction (pack_weight)
    codes = torch.randint(0, 16, (n, k), dtype=torch.int32, generator=g)
    nat = layout.unpack_weight_packed_nibbles(layout.pack_weight(codes).cuda(), n, k).cpu().to(torch.int32)
    assert torch.equal(nat & 0xF, codes[:, 0::2]) and torch.equal(nat >> 4, codes[:, 1::2])
