"""
Constants of the CUDA sources that can be checked without a GPU: the byte tables that turn an int4 code into the e4m3
value the tensor core multiplies (nb_common.cuh, used by both tensor-core GEMMs), read from the source text and decoded with torch's float8_e4m3fn.
"""

import os
import re

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = open(os.path.join(ROOT, "nunchaku_rocm_b200", "csrc", "nb_common.cuh")).read()


def _table(lo_name, hi_name=None, pick=None):
    def words(expr):
        return [int(h, 16) for h in re.findall(r"0x([0-9A-Fa-f]{8})u", expr)]

    m = re.search(r"const uint32_t lo0 = (0x\w+), lo1 = (0x\w+);", SRC)
    lo = words(m.group(0))
    m = re.search(r"const uint32_t hi0 = uns \? (0x\w+) : (0x\w+), hi1 = uns \? (0x\w+) : (0x\w+);", SRC)
    hu0, hs0, hu1, hs1 = words(m.group(0))
    return lo, (hu0, hu1), (hs0, hs1)


def _bytes(words):
    return [(w >> (8 * i)) & 0xFF for w in words for i in range(4)]


def _decode(bs):
    return torch.tensor(bs, dtype=torch.uint8).view(torch.float8_e4m3fn).float().tolist()


def test_e4m3_tables_hold_the_int4_values_exactly():
    lo, hi_unsigned, hi_signed = _table("lo0")
    assert _decode(_bytes(lo)) == [0.0, 1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0]          # codes 0..7, both formats
    assert _decode(_bytes(hi_unsigned)) == [8.0, 9.0, 10.0, 11.0, 12.0, 13.0, 14.0, 15.0]  # codes 8..15, unsigned
    assert _decode(_bytes(hi_signed)) == [-8.0, -7.0, -6.0, -5.0, -4.0, -3.0, -2.0, -1.0]  # codes 8..15, two's complement


def test_group_sums_stay_exact_in_fp32():
    # the largest magnitude of a 64-term sum of products of two codes must be an integer fp32 represents exactly
    worst = 64 * 15 * 8
    assert worst == 7680 and float(worst) == worst and worst < 2**24
