// Checkpoint layout converter for the 4-bit weight, on the device (HBM-bound).
//
// SVDQuant checkpoints store qweight in the register-fragment order of the upstream kernel's mma.m16n8k32
// (reference: nunchaku/ops/triton/layout.py:36-118 unpack_weight / unpack_weight_packed_nibbles, forward direction
// NunchakuWeightPacker.pack_weight, nunchaku/lora/flux/packer.py:187-239): int32 word
//     (((((nt KT + kt) 8 + npk) 8 + nl) 4 + kl) 2 + nps) 2 + kps,  nibble rk
// holds n = ((nt 8 + npk) 2 + nps) 8 + nl, k = kt 64 + kps 32 + kl 8 + rk.  The eight nibbles of a stored word are eight
// consecutive k of one row in the order the natural packing wants them (even k in the low nibble), so the conversion is
// a permutation of 32-bit words: a (nt, kt) block of 128 rows x 64 k is 1024 contiguous words on the stored side and
// 128 segments of 32 bytes on the natural side.  One CTA per block: one 16-byte load per thread, a transpose through
// shared memory, one 16-byte store per thread.
#include "nb_common.cuh"

namespace nb {
namespace {

__global__ void __launch_bounds__(256) layout_unpack_weight_kernel(const uint4* __restrict__ stored, uint32_t* __restrict__ out,
                                                                   int KT, long long out_words_per_row) {
    __shared__ uint32_t tile[128][9];  // (row, word) with one word of padding per row
    const int t = threadIdx.x;
    const long long blk = blockIdx.x;  // nt * KT + kt
    const int nt = (int)(blk / KT), kt = (int)(blk % KT);
    const uint4 w = __ldg(stored + blk * 256 + t);
    // words 4 t + i, i = kps + 2 nps: kl = t & 3, nl = (t >> 2) & 7, npk = t >> 5
    const int kl = t & 3, nl = (t >> 2) & 7, npk = t >> 5;
    const int r0 = npk * 16 + nl;
    tile[r0][kl] = w.x;          // nps 0, kps 0
    tile[r0][4 + kl] = w.y;      // nps 0, kps 1
    tile[r0 + 8][kl] = w.z;      // nps 1, kps 0
    tile[r0 + 8][4 + kl] = w.w;  // nps 1, kps 1
    __syncthreads();
    const int row = t >> 1, half = t & 1;
    const uint4 o = make_uint4(tile[row][4 * half], tile[row][4 * half + 1], tile[row][4 * half + 2], tile[row][4 * half + 3]);
    *reinterpret_cast<uint4*>(out + ((long long)nt * 128 + row) * out_words_per_row + kt * 8 + 4 * half) = o;
}

}  // namespace
}  // namespace nb

extern "C" int nb_layout_unpack_weight(const void* stored, void* out, int32_t n, int32_t k, int64_t stride_on, void* stream) {
    using namespace nb;
    NB_REQUIRE(stored && out);
    NB_REQUIRE(n > 0 && k > 0 && n % 128 == 0 && k % 128 == 0);
    NB_REQUIRE(aligned16(stored) && aligned16(out) && stride_on % 16 == 0 && stride_on >= k / 2);
    const int KT = k / 64;
    const long long blocks = (long long)(n / 128) * KT;
    NB_REQUIRE(blocks <= 0x7fffffffLL);
    layout_unpack_weight_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(stored), static_cast<uint32_t*>(out), KT, stride_on / 4);
    NB_CUDA_CHECK(cudaGetLastError());
    return NB_OK;
}
