// subbyte.cu -- the reference's sub-byte unpack helpers as bulk device operations
// (32bit/src/pulp_nn_utils.c:201-356 element order, :375-438 block forms). Packed 4-bit and 2-bit
// values sit little-endian in their bytes: element i of a byte is bits [w*i, w*i+w), unsigned
// (bitextu) or sign-extended (bitext). No 8-bit kernel of the library uses them (the reference's
// "mixed" tree that would is not part of it); they are here so that a caller that stores
// activations or weights packed can widen them on the device before calling the 8-bit kernels.
//
// One thread widens one aligned 32-bit word (8 or 16 results, one 8- or 16-byte store); a byte-wise
// tail and unaligned buffers go one input byte per thread.
#include "internal.cuh"

namespace pulpnn {

namespace {

template <int BITS, bool SIGNED>
__device__ __forceinline__ unsigned widen4(unsigned packed)        // the low 4*BITS bits -> four bytes
{
  unsigned r = 0;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    unsigned v = (packed >> (BITS * i)) & ((1u << BITS) - 1u);
    if (SIGNED && (v >> (BITS - 1))) v |= 0xffu << BITS;            // sign extension into the byte
    r |= (v & 0xffu) << (8 * i);
  }
  return r;
}

// n_in input bytes -> n_in * (8 / BITS) output bytes
template <int BITS, bool SIGNED>
__global__ void __launch_bounds__(256) unpack_words_kernel(const unsigned *in, uint8_t *out, size_t n_words)
{
  constexpr int PER_WORD = 32 / BITS;                                // 8 or 16 results per input word
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += stride) {
    const unsigned w = __ldg(in + i);
    unsigned r[PER_WORD / 4];
#pragma unroll
    for (int j = 0; j < PER_WORD / 4; j++) r[j] = widen4<BITS, SIGNED>(w >> (4 * BITS * j));
    if constexpr (BITS == 4) *reinterpret_cast<uint2 *>(out + i * PER_WORD) = make_uint2(r[0], r[1]);
    else *reinterpret_cast<uint4 *>(out + i * PER_WORD) = make_uint4(r[0], r[1], r[2], r[3]);
  }
}

template <int BITS, bool SIGNED>
__global__ void __launch_bounds__(256) unpack_bytes_kernel(const uint8_t *in, uint8_t *out, size_t first, size_t n_in)
{
  constexpr int PER_BYTE = 8 / BITS;
  const size_t i = first + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_in) return;
  const unsigned r = widen4<BITS, SIGNED>(in[i]);
#pragma unroll
  for (int j = 0; j < PER_BYTE; j++) out[i * PER_BYTE + j] = (uint8_t)(r >> (8 * j));
}

template <int BITS, bool SIGNED>
void unpack_entry(const char *who, const void *in, void *out, unsigned int n_out)
{
  Context &c = ctx();
  if (!ensure_device(c)) return;
  if (n_out == 0) return;
  if (!in || !out) { set_error(PULPNN_ERR_INVALID_ARG, "%s: NULL pointer", who); return; }
  constexpr unsigned PER_BYTE = 8 / BITS;
  // the reference's tail loops count down by PER_BYTE from blockSize % (4*PER_BYTE) and only stop
  // at exactly zero (pulp_nn_utils.c:408-417,431-437)
  if (n_out % PER_BYTE != 0) {
    set_error(PULPNN_ERR_UNSUPPORTED, "%s: the element count must be a multiple of %u", who, PER_BYTE);
    return;
  }
  const size_t n_in = n_out / PER_BYTE;
  Stager st(c);
  const uint8_t *din = static_cast<const uint8_t *>(st.in(in, n_in));
  uint8_t *dout = static_cast<uint8_t *>(st.out(out, n_out));
  if (!st.ok()) return;
  const bool aligned = (reinterpret_cast<uintptr_t>(din) & 3) == 0 && (reinterpret_cast<uintptr_t>(dout) & 15) == 0;
  const size_t n_words = aligned ? n_in / 4 : 0;
  if (n_words) {
    const size_t want = (n_words + 255) / 256;
    const size_t cap = (size_t)(c.sm_count > 0 ? c.sm_count : 148) * 32;
    unpack_words_kernel<BITS, SIGNED><<<(unsigned)(want < cap ? want : cap), 256, 0, c.stream>>>(
        reinterpret_cast<const unsigned *>(din), dout, n_words);
    count_launch();
  }
  const size_t first = n_words * 4;
  if (first < n_in) {
    unpack_bytes_kernel<BITS, SIGNED><<<(unsigned)((n_in - first + 255) / 256), 256, 0, c.stream>>>(din, dout, first, n_in);
    count_launch();
  }
  if (!cuda_ok(cudaGetLastError(), "unpack launch")) return;
  st.finish();
}

}  // namespace

}  // namespace pulpnn

extern "C" {

void pulp_nn_im2col_u4_to_u8(uint8_t *pInput, uint8_t *pOutput, unsigned int blockSize)
{
  pulpnn::unpack_entry<4, false>("pulp_nn_im2col_u4_to_u8", pInput, pOutput, blockSize);
}
void pulp_nn_im2col_u2_to_u8(uint8_t *pInput, uint8_t *pOutput, unsigned int blockSize)
{
  pulpnn::unpack_entry<2, false>("pulp_nn_im2col_u2_to_u8", pInput, pOutput, blockSize);
}
void pulpnn_i4_to_i8(const int8_t *pSrc, int8_t *pDst, unsigned int n)
{
  pulpnn::unpack_entry<4, true>("pulpnn_i4_to_i8", pSrc, pDst, n);
}
void pulpnn_i2_to_i8(const int8_t *pSrc, int8_t *pDst, unsigned int n)
{
  pulpnn::unpack_entry<2, true>("pulpnn_i2_to_i8", pSrc, pDst, n);
}

}  // extern "C"
