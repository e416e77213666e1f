// subbyte.cu -- the reference's sub-byte unpack helpers as bulk device operations
// (32bit/src/pulp_nn_utils.c:201-356 element order, :375-438 block forms). Packed 4-bit and 2-bit
// values sit little-endian in their bytes: element i of a byte is bits [w*i, w*i+w), unsigned
// (bitextu) or sign-extended (bitext). No 8-bit kernel of the library uses them (the reference's
// "mixed" tree that would is not part of it); they are here so that a caller that stores
// activations or weights packed can widen them on the device before calling the 8-bit kernels.
//
// The scalar requantisers and threshold quantisers of the same header (pulp_nn_bn_quant_u4/u2,
// pulp_nn_quant_u4/u2, pulp_nn_i4_quant, pulp_nn_i2_quant) and pulp_nn_avg_and_replace_int8 follow as
// element-wise bulk operations.
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

// ---- scalar requantisers of the reference as bulk operations -----------------------------------------
// pulp_nn_bn_quant_u8/u4/u2 and pulp_nn_quant_u8/u4/u2 (32bit/src/pulp_nn_utils.c:35-45,148-199; the
// 64-bit tree widens k, lambda and the product to int64 and narrows the multiplier form to int16,
// 64bit/src/pulp_nn_utils.c:34-198). Element i uses the parameters of channel i % channels.
template <typename BN_T>
__global__ void __launch_bounds__(256) bn_quant_bulk_kernel(const int *phi, const BN_T *k, const BN_T *lambda, int d,
                                                            uint8_t *out, unsigned n, unsigned channels, int hi)
{
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const unsigned c = i % channels;
    int x;
    if (sizeof(BN_T) == 4)
      x = (int)((unsigned)(int)__ldg(k + c) * (unsigned)__ldg(phi + i) + (unsigned)(int)__ldg(lambda + c)) >> d;
    else      // the clip builtin takes an int: the shifted 64-bit value is cut to 32 bits first
      x = (int)((long long)((unsigned long long)__ldg(k + c) * (unsigned long long)(long long)__ldg(phi + i) +
                            (unsigned long long)__ldg(lambda + c)) >> d);
    out[i] = (uint8_t)min(max(x, 0), hi);
  }
}

// bits 8: x is cut to int16 in both trees; bits 4 and 2: int32 in the 32-bit tree, int16 in the 64-bit one
__global__ void __launch_bounds__(256) quant_bulk_kernel(const int *phi, int m, int d, uint8_t *out, unsigned n, int hi,
                                                         int narrow16)
{
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    int x = (int)((unsigned)m * (unsigned)__ldg(phi + i)) >> d;
    if (narrow16) x = (int)(short)x;
    out[i] = (uint8_t)min(max(x, 0), hi);
  }
}

// pulp_nn_i4_quant / pulp_nn_i2_quant (32bit/src/pulp_nn_utils.c:438-540): a binary search over
// sorted thresholds; with sorted thresholds its result is (number of thresholds below the input) + the
// lowest level, which is what is computed here by following the same comparisons
__global__ void __launch_bounds__(256) threshold_quant_kernel(const int *in, const short *thr, int8_t *out, unsigned n,
                                                              unsigned channels, int bits)
{
  const unsigned stride = gridDim.x * blockDim.x;
  const int pitch = bits == 4 ? 16 : 4;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const short *t = thr + (size_t)(i % channels) * pitch;
    const int v = __ldg(in + i);
    int lo = 0, width = bits == 4 ? 16 : 4;      // the search tree of the reference: compare with the middle threshold
    while (width > 1) {
      const int mid = lo + width / 2 - 1;
      if (!(v <= (int)__ldg(t + mid))) lo += width / 2;
      width /= 2;
    }
    out[i] = (int8_t)(lo - (bits == 4 ? 8 : 2));
  }
}

// pulp_nn_avg_and_replace_int8 (32bit/src/pulp_nn_utils.c:95-115): base[i] = (base[i] + target[i]) >> 1 on
// signed bytes, for whole words of four only (length >> 2 words)
__global__ void __launch_bounds__(256) avg_replace_kernel(int8_t *base, const int8_t *target, unsigned n)
{
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    base[i] = (int8_t)(((int)base[i] + (int)target[i]) >> 1);
}

unsigned bulk_blocks(const Context &c, unsigned n)
{
  const unsigned want = (n + 255) / 256, cap = (unsigned)(c.sm_count > 0 ? c.sm_count : 148) * 16;
  return want < cap ? want : cap;
}

int level_max(const char *who, int bits)
{
  if (bits == 8) return 255;
  if (bits == 4) return 15;
  if (bits == 2) return 3;
  set_error(PULPNN_ERR_INVALID_ARG, "%s: bits must be 8, 4 or 2", who);
  return -1;
}

template <typename BN_T>
void bn_quant_entry(const char *who, const int32_t *phi, const BN_T *k, const BN_T *lambda, int d, uint8_t *out,
                    unsigned n, unsigned channels, int bits)
{
  Context &c = ctx();
  if (!ensure_device(c) || n == 0) return;
  const int hi = level_max(who, bits);
  if (hi < 0) return;
  if (!phi || !k || !lambda || !out || channels == 0 || d < 0 || d > (sizeof(BN_T) == 4 ? 31 : 63)) {
    set_error(PULPNN_ERR_INVALID_ARG, "%s: NULL pointer, no channels or shift out of range", who);
    return;
  }
  Stager st(c);
  const int *dphi = static_cast<const int *>(st.in(phi, (size_t)n * 4));
  const BN_T *dk = static_cast<const BN_T *>(st.in(k, (size_t)channels * sizeof(BN_T)));
  const BN_T *dl = static_cast<const BN_T *>(st.in(lambda, (size_t)channels * sizeof(BN_T)));
  uint8_t *dout = static_cast<uint8_t *>(st.out(out, n));
  if (!st.ok()) return;
  bn_quant_bulk_kernel<BN_T><<<bulk_blocks(c, n), 256, 0, c.stream>>>(dphi, dk, dl, d, dout, n, channels, hi);
  count_launch();
  if (!cuda_ok(cudaGetLastError(), "bn_quant launch")) return;
  st.finish();
}

void quant_entry(const char *who, int tree_bits, const int32_t *phi, int16_t m, int d, uint8_t *out, unsigned n, int bits)
{
  Context &c = ctx();
  if (!ensure_device(c) || n == 0) return;
  const int hi = level_max(who, bits);
  if (hi < 0) return;
  if (!phi || !out || d < 0 || d > 31) { set_error(PULPNN_ERR_INVALID_ARG, "%s: NULL pointer or shift out of range", who); return; }
  Stager st(c);
  const int *dphi = static_cast<const int *>(st.in(phi, (size_t)n * 4));
  uint8_t *dout = static_cast<uint8_t *>(st.out(out, n));
  if (!st.ok()) return;
  const int narrow16 = (bits == 8 || tree_bits == 64) ? 1 : 0;
  quant_bulk_kernel<<<bulk_blocks(c, n), 256, 0, c.stream>>>(dphi, (int)m, d, dout, n, hi, narrow16);
  count_launch();
  if (!cuda_ok(cudaGetLastError(), "quant launch")) return;
  st.finish();
}

}  // namespace

}  // namespace pulpnn

extern "C" {

void pulpnn_bn_quant_bulk_bn32(const int32_t *phi, const int32_t *k, const int32_t *lambda, int8_t d, uint8_t *out,
                               unsigned int n, unsigned int channels, int bits)
{
  pulpnn::bn_quant_entry<int32_t>("pulpnn_bn_quant_bulk_bn32", phi, k, lambda, d, out, n, channels, bits);
}
void pulpnn_bn_quant_bulk_bn64(const int32_t *phi, const int64_t *k, const int64_t *lambda, int8_t d, uint8_t *out,
                               unsigned int n, unsigned int channels, int bits)
{
  pulpnn::bn_quant_entry<long long>("pulpnn_bn_quant_bulk_bn64", phi, reinterpret_cast<const long long *>(k),
                                    reinterpret_cast<const long long *>(lambda), d, out, n, channels, bits);
}
void pulpnn_quant_bulk_bn32(const int32_t *phi, int16_t m, int8_t d, uint8_t *out, unsigned int n, int bits)
{
  pulpnn::quant_entry("pulpnn_quant_bulk_bn32", 32, phi, m, d, out, n, bits);
}
void pulpnn_quant_bulk_bn64(const int32_t *phi, int16_t m, int8_t d, uint8_t *out, unsigned int n, int bits)
{
  pulpnn::quant_entry("pulpnn_quant_bulk_bn64", 64, phi, m, d, out, n, bits);
}
void pulpnn_threshold_quant_bulk(const int32_t *in, const int16_t *thr, int8_t *out, unsigned int n, unsigned int channels,
                                 int bits)
{
  using namespace pulpnn;
  const char *who = "pulpnn_threshold_quant_bulk";
  Context &c = ctx();
  if (!ensure_device(c) || n == 0) return;
  if (!in || !thr || !out || channels == 0 || (bits != 4 && bits != 2)) {
    set_error(PULPNN_ERR_INVALID_ARG, "%s: NULL pointer, no channels, or bits other than 4 and 2", who);
    return;
  }
  Stager st(c);
  const int *din = static_cast<const int *>(st.in(in, (size_t)n * 4));
  const short *dthr = static_cast<const short *>(st.in(thr, (size_t)channels * (bits == 4 ? 16 : 4) * 2));
  int8_t *dout = static_cast<int8_t *>(st.out(out, n));
  if (!st.ok()) return;
  threshold_quant_kernel<<<bulk_blocks(c, n), 256, 0, c.stream>>>(din, dthr, dout, n, channels, bits);
  count_launch();
  if (!cuda_ok(cudaGetLastError(), "threshold_quant launch")) return;
  st.finish();
}
void pulp_nn_avg_and_replace_int8(int8_t *base, int8_t *target, uint16_t length)
{
  using namespace pulpnn;
  Context &c = ctx();
  if (!ensure_device(c)) return;
  const unsigned n = (unsigned)(length >> 2) * 4u;        // whole words only, as the reference
  if (n == 0) return;
  if (!base || !target) { set_error(PULPNN_ERR_INVALID_ARG, "pulp_nn_avg_and_replace_int8: NULL pointer"); return; }
  Stager st(c);
  int8_t *db = static_cast<int8_t *>(st.inout(base, n));
  const int8_t *dt = static_cast<const int8_t *>(st.in(target, n));
  if (!st.ok()) return;
  avg_replace_kernel<<<bulk_blocks(c, n), 256, 0, c.stream>>>(db, dt, n);
  count_launch();
  if (!cuda_ok(cudaGetLastError(), "avg_and_replace launch")) return;
  st.finish();
}

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
