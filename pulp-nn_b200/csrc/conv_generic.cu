// conv_generic.cu -- CUDA-core implicit GEMM for every shape the API admits.
//
// One kernel covers standard convolution, pointwise convolution and the fully connected layer
// (a 1x1 "image"). It is the path for shapes the tensor-core kernel does not take (reduction
// length not a multiple of 16 bytes, e.g. a 3-channel first layer with K = 27, ragged channel
// counts, spatial kernels). Arithmetic: acc = bias + sum u8*s8 in int32 (dp4a), then the
// reference's requantisation -- see internal.cuh.
//
// Tiling: 64 output pixels x 64 output channels per CTA, 32 bytes of K per step, 256 threads
// with a 4x4 register tile each. The im2col column of a pixel is gathered on the fly: with
// ch_in % 4 == 0 a 4-byte word never straddles two taps, so words are fetched whole; otherwise
// bytes are fetched one at a time. Taps outside the image contribute zero, which is what the
// reference's zero-filled im2col buffer does (32bit/src/pulp_nn_conv_Ho_parallel.c:80-164).
#include "internal.cuh"

namespace pulpnn {

namespace {

constexpr int BM = 64, BN = 64, BKW = 8;          // BKW words = 32 bytes of K per step
constexpr int APITCH = BM + 4, BPITCH = BN + 4;   // word pitches chosen to spread banks

struct GenericParams {
  ConvProblem p;
  int M, K, KW;        // M = B*Ho*Wo, K = ky*kx*Cin, KW = ceil(K/4)
};

template <bool WORDS>
__device__ __forceinline__ unsigned gather_a(const ConvProblem &p, const uint8_t *img, int iy0,
                                             int ix0, int kword, int K)
{
  // returns the 4 bytes k = 4*kword .. 4*kword+3 of the im2col column, zero outside
  const int k0 = kword * 4;
  if (WORDS) {
    if (k0 >= K) return 0u;
    const int tap = k0 / p.Cin, ci = k0 - tap * p.Cin;
    const int fy = tap / p.kx, fx = tap - fy * p.kx;
    const int iy = iy0 + fy, ix = ix0 + fx;
    if ((unsigned)iy >= (unsigned)p.H || (unsigned)ix >= (unsigned)p.W) return 0u;
    return __ldg(reinterpret_cast<const unsigned *>(img + ((size_t)iy * p.W + ix) * p.Cin + ci));
  } else {
    unsigned v = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int k = k0 + j;
      if (k < K) {
        const int tap = k / p.Cin, ci = k - tap * p.Cin;
        const int fy = tap / p.kx, fx = tap - fy * p.kx;
        const int iy = iy0 + fy, ix = ix0 + fx;
        if ((unsigned)iy < (unsigned)p.H && (unsigned)ix < (unsigned)p.W)
          v |= (unsigned)__ldg(img + ((size_t)iy * p.W + ix) * p.Cin + ci) << (8 * j);
      }
    }
    return v;
  }
}

template <bool WORDS>
__device__ __forceinline__ unsigned gather_b(const int8_t *wrow, int kword, int K)
{
  const int k0 = kword * 4;
  if (WORDS) {
    return k0 < K ? __ldg(reinterpret_cast<const unsigned *>(wrow + k0)) : 0u;
  } else {
    unsigned v = 0;
#pragma unroll
    for (int j = 0; j < 4; j++)
      if (k0 + j < K) v |= (unsigned)(uint8_t)__ldg(wrow + k0 + j) << (8 * j);
    return v;
  }
}

template <int MODE, bool WORDS>
__global__ void __launch_bounds__(256) conv_generic_kernel(const GenericParams g)
{
  __shared__ unsigned As[BKW][APITCH];
  __shared__ unsigned Bs[BKW][BPITCH];

  const ConvProblem &p = g.p;
  const int tid = threadIdx.x;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;

  // this thread's two gather rows (A) and two weight rows (B): row = tid/8 (+32), word = tid%8
  const int lrow = tid >> 3, lkw = tid & 7;
  const uint8_t *img[2];
  int iy0[2], ix0[2];
  bool mvalid[2];
  const int8_t *wrow[2];
  bool nvalid[2];
#pragma unroll
  for (int h = 0; h < 2; h++) {
    const int m = m0 + lrow + 32 * h;
    mvalid[h] = m < g.M;
    const int mm = mvalid[h] ? m : 0;
    const int b = mm / (p.Ho * p.Wo);
    const int r = mm - b * (p.Ho * p.Wo);
    const int oy = r / p.Wo, ox = r - oy * p.Wo;
    img[h] = p.in + (size_t)b * p.H * p.W * p.Cin;
    iy0[h] = oy * p.sy - p.pt;
    ix0[h] = ox * p.sx - p.pl;
    const int n = n0 + lrow + 32 * h;
    nvalid[h] = n < p.Cout;
    wrow[h] = p.w + (size_t)(nvalid[h] ? n : 0) * g.K;
  }

  const int ty = tid >> 4, tx = tid & 15;
  int acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0;

  for (int kw0 = 0; kw0 < g.KW; kw0 += BKW) {
#pragma unroll
    for (int h = 0; h < 2; h++) {
      As[lkw][lrow + 32 * h] =
          mvalid[h] ? gather_a<WORDS>(p, img[h], iy0[h], ix0[h], kw0 + lkw, g.K) : 0u;
      Bs[lkw][lrow + 32 * h] = nvalid[h] ? gather_b<WORDS>(wrow[h], kw0 + lkw, g.K) : 0u;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BKW; kk++) {
      unsigned a[4];
      int b[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) b[j] = (int)Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = dp4a_us(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

  // epilogue
  const Epilogue &e = p.epi;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + ty * 4 + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n >= p.Cout) continue;
      int a = acc[i][j];
      if (MODE == EPI_RAW32) {
        if (e.bias) a += __ldg(reinterpret_cast<const int *>(e.bias) + n);
        reinterpret_cast<int *>(p.out)[(size_t)m * p.Cout + n] = a;
      } else {
        if (e.bias) a += (int)__ldg(reinterpret_cast<const int8_t *>(e.bias) + n);
        reinterpret_cast<uint8_t *>(p.out)[(size_t)m * p.Cout + n] = (uint8_t)requant<MODE>(a, n, e);
      }
    }
  }
}

template <bool WORDS>
void launch_mode(const GenericParams &g, dim3 grid, cudaStream_t s)
{
  switch (g.p.epi.mode) {
    case EPI_NONE:  conv_generic_kernel<EPI_NONE, WORDS><<<grid, 256, 0, s>>>(g); break;
    case EPI_MULT:  conv_generic_kernel<EPI_MULT, WORDS><<<grid, 256, 0, s>>>(g); break;
    case EPI_BN32:  conv_generic_kernel<EPI_BN32, WORDS><<<grid, 256, 0, s>>>(g); break;
    case EPI_BN64:  conv_generic_kernel<EPI_BN64, WORDS><<<grid, 256, 0, s>>>(g); break;
    default:        conv_generic_kernel<EPI_RAW32, WORDS><<<grid, 256, 0, s>>>(g); break;
  }
}

}  // namespace

bool launch_conv_generic(Context &c, const ConvProblem &p)
{
  GenericParams g;
  g.p = p;
  const long long M = (long long)p.B * p.Ho * p.Wo;
  if (M > 0x7fffffffLL) { set_error(PULPNN_ERR_UNSUPPORTED, "batch x pixels exceeds 2^31"); return false; }
  g.M = (int)M;
  g.K = p.ky * p.kx * p.Cin;
  g.KW = (g.K + 3) / 4;
  dim3 grid((unsigned)((g.M + BM - 1) / BM), (unsigned)((p.Cout + BN - 1) / BN));
  const bool words = (p.Cin % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.in) & 3) == 0) &&
                     ((reinterpret_cast<uintptr_t>(p.w) & 3) == 0);
  if (words) launch_mode<true>(g, grid, c.stream);
  else       launch_mode<false>(g, grid, c.stream);
  count_launch("conv_generic_kernel");
  return cuda_ok(cudaGetLastError(), "conv_generic launch");
}

}  // namespace pulpnn
