// depthwise.cu -- depthwise convolution, the two layouts.
//
// Arithmetic (32bit/src/pulp_nn_depthwise_generic.c:133-180): per channel,
//   acc = bias[c] + sum over ky x kx taps of in * w[c][fy][fx], zero outside the image,
// followed by the requantisation of internal.cuh with k[c], lambda[c]. Both kernels are
// memory-bound: one pass over the input, one over the output.
//
//  * CHW in / HWC out (the reference layout): a CTA takes one image, a group of 32 channels
//    and a strip of output rows; it stages the input rows the strip needs (contiguous per
//    channel in CHW, fetched with 16-byte loads) in shared memory and then lets lane = channel
//    walk the strip, so that a warp writes 32 consecutive bytes of each HWC output pixel. The
//    per-channel pitch in shared memory is an odd number of words, which makes the 32 lanes of
//    a warp hit 32 different banks.
//  * HWC in / HWC out (what every other kernel of this library produces): a thread owns four
//    adjacent channels (one 32-bit word per pixel) and a run of output pixels along x; a tap
//    costs one dp4a per channel with a weight word that is zero in the other three byte lanes,
//    so no byte unpacking is needed. Neighbouring threads re-read the input through L1.
#include "internal.cuh"

namespace pulpnn {

namespace {

// ------------------------------------------------------------------------------------------
// CHW -> HWC
// ------------------------------------------------------------------------------------------
constexpr int CG = 32;                 // channels per CTA

struct ChwParams {
  DepthwiseProblem p;
  int rows_out;       // output rows per CTA
  int rows_in;        // (rows_out-1)*sy + ky
  int pitch;          // bytes per channel in shared memory, pitch/4 odd
  int vec16;          // 1: rows are fetched with 16-byte loads
};

template <int MODE>
__global__ void __launch_bounds__(256) depthwise_chw_kernel(const ChwParams g)
{
  extern __shared__ __align__(16) uint8_t smem[];
  const DepthwiseProblem &p = g.p;
  const int b = blockIdx.z, c0 = blockIdx.y * CG, oy0 = blockIdx.x * g.rows_out;
  const int nch = min(CG, p.C - c0);
  const int iy_first = oy0 * p.sy - p.pt;           // may be negative
  const int taps = p.ky * p.kx;
  uint8_t *tile = smem;                              // [CG][pitch]
  int8_t *wsm = reinterpret_cast<int8_t *>(smem + (size_t)CG * g.pitch);   // [CG][taps]

  for (int i = threadIdx.x; i < nch * taps; i += blockDim.x)
    wsm[i] = __ldg(p.w + (size_t)c0 * taps + i);

  // stage rows [iy_first, iy_first + rows_in) of each channel; rows outside the image are zero
  const int iy_lo = max(iy_first, 0), iy_hi = min(iy_first + g.rows_in, p.H);
  const int row_off = (iy_lo - iy_first) * p.W;      // byte offset of the first real row
  const int nbytes = max(iy_hi - iy_lo, 0) * p.W;    // contiguous in CHW
  const int total = g.rows_in * p.W;
  for (int c = threadIdx.x >> 5; c < nch; c += blockDim.x >> 5) {
    const int lane = threadIdx.x & 31;
    uint8_t *dst = tile + (size_t)c * g.pitch;
    const uint8_t *src = p.in + (((size_t)b * p.C + c0 + c) * p.H + iy_lo) * p.W;
    for (int i = lane; i < row_off; i += 32) dst[i] = 0;
    for (int i = row_off + nbytes + lane; i < total; i += 32) dst[i] = 0;
    if (g.vec16 && (row_off & 3) == 0) {
      const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
      unsigned *d = reinterpret_cast<unsigned *>(dst + row_off);
      const int n16 = nbytes >> 4;
      for (int i = lane; i < n16; i += 32) {
        const uint4 v = __ldg(s4 + i);
        d[4 * i + 0] = v.x; d[4 * i + 1] = v.y; d[4 * i + 2] = v.z; d[4 * i + 3] = v.w;
      }
      for (int i = (n16 << 4) + lane; i < nbytes; i += 32) dst[row_off + i] = __ldg(src + i);
    } else {
      for (int i = lane; i < nbytes; i += 32) dst[row_off + i] = __ldg(src + i);
    }
  }
  __syncthreads();

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  if (lane >= nch) return;
  const int c = c0 + lane;
  const Epilogue &e = p.epi;
  long long kk = 0, ll = 0;
  if (MODE == EPI_BN32) {
    kk = __ldg(reinterpret_cast<const int *>(e.k) + c);
    ll = __ldg(reinterpret_cast<const int *>(e.lambda) + c);
  } else if (MODE == EPI_BN64) {
    kk = __ldg(reinterpret_cast<const long long *>(e.k) + c);
    ll = __ldg(reinterpret_cast<const long long *>(e.lambda) + c);
  }
  const int bias = e.bias ? (int)__ldg(reinterpret_cast<const int8_t *>(e.bias) + c) : 0;
  const uint8_t *mine = tile + (size_t)lane * g.pitch;
  const int8_t *wmine = wsm + lane * taps;
  const int rows = min(g.rows_out, p.Ho - oy0);
  for (int q = warp; q < rows * p.Wo; q += nwarp) {
    const int r = q / p.Wo, ox = q - r * p.Wo;
    const int ix0 = ox * p.sx - p.pl;
    int acc = bias;
    for (int fy = 0; fy < p.ky; fy++) {
      const uint8_t *row = mine + (r * p.sy + fy) * p.W;
      for (int fx = 0; fx < p.kx; fx++) {
        const int ix = ix0 + fx;
        if ((unsigned)ix < (unsigned)p.W) acc += (int)row[ix] * (int)wmine[fy * p.kx + fx];
      }
    }
    p.out[(((size_t)b * p.Ho + oy0 + r) * p.Wo + ox) * p.C + c] =
        (uint8_t)requant_kl<MODE>(acc, kk, ll, e.out_mult, e.shift);
  }
}

// ------------------------------------------------------------------------------------------
// HWC -> HWC, four channels per thread
// ------------------------------------------------------------------------------------------
constexpr int XRUN = 4;                // output pixels along x per thread

template <int MODE, int KY, int KX>
__global__ void __launch_bounds__(256) depthwise_hwc4_kernel(const DepthwiseProblem p, int C4,
                                                             int xruns, long long total)
{
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  // t -> (b, oy, xrun, c4) with c4 fastest so that a warp reads consecutive words
  const int c4 = (int)(t % C4);
  long long r = t / C4;
  const int xr = (int)(r % xruns); r /= xruns;
  const int oy = (int)(r % p.Ho);
  const int b = (int)(r / p.Ho);
  const int c = c4 * 4;
  const int ky = KY ? KY : p.ky, kx = KX ? KX : p.kx;

  const Epilogue &e = p.epi;
  long long kk[4] = {0, 0, 0, 0}, ll[4] = {0, 0, 0, 0};
  int bias[4] = {0, 0, 0, 0};
#pragma unroll
  for (int j = 0; j < 4; j++) {
    if (MODE == EPI_BN32) {
      kk[j] = __ldg(reinterpret_cast<const int *>(e.k) + c + j);
      ll[j] = __ldg(reinterpret_cast<const int *>(e.lambda) + c + j);
    } else if (MODE == EPI_BN64) {
      kk[j] = __ldg(reinterpret_cast<const long long *>(e.k) + c + j);
      ll[j] = __ldg(reinterpret_cast<const long long *>(e.lambda) + c + j);
    }
    if (e.bias) bias[j] = (int)__ldg(reinterpret_cast<const int8_t *>(e.bias) + c + j);
  }

  const uint8_t *img = p.in + (size_t)b * p.H * p.W * p.C + c;
  const int iy0 = oy * p.sy - p.pt;
  const int ox0 = xr * XRUN;
  int acc[XRUN][4];
#pragma unroll
  for (int x = 0; x < XRUN; x++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[x][j] = bias[j];

  for (int fy = 0; fy < ky; fy++) {
    const int iy = iy0 + fy;
    if ((unsigned)iy >= (unsigned)p.H) continue;
    const uint8_t *row = img + (size_t)iy * p.W * p.C;
    for (int fx = 0; fx < kx; fx++) {
      // weight word of channel j: w[c+j][fy][fx] in byte lane j, zero elsewhere
      int wsel[4];
#pragma unroll
      for (int j = 0; j < 4; j++)
        wsel[j] = (int)((unsigned)(uint8_t)__ldg(p.w + ((size_t)(c + j) * ky + fy) * kx + fx) << (8 * j));
#pragma unroll
      for (int x = 0; x < XRUN; x++) {
        const int ix = (ox0 + x) * p.sx - p.pl + fx;
        if ((unsigned)ix < (unsigned)p.W && ox0 + x < p.Wo) {
          const unsigned v = __ldg(reinterpret_cast<const unsigned *>(row + (size_t)ix * p.C));
#pragma unroll
          for (int j = 0; j < 4; j++) acc[x][j] = dp4a_us(v, wsel[j], acc[x][j]);
        }
      }
    }
  }
#pragma unroll
  for (int x = 0; x < XRUN; x++) {
    if (ox0 + x >= p.Wo) break;
    unsigned o = 0;
#pragma unroll
    for (int j = 0; j < 4; j++)
      o |= (unsigned)requant_kl<MODE>(acc[x][j], kk[j], ll[j], e.out_mult, e.shift) << (8 * j);
    *reinterpret_cast<unsigned *>(p.out + (((size_t)b * p.Ho + oy) * p.Wo + ox0 + x) * p.C + c) = o;
  }
}

// scalar HWC fallback: one thread per output byte (ragged channel counts / unaligned pointers)
template <int MODE>
__global__ void __launch_bounds__(256) depthwise_hwc1_kernel(const DepthwiseProblem p, long long total)
{
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const int c = (int)(t % p.C);
  long long r = t / p.C;
  const int ox = (int)(r % p.Wo); r /= p.Wo;
  const int oy = (int)(r % p.Ho);
  const int b = (int)(r / p.Ho);
  const Epilogue &e = p.epi;
  int acc = e.bias ? (int)__ldg(reinterpret_cast<const int8_t *>(e.bias) + c) : 0;
  const uint8_t *img = p.in + (size_t)b * p.H * p.W * p.C + c;
  for (int fy = 0; fy < p.ky; fy++) {
    const int iy = oy * p.sy - p.pt + fy;
    if ((unsigned)iy >= (unsigned)p.H) continue;
    for (int fx = 0; fx < p.kx; fx++) {
      const int ix = ox * p.sx - p.pl + fx;
      if ((unsigned)ix >= (unsigned)p.W) continue;
      acc += (int)__ldg(img + ((size_t)iy * p.W + ix) * p.C) *
             (int)__ldg(p.w + ((size_t)c * p.ky + fy) * p.kx + fx);
    }
  }
  p.out[t] = (uint8_t)requant<MODE>(acc, c, e);
}

template <int MODE>
bool launch_dw_mode(Context &c, const DepthwiseProblem &p)
{
  if (!p.in_is_hwc) {
    ChwParams g;
    g.p = p;
    // strip height: keep the staged rows of 32 channels within ~48 KB
    int rows_out = p.Ho;
    auto rows_in_of = [&](int ro) { return (ro - 1) * p.sy + p.ky; };
    while (rows_out > 1 && (size_t)rows_in_of(rows_out) * p.W * CG > 48 * 1024) rows_out = (rows_out + 1) / 2;
    g.rows_out = rows_out;
    g.rows_in = rows_in_of(rows_out);
    int pitch = (g.rows_in * p.W + 3) & ~3;
    if (((pitch >> 2) & 1) == 0) pitch += 4;
    g.pitch = pitch;
    g.vec16 = (p.W % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.in) & 15) == 0) ? 1 : 0;
    const size_t smem = (size_t)CG * pitch + (size_t)CG * p.ky * p.kx;
    if (smem > 200 * 1024) {
      set_error(PULPNN_ERR_UNSUPPORTED, "depthwise: one strip of input rows does not fit in shared memory "
                "(%zu bytes)", smem);
      return false;
    }
    if (smem > 48 * 1024 &&
        !cuda_ok(cudaFuncSetAttribute(depthwise_chw_kernel<MODE>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                 "cudaFuncSetAttribute"))
      return false;
    dim3 grid((unsigned)((p.Ho + rows_out - 1) / rows_out), (unsigned)((p.C + CG - 1) / CG), (unsigned)p.B);
    depthwise_chw_kernel<MODE><<<grid, 256, smem, c.stream>>>(g);
  } else {
    const bool vec = (p.C % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.in) & 3) == 0) &&
                     ((reinterpret_cast<uintptr_t>(p.out) & 3) == 0);
    if (vec) {
      const int C4 = p.C / 4, xruns = (p.Wo + XRUN - 1) / XRUN;
      const long long total = (long long)p.B * p.Ho * xruns * C4;
      const unsigned blocks = (unsigned)((total + 255) / 256);
      if (p.ky == 3 && p.kx == 3)
        depthwise_hwc4_kernel<MODE, 3, 3><<<blocks, 256, 0, c.stream>>>(p, C4, xruns, total);
      else
        depthwise_hwc4_kernel<MODE, 0, 0><<<blocks, 256, 0, c.stream>>>(p, C4, xruns, total);
    } else {
      const long long total = (long long)p.B * p.Ho * p.Wo * p.C;
      depthwise_hwc1_kernel<MODE><<<(unsigned)((total + 255) / 256), 256, 0, c.stream>>>(p, total);
    }
  }
  count_launch("depthwise_generic_kernel");
  return cuda_ok(cudaGetLastError(), "depthwise launch");
}

}  // namespace

bool launch_depthwise(Context &c, const DepthwiseProblem &p)
{
  if (!c.opt_force_generic && depthwise_hwc3x3_tma_supported(p)) return launch_depthwise_hwc3x3_tma(c, p);
  if (!c.opt_force_generic && depthwise_hwc3x3_supported(p)) return launch_depthwise_hwc3x3(c, p);
  if (!c.opt_force_generic && depthwise_chw3x3_tma_supported(p)) return launch_depthwise_chw3x3_tma(c, p);
  if (!c.opt_force_generic && depthwise_chw3x3_supported(p)) return launch_depthwise_chw3x3(c, p);
  switch (p.epi.mode) {
    case EPI_NONE: return launch_dw_mode<EPI_NONE>(c, p);
    case EPI_MULT: return launch_dw_mode<EPI_MULT>(c, p);
    case EPI_BN32: return launch_dw_mode<EPI_BN32>(c, p);
    default:       return launch_dw_mode<EPI_BN64>(c, p);
  }
}

}  // namespace pulpnn
