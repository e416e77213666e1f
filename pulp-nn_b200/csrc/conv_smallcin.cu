// conv_smallcin.cu -- standard convolution whose filter row (kx * ch_in bytes) fits in 12 bytes
// and whose ch_out is at most 32: the first layer of an image network (3 input channels, 3x3).
// Same arithmetic as every other convolution here (32bit/src/pulp_nn_conv_Ho_parallel.c:76-186,
// pulp_nn_matmul.c:53-297): acc = bias + sum u8*s8, zero padding, then the requantisation.
//
// With 3 channels the im2col column of a pixel is 27 bytes; the tensor-core path cannot fetch it
// (TMA needs 16-byte rows) and the layer is memory-bound anyway (about 39 op per byte). Layout of
// the work: a CTA stages the input rows of a strip of output rows in shared memory, left/right
// zero padding included, with 4-byte aligned rows. For one output pixel and one filter row the
// kx*ch_in input bytes are CONTIGUOUS in HWC; they are read as three words at an arbitrary byte
// offset (four aligned words + funnel shifts) and multiplied with three weight words per output
// channel whose bytes beyond kx*ch_in are zero, so whatever the third word drags in is ignored.
// A thread computes two output pixels for all 32 output channels: weights are read from shared
// memory as broadcast 16-byte loads (4 channels at a time), one dp4a per channel and word.
#include "internal.cuh"

namespace pulpnn {

namespace {

constexpr int CO = 32;          // output channels held per thread
constexpr int RW = 3;           // weight/input words per filter row

struct SmallParams {
  ConvProblem p;
  int rows_out, rows_in, pitch, lead, row_bytes, vec_rows, vec_store;
};

template <int MODE>
__device__ __forceinline__ void epilogue_px(const int (&acc)[CO], const long long *kS, const long long *lS,
                                            const int *bS, const Epilogue &e, uint8_t *optr, int Cout,
                                            int vec_store)
{
  unsigned w[CO / 4];
#pragma unroll
  for (int c = 0; c < CO; c += 4) {
    int q[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int a = (MODE == EPI_BN32 || MODE == EPI_BN64) ? acc[c + j] : acc[c + j] + bS[c + j];
      if (MODE == EPI_BN32)
        q[j] = (int)((unsigned)(int)kS[c + j] * (unsigned)a + (unsigned)(int)lS[c + j]) >> e.shift;
      else if (MODE == EPI_BN64)
        q[j] = (int)((long long)((unsigned long long)kS[c + j] * (unsigned long long)(long long)a +
                                 (unsigned long long)lS[c + j]) >> e.shift);
      else if (MODE == EPI_MULT)
        q[j] = (int)(short)((int)((unsigned)e.out_mult * (unsigned)a) >> e.shift);
      else
        q[j] = a >> e.shift;
    }
    w[c >> 2] = pack4_sat_u8(q[0], q[1], q[2], q[3]);
  }
  if (vec_store == 2) {
    // all 32 channels of the pixel: one full 32-byte sector
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(optr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
  } else if (vec_store) {
#pragma unroll
    for (int c = 0; c < CO; c += 16)
      if (c < Cout) *reinterpret_cast<uint4 *>(optr + c) = make_uint4(w[c >> 2], w[(c >> 2) + 1], w[(c >> 2) + 2], w[(c >> 2) + 3]);
  } else {
#pragma unroll
    for (int c = 0; c < CO; c++)
      if (c < Cout) optr[c] = (uint8_t)(w[c >> 2] >> (8 * (c & 3)));
  }
}

template <int MODE>
__global__ void __launch_bounds__(256, 2) conv_smallcin_kernel(const SmallParams g)
{
  extern __shared__ __align__(16) uint8_t smem[];
  const ConvProblem &p = g.p;
  const Epilogue &e = p.epi;
  const int tid = threadIdx.x;
  const int b = blockIdx.y, oy0 = blockIdx.x * g.rows_out;
  const int nw = p.ky * RW;                        // weight words per output channel
  unsigned *Ws = reinterpret_cast<unsigned *>(smem);                    // [ky*3][32]
  long long *kS = reinterpret_cast<long long *>(smem + (size_t)nw * CO * 4);   // [32]
  long long *lS = kS + CO;
  int *bS = reinterpret_cast<int *>(lS + CO);
  uint8_t *tile = reinterpret_cast<uint8_t *>(bS + CO);                 // [rows_in][pitch]

  const int rowlen = p.kx * p.Cin;                 // bytes of one filter row
  for (int idx = tid; idx < nw * CO; idx += 256) {
    const int co = idx & (CO - 1), fj = idx >> 5;
    const int fy = fj / RW, j = fj - fy * RW;
    unsigned v = 0;
    if (co < p.Cout) {
      const int8_t *w = p.w + ((size_t)co * p.ky + fy) * rowlen;
#pragma unroll
      for (int t = 0; t < 4; t++)
        if (4 * j + t < rowlen) v |= (unsigned)(uint8_t)__ldg(w + 4 * j + t) << (8 * t);
    }
    Ws[fj * CO + co] = v;
  }
  if (tid < CO) {
    const int c = tid;
    const bool v = c < p.Cout;
    const int bias = (v && e.bias) ? (int)__ldg(reinterpret_cast<const int8_t *>(e.bias) + c) : 0;
    long long k = 0, l = 0;
    if (v && MODE == EPI_BN32) {
      k = __ldg(reinterpret_cast<const int *>(e.k) + c);
      l = (int)((unsigned)(int)k * (unsigned)bias + (unsigned)__ldg(reinterpret_cast<const int *>(e.lambda) + c));
    } else if (v && MODE == EPI_BN64) {
      k = __ldg(reinterpret_cast<const long long *>(e.k) + c);
      l = (long long)((unsigned long long)k * (unsigned long long)(long long)bias +
                      (unsigned long long)__ldg(reinterpret_cast<const long long *>(e.lambda) + c));
    }
    kS[c] = k; lS[c] = l; bS[c] = bias;
  }

  // stage the input rows: [lead zero bytes][row_bytes of data][zeros up to pitch]
  const int iy_first = oy0 * p.sy - p.pt;
  const uint8_t *img = p.in + (size_t)b * p.H * g.row_bytes;
  if (g.vec_rows) {
    const int wpr = g.pitch >> 2, lead_w = g.lead >> 2, data_w = g.row_bytes >> 2;
    for (int idx = tid; idx < g.rows_in * wpr; idx += 256) {
      const int r = idx / wpr, wi = idx - r * wpr;
      const int iy = iy_first + r, dw = wi - lead_w;
      unsigned v = 0;
      if ((unsigned)iy < (unsigned)p.H && (unsigned)dw < (unsigned)data_w)
        v = __ldg(reinterpret_cast<const unsigned *>(img + (size_t)iy * g.row_bytes) + dw);
      reinterpret_cast<unsigned *>(tile)[idx] = v;
    }
  } else {
    for (int idx = tid; idx < g.rows_in * g.pitch; idx += 256) {
      const int r = idx / g.pitch, bi = idx - r * g.pitch;
      const int iy = iy_first + r, db = bi - g.lead;
      uint8_t v = 0;
      if ((unsigned)iy < (unsigned)p.H && (unsigned)db < (unsigned)g.row_bytes)
        v = __ldg(img + (size_t)iy * g.row_bytes + db);
      tile[idx] = v;
    }
  }
  __syncthreads();

  const int rows = min(g.rows_out, p.Ho - oy0);
  const int npix = rows * p.Wo;
  for (int q0 = 2 * tid; q0 < npix; q0 += 512) {
    int acc0[CO], acc1[CO];
#pragma unroll
    for (int c = 0; c < CO; c++) { acc0[c] = 0; acc1[c] = 0; }
    const bool two = q0 + 1 < npix;
    const int r0 = q0 / p.Wo, x0 = q0 - r0 * p.Wo;
    const int q1 = two ? q0 + 1 : q0;
    const int r1 = q1 / p.Wo, x1 = q1 - r1 * p.Wo;
    const int o0 = g.lead + (x0 * p.sx - p.pl) * p.Cin, o1 = g.lead + (x1 * p.sx - p.pl) * p.Cin;
    for (int fy = 0; fy < p.ky; fy++) {
      unsigned col0[RW], col1[RW];
      {
        const unsigned *rp = reinterpret_cast<const unsigned *>(tile + (size_t)(r0 * p.sy + fy) * g.pitch) + (o0 >> 2);
        const unsigned sh = (o0 & 3) * 8;
        const unsigned s0 = rp[0], s1 = rp[1], s2 = rp[2], s3 = rp[3];
        col0[0] = __funnelshift_r(s0, s1, sh); col0[1] = __funnelshift_r(s1, s2, sh); col0[2] = __funnelshift_r(s2, s3, sh);
      }
      {
        const unsigned *rp = reinterpret_cast<const unsigned *>(tile + (size_t)(r1 * p.sy + fy) * g.pitch) + (o1 >> 2);
        const unsigned sh = (o1 & 3) * 8;
        const unsigned s0 = rp[0], s1 = rp[1], s2 = rp[2], s3 = rp[3];
        col1[0] = __funnelshift_r(s0, s1, sh); col1[1] = __funnelshift_r(s1, s2, sh); col1[2] = __funnelshift_r(s2, s3, sh);
      }
#pragma unroll
      for (int j = 0; j < RW; j++) {
        const uint4 *wrow = reinterpret_cast<const uint4 *>(Ws + (fy * RW + j) * CO);
#pragma unroll
        for (int c4 = 0; c4 < CO / 4; c4++) {
          const uint4 w = wrow[c4];
          acc0[4 * c4 + 0] = dp4a_us(col0[j], (int)w.x, acc0[4 * c4 + 0]);
          acc0[4 * c4 + 1] = dp4a_us(col0[j], (int)w.y, acc0[4 * c4 + 1]);
          acc0[4 * c4 + 2] = dp4a_us(col0[j], (int)w.z, acc0[4 * c4 + 2]);
          acc0[4 * c4 + 3] = dp4a_us(col0[j], (int)w.w, acc0[4 * c4 + 3]);
          acc1[4 * c4 + 0] = dp4a_us(col1[j], (int)w.x, acc1[4 * c4 + 0]);
          acc1[4 * c4 + 1] = dp4a_us(col1[j], (int)w.y, acc1[4 * c4 + 1]);
          acc1[4 * c4 + 2] = dp4a_us(col1[j], (int)w.z, acc1[4 * c4 + 2]);
          acc1[4 * c4 + 3] = dp4a_us(col1[j], (int)w.w, acc1[4 * c4 + 3]);
        }
      }
    }
    uint8_t *obase = reinterpret_cast<uint8_t *>(p.out) + ((size_t)b * p.Ho + oy0) * p.Wo * p.Cout;
    epilogue_px<MODE>(acc0, kS, lS, bS, e, obase + (size_t)q0 * p.Cout, p.Cout, g.vec_store);
    if (two) epilogue_px<MODE>(acc1, kS, lS, bS, e, obase + (size_t)q1 * p.Cout, p.Cout, g.vec_store);
  }
}

}  // namespace

bool conv_smallcin_supported(const ConvProblem &p)
{
  if (p.epi.mode == EPI_RAW32) return false;
  if (p.kx * p.Cin > 4 * RW || p.Cout > CO || p.ky > 8) return false;
  if ((long long)p.W * p.Cin > 16384 || p.B > 65535) return false;
  // the last pixel's three words must end inside a staged row (pitch = lead + (W+kx)*Cin + 16)
  if ((p.Wo - 1) * p.sx - p.pl > p.W + p.kx) return false;
  return true;
}

bool launch_conv_smallcin(Context &c, const ConvProblem &p)
{
  SmallParams g;
  g.p = p;
  g.row_bytes = p.W * p.Cin;
  g.lead = (p.pl * p.Cin + 3) & ~3;
  g.pitch = (g.lead + (p.W + p.kx) * p.Cin + 16 + 3) & ~3;
  g.vec_rows = (g.row_bytes % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.in) & 3) == 0);
  g.vec_store = (p.Cout % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
  if (p.Cout == CO && (reinterpret_cast<uintptr_t>(p.out) & 31) == 0) g.vec_store = 2;
  const size_t fixed = (size_t)p.ky * RW * CO * 4 + CO * (8 + 8 + 4);
  // strip height: shared memory under 48 KB, and a pixel-pair count close to a multiple of 256
  int best = 1; double best_waste = 1e9;
  for (int ro = 1; ro <= p.Ho && ro <= 64; ro++) {
    const int rin = (ro - 1) * p.sy + p.ky;
    if (fixed + (size_t)rin * g.pitch > 46 * 1024) break;
    const int pairs = (ro * p.Wo + 1) / 2;
    const int iters = (pairs + 255) / 256;
    const double waste = (double)iters * 256 / pairs + 0.25 * (p.ky - p.sy > 0 ? (double)(p.ky - p.sy) / (ro * p.sy) : 0.0);
    if (waste < best_waste - 1e-9) { best_waste = waste; best = ro; }
  }
  g.rows_out = best;
  g.rows_in = (best - 1) * p.sy + p.ky;
  const size_t smem = fixed + (size_t)g.rows_in * g.pitch;
  if (smem > 48 * 1024) { set_error(PULPNN_ERR_UNSUPPORTED, "conv: one input row strip does not fit in shared memory"); return false; }
  dim3 grid((unsigned)((p.Ho + best - 1) / best), (unsigned)p.B);
  switch (p.epi.mode) {
    case EPI_NONE: conv_smallcin_kernel<EPI_NONE><<<grid, 256, smem, c.stream>>>(g); break;
    case EPI_MULT: conv_smallcin_kernel<EPI_MULT><<<grid, 256, smem, c.stream>>>(g); break;
    case EPI_BN32: conv_smallcin_kernel<EPI_BN32><<<grid, 256, smem, c.stream>>>(g); break;
    default:       conv_smallcin_kernel<EPI_BN64><<<grid, 256, smem, c.stream>>>(g); break;
  }
  count_launch("conv_smallcin_kernel");
  return cuda_ok(cudaGetLastError(), "conv_smallcin launch");
}

}  // namespace pulpnn
