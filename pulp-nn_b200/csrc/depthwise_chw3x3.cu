// depthwise_chw3x3.cu -- the reference's own depthwise layout (CHW in, HWC out,
// 32bit/src/pulp_nn_depthwise_generic.c:74,81) for 3x3 filters with padding 1 and stride 1 or 2.
// Same arithmetic as depthwise.cu; this kernel exists because the third benchmark configuration
// (112x112x64, stride 2, 64-bit batch-norm) is pure memory traffic and should run at memory speed.
//
// In CHW a row of one channel is contiguous, so four horizontally adjacent pixels of a channel
// are simply one aligned 32-bit word: a lane takes four output columns of one channel row, loads
// the one (stride 1) or two (stride 2) words they cover -- lanes of a warp walk along the row, so
// the loads are fully coalesced -- gets the neighbouring word from the next lane with a shuffle,
// forms the shifted windows with funnel shifts and spends one dp4a per output and filter row
// (weights [w0,w1,w2,0] or [0,w0,w1,w2]). A thread does this for four consecutive channels,
// transposes the four result words (4 pixels x 4 channels) in registers and drops them into a
// shared-memory tile laid out as the HWC output (XOR-swizzled so that neither these stores nor the
// read-out conflict). Once the strip is complete the CTA streams the tile to global memory with
// consecutive lanes writing consecutive words, i.e. whole HWC pixels.
#include <type_traits>

#include "internal.cuh"

namespace pulpnn {

namespace {

__device__ __forceinline__ unsigned prmt(unsigned a, unsigned b, unsigned sel)
{
  unsigned d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

struct Chw3Params {
  DepthwiseProblem p;
  int rows_out;     // output rows per CTA
  int groups;       // 4-column groups per output row (<= 32)
  int qpw;          // channel quads handled side by side in one warp (32 / groups)
  int ctile;        // channels per CTA: power of two, 4..64
};

// requantisation of one accumulator with the channel's parameters in registers
template <int MODE>
__device__ __forceinline__ int requant_one(int acc, long long k, long long l, int bias, const Epilogue &e)
{
  if (MODE == EPI_BN32) return (int)((unsigned)(int)k * (unsigned)acc + (unsigned)(int)l) >> e.shift;
  if (MODE == EPI_BN64)   // l already holds k*bias + lambda
    return (int)((long long)((unsigned long long)k * (unsigned long long)(long long)acc + (unsigned long long)l) >> e.shift);
  if (MODE == EPI_MULT) return (int)(short)((int)((unsigned)e.out_mult * (unsigned)(acc + bias)) >> e.shift);
  return (acc + bias) >> e.shift;
}

template <int MODE, int S>
__global__ void __launch_bounds__(256) depthwise_chw3x3_kernel(const Chw3Params g)
{
  extern __shared__ __align__(16) unsigned tile[];      // [rows_out * Wo][ctile / 4] words, swizzled
  const DepthwiseProblem &p = g.p;
  const Epilogue &e = p.epi;
  const int b = blockIdx.z, c_base = blockIdx.y * g.ctile, oy0 = blockIdx.x * g.rows_out;
  const int rows = min(g.rows_out, p.Ho - oy0);
  const int wpp = g.ctile >> 2;                           // words per pixel in the tile
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gidx = lane % g.groups, qsub = lane / g.groups;
  const bool lane_on = qsub < g.qpw;
  const int nquads = (min(g.ctile, p.C - c_base) + 3) >> 2;
  const int ox0 = gidx * 4;
  const int wrow = p.W >> 2;                              // words per input row
  // word index of the first word this lane loads in an input row
  const int w0 = S == 1 ? gidx : 2 * gidx;

  for (int qbase = warp * g.qpw; qbase < nquads; qbase += 8 * g.qpw) {   // warp-uniform
    const int q = qbase + qsub;
    const bool q_on = lane_on && q < nquads;
    const int c0 = c_base + 4 * q;
    int wa[4][3], wb[4][3], bias[4];
    long long kk[4], ll[4];
    bool k32 = true;                     // 64-bit mode: all four k of this thread fit in 32 bits
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const bool c_on = q_on && c0 + j < p.C;
      const int c = c_on ? c0 + j : 0;
      const int8_t *w = p.w + (size_t)c * 9;
#pragma unroll
      for (int fy = 0; fy < 3; fy++) {
        const unsigned v = (unsigned)(uint8_t)__ldg(w + fy * 3) | ((unsigned)(uint8_t)__ldg(w + fy * 3 + 1) << 8) |
                           ((unsigned)(uint8_t)__ldg(w + fy * 3 + 2) << 16);
        wa[j][fy] = c_on ? (int)v : 0;
        wb[j][fy] = c_on ? (int)(v << 8) : 0;
      }
      bias[j] = e.bias ? (int)__ldg(reinterpret_cast<const int8_t *>(e.bias) + c) : 0;
      kk[j] = 0; ll[j] = 0;
      if (MODE == EPI_BN32) {
        const int k = __ldg(reinterpret_cast<const int *>(e.k) + c);
        kk[j] = k;
        ll[j] = (int)((unsigned)k * (unsigned)bias[j] + (unsigned)__ldg(reinterpret_cast<const int *>(e.lambda) + c));
      } else if (MODE == EPI_BN64) {
        const long long k = __ldg(reinterpret_cast<const long long *>(e.k) + c);
        kk[j] = k;
        ll[j] = (long long)((unsigned long long)k * (unsigned long long)(long long)bias[j] +
                            (unsigned long long)__ldg(reinterpret_cast<const long long *>(e.lambda) + c));
        k32 = k32 && (k == (long long)(int)k);
      }
    }
    const unsigned *chan0 = reinterpret_cast<const unsigned *>(p.in + ((size_t)b * p.C + (q_on ? c0 : 0)) * p.H * p.W);
    const size_t chan_words = (size_t)p.H * wrow;

    // Words of the three input rows of the current output row, per channel: x0 (and x1 at stride 2)
    // are the lane's own words, xr (stride 1 only) is the word right of the last column group.
    // Consecutive output rows share 3-S input rows, so only S rows are fetched per output row, and
    // they are fetched one output row ahead.
    unsigned x0[4][3], x1[4][3], xr[4][3];
    unsigned n0[4][S], n1[4][S], nr[4][S];
    auto fetch = [&](int iy, int j, unsigned &a, unsigned &bb, unsigned &rr) {
      a = 0u; bb = 0u; rr = 0u;
      if (q_on && c0 + j < p.C && (unsigned)iy < (unsigned)p.H) {
        const unsigned *rowp = chan0 + (size_t)j * chan_words + (size_t)iy * wrow;
        if (S == 1) {
          if (w0 < wrow) a = __ldg(rowp + w0);
          if (gidx == g.groups - 1 && w0 + 1 < wrow) rr = __ldg(rowp + w0 + 1);
        } else if (w0 + 1 < wrow) {
          const uint2 v = __ldg(reinterpret_cast<const uint2 *>(rowp + w0));
          a = v.x; bb = v.y;
        } else if (w0 < wrow) {
          a = __ldg(rowp + w0);
        }
      }
    };
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
      for (int fy = 0; fy < 3; fy++) fetch(oy0 * S - 1 + fy, j, x0[j][fy], x1[j][fy], xr[j][fy]);

    for (int r = 0; r < rows; r++) {
      if (r + 1 < rows) {
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
          for (int t = 0; t < S; t++) fetch((oy0 + r + 1) * S - 1 + (3 - S) + t, j, n0[j][t], n1[j][t], nr[j][t]);
      }
      unsigned res[4];                                     // per channel: 4 packed output pixels
#pragma unroll
      for (int j = 0; j < 4; j++) {
        int a0 = 0, a1 = 0, a2 = 0, a3 = 0;
#pragma unroll
        for (int fy = 0; fy < 3; fy++) {
          if (S == 1) {
            // outputs ox0..ox0+3 read pixels ox0-1..ox0+4: the lane's word and one byte each of its neighbours'
            const unsigned m = x0[j][fy];
            unsigned hm = __shfl_up_sync(0xffffffffu, m, 1);
            unsigned hp = __shfl_down_sync(0xffffffffu, m, 1);
            if (gidx == 0) hm = 0u;
            if (gidx == g.groups - 1) hp = xr[j][fy];              // no lane holds that word
            const unsigned A = __funnelshift_r(hm, m, 24);           // [p-1, p0, p1, p2]
            const unsigned Bw = __funnelshift_r(m, hp, 16);          // [p2, p3, p4, p5]
            a0 = dp4a_us(A, wa[j][fy], a0);
            a1 = dp4a_us(m, wa[j][fy], a1);
            a2 = dp4a_us(m, wb[j][fy], a2);
            a3 = dp4a_us(Bw, wa[j][fy], a3);
          } else {
            // outputs ox0..ox0+3 read pixels 2*ox0-1..2*ox0+7: two words of the lane, one byte of the left neighbour
            const unsigned m0 = x0[j][fy], m1 = x1[j][fy];
            unsigned hm = __shfl_up_sync(0xffffffffu, m1, 1);
            if (gidx == 0) hm = 0u;
            const unsigned A = __funnelshift_r(hm, m0, 24);          // [p-1, p0, p1, p2]
            const unsigned Cw = __funnelshift_r(m0, m1, 24);         // [p3, p4, p5, p6]
            a0 = dp4a_us(A, wa[j][fy], a0);
            a1 = dp4a_us(m0, wb[j][fy], a1);
            a2 = dp4a_us(Cw, wa[j][fy], a2);
            a3 = dp4a_us(m1, wb[j][fy], a3);
          }
        }
        // slide the window down by S input rows
#pragma unroll
        for (int fy = 0; fy < 3 - S; fy++) { x0[j][fy] = x0[j][fy + S]; x1[j][fy] = x1[j][fy + S]; xr[j][fy] = xr[j][fy + S]; }
#pragma unroll
        for (int t = 0; t < S; t++) { x0[j][3 - S + t] = n0[j][t]; x1[j][3 - S + t] = n1[j][t]; xr[j][3 - S + t] = nr[j][t]; }
        if (MODE == EPI_BN64 && k32) {
          // every k of this thread fits in 32 bits: one wide multiply-add per output
          const long long kj = (long long)(int)kk[j];
          res[j] = pack4_sat_u8((int)((kj * a0 + ll[j]) >> e.shift), (int)((kj * a1 + ll[j]) >> e.shift),
                                (int)((kj * a2 + ll[j]) >> e.shift), (int)((kj * a3 + ll[j]) >> e.shift));
        } else {
          res[j] = pack4_sat_u8(requant_one<MODE>(a0, kk[j], ll[j], bias[j], e), requant_one<MODE>(a1, kk[j], ll[j], bias[j], e),
                                requant_one<MODE>(a2, kk[j], ll[j], bias[j], e), requant_one<MODE>(a3, kk[j], ll[j], bias[j], e));
        }
      }
      // res[j] = channel j, pixels 0..3  ->  pix[i] = pixel i, channels 0..3
      const unsigned ta = prmt(res[0], res[1], 0x5140), tb = prmt(res[0], res[1], 0x7362);
      const unsigned tc = prmt(res[2], res[3], 0x5140), td = prmt(res[2], res[3], 0x7362);
      unsigned pix[4];
      pix[0] = prmt(ta, tc, 0x5410); pix[1] = prmt(ta, tc, 0x7632);
      pix[2] = prmt(tb, td, 0x5410); pix[3] = prmt(tb, td, 0x7632);
      if (q_on) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const int ox = ox0 + i;
          if (ox < p.Wo) {
            const int px = r * p.Wo + ox;
            tile[px * wpp + (q ^ ((px >> 2) & (wpp - 1)))] = pix[i];
          }
        }
      }
    }
  }
  __syncthreads();

  // stream the tile out: consecutive threads take consecutive words of the HWC output
  const int cvalid = min(g.ctile, p.C - c_base) >> 2;       // whole words of real channels per pixel
  const int npx = rows * p.Wo;
  uint8_t *obase = p.out + (((size_t)b * p.Ho + oy0) * p.Wo) * p.C + c_base;
  for (int idx = threadIdx.x; idx < npx * wpp; idx += 256) {
    const int px = idx / wpp, wq = idx - px * wpp;
    if (wq < cvalid)
      *reinterpret_cast<unsigned *>(obase + (size_t)px * p.C + 4 * wq) = tile[px * wpp + (wq ^ ((px >> 2) & (wpp - 1)))];
  }
}

template <int MODE>
bool launch_mode(Context &c, const Chw3Params &g, dim3 grid, size_t smem)
{
  if (g.p.sx == 1) depthwise_chw3x3_kernel<MODE, 1><<<grid, 256, smem, c.stream>>>(g);
  else             depthwise_chw3x3_kernel<MODE, 2><<<grid, 256, smem, c.stream>>>(g);
  count_launch("depthwise_chw3x3_kernel");
  return cuda_ok(cudaGetLastError(), "depthwise_chw3x3 launch");
}

}  // namespace

bool depthwise_chw3x3_supported(const DepthwiseProblem &p)
{
  if (p.in_is_hwc || p.ky != 3 || p.kx != 3 || p.pt != 1 || p.pl != 1) return false;
  if (p.sx != p.sy || (p.sx != 1 && p.sx != 2)) return false;
  if (p.W % 4 != 0 || p.C % 4 != 0 || p.B > 65535) return false;
  if ((reinterpret_cast<uintptr_t>(p.in) & 7) || (reinterpret_cast<uintptr_t>(p.out) & 3)) return false;
  if (p.sx == 2 && ((p.W / 4) & 1) != 0) return false;       // 8-byte loads need an even word count per row
  if ((p.Wo + 3) / 4 > 32) return false;                     // one warp spans an output row
  return true;
}

bool launch_depthwise_chw3x3(Context &c, const DepthwiseProblem &p)
{
  Chw3Params g;
  g.p = p;
  g.groups = (p.Wo + 3) / 4;
  g.qpw = 32 / g.groups;
  int ctile = 4;
  while (ctile < 64 && ctile < p.C) ctile *= 2;
  g.ctile = ctile;
  int rows_out = 8;
  while (rows_out > 1 && (size_t)rows_out * p.Wo * ctile > 40 * 1024) rows_out /= 2;
  if (rows_out > p.Ho) rows_out = p.Ho;
  g.rows_out = rows_out;
  const size_t smem = (size_t)rows_out * p.Wo * ctile;
  dim3 grid((unsigned)((p.Ho + rows_out - 1) / rows_out), (unsigned)((p.C + ctile - 1) / ctile), (unsigned)p.B);
  switch (p.epi.mode) {
    case EPI_NONE: return launch_mode<EPI_NONE>(c, g, grid, smem);
    case EPI_MULT: return launch_mode<EPI_MULT>(c, g, grid, smem);
    case EPI_BN32: return launch_mode<EPI_BN32>(c, g, grid, smem);
    default:       return launch_mode<EPI_BN64>(c, g, grid, smem);
  }
}

}  // namespace pulpnn
