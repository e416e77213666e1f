// depthwise_hwc3x3.cu -- 3x3 depthwise convolution on HWC input, padding 1, stride 1 or 2: the
// shape every depthwise layer of a MobileNet has. Same arithmetic as depthwise.cu
// (32bit/src/pulp_nn_depthwise_generic.c:133-180); this file only changes how the work is laid
// out so that the kernel is limited by memory traffic rather than by instruction issue.
//
// A thread owns four adjacent channels (one 32-bit word of an HWC pixel) and four adjacent output
// columns, and walks down a strip of output rows. Per input row it loads the 6 (stride 1) or 9
// (stride 2) pixels its four outputs touch and transposes each group of four pixel words with
// byte permutes, so that one register holds FOUR HORIZONTALLY ADJACENT PIXELS OF ONE CHANNEL; the
// loads of the following row are issued right after the transposes, into the same registers, and
// fly while the current row is being used. A filter row then costs one dp4a per output: the
// three taps sit in three of the four byte lanes, the fourth lane's weight is zero ([w0,w1,w2,0]
// for a window starting at the left tap, [0,w0,w1,w2] for one starting a pixel earlier). Rows are
// shared vertically: each input row is fetched and transposed once and feeds the three (stride 1)
// or two (stride 2) output rows it belongs to. Pixels outside the image are zero words, which is
// the zero padding.
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

// four pixel words (byte j = channel j) -> four channel words (byte i = pixel i)
__device__ __forceinline__ void transpose4(const unsigned m0, const unsigned m1, const unsigned m2,
                                           const unsigned m3, unsigned (&t)[4])
{
  const unsigned a = prmt(m0, m1, 0x5140), b = prmt(m0, m1, 0x7362);
  const unsigned c = prmt(m2, m3, 0x5140), d = prmt(m2, m3, 0x7362);
  t[0] = prmt(a, c, 0x5410); t[1] = prmt(a, c, 0x7632);
  t[2] = prmt(b, d, 0x5410); t[3] = prmt(b, d, 0x7632);
}

struct Hwc3x3Params {
  DepthwiseProblem p;
  int C4, ngx, nstrips, rows_per_strip;
  unsigned total;
};

// per-channel requantisation parameters of a thread's four channels; BN modes carry the bias
// inside l (k*bias + lambda, exact in wrap-around arithmetic)
template <int MODE> struct Quant {
  typename std::conditional<MODE == EPI_BN64, long long, int>::type k[4], l[4];
  int bias[4];
};

template <int MODE>
__device__ __forceinline__ void finalize_store(const int (&acc)[4][4], const Quant<MODE> &q, const Epilogue &e,
                                               uint8_t *orow, const int (&ooff)[4], unsigned omask)
{
#pragma unroll
  for (int i = 0; i < 4; i++) {
    int v[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      if (MODE == EPI_BN32)
        v[j] = (int)((unsigned)q.k[j] * (unsigned)acc[i][j] + (unsigned)q.l[j]) >> e.shift;
      else if (MODE == EPI_BN64)
        v[j] = (int)((long long)((unsigned long long)q.k[j] * (unsigned long long)(long long)acc[i][j] +
                                 (unsigned long long)q.l[j]) >> e.shift);
      else if (MODE == EPI_MULT)
        v[j] = (int)(short)((int)((unsigned)e.out_mult * (unsigned)(acc[i][j] + q.bias[j])) >> e.shift);
      else
        v[j] = (acc[i][j] + q.bias[j]) >> e.shift;
    }
    if ((omask >> i) & 1u)
      *reinterpret_cast<unsigned *>(orow + ooff[i]) = pack4_sat_u8(v[0], v[1], v[2], v[3]);
  }
}

template <int MODE, int S>
__global__ void __launch_bounds__(128) depthwise_hwc3x3_kernel(const Hwc3x3Params g)
{
  constexpr int NPX = S == 1 ? 6 : 9;        // pixels per input row touched by four outputs
  constexpr unsigned FULL = (1u << NPX) - 1u;
  const DepthwiseProblem &p = g.p;
  unsigned t = blockIdx.x * 128u + threadIdx.x;
  if (t >= g.total) return;
  const int c4 = t % g.C4; t /= g.C4;
  const int gx = t % g.ngx; t /= g.ngx;
  const int strip = t % g.nstrips;
  const int b = t / g.nstrips;
  const int c = c4 * 4, C = p.C;
  const int ox0 = gx * 4;
  const int oyA = strip * g.rows_per_strip, oyB = min(oyA + g.rows_per_strip, p.Ho);

  // weights of the four channels: wa[fy][j] = [w0,w1,w2,0], wb = [0,w0,w1,w2]
  int wa[3][4], wb[3][4];
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const int8_t *w = p.w + (size_t)(c + j) * 9;
#pragma unroll
    for (int fy = 0; fy < 3; fy++) {
      const unsigned v = (unsigned)(uint8_t)__ldg(w + fy * 3) | ((unsigned)(uint8_t)__ldg(w + fy * 3 + 1) << 8) |
                         ((unsigned)(uint8_t)__ldg(w + fy * 3 + 2) << 16);
      wa[fy][j] = (int)v;
      wb[fy][j] = (int)(v << 8);
    }
  }
  const Epilogue &e = p.epi;
  Quant<MODE> q;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    q.bias[j] = e.bias ? (int)__ldg(reinterpret_cast<const int8_t *>(e.bias) + c + j) : 0;
    q.k[j] = 0; q.l[j] = 0;
    if (MODE == EPI_BN32) {
      const int k = __ldg(reinterpret_cast<const int *>(e.k) + c + j);
      const int l = __ldg(reinterpret_cast<const int *>(e.lambda) + c + j);
      q.k[j] = k;
      q.l[j] = (int)((unsigned)k * (unsigned)q.bias[j] + (unsigned)l);
    } else if (MODE == EPI_BN64) {
      const long long k = __ldg(reinterpret_cast<const long long *>(e.k) + c + j);
      const long long l = __ldg(reinterpret_cast<const long long *>(e.lambda) + c + j);
      q.k[j] = k;
      q.l[j] = (long long)((unsigned long long)k * (unsigned long long)(long long)q.bias[j] + (unsigned long long)l);
    }
  }

  // byte offsets of the touched pixels inside an input row, and which of them exist
  const int px0 = ox0 * S - 1;
  int off[NPX];
  unsigned pxmask = 0;
#pragma unroll
  for (int i = 0; i < NPX; i++) {
    const int px = px0 + i;
    off[i] = px * C;
    if ((unsigned)px < (unsigned)p.W) pxmask |= 1u << i;
  }
  int ooff[4];
  unsigned omask = 0;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    ooff[i] = (ox0 + i) * C;
    if (ox0 + i < p.Wo) omask |= 1u << i;
  }
  const uint8_t *img = p.in + (size_t)b * p.H * p.W * C + c;
  uint8_t *oimg = p.out + (size_t)b * p.Ho * p.Wo * C + c;
  const size_t in_pitch = (size_t)p.W * C, out_pitch = (size_t)p.Wo * C;

  auto load_row = [&](int iy, unsigned (&r)[NPX]) {
    if ((unsigned)iy < (unsigned)p.H) {
      const uint8_t *row = img + (size_t)iy * in_pitch;
      if (pxmask == FULL) {
#pragma unroll
        for (int i = 0; i < NPX; i++) r[i] = __ldg(reinterpret_cast<const unsigned *>(row + off[i]));
      } else {
#pragma unroll
        for (int i = 0; i < NPX; i++)
          r[i] = ((pxmask >> i) & 1u) ? __ldg(reinterpret_cast<const unsigned *>(row + off[i])) : 0u;
      }
    } else {
#pragma unroll
      for (int i = 0; i < NPX; i++) r[i] = 0u;
    }
  };

  unsigned cur[NPX];
  if (S == 1) {
    // input row iy feeds output rows iy-1 (filter row 2), iy (row 1) and iy+1 (row 0)
    int acc[3][4][4];
#pragma unroll
    for (int a = 0; a < 3; a++)
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[a][i][j] = 0;
    const int iy_first = oyA - 1, iy_last = oyB;
    load_row(iy_first, cur);
    for (int base = iy_first; base <= iy_last; base += 3) {
#pragma unroll
      for (int ph = 0; ph < 3; ph++) {
        const int iy = base + ph;
        if (iy <= iy_last) {
          unsigned T[4], A[4], Bw[4];
          transpose4(cur[1], cur[2], cur[3], cur[4], T);
#pragma unroll
          for (int j = 0; j < 4; j++) {
            A[j] = prmt(T[j], cur[0], 0x2104u + j);                  // [hm, p0, p1, p2]
            Bw[j] = prmt(T[j], cur[5], 0x0321u | ((4u + j) << 12));   // [p1, p2, p3, hp]
          }
          load_row(iy + 1 <= iy_last ? iy + 1 : -1, cur);            // next row, in flight from here
          // roles: X = acc[ph] completes (filter row 2), Y = acc[(ph+1)%3] (row 1),
          //        Z = acc[(ph+2)%3] starts (row 0)
          int (&X)[4][4] = acc[ph % 3];
          int (&Y)[4][4] = acc[(ph + 1) % 3];
          int (&Z)[4][4] = acc[(ph + 2) % 3];
#pragma unroll
          for (int j = 0; j < 4; j++) {
            X[0][j] = dp4a_us(A[j], wa[2][j], X[0][j]);  X[1][j] = dp4a_us(T[j], wa[2][j], X[1][j]);
            X[2][j] = dp4a_us(T[j], wb[2][j], X[2][j]);  X[3][j] = dp4a_us(Bw[j], wb[2][j], X[3][j]);
            Y[0][j] = dp4a_us(A[j], wa[1][j], Y[0][j]);  Y[1][j] = dp4a_us(T[j], wa[1][j], Y[1][j]);
            Y[2][j] = dp4a_us(T[j], wb[1][j], Y[2][j]);  Y[3][j] = dp4a_us(Bw[j], wb[1][j], Y[3][j]);
            Z[0][j] = dp4a_us(A[j], wa[0][j], 0);        Z[1][j] = dp4a_us(T[j], wa[0][j], 0);
            Z[2][j] = dp4a_us(T[j], wb[0][j], 0);        Z[3][j] = dp4a_us(Bw[j], wb[0][j], 0);
          }
          const int oy = iy - 1;
          if (oy >= oyA && oy < oyB) finalize_store<MODE>(X, q, e, oimg + (size_t)oy * out_pitch, ooff, omask);
        }
      }
    }
  } else {
    // output row m takes input rows 2m-1 (filter row 0), 2m (row 1), 2m+1 (row 2); odd input rows
    // serve two output rows
    int acc[4][4];
    unsigned T[4], U[4], A[4], Cw[4];
    load_row(2 * oyA - 1, cur);
    auto windows = [&]() {
      transpose4(cur[1], cur[2], cur[3], cur[4], T);
      transpose4(cur[5], cur[6], cur[7], cur[8], U);
#pragma unroll
      for (int j = 0; j < 4; j++) {
        A[j] = prmt(T[j], cur[0], 0x2104u + j);     // [hm, p0, p1, p2]
        Cw[j] = prmt(T[j], U[j], 0x6543u);          // [p3, p4, p5, p6]
      }
    };
    windows();
    load_row(2 * oyA, cur);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      acc[0][j] = dp4a_us(A[j], wa[0][j], 0);   acc[1][j] = dp4a_us(T[j], wb[0][j], 0);
      acc[2][j] = dp4a_us(Cw[j], wa[0][j], 0);  acc[3][j] = dp4a_us(U[j], wb[0][j], 0);
    }
    for (int m = oyA; m < oyB; m++) {
      windows();                                  // even row 2m
      load_row(2 * m + 1, cur);
#pragma unroll
      for (int j = 0; j < 4; j++) {
        acc[0][j] = dp4a_us(A[j], wa[1][j], acc[0][j]);   acc[1][j] = dp4a_us(T[j], wb[1][j], acc[1][j]);
        acc[2][j] = dp4a_us(Cw[j], wa[1][j], acc[2][j]);  acc[3][j] = dp4a_us(U[j], wb[1][j], acc[3][j]);
      }
      windows();                                  // odd row 2m+1: closes row m and opens m+1
      load_row(m + 1 < oyB ? 2 * m + 2 : -1, cur);
#pragma unroll
      for (int j = 0; j < 4; j++) {
        acc[0][j] = dp4a_us(A[j], wa[2][j], acc[0][j]);   acc[1][j] = dp4a_us(T[j], wb[2][j], acc[1][j]);
        acc[2][j] = dp4a_us(Cw[j], wa[2][j], acc[2][j]);  acc[3][j] = dp4a_us(U[j], wb[2][j], acc[3][j]);
      }
      finalize_store<MODE>(acc, q, e, oimg + (size_t)m * out_pitch, ooff, omask);
#pragma unroll
      for (int j = 0; j < 4; j++) {
        acc[0][j] = dp4a_us(A[j], wa[0][j], 0);   acc[1][j] = dp4a_us(T[j], wb[0][j], 0);
        acc[2][j] = dp4a_us(Cw[j], wa[0][j], 0);  acc[3][j] = dp4a_us(U[j], wb[0][j], 0);
      }
    }
  }
}

template <int MODE, int S>
bool launch_s(Context &c, const Hwc3x3Params &g)
{
  const unsigned blocks = (g.total + 127u) / 128u;
  depthwise_hwc3x3_kernel<MODE, S><<<blocks, 128, 0, c.stream>>>(g);
  count_launch("depthwise_hwc3x3_kernel");
  return cuda_ok(cudaGetLastError(), "depthwise_hwc3x3 launch");
}

template <int MODE>
bool launch_m(Context &c, const Hwc3x3Params &g)
{
  return g.p.sx == 1 ? launch_s<MODE, 1>(c, g) : launch_s<MODE, 2>(c, g);
}

}  // namespace

bool depthwise_hwc3x3_supported(const DepthwiseProblem &p)
{
  if (!p.in_is_hwc || p.ky != 3 || p.kx != 3 || p.pt != 1 || p.pl != 1) return false;
  if (p.sx != p.sy || (p.sx != 1 && p.sx != 2)) return false;
  if (p.C % 4 != 0) return false;
  if ((reinterpret_cast<uintptr_t>(p.in) & 3) || (reinterpret_cast<uintptr_t>(p.out) & 3)) return false;
  // offsets inside a row are kept in 32-bit registers
  if ((long long)(p.W + 8) * p.C > 0x7fffffffLL) return false;
  return true;
}

bool launch_depthwise_hwc3x3(Context &c, const DepthwiseProblem &p)
{
  Hwc3x3Params g;
  g.p = p;
  g.C4 = p.C / 4;
  g.ngx = (p.Wo + 3) / 4;
  // whole columns per thread unless that leaves the GPU short of threads; a strip boundary costs
  // two extra input rows
  const long long columns = (long long)p.B * g.ngx * g.C4;
  const long long want = (long long)(c.sm_count > 0 ? c.sm_count : 148) * 2048;
  int nstrips = 1;
  while (columns * nstrips < want && p.Ho / (nstrips * 2) >= 8) nstrips *= 2;
  g.rows_per_strip = (p.Ho + nstrips - 1) / nstrips;
  g.nstrips = (p.Ho + g.rows_per_strip - 1) / g.rows_per_strip;
  const long long total = columns * g.nstrips;
  if (total > 0xfffffff0LL) { set_error(PULPNN_ERR_UNSUPPORTED, "depthwise: too many work items"); return false; }
  g.total = (unsigned)total;
  switch (p.epi.mode) {
    case EPI_NONE: return launch_m<EPI_NONE>(c, g);
    case EPI_MULT: return launch_m<EPI_MULT>(c, g);
    case EPI_BN32: return launch_m<EPI_BN32>(c, g);
    default:       return launch_m<EPI_BN64>(c, g);
  }
}

}  // namespace pulpnn
