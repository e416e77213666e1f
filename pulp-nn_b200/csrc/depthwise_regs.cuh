// depthwise_regs.cuh -- the register scheme of the 3x3 depthwise kernels on HWC data staged in shared
// memory: a thread owns four channels (one 32-bit word of a pixel) and four adjacent output columns,
// turns four pixel words into four channel words with byte permutes, and pays one dp4a per output
// and filter row (arithmetic of 32bit/src/pulp_nn_depthwise_generic.c:133-180). Shared by the
// stand-alone depthwise kernel and the fused depthwise + pointwise kernel.
#pragma once

#include <type_traits>

#include "internal.cuh"

namespace pulpnn {
namespace dwregs {

__device__ __forceinline__ unsigned prmt(unsigned a, unsigned b, unsigned sel)
{
  unsigned d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
__device__ __forceinline__ unsigned lds32(uint32_t addr)
{
  unsigned v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts32(uint32_t addr, unsigned v)
{
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// Four pixel words (byte j = channel j) -> four channel words (byte i = pixel i). The registers hold
// the pixels rotated by the lane's rotation r (register i = pixel (i + r) & 3, see the kernel); the
// second level of permutes undoes the rotation through its selectors, so it costs nothing.
struct Rot { unsigned off[4]; unsigned sel_lo, sel_hi; };

template <int CI>
__device__ __forceinline__ Rot make_rot(int r)
{
  Rot rot;
  unsigned sel = 0;
#pragma unroll
  for (int m = 0; m < 4; m++) {
    const unsigned i = (unsigned)(m - r) & 3u;     // the register that holds pixel m
    sel |= ((i & 1u) | ((i & 2u) << 1)) << (4 * m);   // its channel-0 byte after level one: 0, 1, 4, 5
  }
  rot.sel_lo = sel;
  rot.sel_hi = sel + 0x2222u;
#pragma unroll
  for (int i = 0; i < 4; i++) rot.off[i] = (unsigned)(((i + r) & 3) * CI);
  return rot;
}
__device__ __forceinline__ void transpose4(const unsigned m0, const unsigned m1, const unsigned m2,
                                           const unsigned m3, const Rot &rot, unsigned (&t)[4])
{
  const unsigned a = prmt(m0, m1, 0x5140), b = prmt(m0, m1, 0x7362);
  const unsigned c = prmt(m2, m3, 0x5140), d = prmt(m2, m3, 0x7362);
  t[0] = prmt(a, c, rot.sel_lo); t[1] = prmt(a, c, rot.sel_hi);
  t[2] = prmt(b, d, rot.sel_lo); t[3] = prmt(b, d, rot.sel_hi);
}

// a 32 x 32 -> 64-bit multiply-add in one instruction
__device__ __forceinline__ long long mad_wide_s32(int a, int b, long long c)
{
  long long d;
  asm("mad.wide.s32 %0, %1, %2, %3;" : "=l"(d) : "r"(a), "r"(b), "l"(c));
  return d;
}

template <int MODE> struct QuantT {
  typename std::conditional<MODE == EPI_BN64, long long, int>::type k[4], l[4];
  int bias[4];     // accumulators start from it in the modes without batch normalisation
};

// ---- stride 1: six pixels per staged row feed four outputs ---------------------------------------
struct Win1 { unsigned T[4], A[4], B[4]; };

// addr = the thread's first staged pixel of the row (the left neighbour of its four columns);
// ra[i] = address of the i-th of the four middle pixels in the lane's rotated order
template <int CI>
__device__ __forceinline__ void load_row1(uint32_t addr, const uint32_t (&ra)[4], int row_off, unsigned (&cur)[6])
{
  cur[0] = lds32(addr + row_off);
#pragma unroll
  for (int i = 0; i < 4; i++) cur[1 + i] = lds32(ra[i] + row_off);
  cur[5] = lds32(addr + row_off + 5 * CI);
}
__device__ __forceinline__ void windows1(const unsigned (&cur)[6], const Rot &rot, Win1 &w)
{
  transpose4(cur[1], cur[2], cur[3], cur[4], rot, w.T);
#pragma unroll
  for (int j = 0; j < 4; j++) {
    w.A[j] = prmt(w.T[j], cur[0], 0x2104u + j);                   // [left, p0, p1, p2]
    w.B[j] = prmt(w.T[j], cur[5], 0x0321u | ((4u + j) << 12));     // [p1, p2, p3, right]
  }
}
// one staged row: filter row 2 of X (which it completes), row 1 of Y, row 0 of Z (which it opens)
template <bool DOX, bool DOY, bool DOZ = true>
__device__ __forceinline__ void mac1(const Win1 &w, const int (&wa)[3][4], const int (&wb)[3][4], const int (&init)[4],
                                     int (&X)[4][4], int (&Y)[4][4], int (&Z)[4][4])
{
#pragma unroll
  for (int j = 0; j < 4; j++) {
    if (DOX) {
      X[0][j] = dp4a_us(w.A[j], wa[2][j], X[0][j]);  X[1][j] = dp4a_us(w.T[j], wa[2][j], X[1][j]);
      X[2][j] = dp4a_us(w.T[j], wb[2][j], X[2][j]);  X[3][j] = dp4a_us(w.B[j], wb[2][j], X[3][j]);
    }
    if (DOY) {
      Y[0][j] = dp4a_us(w.A[j], wa[1][j], Y[0][j]);  Y[1][j] = dp4a_us(w.T[j], wa[1][j], Y[1][j]);
      Y[2][j] = dp4a_us(w.T[j], wb[1][j], Y[2][j]);  Y[3][j] = dp4a_us(w.B[j], wb[1][j], Y[3][j]);
    }
    if (DOZ) {
      Z[0][j] = dp4a_us(w.A[j], wa[0][j], init[j]);    Z[1][j] = dp4a_us(w.T[j], wa[0][j], init[j]);
      Z[2][j] = dp4a_us(w.T[j], wb[0][j], init[j]);    Z[3][j] = dp4a_us(w.B[j], wb[0][j], init[j]);
    }
  }
}

// ---- stride 2: nine pixels per staged row feed four outputs --------------------------------------
struct Win2 { unsigned T[4], U[4], A[4], C[4]; };

template <int CI>
__device__ __forceinline__ void load_row2(uint32_t addr, const uint32_t (&ra)[4], int row_off, unsigned (&cur)[9])
{
  cur[0] = lds32(addr + row_off);
#pragma unroll
  for (int i = 0; i < 4; i++) cur[1 + i] = lds32(ra[i] + row_off);
#pragma unroll
  for (int i = 0; i < 4; i++) cur[5 + i] = lds32(ra[i] + row_off + 4 * CI);
}
__device__ __forceinline__ void windows2(const unsigned (&cur)[9], const Rot &rot, Win2 &w)
{
  transpose4(cur[1], cur[2], cur[3], cur[4], rot, w.T);
  transpose4(cur[5], cur[6], cur[7], cur[8], rot, w.U);
#pragma unroll
  for (int j = 0; j < 4; j++) {
    w.A[j] = prmt(w.T[j], cur[0], 0x2104u + j);     // [left, p0, p1, p2]
    w.C[j] = prmt(w.T[j], w.U[j], 0x6543u);         // [p3, p4, p5, p6]
  }
}
template <bool OPEN>
__device__ __forceinline__ void mac2(const Win2 &w, const int (&wa)[4], const int (&wb)[4], const int (&init)[4],
                                     int (&acc)[4][4])
{
#pragma unroll
  for (int j = 0; j < 4; j++) {
    acc[0][j] = dp4a_us(w.A[j], wa[j], OPEN ? init[j] : acc[0][j]);
    acc[1][j] = dp4a_us(w.T[j], wb[j], OPEN ? init[j] : acc[1][j]);
    acc[2][j] = dp4a_us(w.C[j], wa[j], OPEN ? init[j] : acc[2][j]);
    acc[3][j] = dp4a_us(w.U[j], wb[j], OPEN ? init[j] : acc[3][j]);
  }
}

// three bytes of a packed weight array starting at byte n, as [b0, b1, b2, 0]
__device__ __forceinline__ int taps3(const unsigned (&W)[9], int n)
{
  const int wi = n >> 2, off = n & 3;
  const unsigned lo = W[wi], hi = wi + 1 < 9 ? W[wi + 1] : 0u;
  return (int)(__funnelshift_r(lo, hi, 8 * off) & 0x00ffffffu);
}

}  // namespace dwregs
}  // namespace pulpnn
