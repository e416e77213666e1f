// depthwise_hwc3x3_tma.cu -- 3x3 depthwise convolution on HWC input (padding 1, stride 1 or 2) for
// channel counts that are a multiple of 32, with input and output staged through shared memory by
// TMA. Arithmetic is that of depthwise.cu (32bit/src/pulp_nn_depthwise_generic.c:133-180) and the
// register scheme is that of depthwise_hwc3x3.cu: a thread owns four channels and four adjacent
// output columns, transposes four pixel words into four channel words with byte permutes, and
// pays one dp4a per output and filter row.
//
// What this file changes is everything around that arithmetic. A CTA owns a tile of CI = 128, 64 or
// 32 channel bytes x 4*NGX output columns and slides down the image. A ring of three groups of
// input rows is kept full by 4-D TMA loads (tensor [B][H][W][C]); rows and columns outside the
// image arrive as zeros from the TMA unit, which IS the zero padding, so the inner loop has no
// boundary test at all. Results go to a double-buffered tile in shared memory and leave with one
// TMA store per group of rows, which also clips columns and rows past the output's edge. With
// CI = 128 one warp = the 32 channel words of one pixel, so every shared-memory access is a
// conflict-free 128-byte row; narrower chunks put several column groups in a warp (see Rot below).
// With the tile width a template parameter every address in the row loop is "one register +
// constant".
//
// Synchronisation per group of rows: one mbarrier wait (data landed), one __syncthreads (all
// threads finished reading the group and writing the output tile), after which thread 0 issues the
// store of the tile and the load that refills the group. Every wait is bounded. When there are more
// whole-image columns than CTAs fit on the GPU at once, a CTA works through several consecutive
// images and its ring of row groups runs on from one image to the next.
//
// The second kernel of this file, depthwise_chw3x3_tma_kernel, does the same for the reference's own
// CHW input layout (see the comment above it): same accumulate / requantise code, different feeding.
#include <type_traits>

#include "internal.cuh"
#include "sm100_primitives.cuh"
#include "depthwise_regs.cuh"

namespace pulpnn {

namespace {

using namespace sm100;
using namespace dwregs;

// CI (template parameter below) = channel bytes per tile: 128, 64 or 32. A warp covers 128/CI
// column groups of CI/4 channel words each.
constexpr int RING = 3;                      // groups of input rows in flight
constexpr int ST_HWC_TMA = 0x400;

// geometry of a tile, all compile-time
template <int S, int NGX, int CI> struct Geo {
  static constexpr int LPC = CI / 4;                          // lanes (channel words) per pixel
  static constexpr int NSUB = 32 / LPC;                       // column groups per warp
  static constexpr int WT = 4 * NGX;                         // output columns per tile
  static constexpr int WBOX = S == 1 ? WT + 2 : 2 * WT + 1;   // input columns per tile (with halo)
  static constexpr int ROWS_IN = S == 1 ? 3 : 4;              // input rows per group
  static constexpr int ROWS_OUT = S == 1 ? 3 : 2;             // output rows a group completes
  static constexpr int IN_PITCH = WBOX * CI;                  // bytes per staged input row
  static constexpr int OUT_PITCH = WT * CI;                   // bytes per staged output row
  static constexpr int GROUP_BYTES = ROWS_IN * IN_PITCH;      // bytes one TMA load brings
  static constexpr int TILE_BYTES = ROWS_OUT * OUT_PITCH;
  static constexpr int GROUP_STRIDE = (GROUP_BYTES + 127) / 128 * 128;   // TMA wants 128-byte aligned boxes
  static constexpr int TILE_STRIDE = (TILE_BYTES + 127) / 128 * 128;
  static constexpr int THREADS = 32 * NGX / NSUB;
  static constexpr int SMEM = 128 + RING * GROUP_STRIDE + 2 * TILE_STRIDE + 64;
  static_assert(NGX % NSUB == 0, "a warp's column groups must all belong to the tile");
};

struct HwcTmaParams {
  DepthwiseProblem p;
  int col_tiles, chunks, strips;   // tiles across the width, 128-channel chunks, strips down the height
  int rows_per_strip;              // output rows per strip (a multiple of the rows a group completes)
  int imgs_per_cta;                // consecutive images one CTA works through (its ring never drains between them)
  int *status;
};

// requantise a completed 4 columns x 4 channels block and put the four pixel words in the tile
template <int MODE, bool K32, int CI>
__device__ __forceinline__ void finalize_k(const int (&acc)[4][4], const QuantT<MODE> &q, const Epilogue &e, uint32_t oaddr)
{
#pragma unroll
  for (int i = 0; i < 4; i++) {
    int v[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      if (MODE == EPI_BN32)
        v[j] = (int)((unsigned)q.k[j] * (unsigned)acc[i][j] + (unsigned)q.l[j]) >> e.shift;
      else if (MODE == EPI_BN64 && K32)      // every k fits in 32 bits: one wide multiply-add
        v[j] = (int)(mad_wide_s32((int)q.k[j], acc[i][j], (long long)q.l[j]) >> e.shift);
      else if (MODE == EPI_BN64)
        v[j] = (int)((long long)((unsigned long long)q.k[j] * (unsigned long long)(long long)acc[i][j] +
                                 (unsigned long long)q.l[j]) >> e.shift);
      else if (MODE == EPI_MULT)
        v[j] = (int)(short)((int)((unsigned)e.out_mult * (unsigned)acc[i][j]) >> e.shift);
      else
        v[j] = acc[i][j] >> e.shift;
    }
    sts32(oaddr + i * CI, pack4_sat_u8(v[0], v[1], v[2], v[3]));
  }
}
template <int MODE, int CI>
__device__ __forceinline__ void finalize_row(const int (&acc)[4][4], const QuantT<MODE> &q, const Epilogue &e,
                                             bool k32, uint32_t oaddr)
{
  if (MODE == EPI_BN64 && k32) finalize_k<MODE, true, CI>(acc, q, e, oaddr);
  else finalize_k<MODE, false, CI>(acc, q, e, oaddr);
}

template <int MODE, int S, int NGX, int CI>
// (Capping the stride-1 kernel at 96 registers, which fits without spilling and lets a third CTA of
// 224 threads onto an SM, was measured: 10-15 % slower on every stride-1 layer.)
__global__ void __launch_bounds__(Geo<S, NGX, CI>::THREADS, 512 / Geo<S, NGX, CI>::THREADS)
depthwise_hwc3x3_tma_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_out,
                            const HwcTmaParams g)
{
  using G = Geo<S, NGX, CI>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t pad = (128u - (smem_u32(smem_raw) & 127u)) & 127u;
  uint8_t *sm = smem_raw + pad;
  const uint32_t ring = smem_u32(sm), tiles = ring + RING * G::GROUP_STRIDE;
  uint64_t *full = reinterpret_cast<uint64_t *>(sm + RING * G::GROUP_STRIDE + 2 * G::TILE_STRIDE);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(full + RING);

  const DepthwiseProblem &p = g.p;
  const Epilogue &e = p.epi;
  // a warp = NSUB column groups x LPC channel words; with CI = 128 that is one column group
  const int tid = threadIdx.x, lane = tid & 31;
  const int c4 = lane % G::LPC, sub = lane / G::LPC, gx = (tid >> 5) * G::NSUB + sub;

  // which tile: column tile fastest, then strip, then channel chunk, then image
  int t = blockIdx.x;
  const int col_tile = t % g.col_tiles; t /= g.col_tiles;
  const int strip = t % g.strips; t /= g.strips;
  const int chunk = t % g.chunks;
  const int b0 = (t / g.chunks) * g.imgs_per_cta;                        // the CTA's first image
  const int nimg = min(g.imgs_per_cta, p.B - b0);
  const int c_base = chunk * CI, ox_base = col_tile * G::WT;
  const int oyA = strip * g.rows_per_strip, oyB = min(oyA + g.rows_per_strip, p.Ho);
  const int ngroups = 1 + (oyB - oyA + G::ROWS_OUT - 1) / G::ROWS_OUT;    // group 0 only opens accumulators
  const int total = nimg * ngroups;                                      // groups of rows over all its images
  const int in_x = S * ox_base - 1;                                      // first staged input column
  const int in_y0 = S == 1 ? oyA - 2 : 2 * oyA - 4;                      // first staged row of group 0

  // thread 0: the groups are numbered through the CTA's images; group n uses slot n % RING
  int issued = 0, next_img = 0, next_j = 0;
  auto issue_next = [&]() {
    const int slot = issued % RING;
    mbar_arrive_expect_tx(&full[slot], (uint32_t)G::GROUP_BYTES);
    tma_load_4d(sm + slot * G::GROUP_STRIDE, &map_in, &full[slot], c_base, in_x, in_y0 + next_j * G::ROWS_IN, b0 + next_img);
    issued++;
    if (++next_j == ngroups) { next_j = 0; next_img++; }
  };
  if (tid == 0) {
    for (int s = 0; s < RING; s++) mbar_init(&full[s], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }

  // the thread's four channels: weights as [w0,w1,w2,0] and [0,w0,w1,w2] per filter row, and the
  // requantisation parameters (fetched while the first loads are in flight)
  const int c = c_base + 4 * c4;
  int wa[3][4], wb[3][4];
  {
    unsigned W[9];
    const unsigned *wp = reinterpret_cast<const unsigned *>(p.w + (size_t)c * 9);
#pragma unroll
    for (int i = 0; i < 9; i++) W[i] = __ldg(wp + i);
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
      for (int fy = 0; fy < 3; fy++) {
        wa[fy][j] = taps3(W, j * 9 + fy * 3);
        wb[fy][j] = (int)((unsigned)wa[fy][j] << 8);
      }
  }
  QuantT<MODE> q;
  int init[4];
  bool k32 = true;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    q.bias[j] = e.bias ? (int)__ldg(reinterpret_cast<const int8_t *>(e.bias) + c + j) : 0;
    q.k[j] = 0; q.l[j] = 0;
    init[j] = (MODE == EPI_BN32 || MODE == EPI_BN64) ? 0 : q.bias[j];
    if (MODE == EPI_BN32) {
      const int k = __ldg(reinterpret_cast<const int *>(e.k) + c + j);
      q.k[j] = k;   // the bias moves into lambda: k*(acc+bias)+l == k*acc + (k*bias+l) in wrap-around arithmetic
      q.l[j] = (int)((unsigned)k * (unsigned)q.bias[j] + (unsigned)__ldg(reinterpret_cast<const int *>(e.lambda) + c + j));
    } else if (MODE == EPI_BN64) {
      const long long k = __ldg(reinterpret_cast<const long long *>(e.k) + c + j);
      q.k[j] = k;
      q.l[j] = (long long)((unsigned long long)k * (unsigned long long)(long long)q.bias[j] +
                           (unsigned long long)__ldg(reinterpret_cast<const long long *>(e.lambda) + c + j));
      k32 = k32 && (k == (long long)(int)k);
    }
  }
  // The filter taps and requantisation parameters above are constants, fetched while the previous
  // kernel may still be running; its output is touched only from here on.
  pdl_wait();
  if (tid == 0) {
    pdl_launch_dependents();
    const int first = total < RING ? total : RING;
    for (int j = 0; j < first; j++) issue_next();
  }
  __syncthreads();                                   // the barriers are initialised

  const uint32_t in_thr = ring + (uint32_t)(4 * S * gx) * CI + 4u * c4;       // thread's first staged pixel
  const uint32_t out_thr = tiles + (uint32_t)(4 * gx) * CI + 4u * c4;
  // Pixels are CI bytes apart, so the column groups of a warp (4 or 4*S pixels apart) would meet in
  // the same shared-memory banks. Each reads its four middle pixels in an order rotated by its
  // index inside the warp instead: one load instruction then touches NSUB different pixels mod 4.
  const Rot rot = make_rot<CI>(sub);
  bool dead = false;             // a wait ran out: keep pace at the barriers, do no more work
  int consumed = 0;              // groups whose data this thread has seen land

  // Accumulators. Stride 1: three sets, one per output row in flight (an input row is filter row 2
  // of one, row 1 of the next and row 0 of the one after). Stride 2: one set.
  int acc[S == 1 ? 3 : 1][4][4];
#pragma unroll
  for (int a = 0; a < (S == 1 ? 3 : 1); a++)
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) acc[a][i][j] = 0;

  int grp = 0, half = 0, j = 0, img = 0;
  uint32_t parity = 0;
  for (int n = 0; n < total; n++) {
    if (!dead && !mbar_wait(&full[grp], parity, abort_flag, g.status, ST_HWC_TMA)) dead = true;
    if (!dead) {
      consumed = n + 1;
      const uint32_t ia = in_thr + grp * G::GROUP_STRIDE, oa = out_thr + half * G::TILE_STRIDE;
      uint32_t ra[4];
#pragma unroll
      for (int i = 0; i < 4; i++) ra[i] = ia + CI + rot.off[i];
      if (j == 0) {
        // ---- an image's group 0: the rows above the strip's first output row only open accumulators
        if constexpr (S == 1) {
          unsigned cur[6]; Win1 w;
          load_row1<CI>(ia, ra, 1 * G::IN_PITCH, cur);          // input row oyA-1
          windows1(cur, rot, w);
          load_row1<CI>(ia, ra, 2 * G::IN_PITCH, cur);          // input row oyA
          mac1<false, false>(w, wa, wb, init, acc[0], acc[0], acc[0]);
          windows1(cur, rot, w);
          mac1<false, true>(w, wa, wb, init, acc[0], acc[0], acc[S == 1 ? 1 : 0]);
        } else {
          unsigned cur[9]; Win2 w;
          load_row2<CI>(ia, ra, 3 * G::IN_PITCH, cur);          // input row 2*oyA-1
          windows2(cur, rot, w);
          mac2<true>(w, wa[0], wb[0], init, acc[0]);
        }
      } else {
        const int rows_here = oyB - (oyA + (j - 1) * G::ROWS_OUT);     // output rows this group still owes
        if constexpr (S == 1) {
          constexpr int A1 = S == 1 ? 1 : 0, A2 = S == 1 ? 2 : 0;
          unsigned cur[6]; Win1 w;
          load_row1<CI>(ia, ra, 0, cur);
          windows1(cur, rot, w);
          if (rows_here > 1) load_row1<CI>(ia, ra, G::IN_PITCH, cur);
          mac1<true, true>(w, wa, wb, init, acc[0], acc[A1], acc[A2]);
          finalize_row<MODE, CI>(acc[0], q, e, k32, oa);
          if (rows_here > 1) {            // the strip's last group may end before its third row
            windows1(cur, rot, w);
            if (rows_here > 2) load_row1<CI>(ia, ra, 2 * G::IN_PITCH, cur);
            mac1<true, true>(w, wa, wb, init, acc[A1], acc[A2], acc[0]);
            finalize_row<MODE, CI>(acc[A1], q, e, k32, oa + G::OUT_PITCH);
            if (rows_here > 2) {
              windows1(cur, rot, w);
              mac1<true, true>(w, wa, wb, init, acc[A2], acc[0], acc[A1]);
              finalize_row<MODE, CI>(acc[A2], q, e, k32, oa + 2 * G::OUT_PITCH);
            }
          }
        } else {
          unsigned cur[9]; Win2 w;
          load_row2<CI>(ia, ra, 0, cur);                          // input row 2m
          windows2(cur, rot, w);
          load_row2<CI>(ia, ra, G::IN_PITCH, cur);                // 2m+1: closes row m, opens m+1
          mac2<false>(w, wa[1], wb[1], init, acc[0]);
          windows2(cur, rot, w);
          if (rows_here > 1) load_row2<CI>(ia, ra, 2 * G::IN_PITCH, cur);
          mac2<false>(w, wa[2], wb[2], init, acc[0]);
          finalize_row<MODE, CI>(acc[0], q, e, k32, oa);
          if (rows_here > 1) {
            mac2<true>(w, wa[0], wb[0], init, acc[0]);
            windows2(cur, rot, w);
            load_row2<CI>(ia, ra, 3 * G::IN_PITCH, cur);
            mac2<false>(w, wa[1], wb[1], init, acc[0]);
            windows2(cur, rot, w);
            mac2<false>(w, wa[2], wb[2], init, acc[0]);
            finalize_row<MODE, CI>(acc[0], q, e, k32, oa + G::OUT_PITCH);
            mac2<true>(w, wa[0], wb[0], init, acc[0]);
          }
        }
        fence_proxy_async();            // the tile words written above, before the TMA store reads them
      }
    }
    // the store issued two groups ago read the half that the NEXT group will write
    if (tid == 0) bulk_wait_read_all();
    __syncthreads();                    // the group has been read, the tile written, by everyone
    if (tid == 0 && !dead) {
      if (j > 0) {
        tma_store_4d(&map_out, sm + RING * G::GROUP_STRIDE + half * G::TILE_STRIDE, c_base, ox_base,
                     oyA + (j - 1) * G::ROWS_OUT, b0 + img);
        bulk_commit();
      }
      if (issued < total) issue_next();      // group n + RING goes into the slot just read
    }
    if (j > 0) half ^= 1;
    if (++j == ngroups) { j = 0; img++; }
    if (++grp == RING) { grp = 0; parity ^= 1; }
  }
  if (tid == 0) {
    // the stores must have read the tile before the CTA's shared memory goes; their writes are
    // complete when the grid is
    bulk_wait_read_all();
    if (*abort_flag) {
      // no TMA write may still be in flight when the CTA's shared memory is released
      for (int qn = consumed; qn < issued; qn++) {
        const unsigned long long t0 = global_ns();
        while (!mbar_try_wait(&full[qn % RING], (uint32_t)(qn / RING) & 1u))
          if (global_ns() - t0 > WAIT_LIMIT_NS) break;
      }
    }
  }
}

// ---- CHW input (the reference's own layout for this kernel, pulp_nn_depthwise_generic.c:74) -------
// The same accumulate / requantise code as above, fed differently: a CTA stages 32 channels x whole
// input rows ([c][row][x], the TMA box of a [B][C][H][W] tensor), a thread owns four channels and
// four adjacent output columns as before, but here the lanes of a warp run along x, so a channel's
// four (stride 1) or eight (stride 2) input bytes ARE the channel word and no byte transpose is
// needed on the way in: two funnel shifts make the shifted windows. The output is HWC: pixel words
// go to a tile whose pixels are 36 bytes apart (so that lanes four pixels apart meet at most
// two-way in a bank), and after the group's barrier all threads copy the tile out, eight words =
// 32 channel bytes per pixel, in whole 32-byte sectors.
template <int S, int LPQ> struct GeoChw {
  static constexpr int CT = 32;                         // channels per tile
  static constexpr int WOP = 4 * LPQ;                   // output columns the lanes of a quad cover
  static constexpr int ROWS_IN = S == 1 ? 3 : 4;
  static constexpr int ROWS_OUT = S == 1 ? 3 : 2;
  static constexpr int PP = CT + 4;                     // pixel pitch of the output tile, bytes
  static constexpr int OUT_PITCH = WOP * PP;
  static constexpr int TILE_BYTES = ROWS_OUT * OUT_PITCH;
  static constexpr int THREADS = 8 * LPQ;               // eight channel quads x LPQ column groups
  static constexpr int HEADER = 128;                    // barriers and the abort flag, ahead of the ring
};

struct ChwTmaParams {
  DepthwiseProblem p;
  int chunks, strips, rows_per_strip;
  int stage_bytes;                 // ROWS_IN * W * 32
  int *status;
};

__device__ __forceinline__ void lds64(uint32_t addr, unsigned &lo, unsigned &hi)
{
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(addr));
}

// one staged row of the thread's four channels -> windows; base[j] = the channel's word at row 0
__device__ __forceinline__ void load_win_chw(const uint32_t (&base)[4], uint32_t roff, unsigned lmask, unsigned rmask, Win1 &w)
{
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const uint32_t a = base[j] + roff;
    const unsigned m = lds32(a), left = lds32(a - 4) & lmask, right = lds32(a + 4) & rmask;
    w.T[j] = m;
    w.A[j] = __funnelshift_r(left, m, 24);        // [left, p0, p1, p2]
    w.B[j] = __funnelshift_r(m, right, 8);        // [p1, p2, p3, right]
  }
}
__device__ __forceinline__ void load_win_chw(const uint32_t (&base)[4], uint32_t roff, unsigned lmask, unsigned, Win2 &w)
{
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const uint32_t a = base[j] + roff;
    unsigned m0, m1;
    lds64(a, m0, m1);
    const unsigned left = lds32(a - 4) & lmask;
    w.T[j] = m0; w.U[j] = m1;
    w.A[j] = __funnelshift_r(left, m0, 24);       // [left, p0, p1, p2]
    w.C[j] = __funnelshift_r(m0, m1, 24);         // [p3, p4, p5, p6]
  }
}

template <int MODE, int S, int LPQ>
__global__ void __launch_bounds__(GeoChw<S, LPQ>::THREADS, 512 / GeoChw<S, LPQ>::THREADS)
depthwise_chw3x3_tma_kernel(const __grid_constant__ CUtensorMap map_in, const ChwTmaParams g)
{
  using G = GeoChw<S, LPQ>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t pad = (128u - (smem_u32(smem_raw) & 127u)) & 127u;
  uint8_t *sm = smem_raw + pad;
  uint64_t *full = reinterpret_cast<uint64_t *>(sm);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(full + RING);
  uint8_t *ring_p = sm + G::HEADER;
  const uint32_t stage = (uint32_t)g.stage_bytes;
  const uint32_t ring = smem_u32(ring_p), tiles = ring + RING * stage;

  const DepthwiseProblem &p = g.p;
  const Epilogue &e = p.epi;
  const int tid = threadIdx.x, gx = tid % LPQ, qd = tid / LPQ;

  int t = blockIdx.x;
  const int strip = t % g.strips; t /= g.strips;
  const int chunk = t % g.chunks;
  const int b = t / g.chunks;
  const int c_base = chunk * G::CT;
  const int oyA = strip * g.rows_per_strip, oyB = min(oyA + g.rows_per_strip, p.Ho);
  const int ngroups = 1 + (oyB - oyA + G::ROWS_OUT - 1) / G::ROWS_OUT;
  const int in_y0 = S == 1 ? oyA - 2 : 2 * oyA - 4;

  if (tid == 0) {
    for (int s = 0; s < RING; s++) mbar_init(&full[s], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  pdl_wait();                      // up to here the kernel may overlap the previous one's tail
  if (tid == 0) {
    pdl_launch_dependents();
    const int first = ngroups < RING ? ngroups : RING;
    for (int j = 0; j < first; j++) {
      mbar_arrive_expect_tx(&full[j], stage);
      tma_load_4d(ring_p + j * stage, &map_in, &full[j], 0, in_y0 + j * G::ROWS_IN, c_base, b);
    }
  }

  // a quad past the last channel (a partial chunk) works on the last real quad; nothing of it is stored
  const int c = min(c_base + 4 * qd, p.C - 4);
  int wa[3][4], wb[3][4];
  {
    unsigned W[9];
    const unsigned *wp = reinterpret_cast<const unsigned *>(p.w + (size_t)c * 9);
#pragma unroll
    for (int i = 0; i < 9; i++) W[i] = __ldg(wp + i);
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
      for (int fy = 0; fy < 3; fy++) {
        wa[fy][j] = taps3(W, j * 9 + fy * 3);
        wb[fy][j] = (int)((unsigned)wa[fy][j] << 8);
      }
  }
  QuantT<MODE> q;
  int init[4];
  bool k32 = true;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    q.bias[j] = e.bias ? (int)__ldg(reinterpret_cast<const int8_t *>(e.bias) + c + j) : 0;
    q.k[j] = 0; q.l[j] = 0;
    init[j] = (MODE == EPI_BN32 || MODE == EPI_BN64) ? 0 : q.bias[j];
    if (MODE == EPI_BN32) {
      const int k = __ldg(reinterpret_cast<const int *>(e.k) + c + j);
      q.k[j] = k;
      q.l[j] = (int)((unsigned)k * (unsigned)q.bias[j] + (unsigned)__ldg(reinterpret_cast<const int *>(e.lambda) + c + j));
    } else if (MODE == EPI_BN64) {
      const long long k = __ldg(reinterpret_cast<const long long *>(e.k) + c + j);
      q.k[j] = k;
      q.l[j] = (long long)((unsigned long long)k * (unsigned long long)(long long)q.bias[j] +
                           (unsigned long long)__ldg(reinterpret_cast<const long long *>(e.lambda) + c + j));
      k32 = k32 && (k == (long long)(int)k);
    }
  }
  __syncthreads();                                   // the barriers are initialised

  // lanes past the last column group read column group 0 (their results are never copied out)
  const uint32_t W = (uint32_t)p.W;
  const bool col_on = 4 * gx < p.Wo;
  const uint32_t xoff = col_on ? (uint32_t)(4 * S * gx) : 0u;
  const unsigned lmask = (col_on && gx) ? 0xffffffffu : 0u;                        // column -1 is padding
  const unsigned rmask = (S == 1 && xoff + 4 < W) ? 0xffffffffu : 0u;              // so is column W
  uint32_t cb[4];
#pragma unroll
  for (int j = 0; j < 4; j++) cb[j] = ring + (uint32_t)((4 * qd + j) * G::ROWS_IN) * W + xoff;
  const uint32_t out_thr = tiles + (uint32_t)(4 * gx) * G::PP + 4u * qd;

  bool dead = false;
  int issued = ngroups < RING ? ngroups : RING;
  int consumed = 0;
  auto refill = [&](int j_next, int grp_) {          // thread 0 only
    mbar_arrive_expect_tx(&full[grp_], stage);
    tma_load_4d(ring_p + grp_ * stage, &map_in, &full[grp_], 0, in_y0 + j_next * G::ROWS_IN, c_base, b);
    issued = j_next + 1;
  };
  // all threads: the finished tile -> HWC output, one 32-bit word (four channels of a pixel) at a time
  const int cw = tid & 7, cp = tid >> 3;
  const bool cw_on = c_base + 4 * cw < p.C;
  auto copy_out = [&](int half, int oy0, int nrows) {
    for (int r = 0; r < nrows; r++) {
      uint8_t *orow = p.out + (((size_t)b * p.Ho + oy0 + r) * p.Wo) * p.C + c_base + 4 * cw;
      const uint32_t trow = tiles + half * G::TILE_BYTES + r * G::OUT_PITCH + 4u * cw;
      if (cw_on)
        for (int px = cp; px < p.Wo; px += G::THREADS / 8)
          *reinterpret_cast<unsigned *>(orow + (size_t)px * p.C) = lds32(trow + px * G::PP);
    }
  };

  int acc[S == 1 ? 3 : 1][4][4];
#pragma unroll
  for (int a = 0; a < (S == 1 ? 3 : 1); a++)
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) acc[a][i][j] = 0;

  // ---- group 0: the rows above the strip's first output row only open accumulators ---------------
  if (!mbar_wait(&full[0], 0, abort_flag, g.status, ST_HWC_TMA)) dead = true;
  if (!dead) {
    consumed = 1;
    if constexpr (S == 1) {
      Win1 w;
      load_win_chw(cb, W, lmask, rmask, w);                       // input row oyA-1
      mac1<false, false>(w, wa, wb, init, acc[0], acc[0], acc[0]);
      load_win_chw(cb, 2 * W, lmask, rmask, w);                   // input row oyA
      mac1<false, true>(w, wa, wb, init, acc[0], acc[0], acc[S == 1 ? 1 : 0]);
    } else {
      Win2 w;
      load_win_chw(cb, 3 * W, lmask, rmask, w);                   // input row 2*oyA-1
      mac2<true>(w, wa[0], wb[0], init, acc[0]);
    }
  }
  __syncthreads();
  if (tid == 0 && !dead && RING < ngroups) refill(RING, 0);

  int grp = 0, half = 0;
  uint32_t parity = 0;
  for (int j = 1; j < ngroups; j++) {
    if (++grp == RING) { grp = 0; parity ^= 1; }
    if (!dead && !mbar_wait(&full[grp], parity, abort_flag, g.status, ST_HWC_TMA)) dead = true;
    const int oy0 = oyA + (j - 1) * G::ROWS_OUT;
    const int rows_here = min(oyB - oy0, G::ROWS_OUT);
    if (!dead) {
      consumed = j + 1;
      const uint32_t oa = out_thr + half * G::TILE_BYTES;
      uint32_t ia[4];
#pragma unroll
      for (int jj = 0; jj < 4; jj++) ia[jj] = cb[jj] + grp * stage;
      if constexpr (S == 1) {
        constexpr int A1 = S == 1 ? 1 : 0, A2 = S == 1 ? 2 : 0;
        Win1 w;
        load_win_chw(ia, 0, lmask, rmask, w);
        mac1<true, true>(w, wa, wb, init, acc[0], acc[A1], acc[A2]);
        finalize_row<MODE, G::PP>(acc[0], q, e, k32, oa);
        if (rows_here > 1) {
          load_win_chw(ia, W, lmask, rmask, w);
          mac1<true, true>(w, wa, wb, init, acc[A1], acc[A2], acc[0]);
          finalize_row<MODE, G::PP>(acc[A1], q, e, k32, oa + G::OUT_PITCH);
          if (rows_here > 2) {
            load_win_chw(ia, 2 * W, lmask, rmask, w);
            mac1<true, true>(w, wa, wb, init, acc[A2], acc[0], acc[A1]);
            finalize_row<MODE, G::PP>(acc[A2], q, e, k32, oa + 2 * G::OUT_PITCH);
          }
        }
      } else {
        Win2 w, v;
        load_win_chw(ia, 0, lmask, rmask, w);                     // input row 2m
        load_win_chw(ia, W, lmask, rmask, v);                     // 2m+1: closes row m, opens m+1
        mac2<false>(w, wa[1], wb[1], init, acc[0]);
        if (rows_here > 1) load_win_chw(ia, 2 * W, lmask, rmask, w);
        mac2<false>(v, wa[2], wb[2], init, acc[0]);
        finalize_row<MODE, G::PP>(acc[0], q, e, k32, oa);
        if (rows_here > 1) {
          mac2<true>(v, wa[0], wb[0], init, acc[0]);
          load_win_chw(ia, 3 * W, lmask, rmask, v);
          mac2<false>(w, wa[1], wb[1], init, acc[0]);
          mac2<false>(v, wa[2], wb[2], init, acc[0]);
          finalize_row<MODE, G::PP>(acc[0], q, e, k32, oa + G::OUT_PITCH);
          mac2<true>(v, wa[0], wb[0], init, acc[0]);
        }
      }
    }
    __syncthreads();           // the group has been read and the tile written by everyone
    if (tid == 0 && !dead && j + RING < ngroups) refill(j + RING, grp);
    // the other half is written by the next group; this half again only after the next barrier
    if (!dead) copy_out(half, oy0, rows_here);
    half ^= 1;
  }
  if (tid == 0 && *abort_flag) {
    // no TMA write may still be in flight when the CTA's shared memory is released
    for (int qn = consumed; qn < issued; qn++) {
      const unsigned long long t0 = global_ns();
      while (!mbar_try_wait(&full[qn % RING], (uint32_t)(qn / RING) & 1u))
        if (global_ns() - t0 > WAIT_LIMIT_NS) break;
    }
  }
}

// ---- host side ----------------------------------------------------------------------------------
bool encode_4d(CUtensorMap *map, const void *base, int C, int Wd, int Hd, int B, int ci, int box_w, int box_h)
{
  cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)Wd, (cuuint64_t)Hd, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)C, (cuuint64_t)Wd * C, (cuuint64_t)Hd * Wd * C};
  cuuint32_t box[4] = {(cuuint32_t)ci, (cuuint32_t)box_w, (cuuint32_t)box_h, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = encode_tiled_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(base), dims, strides, box,
                                       estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error(PULPNN_ERR_CUDA, "cuTensorMapEncodeTiled (depthwise, %dx%dx%dx%d) failed with code %d", B, Hd, Wd, C, (int)r);
    return false;
  }
  return true;
}

// column groups per tile: the candidate that wastes the fewest columns past the right edge (the
// wider one on a tie)
int pick_ngx(int Wo, const int (&cand)[3])
{
  int best = cand[0];
  long long best_cost = -1;
  for (int i = 0; i < 3; i++) {
    const int wt = 4 * cand[i];
    const long long cost = (long long)((Wo + wt - 1) / wt) * wt;
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = cand[i]; }
  }
  return best;
}

template <int MODE, int S, int NGX, int CI>
bool launch_geo(Context &c, const DepthwiseProblem &p)
{
  using G = Geo<S, NGX, CI>;
  HwcTmaParams g;
  g.p = p;
  g.col_tiles = (p.Wo + G::WT - 1) / G::WT;
  g.chunks = p.C / CI;
  g.status = ctx_status_word(c);
  if (!g.status) return false;
  auto kern = depthwise_hwc3x3_tma_kernel<MODE, S, NGX, CI>;
  static PerDeviceInt resident_on;          // CTAs of this instantiation that fit on one SM, per device
  int resident = resident_on.get(c.device);
  if (resident == 0) {
    if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM),
                 "cudaFuncSetAttribute(depthwise_hwc3x3_tma)"))
      return false;
    int n = 0;
    if (!cuda_ok(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, G::THREADS, G::SMEM), "occupancy query")) return false;
    resident = n > 0 ? n : 1;
    resident_on.set(c.device, resident);
  }
  // Strips down the height only when whole columns leave the GPU short of CTAs (small batches): a
  // strip boundary costs one extra group of input rows.
  const long long columns = (long long)p.B * g.chunks * g.col_tiles;
  const long long want = 4LL * (c.sm_count > 0 ? c.sm_count : 148) * resident;
  int strips = 1;
  while (columns * strips < want && p.Ho / (strips * 2) >= 4 * G::ROWS_OUT) strips *= 2;
  int rows = (p.Ho + strips - 1) / strips;
  rows = (rows + G::ROWS_OUT - 1) / G::ROWS_OUT * G::ROWS_OUT;
  g.rows_per_strip = rows;
  g.strips = (p.Ho + rows - 1) / rows;
  // More whole-image columns than CTAs fit on the GPU at once: a CTA takes several consecutive
  // images, enough for one full wave, and its ring of row groups runs on from image to image.
  g.imgs_per_cta = 1;
  const long long per_image = (long long)g.chunks * g.col_tiles;
  const long long slots = (long long)(c.sm_count > 0 ? c.sm_count : 148) * resident;
  if (g.strips == 1 && columns > slots && per_image <= slots) {
    const long long bgroups_max = slots / per_image;
    long long imgs = (p.B + bgroups_max - 1) / bgroups_max;
    if (imgs > 16) imgs = 16;
    g.imgs_per_cta = (int)imgs;
  }
  const long long total = (long long)((p.B + g.imgs_per_cta - 1) / g.imgs_per_cta) * per_image * g.strips;
  if (total > 0x7fffffffLL) { set_error(PULPNN_ERR_UNSUPPORTED, "depthwise: too many tiles"); return false; }
  CUtensorMap map_in, map_out;
  if (!encode_4d(&map_in, p.in, p.C, p.W, p.H, p.B, CI, G::WBOX, G::ROWS_IN)) return false;
  if (!encode_4d(&map_out, p.out, p.C, p.Wo, p.Ho, p.B, CI, G::WT, G::ROWS_OUT)) return false;
  const cudaError_t le = launch_pdl(kern, dim3((unsigned)total), dim3(G::THREADS), G::SMEM, c.stream, map_in, map_out, g);
  count_launch("depthwise_hwc3x3_tma_kernel");
  return cuda_ok(le, "depthwise_hwc3x3_tma launch") && cuda_ok(cudaGetLastError(), "depthwise_hwc3x3_tma launch");
}

// tile widths on offer: 28, 16 or 8 columns per column group of a warp's first lane ... in column
// groups: 7, 4 or 2 warps' worth when a warp is one group (CI = 128); wider when a warp holds more
template <int MODE, int S, int CI>
bool launch_ngx(Context &c, const DepthwiseProblem &p)
{
  constexpr int NSUB = 128 / CI;
  constexpr int N0 = 7 * NSUB, N1 = NSUB == 4 ? 8 : 4, N2 = NSUB == 4 ? 4 : 2;
  const int cand[3] = {N0, N1, N2};
  const int ngx = pick_ngx(p.Wo, cand);
  if (ngx == N0) return launch_geo<MODE, S, N0, CI>(c, p);
  if (ngx == N1) return launch_geo<MODE, S, N1, CI>(c, p);
  return launch_geo<MODE, S, N2, CI>(c, p);
}

template <int MODE, int S>
bool launch_ci(Context &c, const DepthwiseProblem &p)
{
  if (p.C % 128 == 0) return launch_ngx<MODE, S, 128>(c, p);
  if (p.C % 64 == 0) return launch_ngx<MODE, S, 64>(c, p);
  return launch_ngx<MODE, S, 32>(c, p);
}

template <int MODE>
bool launch_stride(Context &c, const DepthwiseProblem &p)
{
  return p.sx == 1 ? launch_ci<MODE, 1>(c, p) : launch_ci<MODE, 2>(c, p);
}

// ---- CHW input ------------------------------------------------------------------------------------
template <int MODE, int S, int LPQ>
bool launch_chw_geo(Context &c, const DepthwiseProblem &p)
{
  using G = GeoChw<S, LPQ>;
  ChwTmaParams g;
  g.p = p;
  g.chunks = (p.C + G::CT - 1) / G::CT;
  g.stage_bytes = G::ROWS_IN * p.W * G::CT;
  g.status = ctx_status_word(c);
  if (!g.status) return false;
  const int smem = 128 + G::HEADER + RING * g.stage_bytes + 2 * G::TILE_BYTES;
  auto kern = depthwise_chw3x3_tma_kernel<MODE, S, LPQ>;
  static PerDeviceInt smem_set;             // largest dynamic shared memory asked for so far, per device
  if (smem > smem_set.get(c.device)) {
    if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                 "cudaFuncSetAttribute(depthwise_chw3x3_tma)"))
      return false;
    smem_set.set(c.device, smem);
  }
  int resident = 0;
  if (!cuda_ok(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, G::THREADS, smem), "occupancy query")) return false;
  if (resident < 1) resident = 1;
  const long long columns = (long long)p.B * g.chunks;
  const long long want = 4LL * (c.sm_count > 0 ? c.sm_count : 148) * resident;
  int strips = 1;
  while (columns * strips < want && p.Ho / (strips * 2) >= 4 * G::ROWS_OUT) strips *= 2;
  int rows = (p.Ho + strips - 1) / strips;
  rows = (rows + G::ROWS_OUT - 1) / G::ROWS_OUT * G::ROWS_OUT;
  g.rows_per_strip = rows;
  g.strips = (p.Ho + rows - 1) / rows;
  const long long total = columns * g.strips;
  if (total > 0x7fffffffLL) { set_error(PULPNN_ERR_UNSUPPORTED, "depthwise: too many tiles"); return false; }
  // [B][C][H][W]: whole rows of 32 channels per box
  CUtensorMap map_in;
  if (!encode_4d(&map_in, p.in, p.W, p.H, p.C, p.B, p.W, G::ROWS_IN, G::CT)) return false;
  const cudaError_t le = launch_pdl(kern, dim3((unsigned)total), dim3(G::THREADS), (size_t)smem, c.stream, map_in, g);
  count_launch("depthwise_chw3x3_tma_kernel");
  return cuda_ok(le, "depthwise_chw3x3_tma launch") && cuda_ok(cudaGetLastError(), "depthwise_chw3x3_tma launch");
}

template <int MODE>
bool launch_chw_stride(Context &c, const DepthwiseProblem &p)
{
  const bool wide = p.Wo > 64;
  if (p.sx == 1) return wide ? launch_chw_geo<MODE, 1, 32>(c, p) : launch_chw_geo<MODE, 1, 16>(c, p);
  return wide ? launch_chw_geo<MODE, 2, 32>(c, p) : launch_chw_geo<MODE, 2, 16>(c, p);
}

}  // namespace

bool depthwise_chw3x3_tma_supported(const DepthwiseProblem &p)
{
  if (p.in_is_hwc || p.ky != 3 || p.kx != 3 || p.pt != 1 || p.pl != 1) return false;
  if (p.sx != p.sy || (p.sx != 1 && p.sx != 2)) return false;
  // whole rows are TMA boxes: 16-byte multiples, at most 256 bytes; the lanes of a quad span a row
  if (p.W % 16 != 0 || p.W > 256 || p.C % 4 != 0) return false;
  if (p.Wo <= 16 || p.Wo > 128) return false;
  if ((reinterpret_cast<uintptr_t>(p.in) & 15) || (reinterpret_cast<uintptr_t>(p.out) & 3)) return false;
  if (reinterpret_cast<uintptr_t>(p.w) & 3) return false;
  return encode_tiled_fn() != nullptr;
}

bool launch_depthwise_chw3x3_tma(Context &c, const DepthwiseProblem &p)
{
  switch (p.epi.mode) {
    case EPI_NONE: return launch_chw_stride<EPI_NONE>(c, p);
    case EPI_MULT: return launch_chw_stride<EPI_MULT>(c, p);
    case EPI_BN32: return launch_chw_stride<EPI_BN32>(c, p);
    default:       return launch_chw_stride<EPI_BN64>(c, p);
  }
}

bool depthwise_hwc3x3_tma_supported(const DepthwiseProblem &p)
{
  if (!p.in_is_hwc || p.ky != 3 || p.kx != 3 || p.pt != 1 || p.pl != 1) return false;
  if (p.sx != p.sy || (p.sx != 1 && p.sx != 2)) return false;
  if (p.C % 32 != 0) return false;
  // TMA wants 16-byte aligned tensors; the weights are read as 32-bit words
  if ((reinterpret_cast<uintptr_t>(p.in) & 15) || (reinterpret_cast<uintptr_t>(p.out) & 15)) return false;
  if (reinterpret_cast<uintptr_t>(p.w) & 3) return false;
  if ((long long)p.H * p.W * p.C > 0x7fffffffffLL) return false;
  return encode_tiled_fn() != nullptr;
}

bool launch_depthwise_hwc3x3_tma(Context &c, const DepthwiseProblem &p)
{
  switch (p.epi.mode) {
    case EPI_NONE: return launch_stride<EPI_NONE>(c, p);
    case EPI_MULT: return launch_stride<EPI_MULT>(c, p);
    case EPI_BN32: return launch_stride<EPI_BN32>(c, p);
    default:       return launch_stride<EPI_BN64>(c, p);
  }
}

}  // namespace pulpnn
