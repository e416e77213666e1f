// dwpw_tcdw.cu -- the 32-channel 3x3 stride-1 depthwise layer and the pointwise layer behind it with BOTH
// layers on the tensor cores. Same chain and same integer results as dwpw_fused.cu
//     pulp_nn_depthwise_generic  -> Im_out  (32bit/src/pulp_nn_depthwise_generic.c:133-180)
//     pulp_nn_pointwise_HoWo_parallel <- pInBuffer (32bit/src/pulp_nn_pointwise_HoWo_parallel.c:103)
// but the depthwise sums are not made by dp4a in builder threads. With 32 channels a pixel is 32 bytes = the
// K of one tcgen05.mma kind::i8, so filter tap (dy, dx) of the depthwise layer is ONE MMA
//     D[pixel][c] += A[pixel + (dy, dx)][c'] * diag(w[dy][dx])[c'][c]            M = 128, N = 32, K = 32
// whose A operand is the input box as TMA left it in shared memory, addressed at a SHIFTED start.
//
// Layout. A box is 18 rows of 36 pixels, fetched as rows of nine 128-byte pieces (four pixels each; 32-byte
// pieces, one per pixel, keep the TMA unit busy four times as long) with the 128-byte swizzle. Seen by the
// MMA, a 128-byte piece is one ROW of a K-major operand whose K runs over four pixels: an MMA that starts j
// pixels into the row reads, as its 128 rows, the pixels 4q + j of eight pieces q of each of 16 box rows
// (eight-row groups one box row = 1 152 bytes apart). So the outputs of a patch of 16 rows x 28 pixels come as
// four "sub-columns" j = 0..3 (pixels x = 4q + j), and tap (dy, dx) of sub-column j only moves the start
// address by dy * 36 + j + dx - 1 pixels. That works because the swizzle, for TMA and for the MMA alike, is a
// function of the absolute shared-memory address.
//
// Sharing the MMAs. Such an MMA costs about 80 cycles whatever its width (it is bound by reading 32 of the 128
// bytes of each of its rows), and the same operand "pixel s of every piece, box row y + dy" is what sub-column
// s + 1 needs for tap dx = 0, sub-column s for dx = 1 and sub-column s - 1 for dx = 2. With the four
// accumulators side by side in tensor memory in the order j = 3, 2, 1, 0, ONE MMA of N = 96 against
// [diag w(dy,0); diag w(dy,1); diag w(dy,2)] feeds all three; at the ends (s = -1, 0, 3, 4) N is 32 or 64 and
// the weight rows start later. 18 MMAs make the depthwise sums of a patch of 448 pixels (the first one, N = 128
// with 32 rows of zeros in front of the weights, also clears the accumulators), against about 4 500 warp
// instructions of builder work.
//
// The depthwise side works a patch at a time, the pointwise side HALF a patch (two sub-columns, 224 pixels: a
// unit); everything changes hands through mbarriers with bounded waits. Roles of a CTA (persistent):
//   warp 0, one lane    TMA: the pointwise weights once, then one box per patch (pixels outside the image
//                       arrive as zeros: the zero padding)
//   warp 1, one lane    depthwise MMAs: 18 per patch into four 32-column accumulators
//   warp 2, one lane    pointwise MMAs: two per unit (K = 32) into two ch_out-column accumulators
//   warps 4..11         two groups of four (one warp per TMEM lane quarter) that take units in turn: tcgen05.ld
//                       of the depthwise sums (lane = row of the MMA = one pixel per sub-column),
//                       requantisation with the depthwise layer's parameters, 32 bytes per pixel stored as a
//                       row of the pointwise MMA's A operand
//   warps 12..27        four groups of four: pointwise epilogue (a group per accumulator pair and sub-column),
//                       32-byte global stores
#include <cuda.h>

#include "internal.cuh"
#include "sm100_primitives.cuh"

namespace pulpnn {

namespace {

using namespace sm100;

constexpr int ST_T_TMA = 0x1000000, ST_T_MMA = 0x2000000, ST_T_RQ = 0x4000000, ST_T_EPI = 0x8000000;

constexpr int TC = 32;                          // input channels = bytes per pixel = K of every MMA
constexpr int TTW = 28, TTH = 16;               // patch: 16 rows of 28 pixels
constexpr int BOX_PX = 36, BOX_H = TTH + 2;     // box row: pixels x0-4 .. x0+31 (nine pieces of four pixels)
constexpr int BOX_PITCH = BOX_PX * TC;          // 1 152 bytes
constexpr int BOX_BYTES = BOX_H * BOX_PITCH;    // 20 736
constexpr int BOX_STRIDE = 21 * 1024;
constexpr int NBOX = 4;                         // ring of input boxes
constexpr int NDACC = 2;                        // depthwise accumulators: per patch four sub-columns of 32 columns
constexpr int WDW_ROWS = 32 + 9 * 32;           // 32 rows of zeros, then per filter row [diag w(dy,0); diag w(dy,1); diag w(dy,2)]
constexpr int NA2 = 4;                          // ring of requantised depthwise tiles: per unit two of 128 rows x 32 bytes
constexpr int A2_BYTES = 128 * TC;
constexpr int RQ_GROUPS = 2;                    // a group per half patch
constexpr int EP_GROUPS = 4;                    // a group per (accumulator pair, sub-column of the unit)
constexpr int FIRST_RQ = 4, FIRST_EP = FIRST_RQ + 4 * RQ_GROUPS;
constexpr int TTHREADS = 32 * (FIRST_EP + 4 * EP_GROUPS);
static_assert(NA2 % RQ_GROUPS == 0 && RQ_GROUPS == 2, "a ring slot must always meet the same group; a group per half patch");

template <int N> struct TG {
  static constexpr int NPACC = (512 - NDACC * 128) / (2 * N);   // pointwise accumulators (pairs: one per unit in flight)
  static_assert(NPACC == 2 && EP_GROUPS == 2 * NPACC, "two epilogue groups per accumulator pair");
  static constexpr int WPW_OFF = 0;                             // pointwise weights [N][32], 32-byte swizzle
  static constexpr int WDW_OFF = (N * TC + 1023) / 1024 * 1024; // the depthwise taps as diagonal blocks (WDW_ROWS rows of 32 bytes)
  static constexpr int A2_OFF = WDW_OFF + WDW_ROWS * TC;
  static constexpr int BOX_OFF = A2_OFF + NA2 * 2 * A2_BYTES;
  static constexpr int PPW_OFF = BOX_OFF + NBOX * BOX_STRIDE;   // pointwise k / lambda (up to 8 bytes each) or bias
  static constexpr int PDW_OFF = PPW_OFF + N * 16;              // depthwise k / lambda or bias
  static constexpr int BAR_OFF = PDW_OFF + TC * 16;
  static constexpr int SMEM = 1024 + BAR_OFF + 1024;
};

struct TcdwParams {
  uint8_t *out;            // [B][H][W][N]
  const int8_t *w_dw;      // [32][3][3]
  Epilogue e_dw, e_pw;
  int B, H, W;
  int tiles_x, tiles_y, patches;
  int ablate;              // measurement only (PULPNN_OPT_TUNE bits 8-12): 1 no epilogue work, 2 no requantisation of the depthwise sums, 4 no depthwise MMAs, 8 no stores, 16 no requantisation in the epilogue
  int *status;
};

// K-major operand; sbo = bytes between eight-row groups; layout 6 = rows of 32 bytes with the 32-byte swizzle,
// 2 = rows of 128 bytes with the 128-byte swizzle
__device__ __forceinline__ uint64_t desc_k(uint32_t saddr, uint32_t sbo, uint64_t layout)
{
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= layout << 61;
  return d;
}
__device__ __forceinline__ uint64_t desc_k32(uint32_t saddr, uint32_t sbo) { return desc_k(saddr, sbo, 6); }

// requantise 32 accumulators of one pixel (column j = channel j) with the parameters staged at `par`
template <int MODE>
__device__ __forceinline__ void requant32(const uint32_t (&v)[32], const uint8_t *par, int nparam, const Epilogue &e,
                                          unsigned (&w)[8])
{
  const int *p_k32 = reinterpret_cast<const int *>(par), *p_l32 = p_k32 + nparam;
  const long long *p_k64 = reinterpret_cast<const long long *>(par), *p_l64 = p_k64 + nparam;
  const int *p_bias = reinterpret_cast<const int *>(par);
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    int q[4];
    if (MODE == EPI_BN32) {
      const int4 kk = *reinterpret_cast<const int4 *>(p_k32 + j);
      const int4 ll = *reinterpret_cast<const int4 *>(p_l32 + j);
      q[0] = (int)((unsigned)kk.x * v[j + 0] + (unsigned)ll.x) >> e.shift;
      q[1] = (int)((unsigned)kk.y * v[j + 1] + (unsigned)ll.y) >> e.shift;
      q[2] = (int)((unsigned)kk.z * v[j + 2] + (unsigned)ll.z) >> e.shift;
      q[3] = (int)((unsigned)kk.w * v[j + 3] + (unsigned)ll.w) >> e.shift;
    } else {
#pragma unroll
      for (int t = 0; t < 4; t++) {
        const int a = (int)v[j + t];
        if (MODE == EPI_BN64)
          q[t] = (int)((long long)((unsigned long long)p_k64[j + t] * (unsigned long long)(long long)a +
                                   (unsigned long long)p_l64[j + t]) >> e.shift);
        else if (MODE == EPI_MULT)
          q[t] = (int)(short)((int)((unsigned)e.out_mult * (unsigned)(a + p_bias[j + t])) >> e.shift);
        else
          q[t] = (a + p_bias[j + t]) >> e.shift;
      }
    }
    w[j >> 2] = pack4_sat_u8(q[0], q[1], q[2], q[3]);
  }
}

// per-channel parameters of one layer -> shared memory, the bias folded into lambda:
// k*(acc+b)+lambda == k*acc + (k*b+lambda) in wrap-around arithmetic
template <int MODE>
__device__ __forceinline__ void stage_params(uint8_t *par, const Epilogue &e, int n_ch, int tid, int nthreads)
{
  for (int n = tid; n < n_ch; n += nthreads) {
    const int bias8 = e.bias ? (int)__ldg(reinterpret_cast<const int8_t *>(e.bias) + n) : 0;
    if (MODE == EPI_BN32) {
      const int k = __ldg(reinterpret_cast<const int *>(e.k) + n);
      reinterpret_cast<int *>(par)[n] = k;
      reinterpret_cast<int *>(par)[n_ch + n] =
          (int)((unsigned)k * (unsigned)bias8 + (unsigned)__ldg(reinterpret_cast<const int *>(e.lambda) + n));
    } else if (MODE == EPI_BN64) {
      const long long k = __ldg(reinterpret_cast<const long long *>(e.k) + n);
      reinterpret_cast<long long *>(par)[n] = k;
      reinterpret_cast<long long *>(par)[n_ch + n] =
          (long long)((unsigned long long)k * (unsigned long long)(long long)bias8 +
                      (unsigned long long)__ldg(reinterpret_cast<const long long *>(e.lambda) + n));
    } else {
      reinterpret_cast<int *>(par)[n] = bias8;
    }
  }
}

template <int MODE, int N>
__global__ void __launch_bounds__(TTHREADS, 1)
dwpw_tcdw_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_w, const TcdwParams g)
{
  using G = TG<N>;
  constexpr int NPACC = G::NPACC;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t *w_pw = sm + G::WPW_OFF;
  uint8_t *w_dw = sm + G::WDW_OFF;
  uint8_t *a2_ring = sm + G::A2_OFF;
  uint8_t *box_ring = sm + G::BOX_OFF;
  uint8_t *par_pw = sm + G::PPW_OFF;
  uint8_t *par_dw = sm + G::PDW_OFF;
  uint64_t *in_full = reinterpret_cast<uint64_t *>(sm + G::BAR_OFF);
  uint64_t *in_empty = in_full + NBOX;
  uint64_t *d_full = in_empty + NBOX;
  uint64_t *d_empty = d_full + NDACC;
  uint64_t *a2_full = d_empty + NDACC;
  uint64_t *a2_empty = a2_full + NA2;
  uint64_t *p_full = a2_empty + NA2;
  uint64_t *p_empty = p_full + NPACC;
  uint64_t *w_bar = p_empty + NPACC;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(w_bar + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const Epilogue &ed = g.e_dw;
  const Epilogue &ep = g.e_pw;

  if (tid == 0) {
    for (int s = 0; s < NBOX; s++) { mbar_init(&in_full[s], 1); mbar_init(&in_empty[s], 1); }
    for (int s = 0; s < NDACC; s++) { mbar_init(&d_full[s], 1); mbar_init(&d_empty[s], 4 * RQ_GROUPS); }
    for (int s = 0; s < NA2; s++) { mbar_init(&a2_full[s], 4); mbar_init(&a2_empty[s], 1); }
    for (int s = 0; s < NPACC; s++) { mbar_init(&p_full[s], 1); mbar_init(&p_empty[s], 8); }
    mbar_init(w_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    // weights and per-channel parameters are constants of the layer: fetched before the wait on the previous kernel
    mbar_arrive_expect_tx(w_bar, (uint32_t)(N * TC));
    tma_load_2d(w_pw, &map_w, w_bar, 0, 0);
  }
  if (warp == 3) tmem_alloc(tmem_slot, 512);
  // the depthwise taps as diagonal 32 x 32 blocks (row = output channel, 32 bytes of K, 32-byte swizzle: the
  // 16-byte halves of rows 4..7 of every eight swap), behind 32 rows of zeros
  for (int i = tid; i < WDW_ROWS * TC / 16; i += TTHREADS) sts128(smem_u32(w_dw) + i * 16, 0u, 0u, 0u, 0u);
  stage_params<MODE>(par_pw, ep, N, tid, TTHREADS);
  stage_params<MODE>(par_dw, ed, TC, tid, TTHREADS);
  __syncthreads();
  for (int i = tid; i < 9 * TC; i += TTHREADS) {
    const int n = i / 9, t = i - n * 9;                       // w_dw is [channel][3][3]: t = dy * 3 + dx
    const int row = 32 + t * 32 + n;
    w_dw[row * 32 + ((((n >> 4) ^ ((row >> 2) & 1)) << 4) | (n & 15))] = (uint8_t)__ldg(g.w_dw + i);
  }
  fence_proxy_async();                  // the tensor cores read what these stores wrote
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // patch pt -> image, first output pixel (x fastest, so neighbours share their halo in L2)
  auto patch_pos = [&](int pt, int &b, int &y0, int &x0) {
    const int r = pt / g.tiles_x;
    x0 = (pt - r * g.tiles_x) * TTW;
    b = r / g.tiles_y;
    y0 = (r - b * g.tiles_y) * TTH;
  };
  // the CTA's units i = 0, 1, ..: unit i is half (i & 1) of the CTA's patch number i >> 1
  const int my_patches = g.patches > (int)blockIdx.x ? (g.patches - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const int my_units = 2 * my_patches;

  if (warp == 0) {
    // ------------------------------ TMA ---------------------------------------------------------
    if (lane == 0) {
      pdl_wait();                       // the input is the previous kernel's output
      pdl_launch_dependents();
      int issued = 0;
      for (int k = 0; k < my_patches; k++) {
        const int s = k % NBOX;
        if (!mbar_wait(&in_empty[s], (((uint32_t)(k / NBOX)) & 1u) ^ 1u, abort_flag, g.status, ST_T_TMA)) break;
        int b, y0, x0;
        patch_pos((int)blockIdx.x + k * (int)gridDim.x, b, y0, x0);
        mbar_arrive_expect_tx(&in_full[s], (uint32_t)BOX_BYTES);
        tma_load_4d(box_ring + s * BOX_STRIDE, &map_in, &in_full[s], 0, x0 / 4 - 1, y0 - 1, b);
        issued++;
      }
      if (*abort_flag && issued) {
        // something gave up: let the loads that are still in flight land before the CTA's memory goes
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ depthwise MMAs ----------------------------------------------
    if (lane == 0) {
      const uint32_t wbase = smem_u32(w_dw);
      for (int k = 0; k < my_patches; k++) {
        const int s = k % NBOX, d = k % NDACC;
        if (!mbar_wait(&d_empty[d], (((uint32_t)(k / NDACC)) & 1u) ^ 1u, abort_flag, g.status, ST_T_MMA)) break;
        if (!mbar_wait(&in_full[s], ((uint32_t)(k / NBOX)) & 1u, abort_flag, g.status, ST_T_MMA)) break;
        tc_fence_after();
        const uint32_t box = smem_u32(box_ring) + s * BOX_STRIDE;
        const uint32_t acc = tmem_base + (uint32_t)(d * 128);          // sub-column j at columns (3 - j) * 32
        // operand "pixel sl of every piece, box row y + dy": rows = the pixels 4q + sl of eight pieces q of 16 box
        // rows; sl = -1 reads the 32 bytes before a box row, which only reach outputs left of the patch (q = 0)
        auto a_desc = [&](int dy, int sl) { return desc_k(box + (uint32_t)((dy * BOX_PX + sl) * TC), BOX_PITCH, 2); };
        if (!(g.ablate & 4)) {
          // clears all four accumulators: [0; w(0,0); w(0,1); w(0,2)] against pixel 1 -> sub-columns -, 2, 1, 0
          umma_i8(acc, a_desc(0, 1), desc_k32(wbase, 8 * TC), umma_idesc_u8s8(128), 0u);
#pragma unroll
          for (int dy = 0; dy < 3; dy++) {
            const uint32_t wrow = wbase + (uint32_t)((32 + dy * 96) * TC);
            umma_i8(acc + 96, a_desc(dy, -1), desc_k32(wrow, 8 * TC), umma_idesc_u8s8(32), 1u);                 // 0 <- dx 0
            umma_i8(acc + 64, a_desc(dy, 0), desc_k32(wrow, 8 * TC), umma_idesc_u8s8(64), 1u);                  // 1 <- dx 0, 0 <- dx 1
            if (dy > 0) umma_i8(acc + 32, a_desc(dy, 1), desc_k32(wrow, 8 * TC), umma_idesc_u8s8(96), 1u);      // 2, 1, 0
            umma_i8(acc, a_desc(dy, 2), desc_k32(wrow, 8 * TC), umma_idesc_u8s8(96), 1u);                       // 3, 2, 1
            umma_i8(acc, a_desc(dy, 3), desc_k32(wrow + 32 * TC, 8 * TC), umma_idesc_u8s8(64), 1u);             // 3 <- dx 1, 2 <- dx 2
            umma_i8(acc, a_desc(dy, 4), desc_k32(wrow + 64 * TC, 8 * TC), umma_idesc_u8s8(32), 1u);             // 3 <- dx 2
          }
        }
        umma_commit(&in_empty[s]);
        umma_commit(&d_full[d]);
      }
    }
  } else if (warp == 2) {
    // ------------------------------ pointwise MMAs ----------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_u8s8(N);
      bool ok = mbar_wait(w_bar, 0, abort_flag, g.status, ST_T_MMA);
      const uint64_t db = desc_k32(smem_u32(w_pw), 8 * TC);
      for (int i = 0; i < my_units && ok; i++) {
        const int a = i % NA2, p = i % NPACC;
        if (!mbar_wait(&p_empty[p], (((uint32_t)(i / NPACC)) & 1u) ^ 1u, abort_flag, g.status, ST_T_MMA)) break;
        if (!mbar_wait(&a2_full[a], ((uint32_t)(i / NA2)) & 1u, abort_flag, g.status, ST_T_MMA)) break;
        tc_fence_after();
#pragma unroll
        for (int jj = 0; jj < 2; jj++)
          umma_i8(tmem_base + (uint32_t)(NDACC * 128 + (p * 2 + jj) * N),
                  desc_k32(smem_u32(a2_ring) + (a * 2 + jj) * A2_BYTES, 8 * TC), db, idesc, 0u);
        umma_commit(&a2_empty[a]);
        umma_commit(&p_full[p]);
      }
    }
  } else if (warp >= FIRST_RQ && warp < FIRST_EP) {
    // ------------------------------ depthwise sums -> requantised rows of the pointwise A operand
    const int grp = (warp - FIRST_RQ) >> 2, quad = warp & 3;
    const int r = quad * 32 + lane;                 // TMEM lane = row of the MMAs
    const uint32_t xr = (uint32_t)((r >> 2) & 1);   // 32-byte swizzle of row r
    for (int i = grp; i < my_units; i += RQ_GROUPS) {         // group h takes half h of every patch
      const int k = i >> 1, h = i & 1, d = k % NDACC, a = i % NA2;
      if (!mbar_wait(&d_full[d], ((uint32_t)(k / NDACC)) & 1u, abort_flag, g.status, ST_T_RQ)) break;
      tc_fence_after();
      // sub-columns j = 2h and 2h + 1 live at columns (3 - j) * 32; one after the other, to stay within the
      // registers that 28 warps leave a thread
      bool ok = true;
#pragma unroll
      for (int jj = 0; jj < 2; jj++) {
        uint32_t v[32];
        tmem_ld_32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(d * 128 + (3 - 2 * h - jj) * 32), v);
        tmem_wait_ld();
        if (jj == 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&d_empty[d]);      // the patch's sums of this half are in registers
        }
        unsigned w[8];
        if (g.ablate & 2) {
#pragma unroll
          for (int t = 0; t < 8; t++) w[t] = v[t];
        } else {
          requant32<MODE>(v, par_dw, TC, ed, w);
        }
        if (jj == 0 && !mbar_wait(&a2_empty[a], (((uint32_t)(i / NA2)) & 1u) ^ 1u, abort_flag, g.status, ST_T_RQ)) { ok = false; break; }
        const uint32_t row = smem_u32(a2_ring) + (a * 2 + jj) * A2_BYTES + (uint32_t)(r * TC);
        sts128(row + (xr << 4), w[0], w[1], w[2], w[3]);
        sts128(row + ((xr ^ 1u) << 4), w[4], w[5], w[6], w[7]);
      }
      if (!ok) break;
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a2_full[a]);
    }
  } else if (warp >= FIRST_EP) {
    // ------------------------------ pointwise epilogue ------------------------------------------
    const int grp = (warp - FIRST_EP) >> 2, quad = warp & 3;
    const int gp = grp >> 1, jj = grp & 1;          // the group's accumulator pair and its sub-column of every unit
    const int r = quad * 32 + lane;
    const int py = r >> 3, q = r & 7;               // box row (= patch row), piece of four pixels
    pdl_wait();                         // the output buffer may still be read by the previous kernel
    for (int i = gp; i < my_units; i += NPACC) {
      const int p = gp, h = i & 1;
      if (!mbar_wait(&p_full[p], ((uint32_t)(i / NPACC)) & 1u, abort_flag, g.status, ST_T_EPI)) break;
      tc_fence_after();
      int b, y0, x0;
      patch_pos((int)blockIdx.x + (i >> 1) * (int)gridDim.x, b, y0, x0);
      const int oy = y0 + py;
      if (!(g.ablate & 1)) {
        const int ox = x0 - 4 + 4 * q + 2 * h + jj;
        const bool store = q > 0 && oy < g.H && ox < g.W;
        uint8_t *orow = g.out + (((size_t)b * g.H + (store ? oy : 0)) * g.W + (store ? ox : 0)) * N;
        const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(NDACC * 128 + (p * 2 + jj) * N);
#pragma unroll
        for (int c0 = 0; c0 < N; c0 += 32) {
          uint32_t v[32];
          tmem_ld_32(t_row + (uint32_t)c0, v);
          tmem_wait_ld();
          unsigned w[8];
          if (g.ablate & 16) {
#pragma unroll
            for (int t = 0; t < 8; t++) w[t] = v[t] ^ v[t + 8] ^ v[t + 16] ^ v[t + 24];
          } else {
            requant32<MODE>(v, par_pw + c0 * (MODE == EPI_BN64 ? 8 : 4), N, ep, w);
          }
          if (store && !(g.ablate & 8))
            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                         ::"l"(orow + c0), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                         : "memory");
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_empty[p]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 3) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int MODE, int N>
bool launch_tcdw(Context &c, const DepthwiseProblem &dw, const ConvProblem &pw)
{
  using G = TG<N>;
  EncodeTiledFn enc = encode_tiled_fn();
  TcdwParams g;
  g.out = static_cast<uint8_t *>(pw.out); g.w_dw = dw.w;
  g.e_dw = dw.epi; g.e_pw = pw.epi;
  g.B = dw.B; g.H = dw.Ho; g.W = dw.Wo;
  g.tiles_x = (dw.Wo + TTW - 1) / TTW;
  g.tiles_y = (dw.Ho + TTH - 1) / TTH;
  const long long patches = (long long)dw.B * g.tiles_x * g.tiles_y;
  if (patches > 0x3fffffffLL) { set_error(PULPNN_ERR_UNSUPPORTED, "fused depthwise+pointwise: too many tiles"); return false; }
  g.patches = (int)patches;
  g.status = ctx_status_word(c);
  if (!g.status) return false;
  g.ablate = (c.opt_tune >> 8) & 31;

  CUtensorMap map_in, map_w;
  {
    // four pixels (128 bytes) are one piece of a box row; pieces left of, right of, above or below the image
    // arrive as zeros
    cuuint64_t dims[4] = {(cuuint64_t)(4 * TC), (cuuint64_t)(dw.W / 4), (cuuint64_t)dw.H, (cuuint64_t)dw.B};
    cuuint64_t strides[3] = {(cuuint64_t)(4 * TC), (cuuint64_t)dw.W * TC, (cuuint64_t)dw.H * dw.W * TC};
    cuuint32_t box[4] = {(cuuint32_t)(4 * TC), (cuuint32_t)(BOX_PX / 4), (cuuint32_t)BOX_H, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = enc(&map_in, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<uint8_t *>(dw.in), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error(PULPNN_ERR_CUDA, "cuTensorMapEncodeTiled (tensor-core depthwise input) failed with code %d", (int)r); return false; }
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)TC, (cuuint64_t)N};
    cuuint64_t strides[1] = {(cuuint64_t)TC};
    cuuint32_t box[2] = {(cuuint32_t)TC, (cuuint32_t)N};
    cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(pw.w), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error(PULPNN_ERR_CUDA, "cuTensorMapEncodeTiled (tensor-core depthwise weights) failed with code %d", (int)r); return false; }
  }
  auto kern = dwpw_tcdw_kernel<MODE, N>;
  static PerDeviceInt attr_set;
  if (!attr_set.get(c.device)) {
    if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM),
                 "cudaFuncSetAttribute(dwpw_tcdw)"))
      return false;
    attr_set.set(c.device, 1);
  }
  const int sms = c.sm_count > 0 ? c.sm_count : 148;
  const int grid = g.patches < sms ? g.patches : sms;
  const cudaError_t le = launch_pdl(kern, dim3(grid), dim3(TTHREADS), (size_t)G::SMEM, c.stream, map_in, map_w, g);
  count_launch("dwpw_tcdw_kernel");
  return cuda_ok(le, "dwpw_tcdw launch") && cuda_ok(cudaGetLastError(), "dwpw_tcdw launch");
}

}  // namespace

// 3x3, stride 1, padding 1, 32 channels in, 64 out, HWC, the same requantisation mode in both layers
bool dwpw_tcdw_supported(const DepthwiseProblem &dw, const ConvProblem &pw)
{
  if (!dw.in_is_hwc || dw.ky != 3 || dw.kx != 3 || dw.pt != 1 || dw.pl != 1 || dw.sx != 1 || dw.sy != 1) return false;
  if (dw.Ho != dw.H || dw.Wo != dw.W || dw.C != TC || pw.Cout != 64) return false;
  if (pw.ky != 1 || pw.kx != 1 || pw.sx != 1 || pw.sy != 1 || pw.pt != 0 || pw.pl != 0) return false;
  if (pw.H != dw.Ho || pw.W != dw.Wo || pw.Ho != pw.H || pw.Wo != pw.W || pw.Cin != dw.C || pw.B != dw.B) return false;
  if (pw.epi.mode != dw.epi.mode || pw.epi.mode == EPI_RAW32) return false;
  if ((reinterpret_cast<uintptr_t>(dw.in) & 15) || (reinterpret_cast<uintptr_t>(pw.out) & 31) ||
      (reinterpret_cast<uintptr_t>(pw.w) & 15))
    return false;
  if (dw.W > 65535 || dw.H > 65535 || dw.W % 4 != 0) return false;       // box rows are pieces of four pixels
  return encode_tiled_fn() != nullptr;
}

bool launch_dwpw_tcdw(Context &c, const DepthwiseProblem &dw, const ConvProblem &pw)
{
  switch (dw.epi.mode) {
    case EPI_NONE: return launch_tcdw<EPI_NONE, 64>(c, dw, pw);
    case EPI_MULT: return launch_tcdw<EPI_MULT, 64>(c, dw, pw);
    case EPI_BN32: return launch_tcdw<EPI_BN32, 64>(c, dw, pw);
    default:       return launch_tcdw<EPI_BN64, 64>(c, dw, pw);
  }
}

}  // namespace pulpnn
