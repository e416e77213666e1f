// dwpw_fused.cu -- a 3x3 depthwise layer (HWC input, padding 1, stride 1 or 2) and the pointwise layer that
// follows it, in one kernel. The chain being fused is the reference's
//     pulp_nn_depthwise_generic  -> Im_out  (32bit/src/pulp_nn_depthwise_generic.c:179)
//     pulp_nn_pointwise_HoWo_parallel <- pInBuffer (32bit/src/pulp_nn_pointwise_HoWo_parallel.c:103)
// whose intermediate tensor (the depthwise output, requantised to uint8) makes one round trip
// through memory. Here it never leaves the SM: the depthwise result of a tile of output pixels is
// written straight into shared memory in the K-major, swizzled layout tcgen05.mma reads as its A
// operand, the pointwise weights stay resident in shared memory as the B operand, the int32
// accumulator lives in tensor memory and the pointwise requantisation runs in the epilogue. The
// arithmetic of both layers is unchanged (same integer operations in the same order per output), so
// the result equals the two-call chain bit for bit.
//
// A unit of work is a patch of TH x TW (<= 128) output pixels of one image, all C channels in,
// all N channels out. Roles in a CTA (persistent over units; two TMA and two MMA warps that take units in
// turn where a layer's units are short, one of each otherwise):
//   TMA warp, one lane  TMA: the resident weights once, then per unit (and per 128-channel chunk) the
//                       (TH+2) x (TW+2) input pixels the patch reads, one 4-D box; pixels outside the
//                       image arrive as zeros, which is the zero padding
//                       (32bit/src/pulp_nn_depthwise_generic.c:82-132)
//   MMA warp, one lane  tcgen05.mma kind::i8, M = 128, N = ch_out, K = 32 per instruction
//   builder warps       depthwise builders, in groups of WPU warps that take units in turn: a thread
//                       owns four channels and four adjacent columns and slides down the patch with
//                       three accumulator sets (depthwise_regs.cuh); finished rows are requantised and
//                       stored as the rows of the A tile
//   epilogue warps      epilogue: tcgen05.ld (lane = pixel), per-channel k / lambda from shared
//                       memory, pack, 32-byte global stores (a pixel's ch_out bytes are contiguous)
// Every mbarrier wait is bounded (sm100_primitives.cuh).
#include <cuda.h>

#include "internal.cuh"
#include "sm100_primitives.cuh"
#include "depthwise_regs.cuh"

namespace pulpnn {

namespace {

using namespace sm100;
using namespace dwregs;

// One thread needs several hundred cycles per unit for its waits, its TMA or MMA issue and its commits
// when busy warps share its scheduler; with the short units of a narrow layer that, not memory or
// arithmetic, set the pace (measured: the kernel took as long with the depthwise arithmetic left out).
// So where the rings allow it two TMA threads and two MMA threads take units in turn.
constexpr int ST_F_TMA = 0x10000, ST_F_BUILD = 0x20000, ST_F_MMA = 0x40000, ST_F_EPI = 0x80000;

// geometry, all compile-time: C input channels, N output channels, patch of TH x TW pixels
template <int C, int N, int TW, int TH, int BW, int EW, int SRV, int S> struct FG {
  static constexpr int NSRV = SRV;            // TMA warps = MMA warps; they take units in turn
  static constexpr int FIRST_MMA = NSRV, FIRST_BUILD = 2 * NSRV;
  static constexpr int BUILD_WARPS = BW;                      // depthwise builder warps
  static constexpr int EPI_WARPS_N = EW;                      // epilogue warps: groups of four (one per TMEM lane quarter)
  static constexpr int EPI_GROUPS = EW / 4;
  static constexpr int FIRST_EPI = FIRST_BUILD + BUILD_WARPS;
  static constexpr int THREADS = 32 * (FIRST_EPI + EPI_WARPS_N);
  static_assert(EW % 4 == 0 && (N != 256 || EW == 8), "epilogue warps come in groups of four; 256 columns take two groups per tile");
  static constexpr int CI = C < 128 ? C : 128;               // channel bytes per chunk = K-slab width
  static constexpr int NCHUNK = C / CI;
  static constexpr int LPC = CI / 4;                          // lanes (channel words) per pixel
  static constexpr int NSUB = 32 / LPC;                       // column groups per warp
  static constexpr int NG = TW / 4;                           // column groups per patch
  static constexpr int WPU = NG * LPC / 32;                   // warps that build one unit
  static constexpr int NBG = BUILD_WARPS / WPU;               // builder groups (units in the making); spare warps idle
  static constexpr int PIX = TW * TH;
  static constexpr int WBOX = S == 1 ? TW + 2 : 2 * TW + 1;   // input columns / rows a patch reads (3x3, padding 1)
  static constexpr int ROWS_IN = S == 1 ? TH + 2 : 2 * TH + 1;
  static_assert(S == 1 || S == 2, "stride 1 or 2");
  static constexpr int IN_PITCH = WBOX * CI;
  static constexpr int IN_BYTES = ROWS_IN * IN_PITCH;         // one TMA box
  static constexpr int IN_STRIDE = (IN_BYTES + 127) / 128 * 128;
  static constexpr int A_SLAB = 128 * CI;                     // 128 rows x one chunk of K
  static constexpr int A_TILE = NCHUNK * A_SLAB;
  static constexpr int NUM_ACC = 512 / N > 8 ? 8 : 512 / N;   // accumulators in tensor memory
  static constexpr int NA = NUM_ACC % NBG == 0 ? NUM_ACC : NBG;   // ring of A tiles: a multiple of the builder groups
  // With all channels in one chunk the (TW+2) pixels of a box row are contiguous in memory: the box is
  // described over [B][H][W*C/4] 32-bit elements, ROWS_IN runs of (TW+2)*C bytes instead of
  // ROWS_IN*(TW+2) pieces of C bytes (the TMA unit works through a box piece by piece, and 32-byte
  // pieces were what bounded the 32-channel kernel).
  static constexpr bool ROW_RUNS = NCHUNK == 1 && WBOX * C / 4 <= 256;
  static constexpr int NIN_WANT = NBG == 1 ? 3 : (NBG * NCHUNK <= 4 ? 4 : 2 * NBG * NCHUNK);   // ring of input boxes
  // ... as many as shared memory has room for beside the weights, the A tiles and the parameters
  static constexpr int NIN_ROOM = (232448 - 4096 - ((N * C + 1023) / 1024 * 1024) - (512 / N > 8 ? 8 : 512 / N) * (C / CI) * 128 * CI -
                                   N * 16) / ((ROWS_IN * WBOX * CI + 127) / 128 * 128);
  static constexpr int NIN = NIN_WANT <= NIN_ROOM ? NIN_WANT : (NBG == 1 ? NIN_ROOM : NIN_ROOM / (NBG * NCHUNK) * (NBG * NCHUNK));
  static_assert(NIN >= 2, "at least two input boxes: one being read, one on its way");
  static constexpr int W_BYTES = N * C;
  static constexpr int PARAM_BYTES = N * 16;                  // k and lambda (up to 8 bytes each) or bias
  static constexpr int W_OFF = 0;
  static constexpr int A_OFF = (W_BYTES + 1023) / 1024 * 1024;
  static constexpr int IN_OFF = A_OFF + NA * A_TILE;
  static constexpr int PARAM_OFF = IN_OFF + NIN * IN_STRIDE;
  static constexpr int BAR_OFF = PARAM_OFF + PARAM_BYTES;
  static constexpr int SMEM = 1024 + BAR_OFF + 1024;
  static_assert(C % CI == 0 && (NG * LPC) % 32 == 0 && WPU <= BUILD_WARPS, "builder warps must tile a unit");
  static_assert(NG % NSUB == 0, "a warp's column groups must all belong to the patch");
  static_assert(PIX <= 128 && TW % 4 == 0, "a patch is at most one 128-row tile");
  static_assert(NA % NBG == 0, "an A tile must always be built by the same group");
  static_assert(NBG == 1 || NIN % (NBG * NCHUNK) == 0, "an input slot must always be read by the same group");
  static_assert(N % 32 == 0 && N >= 32 && N <= 256, "ch_out: a multiple of 32 up to 256");
  static_assert(SMEM <= 232448, "shared memory of one CTA");
  static_assert(NSRV == 1 || (NCHUNK == 1 && NIN % NSRV == 0 && NA % NSRV == 0 && NUM_ACC % NSRV == 0),
                "a ring slot must always be served by the same TMA / MMA warp");
};

struct FusedParams {
  const uint8_t *in;       // [B][H][W][C]
  uint8_t *out;            // [B][H][W][N]
  const int8_t *w_dw;      // [C][3][3]
  Epilogue e_dw, e_pw;
  int B, H, W;             // OUTPUT rows and columns (the input's size lives in the tensor map)
  int tiles_x, tiles_y, units;
  int ablate;              // measurement only (PULPNN_OPT_TUNE bits 8-10): 1 no stores, 2 no depthwise math, 4 no requantisation
  int *status;
};

// byte offset of 32-bit word c4 of row r inside a K-major slab whose rows are CI bytes with the
// CI-byte swizzle: the 16-byte chunk index is XORed with address bits 7.. (as many bits as it has)
template <int CI>
__device__ __forceinline__ uint32_t a_word_off(int r, int c4)
{
  const int chunk = c4 >> 2;
  const int x = CI == 128 ? (r & 7) : (CI == 64 ? ((r >> 1) & 3) : ((r >> 2) & 1));
  return (uint32_t)(r * CI + ((chunk ^ x) << 4) + ((c4 & 3) << 2));
}

// requantise a completed row of 4 columns x 4 channels and store it as rows r0..r0+3 of the A slab
template <int MODE, int CI>
__device__ __forceinline__ void finalize_to_a(const int (&acc)[4][4], const QuantT<MODE> &q, const Epilogue &e,
                                              bool k32, uint32_t slab, int r0, int c4)
{
#pragma unroll
  for (int i = 0; i < 4; i++) {
    int v[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      if (MODE == EPI_BN32)
        v[j] = (int)((unsigned)q.k[j] * (unsigned)acc[i][j] + (unsigned)q.l[j]) >> e.shift;
      else if (MODE == EPI_BN64)
        v[j] = k32 ? (int)(mad_wide_s32((int)q.k[j], acc[i][j], (long long)q.l[j]) >> e.shift)
                   : (int)((long long)((unsigned long long)q.k[j] * (unsigned long long)(long long)acc[i][j] +
                                       (unsigned long long)q.l[j]) >> e.shift);
      else if (MODE == EPI_MULT)
        v[j] = (int)(short)((int)((unsigned)e.out_mult * (unsigned)acc[i][j]) >> e.shift);
      else
        v[j] = acc[i][j] >> e.shift;
    }
    sts32(slab + a_word_off<CI>(r0 + i, c4), pack4_sat_u8(v[0], v[1], v[2], v[3]));
  }
}

template <int MODE, int C, int N, int TW, int TH, int BW, int EW, int SRV, int S>
__global__ void __launch_bounds__((FG<C, N, TW, TH, BW, EW, SRV, S>::THREADS), 1)
dwpw_fused_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_w,
                  const FusedParams g)
{
  using G = FG<C, N, TW, TH, BW, EW, SRV, S>;
  constexpr int CI = G::CI;
  constexpr int THREADS = G::THREADS, FIRST_EPI = G::FIRST_EPI, FIRST_BUILD = G::FIRST_BUILD, FIRST_MMA = G::FIRST_MMA;
  constexpr int NSRV = G::NSRV;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t *w_res = sm + G::W_OFF;
  uint8_t *a_ring = sm + G::A_OFF;
  uint8_t *in_ring = sm + G::IN_OFF;
  uint8_t *params = sm + G::PARAM_OFF;
  uint64_t *in_full = reinterpret_cast<uint64_t *>(sm + G::BAR_OFF);
  uint64_t *in_empty = in_full + G::NIN;
  uint64_t *a_full = in_empty + G::NIN;
  uint64_t *a_empty = a_full + G::NA;
  uint64_t *t_full = a_empty + G::NA;
  uint64_t *t_empty = t_full + G::NUM_ACC;
  uint64_t *w_bar = t_empty + G::NUM_ACC;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(w_bar + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const Epilogue &ed = g.e_dw;
  const Epilogue &ep = g.e_pw;
  // with 256 output channels both halves of the epilogue warps drain every accumulator
  constexpr int EPI_PER_ACC = N == 256 ? 8 : 4;

  if (tid == 0) {
    for (int s = 0; s < G::NIN; s++) { mbar_init(&in_full[s], 1); mbar_init(&in_empty[s], G::WPU); }
    for (int s = 0; s < G::NA; s++) { mbar_init(&a_full[s], G::WPU); mbar_init(&a_empty[s], 1); }
    for (int s = 0; s < G::NUM_ACC; s++) { mbar_init(&t_full[s], 1); mbar_init(&t_empty[s], EPI_PER_ACC); }
    mbar_init(w_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    // Weights and per-channel parameters are constants that no kernel of this library writes once a
    // layer is set up, so they are fetched before the wait on the previous kernel and overlap its tail.
    mbar_arrive_expect_tx(w_bar, (uint32_t)G::W_BYTES);
    for (int ch = 0; ch < G::NCHUNK; ch++) tma_load_2d(w_res + ch * N * CI, &map_w, w_bar, ch * CI, 0);
  }
  if (warp == FIRST_MMA) tmem_alloc(tmem_slot, TMEM_COLS);
  // pointwise per-channel parameters -> shared memory, the bias folded into lambda:
  // k*(acc+b)+lambda == k*acc + (k*b+lambda) in wrap-around arithmetic
  for (int n = tid; n < N; n += THREADS) {
    const int bias8 = ep.bias ? (int)__ldg(reinterpret_cast<const int8_t *>(ep.bias) + n) : 0;
    if (MODE == EPI_BN32) {
      const int k = __ldg(reinterpret_cast<const int *>(ep.k) + n);
      reinterpret_cast<int *>(params)[n] = k;
      reinterpret_cast<int *>(params)[N + n] =
          (int)((unsigned)k * (unsigned)bias8 + (unsigned)__ldg(reinterpret_cast<const int *>(ep.lambda) + n));
    } else if (MODE == EPI_BN64) {
      const long long k = __ldg(reinterpret_cast<const long long *>(ep.k) + n);
      reinterpret_cast<long long *>(params)[n] = k;
      reinterpret_cast<long long *>(params)[N + n] =
          (long long)((unsigned long long)k * (unsigned long long)(long long)bias8 +
                      (unsigned long long)__ldg(reinterpret_cast<const long long *>(ep.lambda) + n));
    } else {
      reinterpret_cast<int *>(params)[n] = bias8;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // unit u -> image, first output pixel of the patch (x fastest, so neighbours share their halo in L2)
  auto unit_pos = [&](int u, int &b, int &y0, int &x0) {
    const int r = u / g.tiles_x;
    x0 = (u - r * g.tiles_x) * TW;
    b = r / g.tiles_y;
    y0 = (r - b * g.tiles_y) * TH;
  };

  if (warp < FIRST_MMA) {
    // ------------------------------ TMA: warp w loads the units i = w, w + NSRV, ... ------------
    if (lane == 0) {
      pdl_wait();                       // the input is the previous kernel's output
      if (warp == 0) pdl_launch_dependents();
      int issued = 0;
      bool ok = true;
      int i = 0;
      for (int u = blockIdx.x; u < g.units && ok; u += gridDim.x, i++) {
        if (NSRV > 1 && i % NSRV != warp) continue;
        int b, y0, x0;
        unit_pos(u, b, y0, x0);
        for (int ch = 0; ch < G::NCHUNK; ch++) {
          const int item = i * G::NCHUNK + ch, s = item % G::NIN;
          const uint32_t ph = ((uint32_t)(item / G::NIN)) & 1u;
          if (!mbar_wait(&in_empty[s], ph ^ 1, abort_flag, g.status, ST_F_TMA)) { ok = false; break; }
          mbar_arrive_expect_tx(&in_full[s], (uint32_t)G::IN_BYTES);
          if (G::ROW_RUNS)      // whole pixels: a row of the box is one run of (TW+2)*C bytes, in 32-bit elements
            tma_load_3d(in_ring + s * G::IN_STRIDE, &map_in, &in_full[s], (S * x0 - 1) * (C / 4), S * y0 - 1, b);
          else
            tma_load_4d(in_ring + s * G::IN_STRIDE, &map_in, &in_full[s], ch * CI, S * x0 - 1, S * y0 - 1, b);
          issued++;
        }
      }
      if (*abort_flag && issued) {
        // something gave up: let the loads that are still in flight land before the CTA's memory goes
        // (a load takes a few microseconds at most)
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp < FIRST_BUILD) {
    // ------------------------------ MMA: warp w issues the units i = w, w + NSRV, ... -----------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_u8s8(N);
      const int me = warp - FIRST_MMA;
      bool ok = mbar_wait(w_bar, 0, abort_flag, g.status, ST_F_MMA);
      int i = 0;
      for (int u = blockIdx.x; u < g.units && ok; u += gridDim.x, i++) {
        if (NSRV > 1 && i % NSRV != me) continue;
        const int slot = i % G::NA, acc = i % G::NUM_ACC;
        if (!mbar_wait(&t_empty[acc], (((uint32_t)(i / G::NUM_ACC)) & 1u) ^ 1u, abort_flag, g.status, ST_F_MMA)) break;
        if (!mbar_wait(&a_full[slot], ((uint32_t)(i / G::NA)) & 1u, abort_flag, g.status, ST_F_MMA)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + (uint32_t)(acc * N);
#pragma unroll
        for (int ch = 0; ch < G::NCHUNK; ch++) {
          const uint64_t da = umma_smem_desc<CI>(smem_u32(a_ring) + slot * G::A_TILE + ch * G::A_SLAB);
          const uint64_t db = umma_smem_desc<CI>(smem_u32(w_res) + ch * N * CI);
#pragma unroll
          for (int j = 0; j < CI / 32; j++)
            umma_i8(d, da + (uint64_t)(j * 2), db + (uint64_t)(j * 2), idesc, (ch > 0 || j > 0) ? 1u : 0u);
        }
        umma_commit(&a_empty[slot]);
        umma_commit(&t_full[acc]);
      }
    }
  } else if (warp < FIRST_EPI) {
    // ------------------------------ depthwise builders ------------------------------------------
    const int bw = warp - FIRST_BUILD;
    const int grp = bw / G::WPU, wig = bw - grp * G::WPU;          // group, warp inside the group
    const int c4 = lane % G::LPC, sub = lane / G::LPC, gx = wig * G::NSUB + sub;
    const Rot rot = make_rot<CI>(sub);
    const uint32_t in_thr = (uint32_t)(4 * S * gx) * CI + 4u * c4; // thread's first staged pixel of a row

    // the thread's four channels of chunk ch: filter taps and requantisation parameters
    int wa[3][4], wb[3][4], init[4];
    QuantT<MODE> q;
    bool k32 = true;
    auto load_channel_params = [&](int ch) {
      const int c = ch * CI + 4 * c4;
      unsigned Wd[9];
      const unsigned *wp = reinterpret_cast<const unsigned *>(g.w_dw + (size_t)c * 9);
#pragma unroll
      for (int i = 0; i < 9; i++) Wd[i] = __ldg(wp + i);
#pragma unroll
      for (int j = 0; j < 4; j++)
#pragma unroll
        for (int fy = 0; fy < 3; fy++) {
          wa[fy][j] = taps3(Wd, j * 9 + fy * 3);
          wb[fy][j] = (int)((unsigned)wa[fy][j] << 8);
        }
      k32 = true;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        q.bias[j] = ed.bias ? (int)__ldg(reinterpret_cast<const int8_t *>(ed.bias) + c + j) : 0;
        q.k[j] = 0; q.l[j] = 0;
        init[j] = (MODE == EPI_BN32 || MODE == EPI_BN64) ? 0 : q.bias[j];
        if (MODE == EPI_BN32) {
          const int k = __ldg(reinterpret_cast<const int *>(ed.k) + c + j);
          q.k[j] = k;
          q.l[j] = (int)((unsigned)k * (unsigned)q.bias[j] + (unsigned)__ldg(reinterpret_cast<const int *>(ed.lambda) + c + j));
        } else if (MODE == EPI_BN64) {
          const long long k = __ldg(reinterpret_cast<const long long *>(ed.k) + c + j);
          q.k[j] = k;
          q.l[j] = (long long)((unsigned long long)k * (unsigned long long)(long long)q.bias[j] +
                               (unsigned long long)__ldg(reinterpret_cast<const long long *>(ed.lambda) + c + j));
          k32 = k32 && (k == (long long)(int)k);
        }
      }
    };
    if (G::NCHUNK == 1) load_channel_params(0);

    bool ok = grp < G::NBG;
    int i = 0;
    for (int u = blockIdx.x; u < g.units && ok; u += gridDim.x, i++) {
      if (i % G::NBG != grp) continue;
      const int slot = i % G::NA;
      if (!mbar_wait(&a_empty[slot], (((uint32_t)(i / G::NA)) & 1u) ^ 1u, abort_flag, g.status, ST_F_BUILD)) break;
#pragma unroll 1
      for (int ch = 0; ch < G::NCHUNK; ch++) {
        const int item = i * G::NCHUNK + ch, is = item % G::NIN;
        if (G::NCHUNK > 1) load_channel_params(ch);
        if (!mbar_wait(&in_full[is], ((uint32_t)(item / G::NIN)) & 1u, abort_flag, g.status, ST_F_BUILD)) { ok = false; break; }
        const uint32_t ia = smem_u32(in_ring) + is * G::IN_STRIDE + in_thr;
        const uint32_t slab = smem_u32(a_ring) + slot * G::A_TILE + ch * G::A_SLAB;
        uint32_t ra[4];
#pragma unroll
        for (int t = 0; t < 4; t++) ra[t] = ia + CI + rot.off[t];
        if constexpr (S == 1) {
          // Staged row ri holds input row y0-1+ri. It is filter row 2 of output row ri-2 (which it
          // completes), row 1 of output row ri-1 and row 0 of output row ri (which it opens); the three
          // accumulator sets rotate, at compile time.
          int acc[3][4][4];
#pragma unroll
          for (int ri = 0; ri < G::ROWS_IN; ri++) {
            if (g.ablate & 2) break;
            unsigned cur[6]; Win1 w;
            load_row1<CI>(ia, ra, ri * G::IN_PITCH, cur);
            windows1(cur, rot, w);
            int (&X)[4][4] = acc[(ri + 1) % 3];     // output row ri-2
            int (&Y)[4][4] = acc[(ri + 2) % 3];     // output row ri-1
            int (&Z)[4][4] = acc[ri % 3];           // output row ri
            if (ri == 0) mac1<false, false, true>(w, wa, wb, init, X, Y, Z);
            else if (ri == 1) mac1<false, true, true>(w, wa, wb, init, X, Y, Z);
            else if (ri < TH) mac1<true, true, true>(w, wa, wb, init, X, Y, Z);
            else if (ri == TH) mac1<true, true, false>(w, wa, wb, init, X, Y, Z);
            else mac1<true, false, false>(w, wa, wb, init, X, Y, Z);
            if (ri >= 2) finalize_to_a<MODE, CI>(X, q, ed, k32, slab, (ri - 2) * TW + 4 * gx, c4);
          }
        } else {
          // Stride 2: staged row ri holds input row 2*y0-1+ri; output row r reads staged rows 2r, 2r+1,
          // 2r+2 (filter rows 0, 1, 2), and row 2r+2 is also filter row 0 of output row r+1. One
          // accumulator set; nine staged pixels per row feed four outputs.
          int acc[4][4];
          unsigned cur[9]; Win2 w;
          if (!(g.ablate & 2)) {
            load_row2<CI>(ia, ra, 0, cur);
            windows2(cur, rot, w);
            mac2<true>(w, wa[0], wb[0], init, acc);
#pragma unroll
            for (int r = 0; r < TH; r++) {
              load_row2<CI>(ia, ra, (2 * r + 1) * G::IN_PITCH, cur);
              windows2(cur, rot, w);
              mac2<false>(w, wa[1], wb[1], init, acc);
              load_row2<CI>(ia, ra, (2 * r + 2) * G::IN_PITCH, cur);
              windows2(cur, rot, w);
              mac2<false>(w, wa[2], wb[2], init, acc);
              finalize_to_a<MODE, CI>(acc, q, ed, k32, slab, r * TW + 4 * gx, c4);
              if (r + 1 < TH) mac2<true>(w, wa[0], wb[0], init, acc);
            }
          }
        }
        // the input box has been read: hand the slot back to the TMA warp
        __syncwarp();
        if (lane == 0) mbar_arrive(&in_empty[is]);
      }
      if (!ok) break;
      fence_proxy_async();              // the tile words written above, before the tensor cores read them
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_full[slot]);
    }
  } else {
    // ------------------------------ epilogue ----------------------------------------------------
    const int ew = warp - FIRST_EPI;
    const int quad = warp & 3;                  // the TMEM lanes this warp may read: 32*quad .. +31
    const int half = ew >> 2;                   // which group of four warps
    const int r = quad * 32 + lane;             // row of the tile = pixel of the patch
    const int py = r / TW, px = r - py * TW;
    // N <= 128: the groups take units in turn; N = 256: two groups work on every unit, 128 columns each
    constexpr int COLS = N == 256 ? 128 : N;
    const int col0 = N == 256 ? half * 128 : 0;
    const int *p_k32 = reinterpret_cast<const int *>(params), *p_l32 = p_k32 + N;
    const long long *p_k64 = reinterpret_cast<const long long *>(params), *p_l64 = p_k64 + N;
    const int *p_bias = reinterpret_cast<const int *>(params);
    pdl_wait();                         // the output buffer may still be read by the previous kernel
    int i = 0;
    for (int u = blockIdx.x; u < g.units; u += gridDim.x, i++) {
      if (N != 256 && i % G::EPI_GROUPS != half) continue;
      const int acc = i % G::NUM_ACC;
      if (!mbar_wait(&t_full[acc], ((uint32_t)(i / G::NUM_ACC)) & 1u, abort_flag, g.status, ST_F_EPI)) break;
      tc_fence_after();
      int b, y0, x0;
      unit_pos(u, b, y0, x0);
      const int oy = y0 + py, ox = x0 + px;
      const bool store = r < G::PIX && oy < g.H && ox < g.W;
      uint8_t *orow = g.out + (((size_t)b * g.H + (store ? oy : 0)) * g.W + (store ? ox : 0)) * N + col0;
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * N + col0);
      // two register buffers: the next 32 columns are on their way from tensor memory while these
      // are requantised
      uint32_t vb[2][32];
      tmem_ld_32(t_row, vb[0]);
#pragma unroll
      for (int c0 = 0; c0 < COLS; c0 += 32) {
        uint32_t (&v)[32] = vb[(c0 >> 5) & 1];
        tmem_wait_ld();
        if (c0 + 32 < COLS) tmem_ld_32(t_row + (uint32_t)(c0 + 32), vb[((c0 >> 5) + 1) & 1]);
        unsigned w[8];
        const int pc = col0 + c0;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          int qv[4];
          if (MODE == EPI_BN32) {
            const int4 kk = *reinterpret_cast<const int4 *>(p_k32 + pc + j);
            const int4 ll = *reinterpret_cast<const int4 *>(p_l32 + pc + j);
            qv[0] = (int)((unsigned)kk.x * v[j + 0] + (unsigned)ll.x) >> ep.shift;
            qv[1] = (int)((unsigned)kk.y * v[j + 1] + (unsigned)ll.y) >> ep.shift;
            qv[2] = (int)((unsigned)kk.z * v[j + 2] + (unsigned)ll.z) >> ep.shift;
            qv[3] = (int)((unsigned)kk.w * v[j + 3] + (unsigned)ll.w) >> ep.shift;
          } else {
#pragma unroll
            for (int t = 0; t < 4; t++) {
              const int a = (int)v[j + t];
              if (MODE == EPI_BN64)
                qv[t] = (int)((long long)((unsigned long long)p_k64[pc + j + t] * (unsigned long long)(long long)a +
                                          (unsigned long long)p_l64[pc + j + t]) >> ep.shift);
              else if (MODE == EPI_MULT)
                qv[t] = (int)(short)((int)((unsigned)ep.out_mult * (unsigned)(a + p_bias[pc + j + t])) >> ep.shift);
              else
                qv[t] = (a + p_bias[pc + j + t]) >> ep.shift;
            }
          }
          w[j >> 2] = pack4_sat_u8(qv[0], qv[1], qv[2], qv[3]);
        }
        if (store && !(g.ablate & 1))
          asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                       ::"l"(orow + c0), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                       : "memory");
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&t_empty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == FIRST_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- host side ----------------------------------------------------------------------------------
template <int MODE, int C, int N, int TW, int TH, int BW, int EW, int SRV, int S = 1>
bool launch_geo(Context &c, const DepthwiseProblem &dw, const ConvProblem &pw)
{
  using G = FG<C, N, TW, TH, BW, EW, SRV, S>;
  EncodeTiledFn enc = encode_tiled_fn();
  FusedParams g;
  g.in = dw.in; g.out = static_cast<uint8_t *>(pw.out); g.w_dw = dw.w;
  g.e_dw = dw.epi; g.e_pw = pw.epi;
  g.B = dw.B; g.H = dw.Ho; g.W = dw.Wo;
  g.tiles_x = (dw.Wo + TW - 1) / TW;
  g.tiles_y = (dw.Ho + TH - 1) / TH;
  const long long units = (long long)dw.B * g.tiles_x * g.tiles_y;
  if (units > 0x7fffffffLL) { set_error(PULPNN_ERR_UNSUPPORTED, "fused depthwise+pointwise: too many tiles"); return false; }
  g.units = (int)units;
  g.status = ctx_status_word(c);
  if (!g.status) return false;
  g.ablate = (c.opt_tune >> 8) & 7;

  CUtensorMap map_in, map_w;
  if (G::ROW_RUNS) {
    cuuint64_t dims[3] = {(cuuint64_t)dw.W * C / 4, (cuuint64_t)dw.H, (cuuint64_t)dw.B};
    cuuint64_t strides[2] = {(cuuint64_t)dw.W * C, (cuuint64_t)dw.H * dw.W * C};
    cuuint32_t box[3] = {(cuuint32_t)(G::WBOX * C / 4), (cuuint32_t)G::ROWS_IN, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(&map_in, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<uint8_t *>(dw.in), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error(PULPNN_ERR_CUDA, "cuTensorMapEncodeTiled (fused input rows) failed with code %d", (int)r); return false; }
  } else {
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)dw.W, (cuuint64_t)dw.H, (cuuint64_t)dw.B};
    cuuint64_t strides[3] = {(cuuint64_t)C, (cuuint64_t)dw.W * C, (cuuint64_t)dw.H * dw.W * C};
    cuuint32_t box[4] = {(cuuint32_t)G::CI, (cuuint32_t)G::WBOX, (cuuint32_t)G::ROWS_IN, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = enc(&map_in, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<uint8_t *>(dw.in), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error(PULPNN_ERR_CUDA, "cuTensorMapEncodeTiled (fused input) failed with code %d", (int)r); return false; }
  }
  {
    // pointwise weights [N][C], K contiguous: one box per 128-channel chunk, rows CI bytes, CI-byte swizzle
    cuuint64_t dims[2] = {(cuuint64_t)C, (cuuint64_t)N};
    cuuint64_t strides[1] = {(cuuint64_t)C};
    cuuint32_t box[2] = {(cuuint32_t)G::CI, (cuuint32_t)N};
    cuuint32_t estr[2] = {1, 1};
    const CUtensorMapSwizzle sw = G::CI == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                : (G::CI == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    const CUresult r = enc(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(pw.w), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error(PULPNN_ERR_CUDA, "cuTensorMapEncodeTiled (fused weights) failed with code %d", (int)r); return false; }
  }
  auto kern = dwpw_fused_kernel<MODE, C, N, TW, TH, BW, EW, SRV, S>;
  static PerDeviceInt attr_set;
  if (!attr_set.get(c.device)) {
    if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM),
                 "cudaFuncSetAttribute(dwpw_fused)"))
      return false;
    attr_set.set(c.device, 1);
  }
  const int sms = c.sm_count > 0 ? c.sm_count : 148;
  const int grid = g.units < sms ? g.units : sms;
  const cudaError_t le = launch_pdl(kern, dim3(grid), dim3(G::THREADS), (size_t)G::SMEM, c.stream, map_in, map_w, g);
  count_launch("dwpw_fused_kernel");
  return cuda_ok(le, "dwpw_fused launch") && cuda_ok(cudaGetLastError(), "dwpw_fused launch");
}

// the geometries on offer: (C, N) and the patch that tiles the image's width best
template <int MODE>
bool launch_shape(Context &c, const DepthwiseProblem &dw, const ConvProblem &pw)
{
  const int C = dw.C, N = pw.Cout;
  // patch shapes: 16 x 8 tiles a 112-wide image exactly; 28 x 4 tiles 56- and 28-wide ones (measured
  // against 8 x 16 on 56 x 56 x 128: 0.243 ms against 0.272 ms at batch 1024). Measured and dropped on
  // the 32-channel pair at batch 1024 (0.342 ms as configured): twelve builder warps (0.375 with one TMA
  // and one MMA warp either way), three epilogue groups (0.345), four TMA and four MMA warps (0.362);
  // on the 128-channel pair two TMA and two MMA warps (0.276 against 0.243)
  if (C == 32 && N == 64) {
    return launch_geo<MODE, 32, 64, 16, 8, 8, 8, 2>(c, dw, pw);
  }
  if (C == 128 && N == 128) {
    return launch_geo<MODE, 128, 128, 28, 4, 14, 8, 1>(c, dw, pw);
  }
  if (C == 256 && N == 256) return launch_geo<MODE, 256, 256, 28, 4, 8, 8, 1>(c, dw, pw);
  if (C == 64 && N == 128 && dw.sx == 2) return launch_geo<MODE, 64, 128, 16, 8, 8, 8, 1, 2>(c, dw, pw);
  if (C == 128 && N == 256 && dw.sx == 2) return launch_geo<MODE, 128, 256, 28, 4, 7, 8, 1, 2>(c, dw, pw);
  set_error(PULPNN_ERR_UNSUPPORTED, "fused depthwise+pointwise: no kernel for %d -> %d channels", C, N);
  return false;
}

}  // namespace

bool dwpw_fused_supported(const DepthwiseProblem &dw, const ConvProblem &pw)
{
  if (!dw.in_is_hwc || dw.ky != 3 || dw.kx != 3 || dw.pt != 1 || dw.pl != 1 || dw.sx != dw.sy) return false;
  if (dw.sx != 1 && dw.sx != 2) return false;
  // the output size of a zero-padded 3x3 convolution with padding 1 on every side
  if (dw.Ho != (dw.H - 1) / dw.sy + 1 || dw.Wo != (dw.W - 1) / dw.sx + 1) return false;
  if (pw.ky != 1 || pw.kx != 1 || pw.sx != 1 || pw.sy != 1 || pw.pt != 0 || pw.pl != 0) return false;
  if (pw.H != dw.Ho || pw.W != dw.Wo || pw.Ho != pw.H || pw.Wo != pw.W || pw.Cin != dw.C || pw.B != dw.B) return false;
  if (pw.epi.mode != dw.epi.mode || pw.epi.mode == EPI_RAW32) return false;      // one requantisation mode per kernel
  const int C = dw.C, N = pw.Cout;
  if (dw.sx == 1) {
    if (!((C == 32 && N == 64) || (C == 128 && N == 128) || (C == 256 && N == 256))) return false;
    // 256 -> 256 channels: measured on 28 x 28 images, the fused kernel wins up to batch 256 (0.049 ms
    // against 0.052 ms for the two kernels; 0.027 against 0.030 at batch 128) and loses at batch 1024
    // (0.171 against 0.165), where the two kernels' larger tiles pay
    if (C == 256 && (long long)dw.B * dw.H * dw.W > 512LL * 28 * 28) return false;
  } else {
    if (!((C == 64 && N == 128) || (C == 128 && N == 256))) return false;
  }
  if ((reinterpret_cast<uintptr_t>(dw.in) & 15) || (reinterpret_cast<uintptr_t>(pw.out) & 31)) return false;
  if ((reinterpret_cast<uintptr_t>(dw.w) & 3) || (reinterpret_cast<uintptr_t>(pw.w) & 15)) return false;
  if (dw.Wo < 4 || dw.Ho < 1 || dw.W > 65535 || dw.H > 65535) return false;
  return encode_tiled_fn() != nullptr;
}

bool launch_dwpw_fused(Context &c, const DepthwiseProblem &dw, const ConvProblem &pw)
{
  // 32 channels: the form with the depthwise sums made by tensor-core MMAs (dwpw_tcdw.cu) is selectable with
  // PULPNN_OPT_TUNE bit 5. Measured on 112 x 112 x 32 -> 64: 0.353 against 0.345 ms at batch 1024, 0.051 against
  // 0.048 at batch 128: both forms are bound by the requantisation's integer work, so the builders stay.
  if ((c.opt_tune & 32) && dwpw_tcdw_supported(dw, pw)) return launch_dwpw_tcdw(c, dw, pw);
  switch (dw.epi.mode) {
    case EPI_NONE: return launch_shape<EPI_NONE>(c, dw, pw);
    case EPI_MULT: return launch_shape<EPI_MULT>(c, dw, pw);
    case EPI_BN32: return launch_shape<EPI_BN32>(c, dw, pw);
    default:       return launch_shape<EPI_BN64>(c, dw, pw);
  }
}

}  // namespace pulpnn
