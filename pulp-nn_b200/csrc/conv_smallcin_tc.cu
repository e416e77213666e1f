// conv_smallcin_tc.cu -- the first layer of an image network (3x3 kernel, 3 input channels,
// 32 or 64 output channels) on the sm_100a tensor cores. Arithmetic is that of the reference's
// im2col + matmul pair (32bit/src/pulp_nn_conv_Ho_parallel.c:77-147, pulp_nn_matmul.c:55-216):
// every output pixel is the dot product of a zero-padded 3x3xCin window with each filter, then
// bias and requantisation.
//
// The im2col matrix is never written to memory: it is built in shared memory, tile by tile, in
// the layout tcgen05.mma reads (K-major rows of 64 bytes with the 64-byte swizzle). A row of it is
// one output pixel; its K axis is laid out as four 16-byte chunks, chunk fy = the kx*Cin (<= 9)
// bytes of filter row fy followed by zeros, chunk 3 = zeros, and the filters are re-packed the same
// way once per CTA. So K = 64, two MMAs of K = 32 per tile of 128 pixels x BN output channels.
//
// Roles in a CTA (15 warps, persistent over units = 4 consecutive output rows of one image):
//   warp 0, one lane   TMA: the 3*SY+3 input rows a unit needs, as one 4-D box of the input seen
//                      as [B][H][pieces of a row][32 or 16 bytes]; rows above and below the image
//                      are zeros
//   warps 1..4         builders: thread = output column. Per input row three aligned words, one
//                      funnel shift each and a mask (columns left/right of the image) give the
//                      window's 9 bytes; 16-byte stores put them into the four tiles of the unit
//   warps 5..6         one lane each issues the two tcgen05.mma of every other tile
//   warps 7..14        epilogue, two groups that take tiles in turn: tcgen05.ld (lane = pixel),
//                      bias, requantisation (k and lambda live in registers for 32 filters with
//                      32-bit batch normalisation), one 32-byte store per 32 output channels
// More MMA warps or epilogue groups were measured and gained nothing.
// Every mbarrier wait is bounded (sm100_primitives.cuh).
#include "internal.cuh"
#include "sm100_primitives.cuh"

namespace pulpnn {

namespace {

using namespace sm100;

// Output rows (= tiles) per unit: the tiles and accumulators are handed from role to role a unit at a
// time (measured with 32 filters: one hand-over per tile 0.198 ms, per four tiles 0.163 ms), and two
// units are in flight, so a unit is as many tiles as half of tensor memory holds accumulators for.
__host__ __device__ constexpr int rows_out_of(int bn) { return bn == 32 ? 8 : 4; }
constexpr int NU = 2;              // units in flight: ring of 2 * rows_out im2col tiles = ring of accumulators
constexpr int NIN = 3;             // ring of input-row stages
constexpr int A_TILE_BYTES = 128 * 64;
// a warp needs about a thousand cycles to drain its quarter of an accumulator (tcgen05.ld, 32 x
// requantise, store: one dependent chain), so four groups keep four tiles in flight
constexpr int BUILD_WARPS = 4, MMA_WARPS = 2, EPI_GROUP_WARPS = 4, EPI_GROUPS_N = 2;
static_assert(NU % EPI_GROUPS_N == 0 && NU % MMA_WARPS == 0, "a ring slot must always meet the same warps");
constexpr int FIRST_BUILD = 1, FIRST_MMA = FIRST_BUILD + BUILD_WARPS, FIRST_EPILOGUE = FIRST_MMA + MMA_WARPS;
constexpr int THREADS = 32 * (FIRST_EPILOGUE + EPI_GROUP_WARPS * EPI_GROUPS_N);
constexpr int ST_C1_TMA = 0x1000, ST_C1_BUILD = 0x2000, ST_C1_MMA = 0x4000, ST_C1_EPI = 0x8000;

struct SmallTcParams {
  ConvProblem p;
  int row_bytes;       // W * Cin
  int stage_bytes;     // (3*SY+3) * row_bytes rounded up to 128
  int groups;          // units per image = ceil(Ho / ROWS_OUT)
  int units;           // B * groups
  int *status;
};

// byte offset of 16-byte chunk c of row r inside a K-major tile with 64-byte rows and the 64-byte
// swizzle (address bits 4..5 are XORed with bits 7..8)
__device__ __forceinline__ uint32_t swz64(int r, int c) { return (uint32_t)(r * 64 + ((c ^ ((r >> 1) & 3)) << 4)); }

__device__ __forceinline__ unsigned lds32(uint32_t addr)
{
  unsigned v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

template <int MODE, int SY, int BN>
__global__ void __launch_bounds__(THREADS, 1)
conv_smallcin_tc_kernel(const __grid_constant__ CUtensorMap map_in, const SmallTcParams g)
{
  constexpr int ROWS_OUT = rows_out_of(BN), NA = NU * ROWS_OUT;
  constexpr int ROWS_IN = (ROWS_OUT - 1) * SY + 3;
  constexpr uint32_t TMEM_COLS = NA * BN;                 // 512: all of tensor memory
  extern __shared__ uint8_t smem_raw[];
  uint8_t *sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t *a_ring = sm;                                   // NA tiles of 128 rows x 64 bytes
  uint8_t *w_tile = a_ring + NA * A_TILE_BYTES;           // BN rows x 64 bytes
  uint8_t *in_ring = w_tile + 4096;                       // NIN stages of input rows
  uint8_t *params = in_ring + NIN * g.stage_bytes;        // per-channel k / lambda / bias
  uint64_t *in_full = reinterpret_cast<uint64_t *>(params + BN * 16);
  uint64_t *in_empty = in_full + NIN;
  uint64_t *a_full = in_empty + NIN;
  uint64_t *a_empty = a_full + NU;
  uint64_t *t_full = a_empty + NU;
  uint64_t *t_empty = t_full + NU;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(t_empty + NU);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const ConvProblem &p = g.p;
  const Epilogue &e = p.epi;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int RB = p.kx * p.Cin;                            // bytes of one filter row (<= 9)

  if (tid == 0) {
    for (int s = 0; s < NIN; s++) { mbar_init(&in_full[s], 1); mbar_init(&in_empty[s], BUILD_WARPS); }
    // the im2col tiles and the accumulators are handed over a UNIT at a time: slot = unit % NU
    for (int s = 0; s < NU; s++) {
      mbar_init(&a_full[s], BUILD_WARPS); mbar_init(&a_empty[s], 1);
      mbar_init(&t_full[s], 1); mbar_init(&t_empty[s], EPI_GROUP_WARPS);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == FIRST_MMA) tmem_alloc(tmem_slot, TMEM_COLS);
  pdl_wait();                      // the set-up above may overlap the previous kernel's tail
  if (tid == 0) pdl_launch_dependents();
  // the im2col ring starts as zeros: chunk 3 of every row (and what lies past a filter row's bytes)
  // is never written again
  for (int idx = tid; idx < NA * A_TILE_BYTES / 16; idx += THREADS) sts128(smem_u32(a_ring) + idx * 16, 0u, 0u, 0u, 0u);
  if (tid < BN) {
    // filter tid, re-packed like an im2col row; per-channel parameters with the bias folded into
    // lambda: k*(acc+b)+lambda == k*acc + (k*b+lambda) in wrap-around arithmetic
    const int n = tid;
    const int8_t *wn = p.w + (size_t)n * 3 * RB;
#pragma unroll
    for (int fy = 0; fy < 3; fy++) {
      unsigned wd[3] = {0u, 0u, 0u};
#pragma unroll
      for (int t = 0; t < 9; t++)
        if (t < RB) wd[t >> 2] |= (unsigned)(uint8_t)__ldg(wn + fy * RB + t) << (8 * (t & 3));
      sts128(smem_u32(w_tile) + swz64(n, fy), wd[0], wd[1], wd[2], 0u);
    }
    sts128(smem_u32(w_tile) + swz64(n, 3), 0u, 0u, 0u, 0u);
    const int bias8 = (e.bias && MODE != EPI_RAW32) ? (int)__ldg(reinterpret_cast<const int8_t *>(e.bias) + n) : 0;
    if (MODE == EPI_BN32) {
      const int k = __ldg(reinterpret_cast<const int *>(e.k) + n);
      reinterpret_cast<int *>(params)[n] = k;
      reinterpret_cast<int *>(params)[BN + n] =
          (int)((unsigned)k * (unsigned)bias8 + (unsigned)__ldg(reinterpret_cast<const int *>(e.lambda) + n));
    } else if (MODE == EPI_BN64) {
      const long long k = __ldg(reinterpret_cast<const long long *>(e.k) + n);
      reinterpret_cast<long long *>(params)[n] = k;
      reinterpret_cast<long long *>(params)[BN + n] =
          (long long)((unsigned long long)k * (unsigned long long)(long long)bias8 +
                      (unsigned long long)__ldg(reinterpret_cast<const long long *>(e.lambda) + n));
    } else {
      reinterpret_cast<int *>(params)[n] = bias8;
    }
  }
  fence_proxy_async();            // the tensor cores read the tiles written above
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA: input rows of a unit ---------------------------------
    if (lane == 0) {
      int s = 0; uint32_t ph = 0; int issued = 0;
      for (int u = blockIdx.x; u < g.units; u += gridDim.x) {
        const int b = u / g.groups, gy = u - b * g.groups;
        if (!mbar_wait(&in_empty[s], ph ^ 1, abort_flag, g.status, ST_C1_TMA)) break;
        mbar_arrive_expect_tx(&in_full[s], (uint32_t)(ROWS_IN * g.row_bytes));
        tma_load_4d(in_ring + s * g.stage_bytes, &map_in, &in_full[s], 0, 0, gy * ROWS_OUT * SY - p.pt, b);
        issued++;
        if (++s == NIN) { s = 0; ph ^= 1; }
      }
      if (*abort_flag) {
        const int pending = issued < NIN ? issued : NIN;
        for (int i = 0; i < pending; i++) {
          if (--s < 0) { s = NIN - 1; ph ^= 1; }
          const unsigned long long t0 = global_ns();
          while (!mbar_try_wait(&in_full[s], ph))
            if (global_ns() - t0 > WAIT_LIMIT_NS) break;
        }
      }
    }
  } else if (warp < FIRST_MMA) {
    // ------------------------------ builders: thread = output column --------------------------
    const int ox = tid - 32 * FIRST_BUILD;
    const int ix0 = ox * p.sx - p.pl;                      // first column of the window
    const int o = ix0 * p.Cin;                             // its byte offset in an input row
    const int a = o & ~3;                                  // the aligned word it starts in
    const unsigned sh = (unsigned)(o & 3) * 8u;
    // bytes of the window that exist: columns inside the image, RB bytes in all
    int lo = (ix0 < 0 ? -ix0 : 0) * p.Cin;
    int hi = (p.W - ix0 < p.kx ? p.W - ix0 : p.kx) * p.Cin;
    if (hi < lo) hi = lo;
    unsigned m[3];
#pragma unroll
    for (int j = 0; j < 3; j++) {
      unsigned mm = 0;
#pragma unroll
      for (int t = 0; t < 4; t++)
        if (4 * j + t >= lo && 4 * j + t < hi) mm |= 0xffu << (8 * t);
      m[j] = mm;
    }
    bool wv[3];
#pragma unroll
    for (int j = 0; j < 3; j++) wv[j] = (a + 4 * j >= 0) && (a + 4 * j < g.row_bytes) && (m[0] | m[1] | m[2]) != 0;
    const uint32_t a_addr = smem_u32(a_ring), in_addr = smem_u32(in_ring);
    int s = 0; uint32_t ph = 0; int i = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < g.units && ok; u += gridDim.x) {
      if (!mbar_wait(&in_full[s], ph, abort_flag, g.status, ST_C1_BUILD)) break;
      unsigned x[ROWS_IN][3];
#pragma unroll
      for (int ri = 0; ri < ROWS_IN; ri++) {
        const uint32_t ra = in_addr + (uint32_t)(s * g.stage_bytes + ri * g.row_bytes + a);
        const unsigned w0 = wv[0] ? lds32(ra) : 0u, w1 = wv[1] ? lds32(ra + 4) : 0u, w2 = wv[2] ? lds32(ra + 8) : 0u;
        x[ri][0] = __funnelshift_r(w0, w1, sh) & m[0];
        x[ri][1] = __funnelshift_r(w1, w2, sh) & m[1];
        x[ri][2] = (w2 >> sh) & m[2];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&in_empty[s]);            // the stage has been read into registers
      if (++s == NIN) { s = 0; ph ^= 1; }
      // one hand-over per unit: wait for the unit's four tile slots, fill them, signal once
      const int us = i % NU;
      if (!mbar_wait(&a_empty[us], ((uint32_t)(i / NU) & 1u) ^ 1u, abort_flag, g.status, ST_C1_BUILD)) { ok = false; break; }
#pragma unroll
      for (int r = 0; r < ROWS_OUT; r++) {
        const uint32_t ta = a_addr + (us * ROWS_OUT + r) * A_TILE_BYTES;
#pragma unroll
        for (int fy = 0; fy < 3; fy++)
          sts128(ta + swz64(ox, fy), x[r * SY + fy][0], x[r * SY + fy][1], x[r * SY + fy][2], 0u);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_full[us]);
      i++;
    }
  } else if (warp < FIRST_EPILOGUE) {
    // ------------------------------ MMA issuers: alternate tiles -------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_u8s8(BN);
      const int me = warp - FIRST_MMA;
      const uint64_t db = umma_smem_desc<64>(smem_u32(w_tile));
      int i = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < g.units && ok; u += gridDim.x, i++) {
        if ((i & (MMA_WARPS - 1)) != me) continue;
        const int us = i % NU;                               // the unit's slot: four tiles, four accumulators
        const uint32_t par = (uint32_t)(i / NU) & 1u;
        if (!mbar_wait(&t_empty[us], par ^ 1, abort_flag, g.status, ST_C1_MMA)) { ok = false; break; }
        if (!mbar_wait(&a_full[us], par, abort_flag, g.status, ST_C1_MMA)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int r = 0; r < ROWS_OUT; r++) {
          const int slot = us * ROWS_OUT + r;
          const uint64_t da = umma_smem_desc<64>(smem_u32(a_ring) + slot * A_TILE_BYTES);
          const uint32_t d = tmem_base + (uint32_t)(slot * BN);
          umma_i8(d, da, db, idesc, 0u);
          umma_i8(d, da + 2, db + 2, idesc, 1u);            // K bytes 32..63: two 16-byte units further
        }
        umma_commit(&a_empty[us]);
        umma_commit(&t_full[us]);
      }
    }
  } else {
    // ------------------------------ epilogue: the groups take tiles in turn ---------------------
    const int grp = (warp - FIRST_EPILOGUE) / EPI_GROUP_WARPS;
    const int quad = warp & 3;                               // the TMEM lanes this warp may read
    const int ox = quad * 32 + lane;
    // 32 filters with 32-bit batch normalisation: k and lambda live in registers for the CTA's
    // lifetime, so a tile costs one multiply-add and one shift per output and no parameter loads
    constexpr bool REG_PARAMS = MODE == EPI_BN32 && BN == 32;
    int kr[32], lr[32];
    if (REG_PARAMS) {
#pragma unroll
      for (int j = 0; j < 32; j++) {
        kr[j] = reinterpret_cast<const int *>(params)[j];
        lr[j] = reinterpret_cast<const int *>(params)[BN + j];
      }
    }
    int i = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < g.units && ok; u += gridDim.x, i++) {
      if ((i & (EPI_GROUPS_N - 1)) != grp) continue;
      const int b = u / g.groups, gy = u - b * g.groups;
      const int us = i % NU;
      if (!mbar_wait(&t_full[us], (uint32_t)(i / NU) & 1u, abort_flag, g.status, ST_C1_EPI)) { ok = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int r = 0; r < ROWS_OUT; r++) {
        const int slot = us * ROWS_OUT + r;
        const int oy = gy * ROWS_OUT + r;
        const bool store = ox < p.Wo && oy < p.Ho;
        uint8_t *orow = reinterpret_cast<uint8_t *>(p.out) + (((size_t)b * p.Ho + (store ? oy : 0)) * p.Wo + (store ? ox : 0)) * BN;
        const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(slot * BN);
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t v[32];
          tmem_ld_32(t_row + (uint32_t)c0, v);
          tmem_wait_ld();
          unsigned w[8];
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            int q[4];
            if (REG_PARAMS) {
#pragma unroll
              for (int t = 0; t < 4; t++) q[t] = (int)((unsigned)kr[j + t] * v[j + t] + (unsigned)lr[j + t]) >> e.shift;
            } else if (MODE == EPI_BN32) {
              const int4 kk = *reinterpret_cast<const int4 *>(reinterpret_cast<const int *>(params) + c0 + j);
              const int4 ll = *reinterpret_cast<const int4 *>(reinterpret_cast<const int *>(params) + BN + c0 + j);
              q[0] = (int)((unsigned)kk.x * v[j + 0] + (unsigned)ll.x) >> e.shift;
              q[1] = (int)((unsigned)kk.y * v[j + 1] + (unsigned)ll.y) >> e.shift;
              q[2] = (int)((unsigned)kk.z * v[j + 2] + (unsigned)ll.z) >> e.shift;
              q[3] = (int)((unsigned)kk.w * v[j + 3] + (unsigned)ll.w) >> e.shift;
            } else {
#pragma unroll
              for (int t = 0; t < 4; t++) {
                const int acc = (int)v[j + t];
                if (MODE == EPI_BN64) {
                  const long long k = reinterpret_cast<const long long *>(params)[c0 + j + t];
                  const long long l = reinterpret_cast<const long long *>(params)[BN + c0 + j + t];
                  q[t] = (int)((long long)((unsigned long long)k * (unsigned long long)(long long)acc + (unsigned long long)l) >> e.shift);
                } else if (MODE == EPI_MULT) {
                  q[t] = (int)(short)((int)((unsigned)e.out_mult * (unsigned)(acc + reinterpret_cast<const int *>(params)[c0 + j + t])) >> e.shift);
                } else {
                  q[t] = (acc + reinterpret_cast<const int *>(params)[c0 + j + t]) >> e.shift;
                }
              }
            }
            w[j >> 2] = pack4_sat_u8(q[0], q[1], q[2], q[3]);
          }
          if (store)
            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                         ::"l"(orow + c0), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                         : "memory");
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&t_empty[us]);
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
int rows_in_of(int sy, int bn) { return (rows_out_of(bn) - 1) * sy + 3; }

template <int MODE, int SY, int BN>
bool launch_cfg(Context &c, const CUtensorMap &map, const SmallTcParams &g)
{
  auto kern = conv_smallcin_tc_kernel<MODE, SY, BN>;
  const size_t smem = 1024 + (size_t)NU * rows_out_of(BN) * A_TILE_BYTES + 4096 + (size_t)NIN * g.stage_bytes + BN * 16 + 512;
  if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
               "cudaFuncSetAttribute(conv_smallcin_tc)"))
    return false;
  const int sms = c.sm_count > 0 ? c.sm_count : 148;
  const int grid = g.units < sms ? g.units : sms;
  const cudaError_t le = launch_pdl(kern, dim3(grid), dim3(THREADS), smem, c.stream, map, g);
  count_launch("conv_smallcin_tc_kernel");
  return cuda_ok(le, "conv_smallcin_tc launch") && cuda_ok(cudaGetLastError(), "conv_smallcin_tc launch");
}

template <int MODE>
bool launch_mode(Context &c, const CUtensorMap &map, const SmallTcParams &g)
{
  const bool wide = g.p.Cout == 64;
  if (g.p.sy == 1) return wide ? launch_cfg<MODE, 1, 64>(c, map, g) : launch_cfg<MODE, 1, 32>(c, map, g);
  return wide ? launch_cfg<MODE, 2, 64>(c, map, g) : launch_cfg<MODE, 2, 32>(c, map, g);
}

}  // namespace

bool conv_smallcin_tc_supported(const ConvProblem &p)
{
  if (p.epi.mode == EPI_RAW32) return false;
  if (p.ky != 3 || p.kx * p.Cin > 9) return false;
  if (p.Cout != 32 && p.Cout != 64) return false;
  if (p.sy != 1 && p.sy != 2) return false;
  if (p.sx < 1 || p.Wo > 128) return false;
  const long long row_bytes = (long long)p.W * p.Cin;
  if (row_bytes % 16 != 0 || row_bytes / 16 > 256) return false;        // one TMA box spans whole rows
  if ((long long)rows_in_of(p.sy, p.Cout) * row_bytes > 24 * 1024) return false;
  if ((reinterpret_cast<uintptr_t>(p.in) & 15) || (reinterpret_cast<uintptr_t>(p.out) & 31)) return false;
  if ((long long)p.B * ((p.Ho + rows_out_of(p.Cout) - 1) / rows_out_of(p.Cout)) > 0x7fffffffLL) return false;
  return encode_tiled_fn() != nullptr;
}

bool launch_conv_smallcin_tc(Context &c, const ConvProblem &p)
{
  SmallTcParams g;
  g.p = p;
  g.row_bytes = p.W * p.Cin;
  g.stage_bytes = (rows_in_of(p.sy, p.Cout) * g.row_bytes + 127) & ~127;
  g.groups = (p.Ho + rows_out_of(p.Cout) - 1) / rows_out_of(p.Cout);
  g.units = p.B * g.groups;
  g.status = ctx_status_word(c);
  if (!g.status) return false;
  // the input as [B][H][row_bytes/piece][piece]: one box = all the pieces of rows_in rows. Pieces
  // of 32 bytes where the row allows it: the TMA unit fetches whole 32-byte sectors either way.
  const unsigned piece = g.row_bytes % 32 == 0 ? 32 : 16;
  CUtensorMap map;
  cuuint64_t dims[4] = {piece, (cuuint64_t)(g.row_bytes / piece), (cuuint64_t)p.H, (cuuint64_t)p.B};
  cuuint64_t strides[3] = {piece, (cuuint64_t)g.row_bytes, (cuuint64_t)p.H * g.row_bytes};
  cuuint32_t box[4] = {piece, (cuuint32_t)(g.row_bytes / piece), (cuuint32_t)rows_in_of(p.sy, p.Cout), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = encode_tiled_fn()(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<uint8_t *>(p.in), dims, strides, box,
                                       estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error(PULPNN_ERR_CUDA, "cuTensorMapEncodeTiled (first-layer input) failed with code %d", (int)r); return false; }
  switch (p.epi.mode) {
    case EPI_NONE: return launch_mode<EPI_NONE>(c, map, g);
    case EPI_MULT: return launch_mode<EPI_MULT>(c, map, g);
    case EPI_BN32: return launch_mode<EPI_BN32>(c, map, g);
    default:       return launch_mode<EPI_BN64>(c, map, g);
  }
}

}  // namespace pulpnn
