// igemm_tc.cu -- u8 x s8 -> s32 GEMM on the sm_100a tensor cores with the requantisation fused
// into the epilogue. It carries the convolutions and the fully connected layers:
//
//     D[m][n] = bias[n] + sum_k A[m][k] * W[n][k]      A: activations, [M][K] uint8, K contiguous
//                                                       W: weights,     [N][K] int8,  K contiguous
//
// The im2col matrix of a 1x1 convolution is the HWC activation tensor itself, and the reference
// keeps weights as [ch_out][ky][kx][ch_in] = [ch_out][K] (32bit/src/pulp_nn_matmul.c:55-59), so both
// operands are K-major exactly as they lie in memory. For a spatial kernel on a multiple of 32
// input channels the im2col matrix is never built: an m-tile is a patch of TH x TW = 128 output
// pixels, a K-slab is (filter tap, chunk of ch_in), and its A operand is one 4-D TMA box of the
// input image (element strides = the convolution's strides, out-of-range fill = the zero padding
// of 32bit/src/pulp_nn_conv_Ho_parallel.c:80-164).
//
// Structure of one CTA (24 warps, persistent over work units = (m-tile, n-tile, k-slice)):
//   warps 0..3, one lane each   TMA producers: a 128-row tile of A and a BN-row tile of W per
//                      pipeline stage, BKB bytes of K wide (32, 64 or 128, matching swizzle),
//                      completion on an mbarrier (no multicast). TMA fetches the whole box from L2
//                      even where it lies outside the tensor, so the box is never wider than K
//                      needs. When the CTA's n-tile of W fits beside four stages of A it is loaded
//                      ONCE per CTA and stays in shared memory; the CTA then keeps that n-tile and
//                      walks down the m-tiles, and the ring carries A only. A stage is always
//                      refilled by the same warp (stage % 4): getting one load on its way costs a
//                      thread several hundred cycles, more than a short-K tile has to spare.
//   warps 4..7, one lane each   issue tcgen05.mma.kind::i8 (M=128, N=BN, K=32 per instruction),
//                      operands from shared-memory descriptors, accumulator in tensor memory;
//                      commits free the stage and publish the accumulator. They alternate tiles
//                      (at most one warp per accumulator), ordered by a "tiles landed" counter.
//   warps 8..23        epilogue: tcgen05.ld the accumulator (lane = output row), requantise with
//                      per-channel k / lambda' (bias folded in) held in shared memory, pack to
//                      bytes. 128- and 256-column tiles go through a swizzled staging tile and
//                      leave with TMA stores (one, or two rounds of 128 columns; 4-D boxes for a
//                      convolution's patch); 64-column tiles, raw int32 output and partial sums are
//                      stored from registers. 64- and 128-column tiles are drained by two groups of
//                      eight warps that alternate tiles, 256-column tiles by all sixteen.
// All 512 columns of tensor memory are used as a ring of 512/BN accumulators, so the MMA issuers run
// several tiles ahead of the epilogue. Integer accumulation is associative, so splitting K over
// several CTAs (used when a problem has very few tiles) gives bit-identical sums; partial sums then
// go to a scratch buffer and a second kernel adds them and requantises. Rows of a short reduction
// (K <= 64, N <= 64) are folded two or more to a GEMM row against a block-diagonal copy of W (see
// launch_igemm_tc).
//
// Every wait on an mbarrier is bounded: after about a second the waiting thread raises a flag in
// shared memory, records a code in a global status word and all roles fall through to the common
// exit, which waits (bounded) for outstanding TMA writes and frees the tensor memory.
#include <cuda.h>
#include <cstdio>
#include <mutex>

#include "internal.cuh"
#include "sm100_primitives.cuh"

namespace pulpnn {

namespace {

using namespace sm100;

constexpr int BM = 128;            // rows per tile = TMEM lanes
constexpr int UMMA_K = 32;         // K per tcgen05.mma for 8-bit operands
constexpr int EPI_WARPS = 8;       // warps that drain one accumulator: two per TMEM lane quarter
constexpr int EPI_GROUPS = 2;      // groups of EPI_WARPS; group g drains the CTA's tiles g, g+2, ...
// One thread needs several hundred cycles to get a TMA load on its way, and a tcgen05.mma plus its
// commits is not much cheaper; with the short K of a pointwise layer that, not the memory system,
// bounded the whole kernel. So both jobs are shared out: producer warp w issues the loads of every
// NPROD-th slab of the CTA's slab sequence, MMA warp m the MMAs of every NMMA-th tile.
constexpr int NPROD = 4;
constexpr int NMMA = 4;            // at most one per accumulator of the ring
constexpr int FIRST_EPI = NPROD + NMMA;
constexpr int NUM_THREADS = 32 * (FIRST_EPI + EPI_WARPS * EPI_GROUPS);
constexpr int MAX_STAGES = 44;     // short-K stages are small: what counts is the bytes in flight
constexpr int PIPE_BYTES = 192 * 1024;   // operand ring (+ resident W) per CTA

// status codes (or-ed into the global status word)
constexpr int ST_PRODUCER = 0x1, ST_MMA_FULL = 0x2, ST_MMA_TMEM = 0x4, ST_EPILOGUE = 0x8, ST_DRAIN = 0x10,
              ST_MMA_WRES = 0x20;

// ---- kernel parameters ---------------------------------------------------------------------
struct TcParams {
  void *out;             // uint8 [M][N], int32 [M][N] (EPI_RAW32) or int32 partials [S][M][N]
  Epilogue epi;
  int M, N, K;
  int m_tiles, n_tiles, k_slices, slabs_per_slice, total_slabs;
  int vec_store;         // 2: 32-byte stores, 1: 16-byte stores, 0: scalar stores
  int w_resident;        // 1: the CTA's n-tile of W sits in shared memory for the CTA's lifetime
  int stationary;        // 1: a CTA keeps one n-tile (blockIdx % n_tiles) and walks down the m-tiles
  int n_stages;          // depth of the operand ring
  // Spatial convolution (conv = 1): an m-tile is a patch of TH x TW output pixels (TH * TW = 128,
  // TW = 1 << tw_log2) of one image, and the A operand of slab s = (filter tap, chunk of Cin) is
  // the 4-D TMA box of the input pixels that tap reads for the patch. Pixels outside the image
  // arrive as zeros from the TMA unit: the zero padding (32bit/src/pulp_nn_conv_Ho_parallel.c:80-164).
  int conv, tw_log2, tiles_x, tiles_y, chunks_per_tap, kx, sx, sy, pl, pt, Ho, Wo;
  int param_period;      // column n takes the per-channel parameters of channel n % param_period (folded rows)
  int *status;
  int ablate;            // measurement only (PULPNN_OPT_TUNE bits 8-10): 1 no epilogue work, 2 no operand loads, 4 no MMAs
};

// Timing trace of the first CTA (a build with -DPULPNN_TRACE only: never in the shipped library):
// role 0 the first producer warp, 1 the MMA warps, 2 the first epilogue warp; clock64 per tile and event.
#ifdef PULPNN_TRACE
__device__ long long g_trace[3][64][8];
#define PULPNN_TRACE_AT(role, tile, ev) \
  do { if (blockIdx.x == 0 && (tile) < 64) g_trace[role][tile][ev] = clock64(); } while (0)
// per launch (the last eight): globaltimer at the stations of block 0
__device__ long long g_ktrace[8][8];
__device__ int g_klaunch;
#define PULPNN_KTRACE(ev) \
  do { if (blockIdx.x == 0) g_ktrace[ktrace_slot & 7][ev] = (long long)global_ns(); } while (0)
#else
#define PULPNN_TRACE_AT(role, tile, ev) do {} while (0)
#define PULPNN_KTRACE(ev) do {} while (0)
#endif

// m-tile index of a convolution -> image and first output pixel of the patch
__device__ __forceinline__ void conv_patch(const TcParams &g, int mt, int &b, int &y0, int &x0)
{
  const int r = mt / g.tiles_x, tx = mt - r * g.tiles_x;
  b = r / g.tiles_y;
  const int ty = r - b * g.tiles_y;
  x0 = tx << g.tw_log2;
  y0 = ty << (7 - g.tw_log2);
}

// bytes of the operand ring (+ resident W). With TMA stores the epilogue stages one output tile
// per group of warps in shared memory, which the ring has to make room for.
__host__ __device__ constexpr int pipe_bytes(int bn, bool tma_out)
{
  if (tma_out && bn == 128) return 176 * 1024;
  return (bn == 256 && !tma_out) ? 208 * 1024 : PIPE_BYTES;      // 256-column tiles: four warps share a lane quarter, smaller copies
}

template <int BN_TILE, bool TMA_OUT>
struct SmemLayout {
  static constexpr int PIPE = pipe_bytes(BN_TILE, TMA_OUT);
  // every epilogue warp keeps its own copy of the k and lambda (up to 8 bytes each) of its columns
  static constexpr int WARP_PARAM_BYTES = BN_TILE / (BN_TILE == 256 ? 4 : 2) * 16;
  static constexpr int PARAM_OFFSET = PIPE;
  // staging tile of the TMA stores: 128 rows of at most 128 bytes, one per group of epilogue warps
  // (a 256-column tile is drained by all sixteen warps and leaves in two halves through one tile)
  static constexpr int OUT_ROW_BYTES = BN_TILE < 128 ? BN_TILE : 128;
  static constexpr int OUT_TILE_BYTES = TMA_OUT ? BM * OUT_ROW_BYTES : 0;
  static constexpr int OUT_OFFSET = PARAM_OFFSET + EPI_WARPS * EPI_GROUPS * WARP_PARAM_BYTES;
  static constexpr int BAR_OFFSET = OUT_OFFSET + (BN_TILE == 256 ? 1 : EPI_GROUPS) * OUT_TILE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 1024 + 1024;  // barriers + slack for 1024-byte alignment
  static_assert(TOTAL <= 232448, "shared memory of one CTA");
  // accumulators in tensor memory: all 512 columns are used, so a narrow tile gets a deep ring
  static constexpr int NUM_ACC = 512 / BN_TILE;
};

// The i-th work unit of this CTA. Stationary: n-tile fixed, m-tiles blockIdx/n_tiles, + gridDim/n_tiles, ...
// (so a resident slice of W serves every unit of the CTA). Otherwise units are dealt round robin.
__device__ __forceinline__ bool unit_at(const TcParams &g, int i, int units, int nt0, int m0, int m_step,
                                        int &nt, int &mt, int &ks);

// unit index -> (n-tile, m-tile, k-slice), n fastest. The common shapes (one n-tile, K not split)
// need no division at all, which matters in the epilogue where this runs once per tile.
__device__ __forceinline__ void decode_unit(const TcParams &g, int u, int &nt, int &mt, int &ks)
{
  int r = u;
  nt = 0;
  if (g.n_tiles != 1) { r = u / g.n_tiles; nt = u - r * g.n_tiles; }
  mt = r; ks = 0;
  if (g.k_slices != 1) { ks = r / g.m_tiles; mt = r - ks * g.m_tiles; }
}

__device__ __forceinline__ bool unit_at(const TcParams &g, int i, int units, int nt0, int m0, int m_step,
                                        int &nt, int &mt, int &ks)
{
  if (g.stationary) {
    nt = nt0; ks = 0;
    mt = m0 + i * m_step;
    return mt < g.m_tiles;
  }
  const int u = blockIdx.x + i * gridDim.x;
  if (u >= units) return false;
  decode_unit(g, u, nt, mt, ks);
  return true;
}

// MODE: the final epilogue; PARTIAL: store raw int32 partial sums instead (split-K); TMA_OUT: the
// uint8 output tile is staged in shared memory and leaves with one TMA store per tile
template <int MODE, int BN_TILE, int BKB, bool PARTIAL, bool TMA_OUT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
igemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_out, const TcParams g)
{
  using L = SmemLayout<BN_TILE, TMA_OUT>;
  static_assert(!TMA_OUT || (!PARTIAL && MODE != EPI_RAW32), "TMA stores carry uint8 tiles");
#ifdef PULPNN_TRACE
  __shared__ int ktrace_slot_s;
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    ktrace_slot_s = atomicAdd(&g_klaunch, 1);
    g_ktrace[ktrace_slot_s & 7][0] = (long long)global_ns();
  }
#endif
  constexpr int A_BYTES = BM * BKB, B_BYTES = BN_TILE * BKB;
  constexpr int NUM_ACC = L::NUM_ACC;
  constexpr uint32_t TMEM_COLS = 512;
  extern __shared__ uint8_t smem_raw[];
  // aligned by an offset, not by a cast, so that the compiler still knows this is shared memory
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t *params_all = smem + L::PARAM_OFFSET;
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + L::BAR_OFFSET);
  uint64_t *empty_bar = full_bar + MAX_STAGES;
  uint64_t *tmem_full = empty_bar + MAX_STAGES;
  uint64_t *tmem_empty = tmem_full + NUM_ACC;
  uint64_t *wres_bar = tmem_empty + NUM_ACC;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(wres_bar + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  volatile int *tiles_landed = abort_flag + 1;      // tiles whose operands have all arrived (MMA warps)
  volatile uint8_t *issued_parity = reinterpret_cast<volatile uint8_t *>(tiles_landed + 1);   // per stage: 1 + parity of its last load

  // operand ring: [resident W: total_slabs * B_BYTES][stage 0][stage 1]...
  const int wres_bytes = g.w_resident ? g.total_slabs * B_BYTES : 0;
  const int stage_bytes = g.w_resident ? A_BYTES : A_BYTES + B_BYTES;
  uint8_t *ring = smem + wres_bytes;
  const int n_stages = g.n_stages;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // stationary CTAs: n-tile and first m-tile of this CTA, distance between its m-tiles
  const int nt0 = g.stationary ? (int)(blockIdx.x % (unsigned)g.n_tiles) : 0;
  const int m0 = g.stationary ? (int)(blockIdx.x / (unsigned)g.n_tiles) : 0;
  const int m_step = g.stationary ? (int)(gridDim.x / (unsigned)g.n_tiles) : 0;

  // the ring's barriers are set up by one thread each (the set-up is not hidden behind the previous kernel: two
  // launches of this kernel cannot share an SM), thread 0 only does what its early weight fetch needs
  if (threadIdx.x >= 32 && threadIdx.x < 32 + MAX_STAGES) {
    const int s = threadIdx.x - 32;
    if (s < g.n_stages) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    issued_parity[s] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (threadIdx.x == 0) {
    // an accumulator is free again once every warp that drains it has arrived (see the epilogue)
    for (int b = 0; b < NUM_ACC; b++) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], BN_TILE == 256 ? 16 : 8); }
    mbar_init(wres_bar, 1);
    *abort_flag = 0;
    *tiles_landed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    // The resident slice of W is fetched right away, before the wait on the previous kernel:
    // weights are constants that no kernel of this library writes after the layer was set up (a
    // block-diagonal copy is made by an ordinary launch, which this kernel cannot overtake), so the
    // fetch may overlap the previous kernel's tail.
    if (g.w_resident) {
      mbar_arrive_expect_tx(wres_bar, (uint32_t)wres_bytes);
      for (int s = 0; s < g.total_slabs; s++) tma_load_2d(smem + s * B_BYTES, &map_b, wres_bar, s * BKB, nt0 * BN_TILE);
    }
  }
  if (warp == NPROD) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
#ifdef PULPNN_TRACE
  const int ktrace_slot = blockIdx.x == 0 ? ktrace_slot_s : 0;
#endif
  if (threadIdx.x == 0) PULPNN_KTRACE(1);
  // everything above overlapped the tail of the previous kernel; nothing below may
  pdl_wait();
  if (threadIdx.x == 0) PULPNN_KTRACE(2);
  if (threadIdx.x == 0) pdl_launch_dependents();

  const int units = g.m_tiles * g.n_tiles * g.k_slices;

  if (warp < NPROD) {
    // ------------------------------ TMA producers -------------------------------------------
    // The CTA's slabs, over all its units, use the stages of the ring in turn. A stage is always
    // refilled by the same warp (stage % NPROD): its parity wait on the stage's "empty" barrier is
    // only meaningful because it has itself seen every earlier round of that stage.
    if (lane == 0) {
      int st = 0; uint32_t ph = 0;           // ring position of the current slab
      bool ok = true;
      for (int i = 0; ok; i++) {
        int nt, mt, ks;
        if (!unit_at(g, i, units, nt0, m0, m_step, nt, mt, ks)) break;
        const int slab0 = ks * g.slabs_per_slice;
        const int slab1 = min(slab0 + g.slabs_per_slice, g.total_slabs);
        int cb = 0, cy = 0, cx = 0;             // convolution: image and first input pixel of the patch
        if (g.conv) {
          conv_patch(g, mt, cb, cy, cx);
          cy = cy * g.sy - g.pt;
          cx = cx * g.sx - g.pl;
        }
        for (int s = slab0; s < slab1; s++) {
          if ((st & (NPROD - 1)) == warp) {
            if (!mbar_wait(&empty_bar[st], ph ^ 1, abort_flag, g.status, ST_PRODUCER)) { ok = false; break; }
            if (warp == 0 && s == slab0) PULPNN_TRACE_AT(0, i, 0);
            uint8_t *a_dst = ring + st * stage_bytes;
            if (g.ablate & 2) { mbar_arrive(&full_bar[st]); issued_parity[st] = (uint8_t)(1u + ph); goto next_slab; }
            mbar_arrive_expect_tx(&full_bar[st], (uint32_t)stage_bytes);
            if (g.conv) {
              const int tap = s / g.chunks_per_tap, chunk = s - tap * g.chunks_per_tap;
              const int fy = tap / g.kx, fx = tap - fy * g.kx;
              tma_load_4d(a_dst, &map_a, &full_bar[st], chunk * BKB, cx + fx, cy + fy, cb);
            } else {
              tma_load_2d(a_dst, &map_a, &full_bar[st], s * BKB, mt * BM);
            }
            if (!g.w_resident) tma_load_2d(a_dst + A_BYTES, &map_b, &full_bar[st], s * BKB, nt * BN_TILE);
            issued_parity[st] = (uint8_t)(1u + ph);
            if (warp == 0 && s == slab0) PULPNN_TRACE_AT(0, i, 1);
          }
        next_slab:
          if (++st == n_stages) { st = 0; ph ^= 1; }
        }
      }
      if (*abort_flag) {
        // something gave up: make sure none of this warp's TMA writes is still in flight into the
        // CTA's memory (the last load into each of its stages)
        for (int s2 = warp; s2 < n_stages; s2 += NPROD) {
          if (issued_parity[s2] == 0) continue;
          const uint32_t par = (uint32_t)issued_parity[s2] - 1u;
          const unsigned long long t0 = global_ns();
          while (!mbar_try_wait(&full_bar[s2], par)) {
            if (global_ns() - t0 > WAIT_LIMIT_NS) { if (g.status) atomicOr(g.status, ST_DRAIN); break; }
          }
        }
        if (warp == 0 && g.w_resident) {
          const unsigned long long t0 = global_ns();
          while (!mbar_try_wait(wres_bar, 0)) {
            if (global_ns() - t0 > WAIT_LIMIT_NS) { if (g.status) atomicOr(g.status, ST_DRAIN); break; }
          }
        }
      }
    }
  } else if (warp < FIRST_EPI) {
    // ------------------------------ MMA issuers ---------------------------------------------
    // tile i of the CTA (accumulator i % NUM_ACC) belongs to MMA warp i % NMMA
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_u8s8(BN_TILE);
      // an accumulator must always be filled by the same MMA warp: no more warps than accumulators
      constexpr int NM = NMMA < NUM_ACC ? NMMA : NUM_ACC;
      static_assert(NUM_ACC % NM == 0, "an accumulator must always be filled by the same MMA warp");
      const int me = warp - NPROD;
      int st_next = 0; uint32_t ph_next = 0;      // ring position of the next tile's first slab
      bool ok = me < NM;
      if (ok && g.w_resident) ok = mbar_wait(wres_bar, 0, abort_flag, g.status, ST_MMA_WRES);
      for (int i = 0; ok; i++) {
        int nt, mt, ks;
        if (!unit_at(g, i, units, nt0, m0, m_step, nt, mt, ks)) break;
        (void)nt; (void)mt;
        const int slab0 = ks * g.slabs_per_slice;
        const int slab1 = min(slab0 + g.slabs_per_slice, g.total_slabs);
        int stage = st_next;
        uint32_t phase = ph_next;
        st_next += slab1 - slab0;
        while (st_next >= n_stages) { st_next -= n_stages; ph_next ^= 1; }
        if ((i & (NM - 1)) != me) continue;
        // A parity wait is only meaningful while the waiter is less than one round of the ring
        // ahead of the barrier. The other MMA warp owns the previous tile, so this one may not
        // look at a stage's barrier before everything up to that tile has arrived.
        if (NMMA > 1 && i > 0) {
          unsigned long long t0 = 0;
          for (unsigned spin = 1; *tiles_landed < i; spin++) {
            if ((spin & 255u) == 0) {
              if (*abort_flag) { ok = false; break; }
              if (t0 == 0) t0 = global_ns();
              else if (global_ns() - t0 > WAIT_LIMIT_NS) {
                *abort_flag = 1;
                if (g.status) atomicOr(g.status, ST_MMA_FULL);
                ok = false;
                break;
              }
            }
          }
          if (!ok) break;
        }
        const int acc = i % NUM_ACC;
        const uint32_t acc_phase = (uint32_t)(i / NUM_ACC) & 1u;
        PULPNN_TRACE_AT(1, i, 0);
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, g.status, ST_MMA_TMEM)) break;
        PULPNN_TRACE_AT(1, i, 1);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN_TILE);
        for (int s = slab0; s < slab1; s++) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, g.status, ST_MMA_FULL)) { ok = false; break; }
          if (s - slab0 < 4) PULPNN_TRACE_AT(1, i, 2 + s - slab0);
          if (i == 0 && s == slab0) PULPNN_KTRACE(3);
          if (NMMA > 1 && s == slab1 - 1) *tiles_landed = i + 1;    // the next tile's warp may go ahead
          tc_fence_after();
          const uint32_t a_addr = smem_u32(ring + stage * stage_bytes);
          const uint32_t b_addr = g.w_resident ? smem_u32(smem + s * B_BYTES) : a_addr + A_BYTES;
          const uint64_t da = umma_smem_desc<BKB>(a_addr), db = umma_smem_desc<BKB>(b_addr);
          // bytes of this slab that lie inside K; the rest of the tile is zero-filled by TMA
          const int kbytes = min(BKB, g.K - s * BKB);
          const int n_mma = (kbytes + UMMA_K - 1) / UMMA_K;
          for (int j = 0; j < n_mma; j++) {
            if (g.ablate & 4) break;
            // advancing K inside the swizzle atom = advancing the start address (16-byte units)
            const uint64_t adv = (uint64_t)((j * UMMA_K) >> 4);
            umma_i8(d_tmem, da + adv, db + adv, idesc, (s > slab0 || j > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);      // stage reusable once these MMAs have read it
          if (++stage == n_stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tmem_full[acc]);          // accumulator complete
        PULPNN_TRACE_AT(1, i, 6);
        if (i == 0) PULPNN_KTRACE(4);
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------------------------
    // A warp may only read the 32 TMEM lanes 32*(warp%4)..+31. NSPLIT warps share each lane quarter
    // of a tile and deal its 32-column chunks out among them. A 256-column tile takes all sixteen
    // warps (there are only two accumulators, so the sooner one is drained the better); narrower
    // tiles take eight, and the two groups of eight alternate tiles.
    constexpr int NSPLIT = BN_TILE == 256 ? 4 : 2;
    constexpr int GROUPS = EPI_WARPS * EPI_GROUPS / (4 * NSPLIT);
    const int quad = warp & 3;
    const int half = ((warp - FIRST_EPI) >> 2) % NSPLIT;      // which share of the chunks
    const int grp = (warp - FIRST_EPI) / (4 * NSPLIT);
    constexpr int HALF_COLS = BN_TILE / NSPLIT;     // columns this warp is responsible for
    // each epilogue warp keeps its own copy of the per-channel parameters of ITS columns, so
    // staging them needs no barrier between warps (a warp that gave up can never strand the others)
    uint8_t *params = params_all + (warp - FIRST_EPI) * L::WARP_PARAM_BYTES;
    static_assert(NUM_ACC % GROUPS == 0, "a group must always meet the same accumulators");
    const Epilogue &e = g.epi;
    int *p_bias = reinterpret_cast<int *>(params);                 // non-BN modes
    int *p_k32 = reinterpret_cast<int *>(params);                  // EPI_BN32: k, lambda'
    int *p_l32 = p_k32 + HALF_COLS;
    long long *p_k64 = reinterpret_cast<long long *>(params);      // EPI_BN64
    long long *p_l64 = p_k64 + HALF_COLS;
    int staged_nt = -1;
    // TMA_OUT: the group's staging tile, and the one thread of the group that issues its stores
    uint8_t *out_tile = smem + L::OUT_OFFSET + grp * L::OUT_TILE_BYTES;
    const bool elected = ((warp - FIRST_EPI) % (4 * NSPLIT)) == 0 && lane == 0;
    constexpr int GROUP_THREADS = 32 * 4 * NSPLIT;       // threads that meet at the group's barrier
    bool dead = false;      // TMA_OUT: a wait ran out; keep meeting the group's barriers, do no work
    // i counts the CTA's tiles; tile i lives in accumulator i % NUM_ACC
    for (int i = grp;; i += GROUPS) {
      int nt, mt, ks;
      if (!unit_at(g, i, units, nt0, m0, m_step, nt, mt, ks)) break;
      const int acc = i % NUM_ACC;
      const uint32_t acc_phase = (uint32_t)(i / NUM_ACC) & 1u;
      const int n0 = nt * BN_TILE;
      if (!PARTIAL && nt != staged_nt) {
        // per-channel parameters of this warp's columns -> shared memory. The bias is folded into
        // lambda: k*(acc+b)+lambda == k*acc + (k*b+lambda) in wrap-around arithmetic.
        // Local slot i holds column (i/32)*32*NSPLIT + half*32 + i%32 of the tile.
        __syncwarp();
        for (int i = lane; i < HALF_COLS; i += 32) {
          const int col = n0 + (i >> 5) * (32 * NSPLIT) + half * 32 + (i & 31);
          const bool v = col < g.N;
          const int n = g.param_period == g.N ? col : col % g.param_period;
          if (MODE == EPI_BN32) {
            const int k = v ? __ldg(reinterpret_cast<const int *>(e.k) + n) : 0;
            const int l = v ? __ldg(reinterpret_cast<const int *>(e.lambda) + n) : 0;
            const int b = (v && e.bias) ? (int)__ldg(reinterpret_cast<const int8_t *>(e.bias) + n) : 0;
            p_k32[i] = k;
            p_l32[i] = (int)((unsigned)k * (unsigned)b + (unsigned)l);
          } else if (MODE == EPI_BN64) {
            const long long k = v ? __ldg(reinterpret_cast<const long long *>(e.k) + n) : 0;
            const long long l = v ? __ldg(reinterpret_cast<const long long *>(e.lambda) + n) : 0;
            const long long b = (v && e.bias) ? (long long)__ldg(reinterpret_cast<const int8_t *>(e.bias) + n) : 0;
            p_k64[i] = k;
            p_l64[i] = (long long)((unsigned long long)k * (unsigned long long)b + (unsigned long long)l);
          } else if (MODE == EPI_RAW32) {
            p_bias[i] = (v && e.bias) ? __ldg(reinterpret_cast<const int *>(e.bias) + n) : 0;
          } else {
            p_bias[i] = (v && e.bias) ? (int)__ldg(reinterpret_cast<const int8_t *>(e.bias) + n) : 0;
          }
        }
        __syncwarp();
        staged_nt = nt;
      }
      if constexpr (TMA_OUT) {
        // requantised bytes of this warp's columns, 8 words per 32-column chunk
        constexpr int NCHUNK = HALF_COLS / 32;
        unsigned w[NCHUNK][8];
        if (warp == FIRST_EPI && lane == 0) PULPNN_TRACE_AT(2, i, 0);
        if (!dead && !mbar_wait(&tmem_full[acc], acc_phase, abort_flag, g.status, ST_EPILOGUE)) dead = true;
        if (warp == FIRST_EPI && lane == 0) PULPNN_TRACE_AT(2, i, 1);
        if (warp == FIRST_EPI && lane == 0 && i == 0) PULPNN_KTRACE(5);
        if (!dead && (g.ablate & 1)) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[acc]);
          continue;
        }
        // The tile leaves in rounds of at most 128 columns (one round, or two for 256 columns), and a round's
        // chunks are fetched from tensor memory and requantised right before it: the arithmetic of the NEXT round
        // (or tile) then runs while the TMA store of this one reads the staging tile, so the wait at (A) finds the
        // store done (measured on 14x14x512 -> 512: the two rounds used to wait 500-700 cycles each).
        constexpr int ROUNDS = BN_TILE == 256 ? 2 : 1;
        constexpr int CPR = NCHUNK / ROUNDS;                 // 32-column chunks of this warp per round
        if (!dead) tc_fence_after();
        const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN_TILE);
#pragma unroll
        for (int rd = 0; rd < ROUNDS; rd++) {
          if (!dead) {
#pragma unroll
            for (int cr = 0; cr < CPR; cr++) {
              const int ch = rd * CPR + cr;
              const int lc = ch * 32, c0 = ch * (32 * NSPLIT) + half * 32;
              uint32_t v[32];
              tmem_ld_32(t_row + (uint32_t)c0, v);
              tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                int q[4];
                if (MODE == EPI_BN32) {
                  const int4 kk = *reinterpret_cast<const int4 *>(p_k32 + lc + j);
                  const int4 ll = *reinterpret_cast<const int4 *>(p_l32 + lc + j);
                  q[0] = (int)((unsigned)kk.x * v[j + 0] + (unsigned)ll.x) >> e.shift;
                  q[1] = (int)((unsigned)kk.y * v[j + 1] + (unsigned)ll.y) >> e.shift;
                  q[2] = (int)((unsigned)kk.z * v[j + 2] + (unsigned)ll.z) >> e.shift;
                  q[3] = (int)((unsigned)kk.w * v[j + 3] + (unsigned)ll.w) >> e.shift;
                } else {
#pragma unroll
                  for (int t = 0; t < 4; t++) {
                    const int a = (int)v[j + t];
                    if (MODE == EPI_BN64)
                      q[t] = (int)((long long)((unsigned long long)p_k64[lc + j + t] * (unsigned long long)(long long)a +
                                               (unsigned long long)p_l64[lc + j + t]) >> e.shift);
                    else if (MODE == EPI_MULT)
                      q[t] = (int)(short)((int)((unsigned)e.out_mult * (unsigned)(a + p_bias[lc + j + t])) >> e.shift);
                    else
                      q[t] = (a + p_bias[lc + j + t]) >> e.shift;
                  }
                }
                w[ch][j >> 2] = pack4_sat_u8(q[0], q[1], q[2], q[3]);
              }
            }
            if (rd == ROUNDS - 1) {
              // the accumulator is in registers: hand it back to the MMA warps before the stores
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&tmem_empty[acc]);
              if (warp == FIRST_EPI && lane == 0) PULPNN_TRACE_AT(2, i, 2);
            }
          }
          // (A) the previous store from the staging tile has finished reading it
          if (elected) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "n"(GROUP_THREADS) : "memory");
          if (warp == FIRST_EPI && lane == 0) PULPNN_TRACE_AT(2, i, 3 + 2 * rd);
          if (!dead) {
            // row r of the staging tile, 16-byte chunks cc, cc+1 of each 32-column chunk, swizzled
            // the way the TMA store expects (rows of OUT_ROW_BYTES with the matching swizzle): no
            // bank conflicts
            const int r = quad * 32 + lane;
            const uint32_t rowaddr = smem_u32(out_tile) + (uint32_t)(r * L::OUT_ROW_BYTES);
            const int x = L::OUT_ROW_BYTES == 128 ? (r & 7) : ((r >> 1) & 3);
#pragma unroll
            for (int cr = 0; cr < CPR; cr++) {
              const int ch = rd * CPR + cr;
              const int cc = ((ch * (32 * NSPLIT) + half * 32) - rd * 128) >> 4;
              sts128(rowaddr + (uint32_t)(((cc) ^ x) << 4), w[ch][0], w[ch][1], w[ch][2], w[ch][3]);
              sts128(rowaddr + (uint32_t)(((cc + 1) ^ x) << 4), w[ch][4], w[ch][5], w[ch][6], w[ch][7]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          }
          // (B) the round's columns are complete
          asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "n"(GROUP_THREADS) : "memory");
          if (elected && !dead) {
            // rows past M (pixels past the image's edge), columns past N are dropped
            if (g.conv) {
              int cb, cy, cx;
              conv_patch(g, mt, cb, cy, cx);
              tma_store_4d(&map_out, out_tile, n0 + rd * 128, cx, cy, cb);
            } else {
              tma_store_2d(&map_out, out_tile, n0 + rd * 128, mt * BM);
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          if (warp == FIRST_EPI && lane == 0) PULPNN_TRACE_AT(2, i, 4 + 2 * rd);
        }
        continue;
      }
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, g.status, ST_EPILOGUE)) break;
      tc_fence_after();
      int m = mt * BM + quad * 32 + lane;
      bool row_ok = m < g.M;
      if (g.conv) {        // row of the tile -> pixel of the patch -> row of the output
        int cb, cy, cx;
        conv_patch(g, mt, cb, cy, cx);
        const int r = quad * 32 + lane;
        cy += r >> g.tw_log2;
        cx += r & ((1 << g.tw_log2) - 1);
        row_ok = cy < g.Ho && cx < g.Wo;
        m = (cb * g.Ho + cy) * g.Wo + cx;
      }
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN_TILE);
#pragma unroll 1
      for (int lc = 0; lc < HALF_COLS; lc += 32) {   // lc: offset inside this warp's parameter copy
        const int c0 = (lc >> 5) * (32 * NSPLIT) + half * 32;   // column offset inside the tile
        if (n0 + c0 >= g.N) break;                   // uniform across the warp
        uint32_t v[32];
        tmem_ld_32(t_row + (uint32_t)c0, v);
        tmem_wait_ld();
        if (PARTIAL || MODE == EPI_RAW32) {
          int *orow = reinterpret_cast<int *>(g.out) +
                      ((size_t)(PARTIAL ? ks : 0) * g.M + (size_t)(row_ok ? m : 0)) * g.N + n0 + c0;
          if (row_ok) {
            if (g.vec_store) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                if (n0 + c0 + i < g.N) {
                  int4 o;
                  o.x = (int)v[i]; o.y = (int)v[i + 1]; o.z = (int)v[i + 2]; o.w = (int)v[i + 3];
                  if (!PARTIAL) {
                    const int4 bb = *reinterpret_cast<const int4 *>(p_bias + lc + i);
                    o.x += bb.x; o.y += bb.y; o.z += bb.z; o.w += bb.w;
                  }
                  *reinterpret_cast<int4 *>(orow + i) = o;
                }
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; i++)
                if (n0 + c0 + i < g.N) orow[i] = (int)v[i] + (PARTIAL ? 0 : p_bias[lc + i]);
            }
          }
        } else {
          unsigned w[8];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            int q[4];
            if (MODE == EPI_BN32) {
              const int4 kk = *reinterpret_cast<const int4 *>(p_k32 + lc + i);
              const int4 ll = *reinterpret_cast<const int4 *>(p_l32 + lc + i);
              q[0] = (int)((unsigned)kk.x * v[i + 0] + (unsigned)ll.x) >> e.shift;
              q[1] = (int)((unsigned)kk.y * v[i + 1] + (unsigned)ll.y) >> e.shift;
              q[2] = (int)((unsigned)kk.z * v[i + 2] + (unsigned)ll.z) >> e.shift;
              q[3] = (int)((unsigned)kk.w * v[i + 3] + (unsigned)ll.w) >> e.shift;
            } else {
#pragma unroll
              for (int j = 0; j < 4; j++) {
                const int a = (int)v[i + j];
                if (MODE == EPI_BN64)
                  q[j] = (int)((long long)((unsigned long long)p_k64[lc + i + j] * (unsigned long long)(long long)a +
                                           (unsigned long long)p_l64[lc + i + j]) >> e.shift);
                else if (MODE == EPI_MULT)
                  q[j] = (int)(short)((int)((unsigned)e.out_mult * (unsigned)(a + p_bias[lc + i + j])) >> e.shift);
                else
                  q[j] = (a + p_bias[lc + i + j]) >> e.shift;
              }
            }
            w[i >> 2] = pack4_sat_u8(q[0], q[1], q[2], q[3]);
          }
          if (row_ok) {
            uint8_t *orow = reinterpret_cast<uint8_t *>(g.out) + (size_t)m * g.N + n0 + c0;
            if (g.vec_store == 2) {
              // one full 32-byte sector per lane and instruction
              asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                           ::"l"(orow), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]),
                             "r"(w[6]), "r"(w[7])
                           : "memory");
            } else if (g.vec_store == 1) {
              if (n0 + c0 < g.N) *reinterpret_cast<uint4 *>(orow) = make_uint4(w[0], w[1], w[2], w[3]);
              if (n0 + c0 + 16 < g.N) *reinterpret_cast<uint4 *>(orow + 16) = make_uint4(w[4], w[5], w[6], w[7]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; i++)
                if (n0 + c0 + i < g.N) orow[i] = (uint8_t)(w[i >> 2] >> (8 * (i & 3)));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
    // the staging tiles must outlive the stores that read them
    // (only until they have READ it: the writes themselves are complete, and visible to the next kernel
    // in the stream, when the grid is: no thread of this kernel reads them back)
    if (TMA_OUT && elected) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    if (warp == FIRST_EPI && lane == 0) PULPNN_KTRACE(6);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == NPROD) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
    if (lane == 0) PULPNN_KTRACE(7);
  }
}

// ---- split-K reduction: sums the int32 partials, adds the bias and requantises ---------------
template <int MODE>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const int *partials, void *out, Epilogue e,
                                                            int M, int N, int S)
{
  const size_t total = (size_t)M * N;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int n = (int)(i % N);
    int acc = 0;
    for (int s = 0; s < S; s++) acc += __ldg(partials + (size_t)s * total + i);
    if (MODE == EPI_RAW32) {
      if (e.bias) acc += __ldg(reinterpret_cast<const int *>(e.bias) + n);
      reinterpret_cast<int *>(out)[i] = acc;
    } else {
      if (e.bias) acc += (int)__ldg(reinterpret_cast<const int8_t *>(e.bias) + n);
      reinterpret_cast<uint8_t *>(out)[i] = (uint8_t)requant<MODE>(acc, n, e);
    }
  }
}

// ---- host side -------------------------------------------------------------------------------
// [rows][K] byte matrix, K contiguous; box = bkb bytes of K x box_rows rows, bkb-byte swizzle.
// Elements outside the matrix read as zero.
bool make_map(CUtensorMap *map, const void *base, int rows, int K, int box_rows, int bkb)
{
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) { set_error(PULPNN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver"); return false; }
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K};
  cuuint32_t box[2] = {(cuuint32_t)bkb, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = bkb == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                              : (bkb == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error(PULPNN_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r); return false; }
  return true;
}

// W [N][K] -> block-diagonal [fold*N][fold*K] (block (p, p) = W, zeros elsewhere), 16 bytes per thread
__global__ void fold_weights_kernel(const int8_t *w, int8_t *wf, int N, int K, int fold)
{
  const int chunks = K * fold / 16;                       // 16-byte chunks per folded row
  const long long total = (long long)N * fold * chunks;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(i / chunks), ch = (int)(i - (long long)row * chunks);
    const int pblk = row / N, n = row - pblk * N;
    const int kk = ch * 16, qblk = kk / K, k = kk - qblk * K;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (pblk == qblk) v = __ldg(reinterpret_cast<const uint4 *>(w + (size_t)n * K + k));
    *reinterpret_cast<uint4 *>(wf + (size_t)row * K * fold + kk) = v;
  }
}

// [B][H][W][C] image, boxes of box_c bytes x box_w x box_h pixels of one image, every sx-th (sy-th)
// pixel of the box taken: the pixels one filter tap reads for a patch of outputs
bool make_map_4d(CUtensorMap *map, const void *base, int C, int Wd, int Hd, int B, int box_c, int box_w, int box_h,
                 int sx, int sy)
{
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) { set_error(PULPNN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver"); return false; }
  cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)Wd, (cuuint64_t)Hd, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)C, (cuuint64_t)Wd * C, (cuuint64_t)Hd * Wd * C};
  cuuint32_t box[4] = {(cuuint32_t)box_c, (cuuint32_t)((box_w - 1) * sx + 1), (cuuint32_t)((box_h - 1) * sy + 1), 1};
  cuuint32_t estr[4] = {1, (cuuint32_t)sx, (cuuint32_t)sy, 1};
  const CUtensorMapSwizzle sw = box_c == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                              : (box_c == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error(PULPNN_ERR_CUDA, "cuTensorMapEncodeTiled (4-D) failed with code %d", (int)r); return false; }
  return true;
}

// patch width (a power of two, the patch has 128 pixels) that covers the output with the fewest
// wasted pixels; the wider one on a tie
int pick_patch_width_log2(int Ho, int Wo, int sx, int sy)
{
  int best = -1;
  long long best_cost = 0;
  for (int l = 3; l <= 7; l++) {
    const int tw = 1 << l, th = 128 >> l;
    if ((tw - 1) * sx + 1 > 256 || (th - 1) * sy + 1 > 256) continue;
    const long long cost = (long long)((Wo + tw - 1) / tw) * ((Ho + th - 1) / th);
    if (best < 0 || cost <= best_cost) { best = l; best_cost = cost; }
  }
  return best;
}

// the three tensor maps of a launch (the output map only matters with TMA stores)
struct TcMaps { CUtensorMap a, b, out; };

template <int MODE, int BN_TILE, int BKB, bool PARTIAL, bool TMA_OUT>
bool launch_cfg(Context &c, const TcMaps &m, const TcParams &g, int grid)
{
  using L = SmemLayout<BN_TILE, TMA_OUT>;
  auto kern = igemm_tc_kernel<MODE, BN_TILE, BKB, PARTIAL, TMA_OUT>;
  static PerDeviceInt attr_set;     // per instantiation and device
  if (!attr_set.get(c.device)) {
    if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL),
                 "cudaFuncSetAttribute(igemm_tc)"))
      return false;
    attr_set.set(c.device, 1);
  }
  // every configuration asks for more than half of an SM's shared memory, so exactly one CTA (and
  // its 512 tensor-memory columns) lives on an SM
  const cudaError_t le = launch_pdl(kern, dim3(grid), dim3(NUM_THREADS), L::TOTAL, c.stream, m.a, m.b, m.out, g);
  count_launch("igemm_tc_kernel");
  return cuda_ok(le, "igemm_tc launch") && cuda_ok(cudaGetLastError(), "igemm_tc launch");
}

template <int MODE, int BN_TILE, bool PARTIAL, bool TMA_OUT>
bool launch_bk(Context &c, const TcMaps &m, const TcParams &g, int bkb, int grid)
{
  if (bkb == 32) return launch_cfg<MODE, BN_TILE, 32, PARTIAL, TMA_OUT>(c, m, g, grid);
  if (bkb == 64) return launch_cfg<MODE, BN_TILE, 64, PARTIAL, TMA_OUT>(c, m, g, grid);
  return launch_cfg<MODE, BN_TILE, 128, PARTIAL, TMA_OUT>(c, m, g, grid);
}

template <int MODE, bool PARTIAL>
bool launch_bn(Context &c, const TcMaps &m, const TcParams &g, int bn, int bkb, int grid, bool tma_out)
{
  if constexpr (!PARTIAL && MODE != EPI_RAW32) {
    if (tma_out && bn == 64)  return launch_bk<MODE, 64, false, true>(c, m, g, bkb, grid);
    if (tma_out && bn == 128) return launch_bk<MODE, 128, false, true>(c, m, g, bkb, grid);
    if (tma_out && bn == 256) return launch_bk<MODE, 256, false, true>(c, m, g, bkb, grid);
  }
  if (bn == 64)  return launch_bk<MODE, 64, PARTIAL, false>(c, m, g, bkb, grid);
  if (bn == 128) return launch_bk<MODE, 128, PARTIAL, false>(c, m, g, bkb, grid);
  return launch_bk<MODE, 256, PARTIAL, false>(c, m, g, bkb, grid);
}

bool launch_final(Context &c, const TcMaps &m, const TcParams &g, int bn, int bkb, int grid, bool tma_out)
{
  switch (g.epi.mode) {
    case EPI_NONE: return launch_bn<EPI_NONE, false>(c, m, g, bn, bkb, grid, tma_out);
    case EPI_MULT: return launch_bn<EPI_MULT, false>(c, m, g, bn, bkb, grid, tma_out);
    case EPI_BN32: return launch_bn<EPI_BN32, false>(c, m, g, bn, bkb, grid, tma_out);
    case EPI_BN64: return launch_bn<EPI_BN64, false>(c, m, g, bn, bkb, grid, tma_out);
    default:       return launch_bn<EPI_RAW32, false>(c, m, g, bn, bkb, grid, false);
  }
}

}  // namespace

// a pointwise convolution or a fully connected layer: A is the plain [M][K] matrix
static bool igemm_is_plain(const ConvProblem &p)
{
  return p.ky == 1 && p.kx == 1 && p.sy == 1 && p.sx == 1 && p.pt == 0 && p.pl == 0 && p.H == p.Ho && p.W == p.Wo;
}

bool igemm_tc_supported(const Context &c, const ConvProblem &p)
{
  (void)c;
  if ((reinterpret_cast<uintptr_t>(p.in) & 15) || (reinterpret_cast<uintptr_t>(p.w) & 15)) return false;
  const long long M = (long long)p.B * p.Ho * p.Wo;
  if (M > 0x7fffffffLL) return false;
  if (igemm_is_plain(p)) return p.Cin >= 16 && p.Cin % 16 == 0;      // TMA: row pitch must be a multiple of 16 bytes
  // spatial convolution: a K-slab is a chunk of one tap's channels, so Cin is a multiple of the slab
  if (p.Cin % 32 != 0 || p.ky * p.kx > 121) return false;
  if (p.sx > 16 || p.sy > 16) return false;
  return pick_patch_width_log2(p.Ho, p.Wo, p.sx, p.sy) >= 0 && encode_tiled_fn() != nullptr;
}

bool launch_igemm_tc(Context &c, const ConvProblem &p)
{
  TcParams g;
  g.M = p.B * p.Ho * p.Wo; g.N = p.Cout; g.K = p.ky * p.kx * p.Cin;
  g.epi = p.epi;
  const bool raw = p.epi.mode == EPI_RAW32;
  g.conv = igemm_is_plain(p) ? 0 : 1;
  g.param_period = p.Cout;
  const int sms = c.sm_count > 0 ? c.sm_count : 148;
  int fold = 1;
  const int8_t *w_used = p.w;
  g.tw_log2 = 7; g.tiles_x = g.tiles_y = 1; g.chunks_per_tap = 1;
  g.kx = p.kx; g.sx = p.sx; g.sy = p.sy; g.pl = p.pl; g.pt = p.pt; g.Ho = p.Ho; g.Wo = p.Wo;
  // K-slab width: the narrowest box that does not fetch bytes beyond K; wider boxes for long K
  int bkb = 128;
  if (g.conv) {
    bkb = p.Cin % 128 == 0 ? 128 : (p.Cin % 64 == 0 ? 64 : 32);
    g.chunks_per_tap = p.Cin / bkb;
    g.tw_log2 = pick_patch_width_log2(p.Ho, p.Wo, p.sx, p.sy);
    g.tiles_x = (p.Wo + (1 << g.tw_log2) - 1) >> g.tw_log2;
    g.tiles_y = (p.Ho + (128 >> g.tw_log2) - 1) / (128 >> g.tw_log2);
    g.m_tiles = p.B * g.tiles_x * g.tiles_y;
  } else {
    // A short reduction makes short-lived tiles, and what bounds the kernel then is the work per
    // tile of its single-thread roles, not memory or the tensor cores. Fold f consecutive rows of A
    // into one (they are contiguous) and multiply by a block-diagonal W' = diag(W, .., W): the
    // output rows fold the same way, so the bytes in memory are the same, for 1/f of the tiles and
    // f times the (plentiful) multiply-adds.
    // Measured on 112x112x32 -> 64 at batch 1024: 0.284 ms unfolded, 0.256 ms with two pixels per
    // row (one 128-column tile, TMA stores), 0.261 ms with four; 64 -> 128 channels loses 5 % when
    // folded, so only outputs of at most 64 channels are, up to one 128-column tile.
    if (g.K <= 64 && g.N <= 64 && g.K % 16 == 0 && c.opt_split_k == 0) {
      fold = 128 / g.K < 128 / g.N ? 128 / g.K : 128 / g.N;
      while (fold > 1 && (fold & (fold - 1))) fold--;                    // a power of two
      while (fold > 1 && (g.M % fold != 0 || g.M / (BM * fold) < 2 * sms)) fold /= 2;
    }
    if (fold > 1) {
      const size_t wbytes = (size_t)g.N * fold * g.K * fold;
      int slot = 0;
      while ((1 << slot) < fold) slot++;
      int8_t *wf = p.folded ? p.folded->w[slot] : nullptr;
      if (!wf) {
        // a layer of a network keeps its folded copy (constant weights: folded once); a one-off
        // call folds into the context's scratch every time
        if (p.folded) {
          void *mem = nullptr;
          if (!cuda_ok(cudaMalloc(&mem, wbytes), "cudaMalloc(folded weights)")) return false;
          wf = p.folded->w[slot] = static_cast<int8_t *>(mem);
        } else {
          wf = static_cast<int8_t *>(ctx_scratch(c, wbytes));
          if (!wf) return false;
        }
        fold_weights_kernel<<<(unsigned)((wbytes / 16 + 255) / 256), 256, 0, c.stream>>>(p.w, wf, g.N, g.K, fold);
        count_launch();
        if (!cuda_ok(cudaGetLastError(), "fold_weights launch")) return false;
      }
      w_used = wf;
      g.M /= fold; g.N *= fold; g.K *= fold;
    }
    if (g.K <= 32) bkb = 32;
    else if (g.K <= 64) bkb = 64;
    else if (g.K < 128 && g.K % 64 != 0) bkb = 32;       // 80, 96, 112: no padded fetch with 32-byte slabs
    g.m_tiles = (g.M + BM - 1) / BM;
  }
  g.total_slabs = (g.K + bkb - 1) / bkb;
  // uint8 tiles can leave through TMA stores (staged in shared memory, at most 128 columns wide)
  const bool out_ok = !raw && g.N % 16 == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;

  int bn = 0, tiles = 0;
  bool tma_out = false;
  auto configure = [&](int bn_try, bool tma_try) {
    bn = bn_try;
    g.n_tiles = (g.N + bn - 1) / bn;
    tiles = g.m_tiles * g.n_tiles;
    // split K only when the tiles alone cannot occupy the GPU and there is enough K to share
    int slices = 1;
    if (c.opt_split_k > 0) slices = c.opt_split_k;
    else if (tiles * 8 <= sms + 8 && g.total_slabs >= 8) {   // measured: from about 32 tiles on the second pass costs more than it saves
      slices = sms / tiles;
      if (slices > g.total_slabs / 4) slices = g.total_slabs / 4;
      if (slices > 16) slices = 16;
    }
    if (slices > g.total_slabs) slices = g.total_slabs;
    if (slices < 1) slices = 1;
    g.slabs_per_slice = (g.total_slabs + slices - 1) / slices;
    g.k_slices = (g.total_slabs + g.slabs_per_slice - 1) / g.slabs_per_slice;
    tma_out = tma_try && g.k_slices == 1;
    // The CTA's n-tile of W stays in shared memory when K is not split and it leaves room for at
    // least four stages of A. Such CTAs keep their n-tile and walk down the m-tiles.
    const int pipe = pipe_bytes(bn, tma_out);
    const int a_bytes = BM * bkb, b_bytes = bn * bkb;
    const long long wres = (long long)g.total_slabs * b_bytes;
    g.w_resident = (g.k_slices == 1 && g.n_tiles <= sms && wres + 4LL * a_bytes <= pipe) ? 1 : 0;
    g.stationary = g.w_resident;
    const int stage_bytes = g.w_resident ? a_bytes : a_bytes + b_bytes;
    int n_stages = (int)((pipe - (g.w_resident ? wres : 0)) / stage_bytes);
    if (n_stages > MAX_STAGES) n_stages = MAX_STAGES;
    g.n_stages = n_stages;
  };
  // Measured on MobileNet's pointwise layers: 64-column tiles are too short-lived for the staging
  // round trip to pay; wide outputs with K above 256 run faster as 256-column tiles (half as many
  // tiles and slabs for the single-thread roles to get through).
  if (g.N <= 64) configure(64, false);
  else if (g.N <= 128 || (out_ok && g.K <= 256)) configure(128, out_ok);
  else configure(256, out_ok);
  // a 128-column slice of a wide W that does not fit is re-streamed for every m-tile: the 256-column
  // tile (plain stores) halves that traffic
  if (g.N > 128 && bn == 128 && !g.w_resident) configure(256, out_ok);

  if (!c.status_word) {
    if (!cuda_ok(cudaMalloc(&c.status_word, sizeof(int)), "cudaMalloc(status)")) return false;
    if (!cuda_ok(cudaMemsetAsync(c.status_word, 0, sizeof(int), c.stream), "cudaMemset(status)")) return false;
  }
  g.status = c.status_word;
  g.ablate = (c.opt_tune >> 8) & 7;

  TcMaps maps;
  const int tw = 1 << g.tw_log2, th = 128 >> g.tw_log2;
  if (g.conv) {
    if (!make_map_4d(&maps.a, p.in, p.Cin, p.W, p.H, p.B, bkb, tw, th, p.sx, p.sy)) return false;
  } else if (!make_map(&maps.a, p.in, g.M, g.K, BM, bkb)) return false;
  if (!make_map(&maps.b, w_used, g.N, g.K, bn, bkb)) return false;
  maps.out = maps.a;
  if (tma_out) {        // box = at most 128 bytes x 128 rows
    if (g.conv) {
      if (!make_map_4d(&maps.out, p.out, g.N, p.Wo, p.Ho, p.B, bn < 128 ? bn : 128, tw, th, 1, 1)) return false;
    } else if (!make_map(&maps.out, p.out, g.M, g.N, BM, bn < 128 ? bn : 128)) return false;
  }

  const int units = tiles * g.k_slices;
  int grid = units < sms ? units : sms;
  if (g.stationary) {
    const int per = sms / g.n_tiles;
    grid = g.n_tiles * (per < g.m_tiles ? per : g.m_tiles);
  }

  if (g.k_slices == 1) {
    g.out = p.out;
    const int align = raw ? 4 : 16;
    g.vec_store = (g.N % align == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    if (!raw && g.vec_store && g.N % 32 == 0 && (reinterpret_cast<uintptr_t>(p.out) & 31) == 0) g.vec_store = 2;
    return launch_final(c, maps, g, bn, bkb, grid, tma_out);
  }
  const size_t part_bytes = (size_t)g.k_slices * g.M * g.N * sizeof(int);
  int *partials = static_cast<int *>(ctx_scratch(c, part_bytes));
  if (!partials) return false;
  g.out = partials;
  g.vec_store = (g.N % 4 == 0);
  // partial sums need no epilogue mode: one instantiation serves them all
  if (!launch_bn<EPI_NONE, true>(c, maps, g, bn, bkb, grid, false)) return false;
  const size_t total = (size_t)g.M * g.N;
  const unsigned blocks = (unsigned)((total + 255) / 256 < (size_t)sms * 8 ? (total + 255) / 256 : (size_t)sms * 8);
  switch (p.epi.mode) {
    case EPI_NONE: splitk_reduce_kernel<EPI_NONE><<<blocks, 256, 0, c.stream>>>(partials, p.out, p.epi, g.M, g.N, g.k_slices); break;
    case EPI_MULT: splitk_reduce_kernel<EPI_MULT><<<blocks, 256, 0, c.stream>>>(partials, p.out, p.epi, g.M, g.N, g.k_slices); break;
    case EPI_BN32: splitk_reduce_kernel<EPI_BN32><<<blocks, 256, 0, c.stream>>>(partials, p.out, p.epi, g.M, g.N, g.k_slices); break;
    case EPI_BN64: splitk_reduce_kernel<EPI_BN64><<<blocks, 256, 0, c.stream>>>(partials, p.out, p.epi, g.M, g.N, g.k_slices); break;
    default:       splitk_reduce_kernel<EPI_RAW32><<<blocks, 256, 0, c.stream>>>(partials, p.out, p.epi, g.M, g.N, g.k_slices); break;
  }
  count_launch();
  return cuda_ok(cudaGetLastError(), "splitk_reduce launch");
}

#ifdef PULPNN_TRACE
}  // namespace pulpnn
extern "C" int pulpnn_ktrace_read(long long *dst, int *launches)
{
  cudaMemcpyFromSymbol(launches, pulpnn::g_klaunch, sizeof(int));
  return (int)cudaMemcpyFromSymbol(dst, pulpnn::g_ktrace, 64 * sizeof(long long));
}
extern "C" int pulpnn_trace_read(long long *dst, int n)
{
  if (n > 3 * 64 * 8) n = 3 * 64 * 8;
  return (int)cudaMemcpyFromSymbol(dst, pulpnn::g_trace, (size_t)n * sizeof(long long));
}
namespace pulpnn {
#endif

// ---- fully connected layer with split K, for callers that must not allocate -------------------
// The split-K path above parks its per-slice partial sums in device memory that the context
// obtains with cudaMalloc on first use (and again when a larger problem comes along). Some callers
// cannot tolerate that: a serving loop that has handed every free byte of the device to its own
// pool (a cudaMalloc there fails, or succeeds only by synchronising the whole device in the
// middle of a request), or a deployment whose memory budget is fixed and audited up front. For
// them the partial sums live in the array below: it is part of the library image, so every GPU
// that loads the library carries these 4 MiB until the process exits, and the entry point that
// uses it touches no allocator at all.
constexpr size_t STATIC_SCRATCH_INTS = 1u << 20;                      // 4 MiB of int32 partial sums
static __device__ __align__(256) int g_static_partials[STATIC_SCRATCH_INTS];
// The ordinary paths report a bounded wait that ran out through a status word obtained with
// cudaMalloc; this path has its own, built into the library image like the array above.
static __device__ int g_static_status;

namespace {
std::atomic<int *> g_static_partials_dev[MAX_DEVICES];    // device address of the array, per device
std::atomic<int *> g_static_status_dev[MAX_DEVICES];      // device address of the status word

// In host code the names g_static_partials / g_static_status are only handles for the runtime; the
// addresses a kernel can use have to be asked for, once per device, with that device current.
bool static_symbols_for_current_device(Context &c, int **partials, int **status)
{
  if (c.device < 0 || c.device >= MAX_DEVICES) {
    set_error(PULPNN_ERR_INVALID_ARG, "device index %d outside 0..%d", c.device, MAX_DEVICES - 1);
    return false;
  }
  int *pp = g_static_partials_dev[c.device].load(std::memory_order_acquire);
  int *ps = g_static_status_dev[c.device].load(std::memory_order_acquire);
  if (!pp || !ps) {
    void *a = nullptr, *b = nullptr;
    if (!cuda_ok(cudaGetSymbolAddress(&a, g_static_partials), "cudaGetSymbolAddress(static scratch)")) return false;
    if (!cuda_ok(cudaGetSymbolAddress(&b, g_static_status), "cudaGetSymbolAddress(static status)")) return false;
    pp = static_cast<int *>(a); ps = static_cast<int *>(b);
    // a module's __device__ variables start at zero, so the status word needs no clearing here
    g_static_status_dev[c.device].store(ps, std::memory_order_release);
    g_static_partials_dev[c.device].store(pp, std::memory_order_release);
  }
  *partials = pp; *status = ps;
  return true;
}
}  // namespace

// Status word of the entry point below on the context's device: 0 if that entry point was never
// used there. Reads and clears it (after the caller has synchronised the stream).
int static_scratch_status_take(Context &c)
{
  if (c.device < 0 || c.device >= MAX_DEVICES) return 0;
  int *ps = g_static_status_dev[c.device].load(std::memory_order_acquire);
  if (!ps) return 0;
  int v = 0;
  if (!cuda_ok(cudaMemcpy(&v, ps, sizeof(int), cudaMemcpyDeviceToHost), "static status read")) return -1;
  if (v != 0) cudaMemset(ps, 0, sizeof(int));
  return v;
}

}  // namespace pulpnn

using namespace pulpnn;

extern "C" int pulpnn_linear_out_32_static_scratch(const uint8_t *pInBuffer, const int32_t *bias,
                                                   int32_t *pOutBuffer, const int8_t *pWeights,
                                                   int dim_vec, int num_o_neurons, int n_vectors,
                                                   int k_slices)
{
  const char *who = "pulpnn_linear_out_32_static_scratch";
  Context &c = ctx();
  if (!ensure_device(c)) return c.err;
  if (!pInBuffer || !pOutBuffer || !pWeights || dim_vec < 1 || num_o_neurons < 1 || n_vectors < 1 || k_slices < 2) {
    set_error(PULPNN_ERR_INVALID_ARG, "%s: NULL pointer, empty dimension or fewer than 2 K slices", who);
    return c.err;
  }
  // host buffers would have to be staged through allocated device memory: refuse them; so is a
  // buffer that lives on another GPU than the context's (the tensor maps are made for this one)
  const void *ptrs[4] = {pInBuffer, pWeights, pOutBuffer, bias};
  for (const void *q : ptrs) {
    if (!q) continue;
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, q) != cudaSuccess ||
        (a.type != cudaMemoryTypeDevice && a.type != cudaMemoryTypeManaged)) {
      cudaGetLastError();
      set_error(PULPNN_ERR_INVALID_ARG, "%s: every buffer must be device (or managed) memory", who);
      return c.err;
    }
    if (a.type == cudaMemoryTypeDevice && a.device != c.device) {
      set_error(PULPNN_ERR_INVALID_ARG, "%s: a buffer lives on device %d, the context is bound to device %d", who,
                a.device, c.device);
      return c.err;
    }
  }
  ConvProblem p;
  p.in = pInBuffer; p.w = pWeights; p.out = pOutBuffer;
  p.B = n_vectors; p.H = p.W = p.Ho = p.Wo = 1; p.Cin = dim_vec; p.Cout = num_o_neurons;
  p.ky = p.kx = 1; p.pt = p.pl = 0; p.sy = p.sx = 1;
  p.epi.k = p.epi.lambda = nullptr; p.epi.bias = bias; p.epi.mode = EPI_RAW32; p.epi.out_mult = 0; p.epi.shift = 0;
  if (!igemm_tc_supported(c, p) || (reinterpret_cast<uintptr_t>(pOutBuffer) & 3) || (reinterpret_cast<uintptr_t>(bias) & 3)) {
    set_error(PULPNN_ERR_UNSUPPORTED, "%s: needs dim_vec a multiple of 16, pInBuffer and pWeights 16-byte aligned, "
              "pOutBuffer and bias 4-byte aligned", who);
    return c.err;
  }

  TcParams g;
  g.M = n_vectors; g.N = num_o_neurons; g.K = dim_vec;
  g.epi = p.epi;
  g.conv = 0; g.tw_log2 = 7; g.tiles_x = g.tiles_y = 1; g.chunks_per_tap = 1;
  g.param_period = g.N;
  g.kx = g.sx = g.sy = 1; g.pl = g.pt = 0; g.Ho = g.Wo = 1;
  const int bn = g.N <= 64 ? 64 : (g.N <= 128 ? 128 : 256);
  int bkb = 128;
  if (g.K <= 32) bkb = 32;
  else if (g.K <= 64) bkb = 64;
  else if (g.K < 128 && g.K % 64 != 0) bkb = 32;
  g.m_tiles = (g.M + BM - 1) / BM;
  g.n_tiles = (g.N + bn - 1) / bn;
  g.total_slabs = (g.K + bkb - 1) / bkb;
  const int slices = k_slices < g.total_slabs ? k_slices : g.total_slabs;
  g.slabs_per_slice = (g.total_slabs + slices - 1) / slices;
  g.k_slices = (g.total_slabs + g.slabs_per_slice - 1) / g.slabs_per_slice;
  if (g.k_slices < 2) {
    set_error(PULPNN_ERR_UNSUPPORTED, "%s: dim_vec %d is too short to split", who, dim_vec);
    return c.err;
  }
  const size_t need = (size_t)g.k_slices * g.M * g.N;
  if (need > STATIC_SCRATCH_INTS) {
    set_error(PULPNN_ERR_UNSUPPORTED,
              "%s: %d slices x %d vectors x %d neurons = %zu partial sums exceed the built-in scratch of %zu "
              "(4 MiB); use fewer slices or vectors, or pulp_nn_linear_out_32",
              who, g.k_slices, g.M, g.N, need, (size_t)STATIC_SCRATCH_INTS);
    return c.err;
  }
  int *partials = nullptr, *status = nullptr;
  if (!static_symbols_for_current_device(c, &partials, &status)) return c.err;

  g.w_resident = 0;
  g.stationary = 0;
  g.n_stages = PIPE_BYTES / (BM * bkb + bn * bkb);
  if (g.n_stages > MAX_STAGES) g.n_stages = MAX_STAGES;
  g.status = status;                       // built into the library too; read by pulpnn_device_status()
  g.out = partials;
  g.vec_store = (g.N % 4 == 0);
  TcMaps maps;
  if (!make_map(&maps.a, p.in, g.M, g.K, BM, bkb)) return c.err;
  if (!make_map(&maps.b, p.w, g.N, g.K, bn, bkb)) return c.err;
  maps.out = maps.a;
  const int sms = c.sm_count > 0 ? c.sm_count : 148;
  const int units = g.m_tiles * g.n_tiles * g.k_slices;
  // Nothing in the scratch has to start at zero: the GEMM below writes every partial sum the
  // reduction reads (each slice owns at least one K slab, every tile of every slice is a unit).
  if (!launch_bn<EPI_NONE, true>(c, maps, g, bn, bkb, units < sms ? units : sms, false)) return c.err;
  const size_t total = (size_t)g.M * g.N;
  const unsigned blocks = (unsigned)((total + 255) / 256 < (size_t)sms * 8 ? (total + 255) / 256 : (size_t)sms * 8);
  splitk_reduce_kernel<EPI_RAW32><<<blocks, 256, 0, c.stream>>>(partials, pOutBuffer, p.epi, g.M, g.N, g.k_slices);
  count_launch();
  if (!cuda_ok(cudaGetLastError(), "splitk_reduce launch")) return c.err;
  return PULPNN_OK;
}
