// igemm_tc2.cu -- the u8 x s8 -> s32 GEMM of igemm_tc.cu for wide layers with a long reduction
// (pointwise layers from 512 input channels on), computed by PAIRS of SMs: a thread-block cluster of
// two CTAs issues tcgen05.mma.cta_group::2, M = 256 (each CTA brings 128 rows of A and holds the
// accumulator of those rows in its own tensor memory), N = 256 (each CTA brings HALF of the weight
// tile). Arithmetic and epilogue are those of igemm_tc.cu (32bit/src/pulp_nn_matmul.c:96-216).
//
// Why pairs: with one CTA per tile a 256-column slice of W with K = 512 fills 128 KB of shared
// memory, the operand ring holds a single tile of A, and A is fetched once per 256 output columns.
// A pair holds the same slice in 64 KB per CTA, so TWO column tiles (all 512 output channels of the
// MobileNet layers) stay resident, A is fetched once for both, and the traffic from L2 into the
// SMs -- what bounds these layers -- halves.
//
// Work: the cluster keeps NT resident column tiles (its "column group") and walks down the row pairs
// (256 rows) assigned to it; per row pair it runs NT passes over the slabs of A, pass t into
// accumulator t of the ring (two accumulators of 256 columns). The slabs of A stay in the ring for
// all passes and are released during the last one. Roles per CTA (18 warps):
//   warp 0, one lane   TMA: its half of the resident weights once, then its 128 rows of every A slab.
//                      Both CTAs' loads complete on the LEADER's "full" barrier (CTA rank 0 of the
//                      pair); no multicast anywhere.
//   warp 1             allocates tensor memory (both CTAs, cta_group::2); in the leader one lane
//                      issues the MMAs and the commits, which arrive on barriers in both CTAs
//   warps 2..17        epilogue of the CTA's own 128 rows: tcgen05.ld, requantise, 32-byte global stores
//                      (every warp on its own: four warps per TMEM lane quarter, two 32-column pieces each)
// Every wait is bounded; the two CTAs meet at a cluster barrier before either frees anything.
#include <cuda.h>
#include <cstdio>
#include <cstdlib>

#include "internal.cuh"
#include "sm100_primitives.cuh"

namespace pulpnn {

namespace {

using namespace sm100;

constexpr int BM = 128, BN = 256, BKB = 128, UMMA_K = 32;
constexpr int A_BYTES = BM * BKB;              // one stage: this CTA's 128 rows of a slab
constexpr int WH_BYTES = (BN / 2) * BKB;       // this CTA's half of one weight slab
constexpr int EPI_WARPS2 = 16, FIRST_EPI2 = 2;
constexpr int THREADS2 = 32 * (FIRST_EPI2 + EPI_WARPS2);
constexpr int MAX_STAGES2 = 8;
constexpr int NUM_ACC2 = 2;
constexpr int ST2_PRODUCER = 0x100000, ST2_MMA = 0x200000, ST2_EPI = 0x400000;

struct Tc2Params {
  void *out;              // uint8 [M][N] (the direct-store epilogue)
  Epilogue epi;
  int M, N, K;
  int slabs;              // K / 128
  int nt;                 // resident column tiles per cluster (1 or 2)
  int col_groups;         // N / (256 * nt)
  int row_pairs;          // ceil(M / 256)
  int n_stages;
  int *status;
  int ablate;             // measurement only (PULPNN_OPT_TUNE bits 8-11): 1 no epilogue work, 2 no loads of A, 4 no MMAs, 8 no stores
};

// shared-memory layout of one CTA (after 1024-byte alignment)
struct Smem2 {
  int w_bytes, ring_off, param_off, bar_off, total;
};
__host__ __device__ inline Smem2 smem2_layout(int slabs, int nt, int n_stages)
{
  Smem2 L;
  L.w_bytes = nt * slabs * WH_BYTES;
  L.ring_off = L.w_bytes;
  L.param_off = L.ring_off + n_stages * A_BYTES;
  L.bar_off = L.param_off + nt * BN * 16;
  L.total = L.bar_off + 1024 + 1024;
  return L;
}

// the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank)
{
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ uint32_t cluster_rank()
{
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// 2-D tiled load whose completion is signalled on a barrier that may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(void *dst, const CUtensorMap *map, uint32_t bar_cluster_addr, int x, int y)
{
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr)
{
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *slot, uint32_t ncols)
{
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
{
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrives (once these MMAs have completed) on the barrier at this shared-memory offset in BOTH CTAs
__device__ __forceinline__ void umma_commit_pair(uint64_t *bar)
{
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3)
               : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void cluster_sync_all()
{
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// instruction descriptor as in umma_idesc_u8s8, for M = 256 over the pair
__host__ __device__ constexpr uint32_t idesc_pair(int n)
{
  return (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

template <int MODE>
__global__ void __launch_bounds__(THREADS2, 1)
igemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const Tc2Params g)
{
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const Smem2 L = smem2_layout(g.slabs, g.nt, g.n_stages);
  uint8_t *ring = smem + L.ring_off;
  uint8_t *params = smem + L.param_off;
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + L.bar_off);      // used in the leader only
  uint64_t *empty_bar = full_bar + MAX_STAGES2;                             // per CTA
  uint64_t *tmem_full = empty_bar + MAX_STAGES2;                            // per CTA
  uint64_t *tmem_empty = tmem_full + NUM_ACC2;                              // used in the leader only
  uint64_t *wres_bar = tmem_empty + NUM_ACC2;                               // used in the leader only
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(wres_bar + 1);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();                 // 0: leader, 1: peer
  const int cluster_id = (int)(blockIdx.x >> 1), n_clusters = (int)(gridDim.x >> 1);
  // the cluster's column group and its row pairs: cg fastest, so the clusters of one row pair run together
  const int cg = cluster_id % g.col_groups;
  const int rp0 = cluster_id / g.col_groups, rp_step = n_clusters / g.col_groups;
  const int n_base = cg * g.nt * BN;                    // first output column of the cluster
  const Epilogue &e = g.epi;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MAX_STAGES2; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < NUM_ACC2; b++) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], 2 * EPI_WARPS2); }
    mbar_init(wres_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, 512);
  // per-channel parameters of the cluster's columns -> shared memory, once; the bias is folded into
  // lambda: k*(acc+b)+lambda == k*acc + (k*b+lambda) in wrap-around arithmetic
  for (int i = threadIdx.x; i < g.nt * BN; i += THREADS2) {
    const int n = n_base + i;
    const int bias8 = e.bias ? (int)__ldg(reinterpret_cast<const int8_t *>(e.bias) + n) : 0;
    if (MODE == EPI_BN32) {
      const int k = __ldg(reinterpret_cast<const int *>(e.k) + n);
      reinterpret_cast<int *>(params)[i] = k;
      reinterpret_cast<int *>(params)[g.nt * BN + i] =
          (int)((unsigned)k * (unsigned)bias8 + (unsigned)__ldg(reinterpret_cast<const int *>(e.lambda) + n));
    } else if (MODE == EPI_BN64) {
      const long long k = __ldg(reinterpret_cast<const long long *>(e.k) + n);
      reinterpret_cast<long long *>(params)[i] = k;
      reinterpret_cast<long long *>(params)[g.nt * BN + i] =
          (long long)((unsigned long long)k * (unsigned long long)(long long)bias8 +
                      (unsigned long long)__ldg(reinterpret_cast<const long long *>(e.lambda) + n));
    } else {
      reinterpret_cast<int *>(params)[i] = bias8;
    }
  }
  tc_fence_before();
  __syncthreads();
  // both CTAs' barriers are initialised before either signals the other's
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------------------------
    if (lane == 0) {
      const uint32_t wres_leader = map_to_cta(smem_u32(wres_bar), 0);
      // this CTA's half (128 rows) of every resident weight slab; constants: before the wait below
      if (rank == 0) mbar_arrive_expect_tx(wres_bar, (uint32_t)(2 * L.w_bytes));
      for (int t = 0; t < g.nt; t++)
        for (int s = 0; s < g.slabs; s++)
          tma_load_2d_pair(smem + (t * g.slabs + s) * WH_BYTES, &map_w, wres_leader, s * BKB,
                           n_base + t * BN + (int)rank * (BN / 2));
      pdl_wait();                      // A is the previous kernel's output
      pdl_launch_dependents();
      int st = 0; uint32_t ph = 0; int issued = 0;
      bool ok = true;
      for (int rp = rp0; rp < g.row_pairs && ok; rp += rp_step) {
        const int row = rp * 2 * BM + (int)rank * BM;
        for (int s = 0; s < g.slabs; s++) {
          if (!mbar_wait(&empty_bar[st], ph ^ 1, abort_flag, g.status, ST2_PRODUCER)) { ok = false; break; }
          if (g.ablate & 2) {
            if (rank == 0) mbar_arrive(&full_bar[st]);
          } else {
            if (rank == 0) mbar_arrive_expect_tx(&full_bar[st], (uint32_t)(2 * A_BYTES));
            tma_load_2d_pair(ring + st * A_BYTES, &map_a, map_to_cta(smem_u32(&full_bar[st]), 0), s * BKB, row);
          }
          issued++;
          if (++st == g.n_stages) { st = 0; ph ^= 1; }
        }
      }
      if (*abort_flag && issued) {
        // something gave up: let the loads that are still in flight land before the CTA's memory goes
        // (a load takes a few microseconds at most; the barriers they signal may be the peer's)
        const unsigned long long t0 = global_ns();
        while (global_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) --------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = idesc_pair(BN);
      bool ok = mbar_wait(wres_bar, 0, abort_flag, g.status, ST2_MMA);
      int st0 = 0; uint32_t ph0 = 0;      // ring position of the row pair's first slab
      int i = 0;                          // tiles issued so far: accumulator i % 2
      for (int rp = rp0; rp < g.row_pairs && ok; rp += rp_step) {
        for (int t = 0; t < g.nt && ok; t++, i++) {
          const int acc = i & 1;
          if (!mbar_wait(&tmem_empty[acc], (((uint32_t)(i >> 1)) & 1u) ^ 1u, abort_flag, g.status, ST2_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d = tmem_base + (uint32_t)(acc * BN);
          int st = st0; uint32_t ph = ph0;
          for (int s = 0; s < g.slabs; s++) {
            // the slabs of A arrive during the first pass and stay for the others
            if (t == 0 && !mbar_wait(&full_bar[st], ph, abort_flag, g.status, ST2_MMA)) { ok = false; break; }
            tc_fence_after();
            const uint64_t da = umma_smem_desc<BKB>(smem_u32(ring + st * A_BYTES));
            const uint64_t db = umma_smem_desc<BKB>(smem_u32(smem + (t * g.slabs + s) * WH_BYTES));
#pragma unroll
            for (int j = 0; j < BKB / UMMA_K; j++)
              if (!(g.ablate & 4)) umma_i8_pair(d, da + (uint64_t)(2 * j), db + (uint64_t)(2 * j), idesc, (s > 0 || j > 0) ? 1u : 0u);
            if (t == g.nt - 1) umma_commit_pair(&empty_bar[st]);       // both producers may refill the stage
            if (++st == g.n_stages) { st = 0; ph ^= 1; }
          }
          if (!ok) break;
          umma_commit_pair(&tmem_full[acc]);                           // both CTAs' epilogues may drain it
          if (t == g.nt - 1) { st0 = st; ph0 = ph; }
        }
      }
    }
  } else {
    // ------------------------------ epilogue of this CTA's 128 rows -----------------------------
    // sixteen warps: four per TMEM lane quarter, each taking every fourth 32-column chunk
    constexpr int NSPLIT = 4, HALF_COLS = BN / NSPLIT, NCHUNK = HALF_COLS / 32;
    const int quad = warp & 3;
    const int ew = warp - FIRST_EPI2;
    const int share = (ew >> 2) % NSPLIT;
    const uint32_t tmem_empty_leader0 = map_to_cta(smem_u32(&tmem_empty[0]), 0);
    const int *p_k32 = reinterpret_cast<const int *>(params), *p_l32 = p_k32 + g.nt * BN;
    const long long *p_k64 = reinterpret_cast<const long long *>(params), *p_l64 = p_k64 + g.nt * BN;
    const int *p_bias = reinterpret_cast<const int *>(params);
    pdl_wait();                          // the output buffer may still be read by the previous kernel
    bool dead = false;
    int i = 0;
    for (int rp = rp0; rp < g.row_pairs && !dead; rp += rp_step) {
      const int row = rp * 2 * BM + (int)rank * BM;
      for (int t = 0; t < g.nt; t++, i++) {
        const int acc = i & 1;
        {   // every warp on its own: nothing to meet the other warps for
          if (!mbar_wait(&tmem_full[acc], ((uint32_t)(i >> 1)) & 1u, abort_flag, g.status, ST2_EPI)) { dead = true; break; }
          tc_fence_after();
          const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
          if (g.ablate & 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tmem_empty_leader0 + (uint32_t)(acc * 8));
            continue;
          }
          const int m = row + quad * 32 + lane;
          uint8_t *orow = reinterpret_cast<uint8_t *>(g.out) + (size_t)(m < g.M ? m : 0) * g.N + n_base + t * BN;
          uint32_t vb[NCHUNK][32];
#pragma unroll
          for (int ch = 0; ch < NCHUNK; ch++) tmem_ld_32(t_row + (uint32_t)(ch * (32 * NSPLIT) + share * 32), vb[ch]);
          tmem_wait_ld();
          // the accumulator is in registers: hand it back to the leader's MMA thread before the stores
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(tmem_empty_leader0 + (uint32_t)(acc * 8));
#pragma unroll
          for (int ch = 0; ch < NCHUNK; ch++) {
            const int c0 = ch * (32 * NSPLIT) + share * 32;
            const int pc = t * BN + c0;
            const uint32_t (&v)[32] = vb[ch];
            unsigned w[8];
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              int q[4];
              if (MODE == EPI_BN32) {
                const int4 kk = *reinterpret_cast<const int4 *>(p_k32 + pc + j);
                const int4 ll = *reinterpret_cast<const int4 *>(p_l32 + pc + j);
                q[0] = (int)((unsigned)kk.x * v[j + 0] + (unsigned)ll.x) >> e.shift;
                q[1] = (int)((unsigned)kk.y * v[j + 1] + (unsigned)ll.y) >> e.shift;
                q[2] = (int)((unsigned)kk.z * v[j + 2] + (unsigned)ll.z) >> e.shift;
                q[3] = (int)((unsigned)kk.w * v[j + 3] + (unsigned)ll.w) >> e.shift;
              } else {
#pragma unroll
                for (int u = 0; u < 4; u++) {
                  const int a = (int)v[j + u];
                  if (MODE == EPI_BN64)
                    q[u] = (int)((long long)((unsigned long long)p_k64[pc + j + u] * (unsigned long long)(long long)a +
                                             (unsigned long long)p_l64[pc + j + u]) >> e.shift);
                  else if (MODE == EPI_MULT)
                    q[u] = (int)(short)((int)((unsigned)e.out_mult * (unsigned)(a + p_bias[pc + j + u])) >> e.shift);
                  else
                    q[u] = (a + p_bias[pc + j + u]) >> e.shift;
                }
              }
              w[j >> 2] = pack4_sat_u8(q[0], q[1], q[2], q[3]);
            }
            if (m < g.M && !(g.ablate & 8))
              asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                           ::"l"(orow + c0), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                           : "memory");
          }
        }
      }
    }
  }

  // neither CTA may release its shared or tensor memory while the other can still reach it
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

bool make_map2(CUtensorMap *map, const void *base, int rows, int row_bytes, int box_rows, int box_bytes)
{
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) { set_error(PULPNN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver"); return false; }
  cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error(PULPNN_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r); return false; }
  return true;
}

// How many clusters of two such CTAs the device runs at once (SM pairs that can form a cluster: fewer
// than half the SM count where a processor cluster has an odd number of SMs). Work is dealt out
// statically, so a grid larger than this would run in two waves.
template <int MODE>
int resident_pairs(Context &c, int smem)
{
  static PerDeviceInt cached;
  int n = cached.get(c.device);
  if (n > 0) return n;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2u * (unsigned)(c.sm_count > 0 ? c.sm_count : 148)); cfg.blockDim = dim3(THREADS2);
  cfg.dynamicSmemBytes = (size_t)smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  if (cudaOccupancyMaxActiveClusters(&n, igemm_tc2_kernel<MODE>, &cfg) != cudaSuccess || n < 1) {
    cudaGetLastError();
    n = (c.sm_count > 0 ? c.sm_count : 148) / 2;
  }
  cached.set(c.device, n);
  return n;
}

template <int MODE>
bool launch_mode2(Context &c, const CUtensorMap &ma, const CUtensorMap &mw, Tc2Params g, int smem)
{
  auto kern = igemm_tc2_kernel<MODE>;
  static PerDeviceInt attr_set;
  if (attr_set.get(c.device) < smem) {
    if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "cudaFuncSetAttribute(igemm_tc2)"))
      return false;
    attr_set.set(c.device, smem);
  }
  // a whole number of clusters per column group, no more than there are row pairs or resident pairs
  int per = resident_pairs<MODE>(c, smem) / g.col_groups;
  if (per < 1) { set_error(PULPNN_ERR_UNSUPPORTED, "igemm_tc2: more column groups than SM pairs"); return false; }
  if (per > g.row_pairs) per = g.row_pairs;
  const int grid = 2 * per * g.col_groups;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(THREADS2); cfg.dynamicSmemBytes = (size_t)smem; cfg.stream = c.stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 2;
  if (getenv("PULPNN_DEBUG")) fprintf(stderr, "igemm_tc2: %d resident pairs, grid %d, nt %d, stages %d\n",
                                      resident_pairs<MODE>(c, smem), grid, g.nt, g.n_stages);
  const cudaError_t le = cudaLaunchKernelEx(&cfg, kern, ma, mw, g);
  count_launch("igemm_tc2_kernel");
  return cuda_ok(le, "igemm_tc2 launch") && cuda_ok(cudaGetLastError(), "igemm_tc2 launch");
}

}  // namespace

// plain GEMM (pointwise / linear), uint8 output, whole 256-column tiles, whole 128-byte K slabs, and a
// weight slice that fits: NT * 64 KB * (K / 512) per CTA beside a ring that holds a whole tile of A
bool igemm_tc2_supported(const Context &c, const ConvProblem &p)
{
  (void)c;
  if (p.ky != 1 || p.kx != 1 || p.sy != 1 || p.sx != 1 || p.pt != 0 || p.pl != 0 || p.H != p.Ho || p.W != p.Wo) return false;
  if (p.epi.mode == EPI_RAW32) return false;
  if (p.Cout % BN != 0 || p.Cin % BKB != 0 || p.Cin < 512 || p.Cin > 1024) return false;
  const long long M = (long long)p.B * p.Ho * p.Wo;
  if (M < 2 * BM || M > 0x7fffffffLL) return false;
  if ((reinterpret_cast<uintptr_t>(p.in) & 15) || (reinterpret_cast<uintptr_t>(p.w) & 15) ||
      (reinterpret_cast<uintptr_t>(p.out) & 31))
    return false;
  return encode_tiled_fn() != nullptr;
}

bool launch_igemm_tc2(Context &c, const ConvProblem &p)
{
  Tc2Params g;
  g.epi = p.epi; g.out = p.out;
  g.M = p.B * p.Ho * p.Wo; g.N = p.Cout; g.K = p.Cin;
  g.slabs = g.K / BKB;
  // two resident column tiles when their halves fit in 128 KB (K <= 512) and the layer has them
  g.nt = (g.slabs * WH_BYTES * 2 <= 128 * 1024 && (g.N / BN) % 2 == 0) ? 2 : 1;
  g.col_groups = g.N / (BN * g.nt);
  g.row_pairs = (g.M + 2 * BM - 1) / (2 * BM);
  const int budget = 216 * 1024 - g.nt * g.slabs * WH_BYTES - g.nt * BN * 16;
  int n_stages = budget / A_BYTES;
  if (n_stages > MAX_STAGES2) n_stages = MAX_STAGES2;
  // with several passes the slabs of a tile stay in the ring for all of them
  if (n_stages < (g.nt > 1 ? g.slabs : 2)) { set_error(PULPNN_ERR_UNSUPPORTED, "igemm_tc2: operand ring too small"); return false; }
  g.n_stages = n_stages;
  g.ablate = (c.opt_tune >> 8) & 15;
  g.status = ctx_status_word(c);
  if (!g.status) return false;
  const Smem2 L = smem2_layout(g.slabs, g.nt, g.n_stages);
  CUtensorMap ma, mw;
  if (!make_map2(&ma, p.in, g.M, g.K, BM, BKB)) return false;
  if (!make_map2(&mw, p.w, g.N, g.K, BN / 2, BKB)) return false;
  switch (p.epi.mode) {
    case EPI_NONE: return launch_mode2<EPI_NONE>(c, ma, mw, g, L.total);
    case EPI_MULT: return launch_mode2<EPI_MULT>(c, ma, mw, g, L.total);
    case EPI_BN32: return launch_mode2<EPI_BN32>(c, ma, mw, g, L.total);
    default:       return launch_mode2<EPI_BN64>(c, ma, mw, g, L.total);
  }
}

}  // namespace pulpnn
