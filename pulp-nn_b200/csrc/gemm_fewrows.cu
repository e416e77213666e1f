// gemm_fewrows.cu -- the u8 x s8 -> s32 contraction for FEW rows (a fully connected layer at a small
// batch: M up to a few hundred, K and N in the thousands), where a tensor-core tile would sit mostly
// empty and the work is to stream the weights once. Arithmetic of 32bit/src/pulp_nn_linear.c:58-108
// and pulp_nn_linear_out_32.c:48-80 (a pointwise layer with few pixels is the same thing).
//
// A CTA owns eight output neurons: their weight rows (8 x K bytes) sit in shared memory, and the
// CTA's eight warps share out the rows of A. For one row a warp's lanes split K in 16-byte pieces
// (a coalesced 512-byte read of A per step), each lane multiplies its piece with the eight weight
// rows by dp4a, and the eight partial sums are added across the lanes by a halving exchange (nine
// shuffles for eight sums). Every CTA reads all of A (from L2) and its own slice of W exactly once.
#include "internal.cuh"

namespace pulpnn {

namespace {

constexpr int NB = 8;            // neurons per CTA
constexpr int FR_WARPS = 8;

template <int MODE>
__global__ void __launch_bounds__(32 * FR_WARPS) gemm_fewrows_kernel(const ConvProblem p, int M, int K)
{
  extern __shared__ uint4 wsm[];                   // [NB][K / 16]
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n0 = blockIdx.x * NB;
  const int kc = K >> 4;                           // 16-byte pieces per row
  const Epilogue &e = p.epi;
  for (int i = threadIdx.x; i < NB * kc; i += 32 * FR_WARPS) {
    const int n = n0 + i / kc;
    wsm[i] = n < p.Cout ? __ldg(reinterpret_cast<const uint4 *>(p.w + (size_t)n * K) + i % kc) : make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  for (int m = warp; m < M; m += FR_WARPS) {
    int acc[NB];
#pragma unroll
    for (int j = 0; j < NB; j++) acc[j] = 0;
    const uint4 *arow = reinterpret_cast<const uint4 *>(p.in + (size_t)m * K);
    for (int c = lane; c < kc; c += 32) {
      const uint4 a = __ldg(arow + c);
#pragma unroll
      for (int j = 0; j < NB; j++) {
        const uint4 w = wsm[j * kc + c];
        acc[j] = dp4a_us(a.x, (int)w.x, acc[j]);
        acc[j] = dp4a_us(a.y, (int)w.y, acc[j]);
        acc[j] = dp4a_us(a.z, (int)w.z, acc[j]);
        acc[j] = dp4a_us(a.w, (int)w.w, acc[j]);
      }
    }
    // eight sums over 32 lanes: each exchange halves the number of sums a lane carries
    int s4[4], s2[2], s1;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const bool up = lane & 16;
      const int keep = up ? acc[j + 4] : acc[j], give = up ? acc[j] : acc[j + 4];
      s4[j] = keep + __shfl_xor_sync(0xffffffffu, give, 16);       // lanes 0-15: neurons 0-3, lanes 16-31: neurons 4-7
    }
#pragma unroll
    for (int j = 0; j < 2; j++) {
      const bool up = lane & 8;
      const int keep = up ? s4[j + 2] : s4[j], give = up ? s4[j] : s4[j + 2];
      s2[j] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
    }
    {
      const bool up = lane & 4;
      const int keep = up ? s2[1] : s2[0], give = up ? s2[0] : s2[1];
      s1 = keep + __shfl_xor_sync(0xffffffffu, give, 4);
    }
    s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
    // lanes 4q..4q+3 now hold the sum of neuron: bit 4 of the lane picks +4, bit 3 picks +2, bit 2 picks +1
    const int n = n0 + ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
    if ((lane & 3) == 0 && n < p.Cout) {
      if (MODE == EPI_RAW32) {
        int a = s1;
        if (e.bias) a += __ldg(reinterpret_cast<const int *>(e.bias) + n);
        reinterpret_cast<int *>(p.out)[(size_t)m * p.Cout + n] = a;
      } else {
        int a = s1;
        if (e.bias) a += (int)__ldg(reinterpret_cast<const int8_t *>(e.bias) + n);
        reinterpret_cast<uint8_t *>(p.out)[(size_t)m * p.Cout + n] = (uint8_t)requant<MODE>(a, n, e);
      }
    }
  }
}

template <int MODE>
bool launch_fr(Context &c, const ConvProblem &p, int M, int K)
{
  const size_t smem = (size_t)NB * K;
  auto kern = gemm_fewrows_kernel<MODE>;
  static PerDeviceInt smem_set;
  if ((int)smem > 48 * 1024 && (int)smem > smem_set.get(c.device)) {
    if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "cudaFuncSetAttribute(gemm_fewrows)"))
      return false;
    smem_set.set(c.device, (int)smem);
  }
  const cudaError_t le = launch_pdl(kern, dim3((unsigned)((p.Cout + NB - 1) / NB)), dim3(32 * FR_WARPS), smem, c.stream, p, M, K);
  count_launch("gemm_fewrows_kernel");
  return cuda_ok(le, "gemm_fewrows launch") && cuda_ok(cudaGetLastError(), "gemm_fewrows launch");
}

}  // namespace

// a plain GEMM (1x1, stride 1, no padding) with few rows, K a multiple of 16 that fits a CTA's shared
// memory eight rows deep, 16-byte aligned operands
bool gemm_fewrows_supported(const ConvProblem &p)
{
  if (p.ky != 1 || p.kx != 1 || p.sy != 1 || p.sx != 1 || p.pt != 0 || p.pl != 0 || p.H != p.Ho || p.W != p.Wo) return false;
  const long long M = (long long)p.B * p.Ho * p.Wo;
  if (M < 1 || M > 256 || p.Cin % 16 != 0 || p.Cin < 256 || p.Cin > 16384) return false;
  if (M * p.Cin > 512 * 1024) return false;        // every CTA streams all of A
  if ((reinterpret_cast<uintptr_t>(p.in) & 15) || (reinterpret_cast<uintptr_t>(p.w) & 15)) return false;
  if (p.epi.mode == EPI_RAW32 && (reinterpret_cast<uintptr_t>(p.out) & 3)) return false;
  return true;
}

bool launch_gemm_fewrows(Context &c, const ConvProblem &p)
{
  const int M = p.B * p.Ho * p.Wo, K = p.Cin;
  switch (p.epi.mode) {
    case EPI_NONE: return launch_fr<EPI_NONE>(c, p, M, K);
    case EPI_MULT: return launch_fr<EPI_MULT>(c, p, M, K);
    case EPI_BN32: return launch_fr<EPI_BN32>(c, p, M, K);
    case EPI_BN64: return launch_fr<EPI_BN64>(c, p, M, K);
    default:       return launch_fr<EPI_RAW32>(c, p, M, K);
  }
}

}  // namespace pulpnn
