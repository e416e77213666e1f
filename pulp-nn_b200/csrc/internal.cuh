// internal.cuh -- shared declarations of the library's translation units.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>
#include <atomic>

#include "../../include/pulpnn_b200.h"

namespace pulpnn {

// ---------------------------------------------------------------------------------------------
// Requantisation epilogues. The mode is decided on the host from (flag_relu, flag_batch_norm)
// exactly as the reference does (32bit/src/pulp_nn_matmul.c:144-216, pulp_nn_linear.c:88-107,
// pulp_nn_depthwise_generic.c:167-178).
// ---------------------------------------------------------------------------------------------
enum EpiMode : int {
  EPI_NONE = 0,   // clip(acc >> d)
  EPI_MULT = 1,   // clip((int16)((int16)out_mult * acc >> d))
  EPI_BN32 = 2,   // clip((int32)(k*acc + lambda) >> d), int32 wrap-around
  EPI_BN64 = 3,   // clip((int32)(((int64)k*acc + lambda) >> d))
  EPI_RAW32 = 4   // store the int32 accumulator (pulp_nn_linear_out_32)
};

struct Epilogue {
  const void *k;        // int32[] or int64[] per output channel (BN modes)
  const void *lambda;
  const void *bias;     // int8[] per output channel, int32[] for EPI_RAW32, or nullptr
  int mode;
  int out_mult;         // already converted to int16 range semantics on the host
  int shift;            // 0..31 (0..63 for EPI_BN64)
};

__device__ __forceinline__ int clip_u8(int x) { return min(max(x, 0), 255); }

template <int MODE>
__device__ __forceinline__ int requant(int acc, int ch, const Epilogue &e)
{
  if (MODE == EPI_BN32) {
    const int k = __ldg(reinterpret_cast<const int *>(e.k) + ch);
    const int l = __ldg(reinterpret_cast<const int *>(e.lambda) + ch);
    const int t = (int)((unsigned)k * (unsigned)acc + (unsigned)l);
    return clip_u8(t >> e.shift);
  } else if (MODE == EPI_BN64) {
    const long long k = __ldg(reinterpret_cast<const long long *>(e.k) + ch);
    const long long l = __ldg(reinterpret_cast<const long long *>(e.lambda) + ch);
    const long long t = (long long)((unsigned long long)k * (unsigned long long)(long long)acc +
                                    (unsigned long long)l);
    return clip_u8((int)(t >> e.shift));
  } else if (MODE == EPI_MULT) {
    const int p = (int)((unsigned)e.out_mult * (unsigned)acc);
    return clip_u8((int)(short)(p >> e.shift));
  } else {
    return clip_u8(acc >> e.shift);
  }
}

// requantisation with the per-channel parameters already in registers / shared memory
template <int MODE>
__device__ __forceinline__ int requant_kl(int acc, long long k, long long l, int out_mult, int shift)
{
  if (MODE == EPI_BN32) {
    const int t = (int)((unsigned)(int)k * (unsigned)acc + (unsigned)(int)l);
    return clip_u8(t >> shift);
  } else if (MODE == EPI_BN64) {
    const long long t = (long long)((unsigned long long)k * (unsigned long long)(long long)acc +
                                    (unsigned long long)l);
    return clip_u8((int)(t >> shift));
  } else if (MODE == EPI_MULT) {
    const int p = (int)((unsigned)out_mult * (unsigned)acc);
    return clip_u8((int)(short)(p >> shift));
  } else {
    return clip_u8(acc >> shift);
  }
}

// Clamp four int32 values to [0,255] and pack them, a in the lowest byte. cvt.pack.sat converts
// two values per instruction: d[7:0] = sat(second), d[15:8] = sat(first), d[31:16] = third[15:0].
__device__ __forceinline__ unsigned pack4_sat_u8(int a, int b, int c, int d)
{
  unsigned hi, r;
  asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(d), "r"(c), "r"(0));
  asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(b), "r"(a), "r"(hi));
  return r;
}

// u8 x s8 dot product of four byte lanes
__device__ __forceinline__ int dp4a_us(unsigned a_u8x4, int b_s8x4, int c)
{
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8x4), "r"(b_s8x4), "r"(c));
  return d;
}

// ---------------------------------------------------------------------------------------------
// Problem descriptions handed from the entry points to the launchers (all pointers are device
// pointers by then).
// ---------------------------------------------------------------------------------------------
// Block-diagonal copies of a layer's weights (see launch_igemm_tc), made once and kept by whoever
// owns the layer; slot i holds the copy for 2^i pixels per GEMM row. Device memory, freed by the owner.
struct FoldedWeights { int8_t *w[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr}; };

struct ConvProblem {
  const uint8_t *in;     // [B][H][W][Cin]
  const int8_t *w;       // [Cout][ky][kx][Cin]
  void *out;             // [B][Ho][Wo][Cout] uint8 (int32 for EPI_RAW32)
  int B, H, W, Cin, Ho, Wo, Cout, ky, kx, pt, pl, sy, sx;
  Epilogue epi;
  FoldedWeights *folded = nullptr;   // optional: where constant weights keep their folded copies
};

struct DepthwiseProblem {
  const uint8_t *in;     // [B][C][H][W] (chw) or [B][H][W][C]
  const int8_t *w;       // [C][ky][kx]
  uint8_t *out;          // [B][Ho][Wo][C]
  int B, H, W, C, Ho, Wo, ky, kx, pt, pl, sy, sx;
  bool in_is_hwc;
  Epilogue epi;
};

struct PoolProblem {
  const uint8_t *in;     // [B][H][W][C]
  uint8_t *out;          // [B][Ho][Wo][C]
  int B, H, W, C, Ho, Wo, ky, kx, pt, pb, pl, pr, sy, sx;
  // avgpool only
  int bn_bits, requant, shift;
  long long lambda, out_add;
};

// ---------------------------------------------------------------------------------------------
// Per-thread context
// ---------------------------------------------------------------------------------------------
struct StageSlot { void *dev = nullptr; size_t cap = 0; };

struct Context {
  int device = -1;
  cudaStream_t stream = nullptr;
  int batch = 1;
  int err = PULPNN_OK;
  char msg[512] = {0};
  int opt_force_generic = 0;
  int opt_maxpool_clobber = 0;
  int opt_split_k = 0;
  int opt_tune = 0;               // experiment switch: alternative kernel configurations (bit mask)
  int opt_fuse_dwpw = 1;          // the network runner pairs depthwise + pointwise layers into one kernel
  StageSlot slots[8];
  // device scratch owned by the context (split-K partial sums, status word)
  void *scratch = nullptr; size_t scratch_cap = 0;
  int *status_word = nullptr;     // device int, 0 = fine
  int sm_count = 0;
};

Context &ctx();
bool ensure_device(Context &c);
void set_error(int code, const char *fmt, ...);
bool cuda_ok(cudaError_t e, const char *what);
void count_launch(unsigned n = 1);
void count_launch(const char *kernel_name);     // one launch, and remembers which kernel family it was
unsigned long long thread_launch_count();       // launches made by the calling thread so far
const char *thread_last_kernel();               // the kernel family of the calling thread's latest named launch

// Programmatic dependent launch. A kernel launched this way may become resident and run its
// prologue while the previous kernel of the stream is still draining; it must execute pdl_wait()
// before it reads anything an earlier kernel wrote or writes anything an earlier kernel may still
// read (the wait returns once the earlier grids have completed and their writes are visible).
// pdl_launch_dependents() lets the NEXT kernel of the stream do the same with respect to this one.
// Both are no-ops in a kernel launched the ordinary way.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args &&...args)
{
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif
void *ctx_scratch(Context &c, size_t bytes);    // grow-only device scratch, nullptr on failure

// A per-kernel setting that belongs to a device (cudaFuncSetAttribute, an occupancy figure) is
// cached per device, not per process or per thread: one process may drive several GPUs, from one
// thread that rebinds its context or from a thread per GPU.
constexpr int MAX_DEVICES = 64;
struct PerDeviceInt {
  std::atomic<int> v[MAX_DEVICES];
  PerDeviceInt() { for (auto &x : v) x.store(0, std::memory_order_relaxed); }
  int get(int dev) const { return (dev >= 0 && dev < MAX_DEVICES) ? v[dev].load(std::memory_order_acquire) : 0; }
  void set(int dev, int val) { if (dev >= 0 && dev < MAX_DEVICES) v[dev].store(val, std::memory_order_release); }
};

// Stages host buffers through device memory. Device pointers pass through untouched.
class Stager {
 public:
  explicit Stager(Context &c) : c_(c) {}
  const void *in(const void *p, size_t bytes);
  void *out(void *p, size_t bytes);
  void *inout(void *p, size_t bytes);
  bool ok() const { return ok_; }
  // copies results back and waits if any buffer was staged; returns false on a CUDA error
  bool finish();
 private:
  void *stage(const void *p, size_t bytes, bool copy_in, bool copy_out);
  Context &c_;
  struct Pending { void *host; void *dev; size_t bytes; } pend_[8];
  int n_pend_ = 0, n_slot_ = 0;
  bool ok_ = true, staged_ = false;
};

// ---------------------------------------------------------------------------------------------
// Launchers (each returns false and records an error when the launch could not be made)
// ---------------------------------------------------------------------------------------------
bool launch_conv(Context &c, const ConvProblem &p);             // picks tensor-core or generic
bool launch_conv_generic(Context &c, const ConvProblem &p);
bool conv_smallcin_tc_supported(const ConvProblem &p);
bool launch_conv_smallcin_tc(Context &c, const ConvProblem &p);
bool conv_smallcin_supported(const ConvProblem &p);
bool launch_conv_smallcin(Context &c, const ConvProblem &p);
bool igemm_tc_supported(const Context &c, const ConvProblem &p);
bool launch_igemm_tc(Context &c, const ConvProblem &p);
// the same GEMM computed by pairs of SMs (tcgen05 cta_group::2), for wide layers with a long reduction
bool igemm_tc2_supported(const Context &c, const ConvProblem &p);
bool launch_igemm_tc2(Context &c, const ConvProblem &p);
// the same contraction for few rows (a fully connected layer at a small batch), on dp4a
bool gemm_fewrows_supported(const ConvProblem &p);
bool launch_gemm_fewrows(Context &c, const ConvProblem &p);
bool launch_depthwise(Context &c, const DepthwiseProblem &p);
bool depthwise_hwc3x3_supported(const DepthwiseProblem &p);
bool launch_depthwise_hwc3x3(Context &c, const DepthwiseProblem &p);
bool depthwise_hwc3x3_tma_supported(const DepthwiseProblem &p);
bool launch_depthwise_hwc3x3_tma(Context &c, const DepthwiseProblem &p);
bool depthwise_chw3x3_tma_supported(const DepthwiseProblem &p);
bool launch_depthwise_chw3x3_tma(Context &c, const DepthwiseProblem &p);
// a 3x3 stride-1 depthwise layer and the pointwise layer behind it in one kernel (dwpw_fused.cu)
bool dwpw_fused_supported(const DepthwiseProblem &dw, const ConvProblem &pw);
bool launch_dwpw_fused(Context &c, const DepthwiseProblem &dw, const ConvProblem &pw);
// the 32 -> 64 channel pair with the depthwise layer on the tensor cores too (dwpw_tcdw.cu)
bool dwpw_tcdw_supported(const DepthwiseProblem &dw, const ConvProblem &pw);
bool launch_dwpw_tcdw(Context &c, const DepthwiseProblem &dw, const ConvProblem &pw);
bool depthwise_chw3x3_supported(const DepthwiseProblem &p);
bool launch_depthwise_chw3x3(Context &c, const DepthwiseProblem &p);
int *ctx_status_word(Context &c);               // allocated on first use; nullptr on failure
int static_scratch_status_take(Context &c);     // status of the no-allocation entry point (0: unused or fine)
bool launch_maxpool(Context &c, const PoolProblem &p, uint8_t *clobber_in);
bool launch_avgpool(Context &c, const PoolProblem &p);
bool launch_add(Context &c, const uint8_t *a, const uint8_t *b, uint8_t *out, size_t n, int m1,
                int m2, int shift);

}  // namespace pulpnn
