// diagnostics.cu -- a self-test of the bounded-wait machinery: a kernel whose wait is meant to run out.
#include "internal.cuh"
#include "sm100_primitives.cuh"

namespace pulpnn {
namespace {

using namespace sm100;
constexpr int ST_SELFTEST = 0x4000;

// One warp; lane 0 waits on an mbarrier that expects one arrival nobody makes. The wait gives up
// after limit_ns, raises the (shared-memory) abort flag and ors ST_SELFTEST into the status word:
// the same code path a protocol error inside a production kernel would take.
__global__ void __launch_bounds__(32) wait_timeout_probe_kernel(int *status, unsigned long long limit_ns)
{
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) mbar_wait(&bar, 0, &abort_flag, status, ST_SELFTEST, limit_ns);
}

}  // namespace
}  // namespace pulpnn

using namespace pulpnn;

extern "C" int pulpnn_selftest_wait_timeout(unsigned int limit_us)
{
  Context &c = ctx();
  if (!ensure_device(c)) return c.err;
  if (limit_us < 1) limit_us = 1;
  if (limit_us > 100000) limit_us = 100000;
  int *status = ctx_status_word(c);
  if (!status) return c.err;
  wait_timeout_probe_kernel<<<1, 32, 0, c.stream>>>(status, (unsigned long long)limit_us * 1000ull);
  count_launch();
  if (!cuda_ok(cudaGetLastError(), "wait_timeout_probe launch")) return c.err;
  return PULPNN_OK;
}
