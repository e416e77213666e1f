// context.cu -- per-thread context, error reporting, host-buffer staging.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <atomic>

#include "internal.cuh"

namespace pulpnn {

static std::atomic<unsigned long long> g_launches{0};

Context &ctx()
{
  static thread_local Context c;
  return c;
}

static thread_local unsigned long long t_launches = 0;

void count_launch(unsigned n)
{
  g_launches.fetch_add(n, std::memory_order_relaxed);
  t_launches += n;
}
unsigned long long thread_launch_count() { return t_launches; }

static thread_local const char *t_last_kernel = "";
void count_launch(const char *kernel_name)
{
  count_launch(1u);
  t_last_kernel = kernel_name;
}
const char *thread_last_kernel() { return t_last_kernel; }

void set_error(int code, const char *fmt, ...)
{
  Context &c = ctx();
  c.err = code;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(c.msg, sizeof(c.msg), fmt, ap);
  va_end(ap);
}

bool cuda_ok(cudaError_t e, const char *what)
{
  if (e == cudaSuccess) return true;
  set_error(PULPNN_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return false;
}

// Binds the context to a device on first use. Without a GPU every entry point fails here:
// nothing in this library computes on the host.
bool ensure_device(Context &c)
{
  if (c.device >= 0) {
    int cur = -1;
    if (cudaGetDevice(&cur) == cudaSuccess && cur != c.device) cudaSetDevice(c.device);
    return true;
  }
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n <= 0) {
    cudaGetLastError();
    set_error(PULPNN_ERR_NO_DEVICE, "no CUDA device is available (%s); this library has no CPU path",
              e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    return false;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) dev = 0;
  if (!cuda_ok(cudaSetDevice(dev), "cudaSetDevice")) return false;
  c.device = dev;
  cudaDeviceProp prop;
  if (cuda_ok(cudaGetDeviceProperties(&prop, dev), "cudaGetDeviceProperties")) {
    c.sm_count = prop.multiProcessorCount;
    if (prop.major != 10) {
      set_error(PULPNN_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only",
                dev, prop.major, prop.minor);
      c.device = -1;
      return false;
    }
  }
  return true;
}

void *ctx_scratch(Context &c, size_t bytes)
{
  if (bytes <= c.scratch_cap) return c.scratch;
  if (c.scratch) {
    cudaStreamSynchronize(c.stream);
    cudaFree(c.scratch);
    c.scratch = nullptr; c.scratch_cap = 0;
  }
  size_t cap = (bytes + (1u << 20) - 1) & ~(size_t)((1u << 20) - 1);
  if (!cuda_ok(cudaMalloc(&c.scratch, cap), "cudaMalloc(scratch)")) return nullptr;
  c.scratch_cap = cap;
  return c.scratch;
}

// device word that kernels with bounded waits report into (read by pulpnn_device_status)
int *ctx_status_word(Context &c)
{
  if (!c.status_word) {
    if (!cuda_ok(cudaMalloc(&c.status_word, sizeof(int)), "cudaMalloc(status)")) return nullptr;
    if (!cuda_ok(cudaMemsetAsync(c.status_word, 0, sizeof(int), c.stream), "cudaMemset(status)")) return nullptr;
  }
  return c.status_word;
}

// ---- staging ------------------------------------------------------------------------------
static bool is_device_pointer(const void *p)
{
  cudaPointerAttributes a;
  cudaError_t e = cudaPointerGetAttributes(&a, p);
  if (e != cudaSuccess) { cudaGetLastError(); return false; }
  return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

void *Stager::stage(const void *p, size_t bytes, bool copy_in, bool copy_out)
{
  if (!p || !ok_) return const_cast<void *>(p);
  if (is_device_pointer(p)) return const_cast<void *>(p);
  if (n_slot_ >= 8) { ok_ = false; set_error(PULPNN_ERR_INVALID_ARG, "too many host buffers"); return nullptr; }
  StageSlot &s = c_.slots[n_slot_++];
  if (s.cap < bytes) {
    if (s.dev) { cudaStreamSynchronize(c_.stream); cudaFree(s.dev); s.dev = nullptr; s.cap = 0; }
    size_t cap = (bytes + 4095) & ~(size_t)4095;
    if (!cuda_ok(cudaMalloc(&s.dev, cap), "cudaMalloc(staging)")) { ok_ = false; return nullptr; }
    s.cap = cap;
  }
  staged_ = true;
  if (copy_in &&
      !cuda_ok(cudaMemcpyAsync(s.dev, p, bytes, cudaMemcpyHostToDevice, c_.stream), "H2D copy")) {
    ok_ = false;
    return nullptr;
  }
  if (copy_out) {
    pend_[n_pend_].host = const_cast<void *>(p);
    pend_[n_pend_].dev = s.dev;
    pend_[n_pend_].bytes = bytes;
    n_pend_++;
  }
  return s.dev;
}

const void *Stager::in(const void *p, size_t bytes) { return stage(p, bytes, true, false); }
void *Stager::out(void *p, size_t bytes) { return stage(p, bytes, false, true); }
void *Stager::inout(void *p, size_t bytes) { return stage(p, bytes, true, true); }

bool Stager::finish()
{
  if (!staged_) return ok_;
  for (int i = 0; i < n_pend_ && ok_; i++)
    ok_ = cuda_ok(cudaMemcpyAsync(pend_[i].host, pend_[i].dev, pend_[i].bytes,
                                  cudaMemcpyDeviceToHost, c_.stream), "D2H copy");
  if (!cuda_ok(cudaStreamSynchronize(c_.stream), "cudaStreamSynchronize")) ok_ = false;
  return ok_;
}

}  // namespace pulpnn

using namespace pulpnn;

extern "C" {

int pulpnn_set_device(int device)
{
  Context &c = ctx();
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n <= 0) {
    cudaGetLastError();
    set_error(PULPNN_ERR_NO_DEVICE, "no CUDA device is available; this library has no CPU path");
    return c.err;
  }
  if (device < 0 || device >= n) {
    set_error(PULPNN_ERR_INVALID_ARG, "device %d out of range (0..%d)", device, n - 1);
    return c.err;
  }
  if (!cuda_ok(cudaSetDevice(device), "cudaSetDevice")) return c.err;
  if (c.device != device) {
    // buffers owned by the context belong to the old device
    for (auto &s : c.slots) { if (s.dev) cudaFree(s.dev); s.dev = nullptr; s.cap = 0; }
    if (c.scratch) cudaFree(c.scratch);
    c.scratch = nullptr; c.scratch_cap = 0;
    if (c.status_word) cudaFree(c.status_word);
    c.status_word = nullptr;
    c.device = -1;
  }
  if (!ensure_device(c)) return c.err;
  return PULPNN_OK;
}

int pulpnn_set_stream(void *cuda_stream)
{
  ctx().stream = reinterpret_cast<cudaStream_t>(cuda_stream);
  return PULPNN_OK;
}

int pulpnn_set_batch(int n)
{
  if (n < 1) { set_error(PULPNN_ERR_INVALID_ARG, "batch must be >= 1 (got %d)", n); return ctx().err; }
  ctx().batch = n;
  return PULPNN_OK;
}

int pulpnn_get_batch(void) { return ctx().batch; }

int pulpnn_synchronize(void)
{
  Context &c = ctx();
  if (!ensure_device(c)) return c.err;
  if (!cuda_ok(cudaStreamSynchronize(c.stream), "cudaStreamSynchronize")) return c.err;
  return PULPNN_OK;
}

int pulpnn_last_error(void) { return ctx().err; }
const char *pulpnn_last_error_message(void) { return ctx().msg; }
void pulpnn_clear_error(void) { ctx().err = PULPNN_OK; ctx().msg[0] = 0; }
unsigned long long pulpnn_launch_count(void) { return g_launches.load(); }

int pulpnn_device_status(void)
{
  Context &c = ctx();
  if (!ensure_device(c)) return -1;
  if (!cuda_ok(cudaStreamSynchronize(c.stream), "cudaStreamSynchronize")) return -1;
  int v = 0;
  if (c.status_word) {
    if (!cuda_ok(cudaMemcpy(&v, c.status_word, sizeof(int), cudaMemcpyDeviceToHost), "status read")) return -1;
    if (v != 0) cudaMemset(c.status_word, 0, sizeof(int));
  }
  // the entry point that must not allocate keeps its own word inside the library image
  const int s = static_scratch_status_take(c);
  if (s < 0) return -1;
  v |= s;
  if (v != 0)
    set_error(PULPNN_ERR_DEVICE_WAIT, "a bounded wait inside a tensor-core kernel ran out (code 0x%x)", v);
  return v;
}

int pulpnn_set_option(int option, int value)
{
  Context &c = ctx();
  switch (option) {
    case PULPNN_OPT_FORCE_GENERIC: c.opt_force_generic = value != 0; return PULPNN_OK;
    case PULPNN_OPT_MAXPOOL_CLOBBER: c.opt_maxpool_clobber = value != 0; return PULPNN_OK;
    case PULPNN_OPT_SPLIT_K: c.opt_split_k = value < 0 ? 0 : value; return PULPNN_OK;
    case PULPNN_OPT_FUSE_DWPW: c.opt_fuse_dwpw = value != 0; return PULPNN_OK;
    case PULPNN_OPT_TUNE: c.opt_tune = value; return PULPNN_OK;
    default: set_error(PULPNN_ERR_INVALID_ARG, "unknown option %d", option); return c.err;
  }
}

int pulpnn_get_option(int option)
{
  Context &c = ctx();
  switch (option) {
    case PULPNN_OPT_FORCE_GENERIC: return c.opt_force_generic;
    case PULPNN_OPT_MAXPOOL_CLOBBER: return c.opt_maxpool_clobber;
    case PULPNN_OPT_SPLIT_K: return c.opt_split_k;
    case PULPNN_OPT_FUSE_DWPW: return c.opt_fuse_dwpw;
    case PULPNN_OPT_TUNE: return c.opt_tune;
    default: return -1;
  }
}

}  // extern "C"
