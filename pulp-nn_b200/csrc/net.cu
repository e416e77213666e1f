// net.cu -- sequential network runner: the chain of kernel calls a user of the reference library
// writes by hand, held as a list of layers with device-resident parameters and two ping-pong
// activation buffers. Images are independent, so a batch is pushed through the stack in
// micro-batches; every layer call goes through the same launchers as the C entry points.
#include <cstring>
#include <new>
#include <vector>

#include "internal.cuh"

using namespace pulpnn;

namespace {

struct Layer {
  pulpnn_layer_desc_t d;
  const int8_t *w = nullptr;
  const void *bias = nullptr, *k = nullptr, *lambda = nullptr;
  size_t in_bytes = 0, out_bytes = 0;      // per image
  int mode = EPI_NONE;
  FoldedWeights folded;                    // device copies owned by the network
};

bool is_device_ptr(const void *p)
{
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
  return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

}  // namespace

struct pulpnn_net {
  int bn_bits = 32, max_batch = 1, micro = 0;
  bool finalized = false;
  std::vector<Layer> layers;
  std::vector<void *> owned;               // device allocations holding parameters
  uint8_t *act[2] = {nullptr, nullptr};
  size_t act_bytes = 0;                    // per buffer
  uint8_t *stage_in = nullptr; size_t stage_in_cap = 0;
  uint8_t *stage_out = nullptr; size_t stage_out_cap = 0;
  cudaStream_t copy_stream = nullptr;
  // pipelined host-buffer runs (pulpnn_net_submit / pulpnn_net_wait): two staging slots, so that the
  // copies of one batch overlap the compute of the other
  uint8_t *slot_in[2] = {nullptr, nullptr}, *slot_out[2] = {nullptr, nullptr};
  size_t slot_in_cap[2] = {0, 0}, slot_out_cap[2] = {0, 0};
  cudaStream_t out_stream = nullptr;
  cudaEvent_t ev_compute[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
  bool slot_busy[2] = {false, false};
  unsigned long long submitted = 0;
  unsigned long long launches_last_run = 0;
  std::vector<char> role_last_run;         // per layer: 0 own kernel, 1 / 2 first / second layer of a fused pair
  std::vector<const char *> kernel_last_run;   // per layer: the kernel family that ran it
  cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_done[2] = {nullptr, nullptr};
};

namespace {

const void *upload(pulpnn_net *net, const void *src, size_t bytes)
{
  if (!src || bytes == 0) return nullptr;
  void *dev = nullptr;
  if (!cuda_ok(cudaMalloc(&dev, (bytes + 255) & ~(size_t)255), "cudaMalloc(parameters)")) return nullptr;
  net->owned.push_back(dev);
  const cudaMemcpyKind kind = is_device_ptr(src) ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
  if (!cuda_ok(cudaMemcpy(dev, src, bytes, kind), "parameter upload")) return nullptr;
  return dev;
}

Epilogue layer_epilogue(const Layer &L)
{
  Epilogue e;
  e.k = L.k; e.lambda = L.lambda; e.bias = L.bias; e.mode = L.mode;
  e.out_mult = (int)(int16_t)(uint16_t)L.d.out_mult; e.shift = L.d.out_shift;
  return e;
}

ConvProblem conv_problem(Layer &L, const uint8_t *in, void *out, int n)
{
  const pulpnn_layer_desc_t &d = L.d;
  ConvProblem p;
  p.in = in; p.w = L.w; p.out = out; p.epi = layer_epilogue(L); p.folded = &L.folded;
  p.B = n; p.H = d.dim_in_y; p.W = d.dim_in_x; p.Cin = d.ch_in; p.Ho = d.dim_out_y; p.Wo = d.dim_out_x;
  p.Cout = d.ch_out;
  if (d.type == PULPNN_LAYER_CONV) {
    p.ky = d.dim_kernel_y; p.kx = d.dim_kernel_x; p.pt = d.padding_y_top; p.pl = d.padding_x_left;
    p.sy = d.stride_y; p.sx = d.stride_x;
  } else {
    p.ky = p.kx = 1; p.pt = p.pl = 0; p.sy = p.sx = 1;
  }
  return p;
}

DepthwiseProblem depthwise_problem(const Layer &L, const uint8_t *in, void *out, int n)
{
  const pulpnn_layer_desc_t &d = L.d;
  DepthwiseProblem p;
  p.in = in; p.w = L.w; p.out = static_cast<uint8_t *>(out); p.epi = layer_epilogue(L);
  p.B = n; p.H = d.dim_in_y; p.W = d.dim_in_x; p.C = d.ch_in; p.Ho = d.dim_out_y; p.Wo = d.dim_out_x;
  p.ky = d.dim_kernel_y; p.kx = d.dim_kernel_x; p.pt = d.padding_y_top; p.pl = d.padding_x_left;
  p.sy = d.stride_y; p.sx = d.stride_x; p.in_is_hwc = true;
  return p;
}

bool run_layer(Context &c, const pulpnn_net *net, Layer &L, const uint8_t *in, void *out, int n)
{
  const pulpnn_layer_desc_t &d = L.d;
  switch (d.type) {
    case PULPNN_LAYER_CONV:
    case PULPNN_LAYER_POINTWISE:
    case PULPNN_LAYER_LINEAR_OUT_32:
      return launch_conv(c, conv_problem(L, in, out, n));
    case PULPNN_LAYER_DEPTHWISE:
      return launch_depthwise(c, depthwise_problem(L, in, out, n));
    case PULPNN_LAYER_AVGPOOL:
    case PULPNN_LAYER_MAXPOOL: {
      PoolProblem p{};
      p.in = in; p.out = static_cast<uint8_t *>(out);
      p.B = n; p.H = d.dim_in_y; p.W = d.dim_in_x; p.C = d.ch_in; p.Ho = d.dim_out_y; p.Wo = d.dim_out_x;
      p.ky = d.dim_kernel_y; p.kx = d.dim_kernel_x; p.pt = d.padding_y_top; p.pb = d.padding_y_bottom;
      p.pl = d.padding_x_left; p.pr = d.padding_x_right; p.sy = d.stride_y; p.sx = d.stride_x;
      p.bn_bits = net->bn_bits; p.requant = 0; p.shift = 0; p.lambda = 0; p.out_add = 0;
      return d.type == PULPNN_LAYER_AVGPOOL ? launch_avgpool(c, p) : launch_maxpool(c, p, nullptr);
    }
    default:
      set_error(PULPNN_ERR_INVALID_ARG, "unknown layer type %d", d.type);
      return false;
  }
}

// Layers l (depthwise) and l+1 (pointwise) as one kernel, the depthwise output never leaving the
// SM? Only where a fused kernel exists for the pair's shape and both layers requantise the same way.
bool pair_is_fusable(Context &c, pulpnn_net *net, int l, int n_layers, const uint8_t *in, void *out, int n)
{
  if (!c.opt_fuse_dwpw || l + 1 >= n_layers) return false;
  Layer &A = net->layers[l], &B = net->layers[l + 1];
  if (A.d.type != PULPNN_LAYER_DEPTHWISE || B.d.type != PULPNN_LAYER_POINTWISE) return false;
  return dwpw_fused_supported(depthwise_problem(A, in, nullptr, n), conv_problem(B, nullptr, out, n));
}

// pushes images [0, n) that already sit in device memory through layers [0, n_layers)
bool run_device(Context &c, pulpnn_net *net, const uint8_t *din, uint8_t *dout, int n, int n_layers,
                std::vector<cudaEvent_t> *marks = nullptr)
{
  const int micro = net->micro > 0 ? net->micro : n;
  const size_t in_b = net->layers.front().in_bytes;
  const size_t out_b = net->layers[n_layers - 1].out_bytes;
  for (int i0 = 0; i0 < n; i0 += micro) {
    const int nb = n - i0 < micro ? n - i0 : micro;
    const uint8_t *cur = din + (size_t)i0 * in_b;
    int cur_buf = -1;                      // which ping-pong buffer holds `cur` (-1: the caller's input)
    for (int l = 0; l < n_layers; l++) {
      auto mark = [&]() {
        if (!marks) return true;
        cudaEvent_t ev;
        if (!cuda_ok(cudaEventCreate(&ev), "cudaEventCreate")) return false;
        cudaEventRecord(ev, c.stream);
        marks->push_back(ev);
        return true;
      };
      // where the output of layer `last` goes: the caller's buffer for the final layer, else the
      // ping-pong buffer that does not hold the current input
      const int other = cur_buf == 0 ? 1 : 0;
      auto dest = [&](int last) -> void * {
        if (last == n_layers - 1) return static_cast<void *>(dout + (size_t)i0 * out_b);
        return static_cast<void *>(net->act[other]);
      };
      if (!mark()) return false;
      if (pair_is_fusable(c, net, l, n_layers, cur, dest(l + 1), nb)) {
        void *dst = dest(l + 1);
        if (!launch_dwpw_fused(c, depthwise_problem(net->layers[l], cur, nullptr, nb),
                               conv_problem(net->layers[l + 1], nullptr, dst, nb)))
          return false;
        cur = static_cast<const uint8_t *>(dst);
        cur_buf = other;
        net->role_last_run[l] = 1; net->role_last_run[l + 1] = 2;
        net->kernel_last_run[l] = net->kernel_last_run[l + 1] = thread_last_kernel();
        l++;
        if (!mark()) return false;         // the pair's time is booked on the depthwise layer, none on the pointwise
        continue;
      }
      cur_buf = other;
      net->role_last_run[l] = 0;
      void *dst = dest(l);
      if (!run_layer(c, net, net->layers[l], cur, dst, nb)) return false;
      net->kernel_last_run[l] = thread_last_kernel();
      cur = static_cast<const uint8_t *>(dst);
    }
  }
  if (marks) {
    cudaEvent_t ev;
    if (!cuda_ok(cudaEventCreate(&ev), "cudaEventCreate")) return false;
    cudaEventRecord(ev, c.stream);
    marks->push_back(ev);
  }
  return true;
}

// Host input: copied in a few slices on a second stream, each slice going through the whole stack as
// soon as it has landed, so that the copy of slice i+1 overlaps the compute of slice i. With a
// micro-batch set, a slice is a whole number of micro-batches.
bool enqueue_sliced(Context &c, pulpnn_net *net, const uint8_t *input, uint8_t *stage, uint8_t *dout, int n, int n_layers)
{
  const int micro = net->micro > 0 ? net->micro : n;
  int sizes[64];
  int n_slices = 0;
  {
    const int want = 4;        // measured at batch 1024: 5 slices lose 2 %, 6 lose 5 %, 8 lose 7 %
    const int part = (n + want - 1) / want;
    int slice = micro < part ? micro : part;
    while (slice < n && slice * want < n) slice += micro;
    for (int left = n; left > 0 && n_slices < 64; left -= slice) sizes[n_slices++] = left < slice ? left : slice;
  }
  const size_t img_in = net->layers.front().in_bytes, img_out = net->layers[n_layers - 1].out_bytes;
  int i0 = 0;
  for (int idx = 0; idx < n_slices; idx++) {
    const int nb = sizes[idx];
    cudaEvent_t ev = net->ev_in[idx & 1];
    if (!cuda_ok(cudaMemcpyAsync(stage + (size_t)i0 * img_in, input + (size_t)i0 * img_in,
                                 (size_t)nb * img_in, cudaMemcpyHostToDevice, net->copy_stream), "H2D copy"))
      return false;
    cudaEventRecord(ev, net->copy_stream);
    cudaStreamWaitEvent(c.stream, ev, 0);
    if (!run_device(c, net, stage + (size_t)i0 * img_in, dout + (size_t)i0 * img_out, nb, n_layers)) return false;
    i0 += nb;
  }
  return true;
}

int run_impl(pulpnn_net *net, const uint8_t *input, void *output, int n, int n_layers)
{
  Context &c = ctx();
  if (!ensure_device(c)) return c.err;
  if (!net || !net->finalized) { set_error(PULPNN_ERR_INVALID_ARG, "network is not finalized"); return c.err; }
  if (!input || !output || n < 1 || n > net->max_batch || n_layers < 1 || n_layers > (int)net->layers.size()) {
    set_error(PULPNN_ERR_INVALID_ARG, "pulpnn_net_run: bad arguments (n=%d, max_batch=%d)", n, net->max_batch);
    return c.err;
  }
  const size_t in_b = net->layers.front().in_bytes * n;
  const size_t out_b = net->layers[n_layers - 1].out_bytes * n;
  const bool in_dev = is_device_ptr(input), out_dev = is_device_ptr(output);
  const unsigned long long launches0 = thread_launch_count();
  const uint8_t *din = input;
  uint8_t *dout = static_cast<uint8_t *>(output);
  if (!in_dev) {
    if (net->stage_in_cap < in_b) {
      if (net->stage_in) { cudaStreamSynchronize(c.stream); cudaFree(net->stage_in); }
      net->stage_in = nullptr; net->stage_in_cap = 0;
      if (!cuda_ok(cudaMalloc(&net->stage_in, in_b), "cudaMalloc(input staging)")) return c.err;
      net->stage_in_cap = in_b;
    }
    din = net->stage_in;
  }
  if (!out_dev) {
    if (net->stage_out_cap < out_b) {
      if (net->stage_out) { cudaStreamSynchronize(c.stream); cudaFree(net->stage_out); }
      net->stage_out = nullptr; net->stage_out_cap = 0;
      if (!cuda_ok(cudaMalloc(&net->stage_out, out_b), "cudaMalloc(output staging)")) return c.err;
      net->stage_out_cap = out_b;
    }
    dout = net->stage_out;
  }

  if (in_dev) {
    if (!run_device(c, net, din, dout, n, n_layers)) return c.err;
  } else {
    // The copy is the longer of the two (154 MB of images take longer to cross PCIe than to classify),
    // so what the overlap inside one call cannot hide is the compute of the last slice; equal slices
    // measured best. pulpnn_net_submit / pulpnn_net_wait hide that too, under the next batch's copy.
    if (!enqueue_sliced(c, net, input, net->stage_in, dout, n, n_layers)) return c.err;
  }
  net->launches_last_run = thread_launch_count() - launches0;
  if (!out_dev) {
    if (!cuda_ok(cudaMemcpyAsync(output, dout, out_b, cudaMemcpyDeviceToHost, c.stream), "D2H copy")) return c.err;
  }
  if (!in_dev || !out_dev) {
    if (!cuda_ok(cudaStreamSynchronize(c.stream), "cudaStreamSynchronize")) return c.err;
  }
  return PULPNN_OK;
}

}  // namespace

extern "C" {

pulpnn_net_t *pulpnn_net_create(int bn_bits, int max_batch)
{
  Context &c = ctx();
  if (!ensure_device(c)) return nullptr;
  if ((bn_bits != 32 && bn_bits != 64) || max_batch < 1) {
    set_error(PULPNN_ERR_INVALID_ARG, "pulpnn_net_create: bn_bits must be 32 or 64 and max_batch >= 1");
    return nullptr;
  }
  pulpnn_net *net = new (std::nothrow) pulpnn_net;
  if (!net) return nullptr;
  net->bn_bits = bn_bits;
  net->max_batch = max_batch;
  return net;
}

int pulpnn_net_add_layer(pulpnn_net_t *net, const pulpnn_layer_desc_t *desc)
{
  Context &c = ctx();
  if (!net || !desc || net->finalized) { set_error(PULPNN_ERR_INVALID_ARG, "pulpnn_net_add_layer: bad arguments"); return c.err; }
  if (!ensure_device(c)) return c.err;
  Layer L;
  L.d = *desc;
  const pulpnn_layer_desc_t &d = L.d;
  if (d.dim_in_x < 1 || d.dim_in_y < 1 || d.ch_in < 1 || d.dim_out_x < 1 || d.dim_out_y < 1 || d.ch_out < 1) {
    set_error(PULPNN_ERR_INVALID_ARG, "layer %zu: zero dimension", net->layers.size());
    return c.err;
  }
  L.in_bytes = (size_t)d.dim_in_x * d.dim_in_y * d.ch_in;
  L.out_bytes = (size_t)d.dim_out_x * d.dim_out_y * d.ch_out * (d.type == PULPNN_LAYER_LINEAR_OUT_32 ? 4 : 1);
  if (!net->layers.empty() && net->layers.back().out_bytes != L.in_bytes) {
    set_error(PULPNN_ERR_INVALID_ARG, "layer %zu: input size %zu does not match the previous output %zu",
              net->layers.size(), L.in_bytes, net->layers.back().out_bytes);
    return c.err;
  }
  if (!net->layers.empty() && net->layers.back().d.type == PULPNN_LAYER_LINEAR_OUT_32) {
    set_error(PULPNN_ERR_INVALID_ARG, "an int32-output layer must be the last one");
    return c.err;
  }
  const size_t bn_sz = net->bn_bits / 8;
  const int bn_mode = net->bn_bits == 32 ? EPI_BN32 : EPI_BN64;
  size_t wbytes = 0;
  switch (d.type) {
    case PULPNN_LAYER_CONV:
      wbytes = (size_t)d.ch_out * d.dim_kernel_x * d.dim_kernel_y * d.ch_in;
      L.mode = (d.flag_batch_norm && d.flag_relu) ? bn_mode : (d.flag_relu == 1 ? EPI_MULT : EPI_NONE);
      if ((d.dim_out_x - 1) * d.stride_x + d.dim_kernel_x > d.dim_in_x + d.padding_x_left + d.padding_x_right ||
          (d.dim_out_y - 1) * d.stride_y + d.dim_kernel_y > d.dim_in_y + d.padding_y_top + d.padding_y_bottom) {
        set_error(PULPNN_ERR_UNSUPPORTED, "layer %zu: inconsistent output size", net->layers.size());
        return c.err;
      }
      break;
    case PULPNN_LAYER_POINTWISE:
      wbytes = (size_t)d.ch_out * d.ch_in;
      L.mode = (d.flag_batch_norm && d.flag_relu) ? bn_mode : (d.flag_relu == 1 ? EPI_MULT : EPI_NONE);
      if (d.dim_in_x != d.dim_out_x || d.dim_in_y != d.dim_out_y) {
        set_error(PULPNN_ERR_UNSUPPORTED, "layer %zu: pointwise needs dim_in == dim_out", net->layers.size());
        return c.err;
      }
      break;
    case PULPNN_LAYER_DEPTHWISE:
      wbytes = (size_t)d.ch_in * d.dim_kernel_x * d.dim_kernel_y;
      L.mode = (d.flag_batch_norm && d.flag_relu) ? bn_mode : (d.flag_relu ? EPI_MULT : EPI_NONE);
      if (d.ch_in != d.ch_out) { set_error(PULPNN_ERR_UNSUPPORTED, "layer %zu: depthwise needs ch_in == ch_out", net->layers.size()); return c.err; }
      break;
    case PULPNN_LAYER_LINEAR_OUT_32:
      wbytes = (size_t)d.ch_out * L.in_bytes;
      L.d.ch_in = (int)L.in_bytes; L.d.dim_in_x = L.d.dim_in_y = 1;
      L.mode = EPI_RAW32;
      break;
    case PULPNN_LAYER_AVGPOOL:
    case PULPNN_LAYER_MAXPOOL:
      if (d.ch_in != d.ch_out) { set_error(PULPNN_ERR_UNSUPPORTED, "layer %zu: pooling needs ch_in == ch_out", net->layers.size()); return c.err; }
      break;
    default:
      set_error(PULPNN_ERR_INVALID_ARG, "layer %zu: unknown type %d", net->layers.size(), d.type);
      return c.err;
  }
  if (L.mode != EPI_RAW32 && wbytes) {
    const int hi = L.mode == EPI_BN64 ? 63 : 31;
    if (d.out_shift < 0 || d.out_shift > hi) { set_error(PULPNN_ERR_INVALID_ARG, "layer %zu: out_shift %d", net->layers.size(), d.out_shift); return c.err; }
  }
  if (wbytes) {
    if (!d.weights) { set_error(PULPNN_ERR_INVALID_ARG, "layer %zu: weights missing", net->layers.size()); return c.err; }
    L.w = static_cast<const int8_t *>(upload(net, d.weights, wbytes));
    if (!L.w) return c.err;
    if (d.bias) {
      L.bias = upload(net, d.bias, (size_t)d.ch_out * (d.type == PULPNN_LAYER_LINEAR_OUT_32 ? 4 : 1));
      if (!L.bias) return c.err;
    }
    if (L.mode == EPI_BN32 || L.mode == EPI_BN64) {
      if (!d.k || !d.lambda) { set_error(PULPNN_ERR_INVALID_ARG, "layer %zu: batch-norm parameters missing", net->layers.size()); return c.err; }
      L.k = upload(net, d.k, bn_sz * d.ch_out);
      L.lambda = upload(net, d.lambda, bn_sz * d.ch_out);
      if (!L.k || !L.lambda) return c.err;
    }
  }
  L.d.weights = nullptr; L.d.bias = nullptr; L.d.k = L.d.lambda = nullptr;
  net->layers.push_back(L);
  return PULPNN_OK;
}

int pulpnn_net_finalize(pulpnn_net_t *net, int micro_batch)
{
  Context &c = ctx();
  if (!net || net->finalized || net->layers.empty()) { set_error(PULPNN_ERR_INVALID_ARG, "pulpnn_net_finalize: bad arguments"); return c.err; }
  if (!ensure_device(c)) return c.err;
  size_t biggest = 0;
  for (size_t l = 0; l + 1 < net->layers.size(); l++) biggest = net->layers[l].out_bytes > biggest ? net->layers[l].out_bytes : biggest;
  int micro = micro_batch > 0 ? micro_batch : net->max_batch;
  if (micro > net->max_batch) micro = net->max_batch;
  net->micro = micro;
  net->act_bytes = biggest * micro;
  for (int i = 0; i < 2; i++) {
    if (net->act_bytes && !cuda_ok(cudaMalloc(&net->act[i], net->act_bytes), "cudaMalloc(activations)")) return c.err;
    if (!cuda_ok(cudaEventCreateWithFlags(&net->ev_in[i], cudaEventDisableTiming), "cudaEventCreate")) return c.err;
    if (!cuda_ok(cudaEventCreateWithFlags(&net->ev_done[i], cudaEventDisableTiming), "cudaEventCreate")) return c.err;
  }
  if (!cuda_ok(cudaStreamCreateWithFlags(&net->copy_stream, cudaStreamNonBlocking), "cudaStreamCreate")) return c.err;
  net->role_last_run.assign(net->layers.size(), 0);
  net->kernel_last_run.assign(net->layers.size(), "");
  net->finalized = true;
  return PULPNN_OK;
}

int pulpnn_net_run(pulpnn_net_t *net, const uint8_t *input, void *output, int n_images)
{
  return run_impl(net, input, output, n_images, net ? (int)net->layers.size() : 0);
}

int pulpnn_net_submit(pulpnn_net_t *net, const uint8_t *input, void *output, int n_images)
{
  Context &c = ctx();
  if (!ensure_device(c)) return -c.err;
  if (!net || !net->finalized || !input || !output || n_images < 1 || n_images > net->max_batch) {
    set_error(PULPNN_ERR_INVALID_ARG, "pulpnn_net_submit: bad arguments");
    return -c.err;
  }
  if (is_device_ptr(input) || is_device_ptr(output)) {
    set_error(PULPNN_ERR_INVALID_ARG, "pulpnn_net_submit is for host buffers; device buffers need no staging: use pulpnn_net_run");
    return -c.err;
  }
  const int nl = (int)net->layers.size();
  const int b = (int)(net->submitted & 1);
  if (net->slot_busy[b]) {            // the caller did not collect this slot's previous batch: do it for him
    if (!cuda_ok(cudaEventSynchronize(net->ev_out[b]), "cudaEventSynchronize")) return -c.err;
    net->slot_busy[b] = false;
  }
  const size_t in_b = net->layers.front().in_bytes * n_images, out_b = net->layers[nl - 1].out_bytes * n_images;
  if (!net->out_stream) {
    if (!cuda_ok(cudaStreamCreateWithFlags(&net->out_stream, cudaStreamNonBlocking), "cudaStreamCreate")) return -c.err;
    for (int i = 0; i < 2; i++) {
      if (!cuda_ok(cudaEventCreateWithFlags(&net->ev_compute[i], cudaEventDisableTiming), "cudaEventCreate")) return -c.err;
      if (!cuda_ok(cudaEventCreateWithFlags(&net->ev_out[i], cudaEventDisableTiming), "cudaEventCreate")) return -c.err;
    }
  }
  if (net->slot_in_cap[b] < in_b) {
    if (net->slot_in[b]) { cudaDeviceSynchronize(); cudaFree(net->slot_in[b]); net->slot_in[b] = nullptr; net->slot_in_cap[b] = 0; }
    if (!cuda_ok(cudaMalloc(&net->slot_in[b], in_b), "cudaMalloc(input staging)")) return -c.err;
    net->slot_in_cap[b] = in_b;
  }
  if (net->slot_out_cap[b] < out_b) {
    if (net->slot_out[b]) { cudaDeviceSynchronize(); cudaFree(net->slot_out[b]); net->slot_out[b] = nullptr; net->slot_out_cap[b] = 0; }
    if (!cuda_ok(cudaMalloc(&net->slot_out[b], out_b), "cudaMalloc(output staging)")) return -c.err;
    net->slot_out_cap[b] = out_b;
  }
  // this slot's staging buffers were last used two batches ago: the copies wait for that batch's
  // compute to have read the input, the compute for its results to have left
  if (net->submitted >= 2) {
    cudaStreamWaitEvent(net->copy_stream, net->ev_compute[b], 0);
    cudaStreamWaitEvent(c.stream, net->ev_out[b], 0);
  }
  const unsigned long long launches0 = thread_launch_count();
  if (!enqueue_sliced(c, net, input, net->slot_in[b], net->slot_out[b], n_images, nl)) return -c.err;
  net->launches_last_run = thread_launch_count() - launches0;
  cudaEventRecord(net->ev_compute[b], c.stream);
  cudaStreamWaitEvent(net->out_stream, net->ev_compute[b], 0);
  if (!cuda_ok(cudaMemcpyAsync(output, net->slot_out[b], out_b, cudaMemcpyDeviceToHost, net->out_stream), "D2H copy")) return -c.err;
  cudaEventRecord(net->ev_out[b], net->out_stream);
  net->slot_busy[b] = true;
  net->submitted++;
  return b;
}

int pulpnn_net_wait(pulpnn_net_t *net, int ticket)
{
  Context &c = ctx();
  if (!net || ticket < 0 || ticket > 1) { set_error(PULPNN_ERR_INVALID_ARG, "pulpnn_net_wait: bad ticket"); return c.err; }
  if (!net->slot_busy[ticket]) return PULPNN_OK;
  if (!cuda_ok(cudaEventSynchronize(net->ev_out[ticket]), "cudaEventSynchronize")) return c.err;
  net->slot_busy[ticket] = false;
  return PULPNN_OK;
}

int pulpnn_net_run_prefix(pulpnn_net_t *net, const uint8_t *input, void *output, int n_images, int n_layers)
{
  return run_impl(net, input, output, n_images, n_layers);
}

int pulpnn_net_run_timed(pulpnn_net_t *net, const uint8_t *input, void *output, int n_images, float *layer_ms)
{
  Context &c = ctx();
  if (!ensure_device(c)) return c.err;
  if (!net || !net->finalized || !input || !output || !layer_ms || n_images < 1 || n_images > net->max_batch) {
    set_error(PULPNN_ERR_INVALID_ARG, "pulpnn_net_run_timed: bad arguments");
    return c.err;
  }
  if (!is_device_ptr(input) || !is_device_ptr(output)) {
    set_error(PULPNN_ERR_INVALID_ARG, "pulpnn_net_run_timed: buffers must be device memory");
    return c.err;
  }
  const int nl = (int)net->layers.size();
  std::vector<cudaEvent_t> marks;
  const unsigned long long launches0 = thread_launch_count();
  bool ok = run_device(c, net, input, static_cast<uint8_t *>(output), n_images, nl, &marks);
  net->launches_last_run = thread_launch_count() - launches0;
  ok = ok && cuda_ok(cudaStreamSynchronize(c.stream), "cudaStreamSynchronize");
  if (ok) {
    for (int l = 0; l < nl; l++) layer_ms[l] = 0.f;
    // marks: one event before every layer call of every micro-batch, plus one at the very end
    for (size_t i = 0; i + 1 < marks.size(); i++) {
      float ms = 0.f;
      cudaEventElapsedTime(&ms, marks[i], marks[i + 1]);
      layer_ms[i % nl] += ms;
    }
  }
  for (cudaEvent_t ev : marks) cudaEventDestroy(ev);
  // only this call's own failures count: an error left on the thread by an earlier call is not ours
  return ok ? PULPNN_OK : (c.err ? c.err : PULPNN_ERR_CUDA);
}

int pulpnn_net_num_layers(const pulpnn_net_t *net) { return net ? (int)net->layers.size() : 0; }

size_t pulpnn_net_layer_output_bytes(const pulpnn_net_t *net, int layer)
{
  if (!net || layer < 0 || layer >= (int)net->layers.size()) return 0;
  return net->layers[layer].out_bytes;
}

int pulpnn_net_layer_role(const pulpnn_net_t *net, int layer)
{
  if (!net || layer < 0 || layer >= (int)net->role_last_run.size()) return -1;
  return net->role_last_run[layer];
}

const char *pulpnn_net_layer_kernel(const pulpnn_net_t *net, int layer)
{
  if (!net || layer < 0 || layer >= (int)net->kernel_last_run.size()) return "";
  return net->kernel_last_run[layer];
}

unsigned long long pulpnn_net_launches_per_run(const pulpnn_net_t *net, int n_images)
{
  (void)n_images;
  return net ? net->launches_last_run : 0;
}

void pulpnn_net_destroy(pulpnn_net_t *net)
{
  if (!net) return;
  cudaDeviceSynchronize();
  for (void *p : net->owned) cudaFree(p);
  for (Layer &L : net->layers)
    for (int8_t *wf : L.folded.w) if (wf) cudaFree(wf);
  for (int i = 0; i < 2; i++) {
    if (net->act[i]) cudaFree(net->act[i]);
    if (net->ev_in[i]) cudaEventDestroy(net->ev_in[i]);
    if (net->ev_done[i]) cudaEventDestroy(net->ev_done[i]);
  }
  if (net->stage_in) cudaFree(net->stage_in);
  if (net->stage_out) cudaFree(net->stage_out);
  for (int i = 0; i < 2; i++) {
    if (net->slot_in[i]) cudaFree(net->slot_in[i]);
    if (net->slot_out[i]) cudaFree(net->slot_out[i]);
    if (net->ev_compute[i]) cudaEventDestroy(net->ev_compute[i]);
    if (net->ev_out[i]) cudaEventDestroy(net->ev_out[i]);
  }
  if (net->out_stream) cudaStreamDestroy(net->out_stream);
  if (net->copy_stream) cudaStreamDestroy(net->copy_stream);
  delete net;
}

}  // extern "C"
