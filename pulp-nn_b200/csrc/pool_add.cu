// pool_add.cu -- max pooling, average pooling and the residual add. All three are one pass over
// the input and one over the output; threads are laid out along the channel axis (HWC), four
// channels (one 32-bit word) per thread where the channel count allows, sixteen for the add.
#include "internal.cuh"

namespace pulpnn {

namespace {

__device__ __forceinline__ unsigned ld_bytes(const uint8_t *p, int n)
{
  unsigned v = 0;
  for (int j = 0; j < n; j++) v |= (unsigned)__ldg(p + j) << (8 * j);
  return v;
}
__device__ __forceinline__ void st_bytes(uint8_t *p, unsigned v, int n)
{
  for (int j = 0; j < n; j++) p[j] = (uint8_t)(v >> (8 * j));
}

// ---- max pooling ---------------------------------------------------------------------------
// The reference pools along x in place and then along y (32bit/src/pulp_nn_maxpool.c:58-144);
// with stride_x > padding_l (checked on the host) that equals the maximum over the window
// clipped to the image: rows [max(0, oy*sy - pt), min(oy*sy - pt + ky, H)), columns likewise
// with padding_l. padding_b / padding_r are never read by the reference.
template <bool VEC>
__global__ void __launch_bounds__(256) maxpool_kernel(const PoolProblem p, int CW, long long total)
{
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const int cw = (int)(t % CW);
  long long r = t / CW;
  const int ox = (int)(r % p.Wo); r /= p.Wo;
  const int oy = (int)(r % p.Ho);
  const int b = (int)(r / p.Ho);
  const int c = VEC ? cw * 4 : cw, nb = VEC ? 4 : 1;
  const int y0 = max(oy * p.sy - p.pt, 0), y1 = min(oy * p.sy - p.pt + p.ky, p.H);
  const int x0 = max(ox * p.sx - p.pl, 0), x1 = min(ox * p.sx - p.pl + p.kx, p.W);
  const uint8_t *img = p.in + (size_t)b * p.H * p.W * p.C + c;
  unsigned m = 0;
  for (int y = y0; y < y1; y++)
    for (int x = x0; x < x1; x++) {
      const uint8_t *q = img + ((size_t)y * p.W + x) * p.C;
      const unsigned v = VEC ? __ldg(reinterpret_cast<const unsigned *>(q)) : ld_bytes(q, nb);
      m = __vmaxu4(m, v);
    }
  uint8_t *o = p.out + (((size_t)b * p.Ho + oy) * p.Wo + ox) * p.C + c;
  if (VEC) *reinterpret_cast<unsigned *>(o) = m; else st_bytes(o, m, nb);
}

// The same for 16 channels per thread (C a multiple of 16, 16-byte aligned tensors, fewer than 2^31
// threads): 16-byte accesses and 32-bit index arithmetic. The four-channel kernel above spends its
// time on 64-bit divisions; this one reaches the memory system.
__global__ void __launch_bounds__(256) maxpool16_kernel(const PoolProblem p, int CW, unsigned total)
{
  const unsigned t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const unsigned cw = t % (unsigned)CW;
  unsigned r = t / (unsigned)CW;
  const int ox = (int)(r % (unsigned)p.Wo); r /= (unsigned)p.Wo;
  const int oy = (int)(r % (unsigned)p.Ho);
  const int b = (int)(r / (unsigned)p.Ho);
  const int y0 = max(oy * p.sy - p.pt, 0), y1 = min(oy * p.sy - p.pt + p.ky, p.H);
  const int x0 = max(ox * p.sx - p.pl, 0), x1 = min(ox * p.sx - p.pl + p.kx, p.W);
  const uint8_t *img = p.in + (size_t)b * p.H * p.W * p.C + cw * 16;
  uint4 m = make_uint4(0, 0, 0, 0);
  // the window's pixels in one sequence, four loads in flight at a time (a 2x2 window: all of it)
  const int tot = (x1 > x0 && y1 > y0) ? (x1 - x0) * (y1 - y0) : 0;
  int yy = y0, xx = x0;
  for (int n = 0; n < tot; n += 4) {
    uint4 v[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      v[i] = make_uint4(0, 0, 0, 0);
      if (n + i < tot) {
        v[i] = __ldg(reinterpret_cast<const uint4 *>(img + ((size_t)yy * p.W + xx) * p.C));
        if (++xx == x1) { xx = x0; yy++; }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      m.x = __vmaxu4(m.x, v[i].x); m.y = __vmaxu4(m.y, v[i].y); m.z = __vmaxu4(m.z, v[i].z); m.w = __vmaxu4(m.w, v[i].w);
    }
  }
  *reinterpret_cast<uint4 *>(p.out + (((size_t)b * p.Ho + oy) * p.Wo + ox) * p.C + cw * 16) = m;
}

// Reproduces what the reference leaves in Im_in: after its x pass, column ox of every input row
// holds the maximum over that row's window for output column ox (pulp_nn_maxpool.c:63,85-92).
// Reads the untouched input copy `src` and writes into `dst` (the caller's Im_in).
__global__ void __launch_bounds__(256) maxpool_clobber_kernel(const PoolProblem p, const uint8_t *src,
                                                              uint8_t *dst, long long total)
{
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const int c = (int)(t % p.C);
  long long r = t / p.C;
  const int ox = (int)(r % p.Wo); r /= p.Wo;
  const int y = (int)(r % p.H);
  const int b = (int)(r / p.H);
  const int x0 = max(ox * p.sx - p.pl, 0), x1 = min(ox * p.sx - p.pl + p.kx, p.W);
  const uint8_t *row = src + (((size_t)b * p.H + y) * p.W) * p.C + c;
  int m = 0;
  for (int x = x0; x < x1; x++) m = max(m, (int)__ldg(row + (size_t)x * p.C));
  dst[(((size_t)b * p.H + y) * p.W + ox) * p.C + c] = (uint8_t)m;
}

// ---- average pooling -----------------------------------------------------------------------
// 32bit/src/pulp_nn_avgpool.c:71-119. Window start in y uses padding_b and window end in x uses
// padding_r, as written there; the divisor is always kx*ky. The requantised form is unsigned
// 32-bit arithmetic in the 32-bit tree and signed 64-bit arithmetic in the 64-bit tree.
template <bool VEC>
__global__ void __launch_bounds__(256) avgpool_kernel(const PoolProblem p, int CW, long long total)
{
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const int cw = (int)(t % CW);
  long long r = t / CW;
  const int ox = (int)(r % p.Wo); r /= p.Wo;
  const int oy = (int)(r % p.Ho);
  const int b = (int)(r / p.Ho);
  const int c = VEC ? cw * 4 : cw, nb = VEC ? 4 : 1;
  const int y0 = max(oy * p.sy - p.pb, 0), y1 = min(oy * p.sy - p.pt + p.ky, p.H);
  const int x0 = max(ox * p.sx - p.pl, 0), x1 = min(ox * p.sx - p.pr + p.kx, p.W);
  const uint8_t *img = p.in + (size_t)b * p.H * p.W * p.C + c;
  unsigned s[4] = {0, 0, 0, 0};
  for (int y = y0; y < y1; y++)
    for (int x = x0; x < x1; x++) {
      const uint8_t *q = img + ((size_t)y * p.W + x) * p.C;
      const unsigned v = VEC ? __ldg(reinterpret_cast<const unsigned *>(q)) : ld_bytes(q, nb);
      s[0] += v & 0xff; s[1] += (v >> 8) & 0xff; s[2] += (v >> 16) & 0xff; s[3] += v >> 24;
    }
  const unsigned ktot = (unsigned)(p.kx * p.ky);
  unsigned o = 0;
  for (int j = 0; j < nb; j++) {
    int res;
    if (p.requant) {
      if (p.bn_bits == 32) {
        const unsigned tq = s[j] * (unsigned)(int)p.lambda / ktot + (unsigned)(int)p.out_add;
        res = (int)(tq >> p.shift);
      } else {
        const long long tq = (long long)s[j] * p.lambda / (long long)ktot + p.out_add;
        res = (int)(tq >> p.shift);
      }
    } else {
      res = (int)(s[j] / ktot);
    }
    o |= (unsigned)clip_u8(res) << (8 * j);
  }
  uint8_t *dst = p.out + (((size_t)b * p.Ho + oy) * p.Wo + ox) * p.C + c;
  if (VEC) *reinterpret_cast<unsigned *>(dst) = o; else st_bytes(dst, o, nb);
}

// The same for 16 channels per thread (C a multiple of 16, 16-byte aligned tensors): 16-byte loads,
// four of them in flight, so that a window of many pixels (a global pool) keeps HBM busy.
__global__ void __launch_bounds__(256) avgpool16_kernel(const PoolProblem p, int CW, long long total)
{
  pdl_wait();
  pdl_launch_dependents();
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const int cw = (int)(t % CW);
  long long r = t / CW;
  const int ox = (int)(r % p.Wo); r /= p.Wo;
  const int oy = (int)(r % p.Ho);
  const int b = (int)(r / p.Ho);
  const int c = cw * 16;
  const int y0 = max(oy * p.sy - p.pb, 0), y1 = min(oy * p.sy - p.pt + p.ky, p.H);
  const int x0 = max(ox * p.sx - p.pl, 0), x1 = min(ox * p.sx - p.pr + p.kx, p.W);
  const uint8_t *img = p.in + (size_t)b * p.H * p.W * p.C + c;
  unsigned s[16];
#pragma unroll
  for (int j = 0; j < 16; j++) s[j] = 0;
  auto add16 = [&](const uint4 &v) {
    const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      s[4 * i + 0] += w[i] & 0xff; s[4 * i + 1] += (w[i] >> 8) & 0xff;
      s[4 * i + 2] += (w[i] >> 16) & 0xff; s[4 * i + 3] += w[i] >> 24;
    }
  };
  // the window's pixels in one sequence, eight loads in flight at a time
  const int tot = (x1 > x0 && y1 > y0) ? (x1 - x0) * (y1 - y0) : 0;
  int yy = y0, xx = x0;
  for (int n = 0; n < tot; n += 8) {
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
      v[i] = make_uint4(0, 0, 0, 0);
      if (n + i < tot) {
        v[i] = __ldg(reinterpret_cast<const uint4 *>(img + ((size_t)yy * p.W + xx) * p.C));
        if (++xx == x1) { xx = x0; yy++; }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; i++) add16(v[i]);
  }
  const unsigned ktot = (unsigned)(p.kx * p.ky);
  unsigned o[4] = {0, 0, 0, 0};
#pragma unroll
  for (int j = 0; j < 16; j++) {
    int res;
    if (p.requant) {
      if (p.bn_bits == 32) {
        const unsigned tq = s[j] * (unsigned)(int)p.lambda / ktot + (unsigned)(int)p.out_add;
        res = (int)(tq >> p.shift);
      } else {
        const long long tq = (long long)s[j] * p.lambda / (long long)ktot + p.out_add;
        res = (int)(tq >> p.shift);
      }
    } else {
      res = (int)(s[j] / ktot);
    }
    o[j >> 2] |= (unsigned)clip_u8(res) << (8 * (j & 3));
  }
  uint8_t *dst = p.out + (((size_t)b * p.Ho + oy) * p.Wo + ox) * p.C + c;
  *reinterpret_cast<uint4 *>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
}

// Large windows (a global pool): one thread per window would leave most of the GPU idle and make
// every thread walk the whole window alone. Here a block takes one output pixel and 128 channels:
// lane = four channels (a warp reads 128 contiguous bytes of a pixel), the block's eight warps share
// out the window's pixels, and shared memory adds up the eight partial sums. Same arithmetic.
__global__ void __launch_bounds__(256) avgpool_window_kernel(const PoolProblem p, int chunks)
{
  __shared__ unsigned part[8][32][4];
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned t = blockIdx.x;
  const int chunk = (int)(t % (unsigned)chunks); t /= (unsigned)chunks;
  const int ox = (int)(t % (unsigned)p.Wo); t /= (unsigned)p.Wo;
  const int oy = (int)(t % (unsigned)p.Ho);
  const int b = (int)(t / (unsigned)p.Ho);
  const int c = chunk * 128 + lane * 4;
  const bool on = c < p.C;
  const int y0 = max(oy * p.sy - p.pb, 0), y1 = min(oy * p.sy - p.pt + p.ky, p.H);
  const int x0 = max(ox * p.sx - p.pl, 0), x1 = min(ox * p.sx - p.pr + p.kx, p.W);
  const int wx = x1 - x0, tot = (wx > 0 && y1 > y0) ? wx * (y1 - y0) : 0;
  const uint8_t *img = p.in + (size_t)b * p.H * p.W * p.C + (on ? c : 0);
  unsigned s[4] = {0, 0, 0, 0};
  // a window as wide as the image (a global pool) is one contiguous run of pixels: no division
  const bool run = wx == p.W;
  for (int n = warp; n < tot; n += 32) {          // four loads in flight per thread
    unsigned v[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int q = n + 8 * i;
      v[i] = 0;
      if (q < tot && on) {
        const size_t pix = run ? (size_t)y0 * p.W + q : (size_t)(y0 + q / wx) * p.W + x0 + q % wx;
        v[i] = __ldg(reinterpret_cast<const unsigned *>(img + pix * p.C));
      }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      s[0] += v[i] & 0xff; s[1] += (v[i] >> 8) & 0xff; s[2] += (v[i] >> 16) & 0xff; s[3] += v[i] >> 24;
    }
  }
#pragma unroll
  for (int j = 0; j < 4; j++) part[warp][lane][j] = s[j];
  __syncthreads();
  if (warp != 0 || !on) return;
#pragma unroll
  for (int w = 1; w < 8; w++)
#pragma unroll
    for (int j = 0; j < 4; j++) s[j] += part[w][lane][j];
  const unsigned ktot = (unsigned)(p.kx * p.ky);
  unsigned o = 0;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    int res;
    if (p.requant) {
      if (p.bn_bits == 32) {
        const unsigned tq = s[j] * (unsigned)(int)p.lambda / ktot + (unsigned)(int)p.out_add;
        res = (int)(tq >> p.shift);
      } else {
        const long long tq = (long long)s[j] * p.lambda / (long long)ktot + p.out_add;
        res = (int)(tq >> p.shift);
      }
    } else {
      res = (int)(s[j] / ktot);
    }
    o |= (unsigned)clip_u8(res) << (8 * j);
  }
  *reinterpret_cast<unsigned *>(p.out + (((size_t)b * p.Ho + oy) * p.Wo + ox) * p.C + c) = o;
}

// ---- residual add --------------------------------------------------------------------------
// 32bit/src/pulp_nn_utils.c:47-60: uint32 sum of the two int16-scaled bytes, logical shift,
// cut to 16 bits, then clamp to 255.
__device__ __forceinline__ unsigned add_word(unsigned a, unsigned b, int m1, int m2, int d)
{
  unsigned o = 0;
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const unsigned t = (unsigned)((int)((a >> (8 * j)) & 0xff) * m1 + (int)((b >> (8 * j)) & 0xff) * m2);
    const unsigned x = (t >> d) & 0xffffu;
    o |= min(x, 255u) << (8 * j);
  }
  return o;
}

__global__ void __launch_bounds__(256) add_vec_kernel(const uint4 *a, const uint4 *b, uint4 *out,
                                                      size_t n16, int m1, int m2, int d)
{
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
    const uint4 x = __ldg(a + i), y = __ldg(b + i);
    uint4 o;
    o.x = add_word(x.x, y.x, m1, m2, d); o.y = add_word(x.y, y.y, m1, m2, d);
    o.z = add_word(x.z, y.z, m1, m2, d); o.w = add_word(x.w, y.w, m1, m2, d);
    out[i] = o;
  }
}

__global__ void __launch_bounds__(256) add_byte_kernel(const uint8_t *a, const uint8_t *b, uint8_t *out,
                                                       size_t first, size_t n, int m1, int m2, int d)
{
  const size_t i = first + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  out[i] = (uint8_t)add_word(a[i], b[i], m1, m2, d);
}

}  // namespace

bool launch_maxpool(Context &c, const PoolProblem &p, uint8_t *clobber_in)
{
  const bool vec = (p.C % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.in) & 3) == 0) &&
                   ((reinterpret_cast<uintptr_t>(p.out) & 3) == 0);
  const int CW = vec ? p.C / 4 : p.C;
  const long long total = (long long)p.B * p.Ho * p.Wo * CW;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  const long long total16 = (long long)p.B * p.Ho * p.Wo * (p.C / 16);
  if (p.C % 16 == 0 && total16 < 0x7fffffffLL &&
      ((reinterpret_cast<uintptr_t>(p.in) | reinterpret_cast<uintptr_t>(p.out)) & 15) == 0)
    maxpool16_kernel<<<(unsigned)((total16 + 255) / 256), 256, 0, c.stream>>>(p, p.C / 16, (unsigned)total16);
  else if (vec) maxpool_kernel<true><<<blocks, 256, 0, c.stream>>>(p, CW, total);
  else     maxpool_kernel<false><<<blocks, 256, 0, c.stream>>>(p, CW, total);
  count_launch();
  if (!cuda_ok(cudaGetLastError(), "maxpool launch")) return false;
  if (clobber_in) {
    // the x-pass image must be computed from the untouched input: copy it aside first
    const size_t bytes = (size_t)p.B * p.H * p.W * p.C;
    void *copy = ctx_scratch(c, bytes);
    if (!copy) return false;
    if (!cuda_ok(cudaMemcpyAsync(copy, clobber_in, bytes, cudaMemcpyDeviceToDevice, c.stream), "D2D copy"))
      return false;
    const long long tot2 = (long long)p.B * p.H * p.Wo * p.C;
    maxpool_clobber_kernel<<<(unsigned)((tot2 + 255) / 256), 256, 0, c.stream>>>(
        p, static_cast<const uint8_t *>(copy), clobber_in, tot2);
    count_launch();
    if (!cuda_ok(cudaGetLastError(), "maxpool clobber launch")) return false;
  }
  return true;
}

bool launch_avgpool(Context &c, const PoolProblem &p)
{
  const bool vec = (p.C % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.in) & 3) == 0) &&
                   ((reinterpret_cast<uintptr_t>(p.out) & 3) == 0);
  // windows of at least 32 pixels: a block per output pixel and 128 channels
  const int chunks = (p.C + 127) / 128;
  const long long blocks_w = (long long)p.B * p.Ho * p.Wo * chunks;
  const long long threads16 = (long long)p.B * p.Ho * p.Wo * (p.C / 16);
  const bool fills_gpu = p.C % 16 == 0 && threads16 >= 32768;      // measured: from batch 512 of a 7x7x1024 pool on
  if (vec && p.kx * p.ky >= 32 && blocks_w < 0x7fffffffLL && !fills_gpu) {
    const cudaError_t le = launch_pdl(avgpool_window_kernel, dim3((unsigned)blocks_w), dim3(256), 0, c.stream, p, chunks);
    count_launch("avgpool_window_kernel");
    return cuda_ok(le, "avgpool launch") && cuda_ok(cudaGetLastError(), "avgpool launch");
  }
  // windows of at least 16 pixels: fewer threads with more bytes in flight each
  if (p.C % 16 == 0 && p.kx * p.ky >= 16 && ((reinterpret_cast<uintptr_t>(p.in) | reinterpret_cast<uintptr_t>(p.out)) & 15) == 0) {
    const int CW16 = p.C / 16;
    const long long total16 = (long long)p.B * p.Ho * p.Wo * CW16;
    const cudaError_t le = launch_pdl(avgpool16_kernel, dim3((unsigned)((total16 + 255) / 256)), dim3(256), 0, c.stream,
                                      p, CW16, total16);
    count_launch("avgpool16_kernel");
    return cuda_ok(le, "avgpool launch") && cuda_ok(cudaGetLastError(), "avgpool launch");
  }
  const int CW = vec ? p.C / 4 : p.C;
  const long long total = (long long)p.B * p.Ho * p.Wo * CW;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (vec) avgpool_kernel<true><<<blocks, 256, 0, c.stream>>>(p, CW, total);
  else     avgpool_kernel<false><<<blocks, 256, 0, c.stream>>>(p, CW, total);
  count_launch();
  return cuda_ok(cudaGetLastError(), "avgpool launch");
}

bool launch_add(Context &c, const uint8_t *a, const uint8_t *b, uint8_t *out, size_t n, int m1,
                int m2, int shift)
{
  const bool aligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                         reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  const size_t n16 = aligned ? n / 16 : 0;
  if (n16) {
    const size_t want = (n16 + 255) / 256;
    const unsigned blocks = (unsigned)(want < (size_t)c.sm_count * 16 ? want : (size_t)c.sm_count * 16);
    add_vec_kernel<<<blocks, 256, 0, c.stream>>>(reinterpret_cast<const uint4 *>(a),
                                                 reinterpret_cast<const uint4 *>(b),
                                                 reinterpret_cast<uint4 *>(out), n16, m1, m2, shift);
    count_launch();
  }
  const size_t first = n16 * 16;
  if (first < n) {
    add_byte_kernel<<<(unsigned)((n - first + 255) / 256), 256, 0, c.stream>>>(a, b, out, first, n, m1, m2, shift);
    count_launch();
  }
  return cuda_ok(cudaGetLastError(), "add launch");
}

}  // namespace pulpnn
