// layout.cu -- CHW <-> HWC layout change of uint8 activations. The reference has no such
// function although its depthwise kernel wants CHW input and every other kernel produces HWC
// (32bit/src/pulp_nn_depthwise_generic.c:74,81); a caller that chains them needs one. Both
// directions are the same byte-matrix transpose per image: [rows][cols] -> [cols][rows] with
// (rows, cols) = (C, H*W) for CHW -> HWC and (H*W, C) for HWC -> CHW.
//
// A CTA moves a 64 x 64 tile through shared memory: 32-bit loads along the input's contiguous
// dimension, four byte reads down a tile column packed into one 32-bit store along the output's.
#include "internal.cuh"

namespace pulpnn {

namespace {

constexpr int TS = 64;            // tile side in bytes
constexpr int PITCH = TS + 4;     // row pitch of the tile in shared memory

__global__ void __launch_bounds__(256) transpose_u8_kernel(const uint8_t *in, uint8_t *out, int rows, int cols,
                                                           int tiles_r, int tiles_c, int vec_in, int vec_out)
{
  __shared__ __align__(4) uint8_t tile[TS][PITCH];
  int t = blockIdx.x;
  const int tc = t % tiles_c; t /= tiles_c;
  const int tr = t % tiles_r;
  const int b = t / tiles_r;
  const int r0 = tr * TS, c0 = tc * TS;
  const uint8_t *src = in + (size_t)b * rows * cols;
  uint8_t *dst = out + (size_t)b * rows * cols;
  const int q = (threadIdx.x & 15) * 4, l = threadIdx.x >> 4;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int r = r0 + l + 16 * i, c = c0 + q;
    unsigned v = 0;
    if (r < rows) {
      const uint8_t *p = src + (size_t)r * cols + c;
      if (vec_in && c + 3 < cols) v = __ldg(reinterpret_cast<const unsigned *>(p));
      else {
#pragma unroll
        for (int k = 0; k < 4; k++)
          if (c + k < cols) v |= (unsigned)__ldg(p + k) << (8 * k);
      }
    }
    *reinterpret_cast<unsigned *>(&tile[l + 16 * i][q]) = v;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int oc = l + 16 * i;                 // column of the tile = row of the output
    const int c = c0 + oc, r = r0 + q;
    if (c < cols) {
      const unsigned v = (unsigned)tile[q][oc] | ((unsigned)tile[q + 1][oc] << 8) | ((unsigned)tile[q + 2][oc] << 16) |
                         ((unsigned)tile[q + 3][oc] << 24);
      uint8_t *p = dst + (size_t)c * rows + r;
      if (vec_out && r + 3 < rows) *reinterpret_cast<unsigned *>(p) = v;
      else {
#pragma unroll
        for (int k = 0; k < 4; k++)
          if (r + k < rows) p[k] = (uint8_t)(v >> (8 * k));
      }
    }
  }
}

// The fast path: 128 x 128 byte tiles. Phase 1: 16-byte loads along the input's rows, the words
// stored in shared memory at word position w ^ ((r >> 2) ^ (r & 3)) of row r. Phase 2: a lane takes
// four consecutive rows of one word column (four conflict-free 32-bit loads thanks to the swizzle),
// transposes the 4 x 4 bytes with byte permutes and writes one word to each of four output rows;
// the lanes of a warp cover 128 consecutive bytes of an output row. Needs cols % 16 == 0,
// rows % 4 == 0 and aligned buffers; tiles at the edges are clipped chunk-wise.
constexpr int TB = 128;

__device__ __forceinline__ unsigned prmt(unsigned a, unsigned b, unsigned sel)
{
  unsigned d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

__global__ void __launch_bounds__(256) transpose_u8_fast_kernel(const uint8_t *in, uint8_t *out, int rows, int cols,
                                                                int tiles_r, int tiles_c)
{
  __shared__ unsigned tile[TB][TB / 4];
  int t = blockIdx.x;
  const int tc = t % tiles_c; t /= tiles_c;
  const int tr = t % tiles_r;
  const int b = t / tiles_r;
  const int r0 = tr * TB, c0 = tc * TB;
  const uint8_t *src = in + (size_t)b * rows * cols;
  uint8_t *dst = out + (size_t)b * rows * cols;
  const int tid = threadIdx.x;
  // phase 1: thread -> (row, 16-byte chunk): 8 chunks per row, 32 rows per pass, 4 passes
  {
    const int ch = tid & 7, rl = tid >> 3;
    uint4 v[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int r = r0 + rl + 32 * i, c = c0 + 16 * ch;
      v[i] = make_uint4(0, 0, 0, 0);
      if (r < rows && c < cols) v[i] = __ldg(reinterpret_cast<const uint4 *>(src + (size_t)r * cols + c));
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int r = rl + 32 * i;
      const int f = ((r >> 2) ^ (r & 3)) & 31;
      tile[r][(4 * ch + 0) ^ f] = v[i].x; tile[r][(4 * ch + 1) ^ f] = v[i].y;
      tile[r][(4 * ch + 2) ^ f] = v[i].z; tile[r][(4 * ch + 3) ^ f] = v[i].w;
    }
  }
  __syncthreads();
  // phase 2: lane = group of four rows, warp = word column (four of them per warp)
  const int rg = tid & 31, warp = tid >> 5;
  const int r = r0 + 4 * rg;
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const int cg = warp + 8 * k;
    unsigned m[4];
#pragma unroll
    for (int i = 0; i < 4; i++) m[i] = tile[4 * rg + i][cg ^ ((rg ^ i) & 31)];
    // 4 x 4 byte transpose: w[j] = byte j of m[0..3]
    const unsigned a = prmt(m[0], m[1], 0x5140), bb = prmt(m[0], m[1], 0x7362);
    const unsigned cc = prmt(m[2], m[3], 0x5140), d = prmt(m[2], m[3], 0x7362);
    const unsigned w0 = prmt(a, cc, 0x5410), w1 = prmt(a, cc, 0x7632);
    const unsigned w2 = prmt(bb, d, 0x5410), w3 = prmt(bb, d, 0x7632);
    const int c = c0 + 4 * cg;
    if (r < rows) {
      if (c + 0 < cols) *reinterpret_cast<unsigned *>(dst + (size_t)(c + 0) * rows + r) = w0;
      if (c + 1 < cols) *reinterpret_cast<unsigned *>(dst + (size_t)(c + 1) * rows + r) = w1;
      if (c + 2 < cols) *reinterpret_cast<unsigned *>(dst + (size_t)(c + 2) * rows + r) = w2;
      if (c + 3 < cols) *reinterpret_cast<unsigned *>(dst + (size_t)(c + 3) * rows + r) = w3;
    }
  }
}

void layout_entry(const char *who, const uint8_t *in, uint8_t *out, int dim_x, int dim_y, int ch, bool to_hwc)
{
  Context &c = ctx();
  if (!ensure_device(c)) return;
  if (!in || !out) { set_error(PULPNN_ERR_INVALID_ARG, "%s: NULL pointer", who); return; }
  if (dim_x <= 0 || dim_y <= 0 || ch <= 0) { set_error(PULPNN_ERR_INVALID_ARG, "%s: zero dimension", who); return; }
  const size_t n = (size_t)c.batch * dim_x * dim_y * ch;
  Stager st(c);
  const uint8_t *din = static_cast<const uint8_t *>(st.in(in, n));
  uint8_t *dout = static_cast<uint8_t *>(st.out(out, n));
  if (!st.ok()) return;
  const int hw = dim_x * dim_y;
  const int rows = to_hwc ? ch : hw, cols = to_hwc ? hw : ch;
  if (cols % 16 == 0 && rows % 4 == 0 && (reinterpret_cast<uintptr_t>(din) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(dout) & 3) == 0) {
    const int fr = (rows + TB - 1) / TB, fc = (cols + TB - 1) / TB;
    const long long ftotal = (long long)c.batch * fr * fc;
    if (ftotal <= 0x7fffffffLL) {
      transpose_u8_fast_kernel<<<(unsigned)ftotal, 256, 0, c.stream>>>(din, dout, rows, cols, fr, fc);
      count_launch();
      if (!cuda_ok(cudaGetLastError(), "transpose launch")) return;
      st.finish();
      return;
    }
  }
  const int tiles_r = (rows + TS - 1) / TS, tiles_c = (cols + TS - 1) / TS;
  const long long total = (long long)c.batch * tiles_r * tiles_c;
  if (total > 0x7fffffffLL) { set_error(PULPNN_ERR_UNSUPPORTED, "%s: too many tiles", who); return; }
  // whole words only when every row of every image starts on a word boundary
  const int vec_in = (cols % 4 == 0 && (reinterpret_cast<uintptr_t>(din) & 3) == 0) ? 1 : 0;
  const int vec_out = (rows % 4 == 0 && (reinterpret_cast<uintptr_t>(dout) & 3) == 0) ? 1 : 0;
  transpose_u8_kernel<<<(unsigned)total, 256, 0, c.stream>>>(din, dout, rows, cols, tiles_r, tiles_c, vec_in, vec_out);
  count_launch();
  if (!cuda_ok(cudaGetLastError(), "transpose launch")) return;
  st.finish();
}

}  // namespace

}  // namespace pulpnn

extern "C" {

void pulpnn_chw_to_hwc(const uint8_t *Im_in, uint8_t *Im_out, uint16_t dim_im_x, uint16_t dim_im_y, uint16_t ch_im)
{
  pulpnn::layout_entry("pulpnn_chw_to_hwc", Im_in, Im_out, dim_im_x, dim_im_y, ch_im, true);
}

void pulpnn_hwc_to_chw(const uint8_t *Im_in, uint8_t *Im_out, uint16_t dim_im_x, uint16_t dim_im_y, uint16_t ch_im)
{
  pulpnn::layout_entry("pulpnn_hwc_to_chw", Im_in, Im_out, dim_im_x, dim_im_y, ch_im, false);
}

}  // extern "C"
