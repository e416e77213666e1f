/*
 * pulpnn_oracle.c -- CPU restatement of the PULP-NN 8-bit kernels.
 *
 * TEST INFRASTRUCTURE ONLY. This file states, in plain loops, what each
 * reference kernel computes, so that the CUDA library can be checked on a
 * machine where the reference tree itself is not present. It is pinned against
 * the compiled reference (oracle/_ref, built from the reference sources in
 * place) by tests/test_oracle_vs_reference.py and against the fixtures under
 * tests/golden/, which were produced by that compiled reference. Only tests/,
 * the smoke check and bench.py's CPU-baseline legs may load it; the shipped
 * library never does.
 *
 * Citations are file:line inside the PULP-NN tree (32bit/ unless noted; the
 * 64bit/ twin has the same line numbers except where stated).
 *
 * All entry points take `batch` contiguous images; weights and batch-norm
 * parameters are shared by the whole batch. `bn_bits` selects the tree:
 * 32 -> k/lambda are int32_t[], 64 -> int64_t[].
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include <stdlib.h>

/* clamp of a 32-bit register to [0,255]: __builtin_pulp_clipu_r(x,255),
 * src/pulp_nn_utils.c:43. A wider value is truncated to 32 bits first. */
static inline uint8_t clip_u8(int32_t x)
{
  return (uint8_t)(x < 0 ? 0 : (x > 255 ? 255 : x));
}

/* src/pulp_nn_utils.c:35-45 (32-bit tree): int32 wrap-around product and sum,
 * arithmetic shift by (int8_t)d. */
static inline uint8_t bn_quant_32(int32_t phi, int32_t k, int32_t lambda, int d)
{
  int32_t t = (int32_t)((uint32_t)k * (uint32_t)phi + (uint32_t)lambda);
  return clip_u8(t >> d);
}

/* 64bit/src/pulp_nn_utils.c:34-44: the same in int64, truncated to 32 bits
 * only where the clip instruction takes its operand. */
static inline uint8_t bn_quant_64(int32_t phi, int64_t k, int64_t lambda, int d)
{
  int64_t t = (int64_t)((uint64_t)k * (uint64_t)(int64_t)phi + (uint64_t)lambda);
  return clip_u8((int32_t)(t >> d));
}

/* src/pulp_nn_utils.c:148-156: int32 product, shifted, then cut to int16. */
static inline uint8_t mult_quant(int32_t phi, int out_mult, int d)
{
  int16_t m = (int16_t)(uint16_t)out_mult;
  int32_t p = (int32_t)((uint32_t)(int32_t)m * (uint32_t)phi);
  int16_t x = (int16_t)(p >> d);
  return clip_u8(x);
}

enum { MODE_NONE = 0, MODE_MULT = 1, MODE_BN = 2 };

/* Epilogue selection, src/pulp_nn_matmul.c:144-216 and src/pulp_nn_linear.c:88-107:
 * BN needs both flags (truthiness); the multiplier path needs flag_relu == 1
 * exactly; everything else is a bare shift and clip. */
static int mode_conv(int flag_relu, int flag_bn)
{
  if (flag_bn && flag_relu) return MODE_BN;
  if (flag_relu == 1) return MODE_MULT;
  return MODE_NONE;
}
/* src/pulp_nn_depthwise_generic.c:167-178: here the middle test is truthiness. */
static int mode_dw(int flag_relu, int flag_bn)
{
  if (flag_bn && flag_relu) return MODE_BN;
  if (flag_relu) return MODE_MULT;
  return MODE_NONE;
}

static inline uint8_t requant(int32_t acc, int mode, int bn_bits, const void *k, const void *lambda,
                              int ch, int out_mult, int d)
{
  if (mode == MODE_BN) {
    if (bn_bits == 32)
      return bn_quant_32(acc, ((const int32_t *)k)[ch], ((const int32_t *)lambda)[ch], d);
    return bn_quant_64(acc, ((const int64_t *)k)[ch], ((const int64_t *)lambda)[ch], d);
  }
  if (mode == MODE_MULT) return mult_quant(acc, out_mult, d);
  return clip_u8(acc >> d);
}

/* the shift operand reaches the helpers as int8_t (src/pulp_nn_utils.c:39,151) */
static inline int shift_arg(int out_shift) { return (int)(int8_t)out_shift; }

/* ---------------------------------------------------------------------------
 * Standard convolution, HWC in / HWC out, weights [ch_out][ky][kx][ch_in].
 * src/pulp_nn_conv_Ho_parallel.c:76-186 builds, per output pixel, the column
 * of kx*ky*ch_in input bytes with zeros outside the image (:89,:109,:135,:155)
 * and src/pulp_nn_matmul.c:53-297 takes its dot product with every filter,
 * starting from the int8 bias (:70-92). src/pulp_nn_conv_HoWo_parallel.c
 * differs only in which core computes which pixels.
 * If acc_out is not NULL the raw accumulators are stored there as well.
 * ------------------------------------------------------------------------- */
void oracle_conv(int bn_bits, const uint8_t *in, const int8_t *bias, uint8_t *out, const int8_t *w,
                 const void *k, const void *lambda, int out_mult, int out_shift,
                 int dim_in_x, int dim_in_y, int ch_in, int dim_out_x, int dim_out_y, int ch_out,
                 int kx, int ky, int pt, int pb, int pl, int pr, int sx, int sy,
                 int flag_relu, int flag_bn, int batch, int32_t *acc_out)
{
  (void)pb; (void)pr;
  const int mode = mode_conv(flag_relu, flag_bn);
  const int d = shift_arg(out_shift);
  const size_t in_sz = (size_t)dim_in_x * dim_in_y * ch_in;
  const size_t out_sz = (size_t)dim_out_x * dim_out_y * ch_out;
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < batch; b++)
    for (int oy = 0; oy < dim_out_y; oy++)
      for (int ox = 0; ox < dim_out_x; ox++)
        for (int co = 0; co < ch_out; co++) {
          int32_t acc = bias ? (int32_t)bias[co] : 0;
          for (int fy = 0; fy < ky; fy++) {
            int iy = oy * sy - pt + fy;
            if (iy < 0 || iy >= dim_in_y) continue;
            for (int fx = 0; fx < kx; fx++) {
              int ix = ox * sx - pl + fx;
              if (ix < 0 || ix >= dim_in_x) continue;
              const uint8_t *px = in + (size_t)b * in_sz + ((size_t)iy * dim_in_x + ix) * ch_in;
              const int8_t *pw = w + (((size_t)co * ky + fy) * kx + fx) * ch_in;
              for (int ci = 0; ci < ch_in; ci++) acc += (int32_t)px[ci] * (int32_t)pw[ci];
            }
          }
          size_t o = (size_t)b * out_sz + ((size_t)oy * dim_out_x + ox) * ch_out + co;
          if (acc_out) acc_out[o] = acc;
          out[o] = requant(acc, mode, bn_bits, k, lambda, co, out_mult, d);
        }
}

/* ---------------------------------------------------------------------------
 * Pointwise (1x1) convolution. src/pulp_nn_pointwise_HoWo_parallel.c:98-181
 * hands pairs of adjacent HWC pixels straight to the matmul; the kernel-size,
 * padding and stride arguments are never read and the input pixel of output
 * (y,x) is in[(y*dim_in_x + x)*ch_in] (:103).
 * ------------------------------------------------------------------------- */
void oracle_pointwise(int bn_bits, const uint8_t *in, const int8_t *bias, uint8_t *out,
                      const int8_t *w, const void *k, const void *lambda, int out_mult,
                      int out_shift, int dim_in_x, int dim_in_y, int ch_in, int dim_out_x,
                      int dim_out_y, int ch_out, int flag_relu, int flag_bn, int batch,
                      int32_t *acc_out)
{
  const int mode = mode_conv(flag_relu, flag_bn);
  const int d = shift_arg(out_shift);
  const size_t in_sz = (size_t)dim_in_x * dim_in_y * ch_in;
  const size_t out_sz = (size_t)dim_out_x * dim_out_y * ch_out;
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < batch; b++)
    for (int oy = 0; oy < dim_out_y; oy++)
      for (int ox = 0; ox < dim_out_x; ox++) {
        const uint8_t *px = in + (size_t)b * in_sz + ((size_t)oy * dim_in_x + ox) * ch_in;
        for (int co = 0; co < ch_out; co++) {
          const int8_t *pw = w + (size_t)co * ch_in;
          int32_t acc = bias ? (int32_t)bias[co] : 0;
          for (int ci = 0; ci < ch_in; ci++) acc += (int32_t)px[ci] * (int32_t)pw[ci];
          size_t o = (size_t)b * out_sz + ((size_t)oy * dim_out_x + ox) * ch_out + co;
          if (acc_out) acc_out[o] = acc;
          out[o] = requant(acc, mode, bn_bits, k, lambda, co, out_mult, d);
        }
      }
}

/* ---------------------------------------------------------------------------
 * Depthwise convolution. src/pulp_nn_depthwise_generic.c:72-389: input is CHW
 * (:74 channel offset = c*H*W), weights [c][ky][kx] (:75), output HWC (:81,
 * :179). Per channel and output column the reference builds a zero-padded
 * strip (:82-132 left zone, :189-228 middle, :285-337 right zone) and takes
 * ky*kx-tap dot products down it (:133-180). Inside the domain the library
 * accepts (odd kx, pad_left == kx/2, kx*ky >= 4, see the validation in the
 * shipped library) that equals the zero-padded depthwise convolution below.
 * Batch-norm parameters are indexed by channel (:169 with k++ at :387).
 * in_is_hwc != 0 selects the HWC-input variant the network runner uses; the
 * arithmetic is identical.
 * ------------------------------------------------------------------------- */
void oracle_depthwise(int bn_bits, const uint8_t *in, const int8_t *bias, uint8_t *out,
                      const int8_t *w, const void *k, const void *lambda, int out_mult,
                      int out_shift, int dim_in_x, int dim_in_y, int ch, int dim_out_x,
                      int dim_out_y, int kx, int ky, int pt, int pb, int pl, int pr, int sx, int sy,
                      int flag_relu, int flag_bn, int in_is_hwc, int batch, int32_t *acc_out)
{
  (void)pb; (void)pr;
  const int mode = mode_dw((int)(int8_t)flag_relu, (int)(int8_t)flag_bn);
  const int d = shift_arg(out_shift);
  const size_t in_sz = (size_t)dim_in_x * dim_in_y * ch;
  const size_t out_sz = (size_t)dim_out_x * dim_out_y * ch;
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < batch; b++)
    for (int oy = 0; oy < dim_out_y; oy++)
      for (int ox = 0; ox < dim_out_x; ox++)
        for (int c = 0; c < ch; c++) {
          int32_t acc = bias ? (int32_t)bias[c] : 0;
          for (int fy = 0; fy < ky; fy++) {
            int iy = oy * sy - pt + fy;
            if (iy < 0 || iy >= dim_in_y) continue;
            for (int fx = 0; fx < kx; fx++) {
              int ix = ox * sx - pl + fx;
              if (ix < 0 || ix >= dim_in_x) continue;
              size_t ii = in_is_hwc ? ((size_t)iy * dim_in_x + ix) * ch + c
                                    : ((size_t)c * dim_in_y + iy) * dim_in_x + ix;
              acc += (int32_t)in[(size_t)b * in_sz + ii] * (int32_t)w[((size_t)c * ky + fy) * kx + fx];
            }
          }
          size_t o = (size_t)b * out_sz + ((size_t)oy * dim_out_x + ox) * ch + c;
          if (acc_out) acc_out[o] = acc;
          out[o] = requant(acc, mode, bn_bits, k, lambda, c, out_mult, d);
        }
}

/* ---------------------------------------------------------------------------
 * Fully connected layer. src/pulp_nn_linear.c:58-108: acc = int8 bias[i] +
 * dot(in, w[i]); epilogue as for conv; out_shift arrives as int8_t (:37).
 * ------------------------------------------------------------------------- */
void oracle_linear(int bn_bits, const uint8_t *in, const int8_t *bias, uint8_t *out,
                   const int8_t *w, const void *k, const void *lambda, int out_mult, int out_shift,
                   int dim_vec, int num_o, int flag_relu, int flag_bn, int batch)
{
  const int mode = mode_conv(flag_relu, flag_bn);
  const int d = shift_arg(out_shift);
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < batch; b++)
    for (int o = 0; o < num_o; o++) {
      int32_t acc = bias ? (int32_t)bias[o] : 0;
      const uint8_t *pi = in + (size_t)b * dim_vec;
      const int8_t *pw = w + (size_t)o * dim_vec;
      for (int j = 0; j < dim_vec; j++) acc += (int32_t)pi[j] * (int32_t)pw[j];
      out[(size_t)b * num_o + o] = requant(acc, mode, bn_bits, k, lambda, o, out_mult, d);
    }
}

/* src/pulp_nn_linear_out_32.c:48-80: no requantisation, the int32 accumulator
 * is stored. The bias argument is declared int8_t* but is read as a 32-bit
 * word at byte offset 4*i (:54), i.e. it is an int32_t[num_o] array. */
void oracle_linear_out_32(const uint8_t *in, const int8_t *bias, int32_t *out, const int8_t *w,
                          int dim_vec, int num_o, int batch)
{
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < batch; b++)
    for (int o = 0; o < num_o; o++) {
      int32_t acc = 0;
      if (bias) memcpy(&acc, bias + 4 * (size_t)o, 4);
      const uint8_t *pi = in + (size_t)b * dim_vec;
      const int8_t *pw = w + (size_t)o * dim_vec;
      for (int j = 0; j < dim_vec; j++) acc += (int32_t)pi[j] * (int32_t)pw[j];
      out[(size_t)b * num_o + o] = acc;
    }
}

/* ---------------------------------------------------------------------------
 * Max pooling, HWC. src/pulp_nn_maxpool.c works in two passes: first along x,
 * writing the running maxima INTO THE INPUT rows at column i_x (:58-94), then
 * along y from those rows into the output (:107-144). Windows are clipped to
 * the image; padding_b and padding_r are never read. This restatement runs the
 * same two passes on a private copy; when in_after is not NULL it receives
 * that copy, i.e. the state the reference leaves its input buffer in.
 * ------------------------------------------------------------------------- */
void oracle_maxpool(const uint8_t *in, uint8_t *out, uint8_t *in_after, int dim_in_x, int dim_in_y,
                    int ch, int dim_out_x, int dim_out_y, int kx, int ky, int pt, int pl, int sx,
                    int sy, int batch)
{
  const size_t in_sz = (size_t)dim_in_x * dim_in_y * ch;
  const size_t out_sz = (size_t)dim_out_x * dim_out_y * ch;
#pragma omp parallel for schedule(static)
  for (int b = 0; b < batch; b++) {
    uint8_t *tmp = (uint8_t *)malloc(in_sz ? in_sz : 1);
    memcpy(tmp, in + (size_t)b * in_sz, in_sz);
    for (int y = 0; y < dim_in_y; y++)
      for (int ox = 0; ox < dim_out_x; ox++) {
        int x0 = ox * sx - pl;
        int start = x0 < 0 ? ox : x0;                       /* :66-73 */
        int stop = x0 + kx >= dim_in_x ? dim_in_x : x0 + kx; /* :75-82 */
        uint8_t *target = tmp + ((size_t)y * dim_in_x + ox) * ch;
        const uint8_t *p = tmp + ((size_t)y * dim_in_x + start) * ch;
        for (int c = 0; c < ch; c++) target[c] = p[c];       /* :85 */
        for (int x = start + 1; x < stop; x++) {             /* :88-92 */
          p = tmp + ((size_t)y * dim_in_x + x) * ch;
          for (int c = 0; c < ch; c++) if (target[c] < p[c]) target[c] = p[c];
        }
      }
    for (int oy = 0; oy < dim_out_y; oy++) {
      int y0 = oy * sy - pt;
      int start = y0 < 0 ? 0 : y0;                           /* :114-121 */
      int stop = y0 + ky >= dim_in_y ? dim_in_y : y0 + ky;   /* :123-130 */
      uint8_t *target = out + (size_t)b * out_sz + (size_t)oy * dim_out_x * ch;
      const size_t n = (size_t)dim_out_x * ch;
      memcpy(target, tmp + (size_t)start * dim_in_x * ch, n); /* :133-136 */
      for (int y = start + 1; y < stop; y++) {               /* :140-143 */
        const uint8_t *p = tmp + (size_t)y * dim_in_x * ch;
        for (size_t i = 0; i < n; i++) if (target[i] < p[i]) target[i] = p[i];
      }
    }
    if (in_after) memcpy(in_after + (size_t)b * in_sz, tmp, in_sz);
    free(tmp);
  }
}

/* ---------------------------------------------------------------------------
 * Average pooling, HWC. src/pulp_nn_avgpool.c:71-119. The window is
 * [max(0, oy*sy - padding_b), min(oy*sy - padding_t + ky, H)) in y (:82-83) and
 * [max(0, ox*sx - padding_l), min(ox*sx - padding_r + kx, W)) in x (:85-86);
 * the divisor is always kx*ky (:66). Without requantisation the result is
 * clip(sum / (kx*ky)) (:112-113). With it (:108):
 *   32-bit tree: every operand converts to uint32 (sum is uint32_t, :70), so the
 *     product, the division and the shift are unsigned and the result is read
 *     back as int32 before the clip;
 *   64-bit tree: int64 arithmetic (64bit/src/pulp_nn_avgpool.c:106-108), signed
 *     division truncating toward zero, arithmetic shift, then the 32-bit clip.
 * ------------------------------------------------------------------------- */
void oracle_avgpool(int bn_bits, const uint8_t *in, uint8_t *out, int64_t lambda, int out_shift,
                    int64_t out_add, int dim_in_x, int dim_in_y, int ch, int dim_out_x,
                    int dim_out_y, int kx, int ky, int pt, int pb, int pl, int pr, int sx, int sy,
                    int flag_requant, int batch)
{
  const size_t in_sz = (size_t)dim_in_x * dim_in_y * ch;
  const size_t out_sz = (size_t)dim_out_x * dim_out_y * ch;
  const uint32_t ktot = (uint32_t)kx * (uint32_t)ky;
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < batch; b++)
    for (int oy = 0; oy < dim_out_y; oy++)
      for (int ox = 0; ox < dim_out_x; ox++) {
        int ys = oy * sy - pb; if (ys < 0) ys = 0;
        int ye = oy * sy - pt + ky; if (ye > dim_in_y) ye = dim_in_y;
        int xs = ox * sx - pl; if (xs < 0) xs = 0;
        int xe = ox * sx - pr + kx; if (xe > dim_in_x) xe = dim_in_x;
        for (int c = 0; c < ch; c++) {
          uint32_t sum = 0;
          for (int y = ys; y < ye; y++)
            for (int x = xs; x < xe; x++)
              sum += in[(size_t)b * in_sz + ((size_t)y * dim_in_x + x) * ch + c];
          int32_t r;
          if (flag_requant) {
            if (bn_bits == 32) {
              uint32_t t = sum * (uint32_t)(int32_t)lambda / ktot + (uint32_t)(int32_t)out_add;
              r = (int32_t)(t >> out_shift);
            } else {
              int64_t t = (int64_t)sum * lambda / (int64_t)ktot + out_add;
              r = (int32_t)(t >> out_shift);
            }
          } else {
            r = (int32_t)(sum / ktot);
          }
          out[(size_t)b * out_sz + ((size_t)oy * dim_out_x + ox) * ch + c] = clip_u8(r);
        }
      }
}

/* ---------------------------------------------------------------------------
 * Residual add. src/pulp_nn_add.c:54-60 applies src/pulp_nn_utils.c:47-60 to
 * every byte: the multipliers are read as int16, the sum is held in a uint32,
 * shifted logically, CUT TO 16 BITS, and only then clamped to 255.
 * ------------------------------------------------------------------------- */
void oracle_add(const uint8_t *in1, const uint8_t *in2, uint8_t *out, int out_mult1, int out_mult2,
                int out_shift, size_t count)
{
  const int16_t m1 = (int16_t)(uint16_t)out_mult1, m2 = (int16_t)(uint16_t)out_mult2;
  const int d = shift_arg(out_shift);
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < count; i++) {
    uint32_t t = (uint32_t)((int32_t)in1[i] * m1 + (int32_t)in2[i] * m2);
    uint16_t x = (uint16_t)(t >> d);
    out[i] = (uint8_t)(x > 255 ? 255 : x);
  }
}
