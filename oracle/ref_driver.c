/*
 * ref_driver.c -- batch/thread harness around the UNMODIFIED PULP-NN reference
 * kernels. TEST INFRASTRUCTURE ONLY: it is linked with the reference objects
 * (compiled in place from the reference tree, see oracle/Makefile) into
 * oracle/_ref/libpulpnn_ref{32,64}.so and is used by tests/, the smoke check
 * and bench.py's CPU-baseline legs as the checker / timed CPU baseline. The
 * shipped library never links or loads it.
 *
 * Why a harness is needed at all:
 *  - the reference API is one image per call; the harness loops over a batch,
 *    one worker thread per slice of images (images are independent);
 *  - pulp_nn_depthwise_generic keeps an input address in an `int`
 *    (32bit/src/pulp_nn_depthwise_generic.c:101,205,301), which only survives
 *    on a 64-bit host when the buffer lives below 2 GiB, and its strip builder
 *    loads 4 bytes for a 3-byte row (ibid. :113,211,310) so it reads a few
 *    bytes past the input. Every per-image buffer handed to the reference is
 *    therefore a padded slot of a low-address arena; inputs are copied in and
 *    outputs copied out.
 *
 * Compile with -DBN_T=int32_t against the 32bit tree or -DBN_T=int64_t against
 * the 64bit tree. Every entry returns the wall-clock seconds spent inside the
 * threaded region (copies included), or a negative value on failure.
 */
#define _GNU_SOURCE
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include <stdlib.h>
#include <pthread.h>
#include <time.h>
#include <sys/mman.h>

#ifndef BN_T
#error "define BN_T as int32_t or int64_t"
#endif
typedef BN_T bn_t;

/* the reference header has no include guard and no includes of its own */
#include "pulp_nn_kernels.h"

#define GUARD 64u

static uint8_t *g_arena = NULL;
static size_t   g_arena_size = 0;

static double now_s(void)
{
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

/* Map (once) a region whose addresses all fit in a positive 32-bit int. */
int refdrv_init(size_t bytes)
{
  if (g_arena && g_arena_size >= bytes) return 0;
  if (g_arena) { munmap(g_arena, g_arena_size); g_arena = NULL; g_arena_size = 0; }
  /* try every 64 MiB step below 2 GiB until a free range is found */
  for (uintptr_t base = 0x10000000u; base + bytes < 0x7ff00000u; base += 0x04000000u) {
    void *p = mmap((void *)base, bytes, PROT_READ | PROT_WRITE,
                   MAP_PRIVATE | MAP_ANONYMOUS | MAP_FIXED_NOREPLACE, -1, 0);
    if (p == MAP_FAILED) continue;
    if ((uintptr_t)p != base) { munmap(p, bytes); continue; }
    g_arena = (uint8_t *)p;
    g_arena_size = bytes;
    return 0;
  }
  return -1;
}

int refdrv_bn_bits(void) { return (int)(8 * sizeof(bn_t)); }
int refdrv_num_cores(void) { return NUM_CORES; }

/* --- a tiny bump allocator over the arena, reset per call ---------------- */
typedef struct { size_t off; } bump_t;
static uint8_t *bump(bump_t *b, size_t n)
{
  size_t need = ((n + GUARD + 63u) & ~(size_t)63u) + GUARD;
  if (!g_arena || b->off + need > g_arena_size) return NULL;
  uint8_t *p = g_arena + b->off + GUARD;
  b->off += need;
  return p;
}

typedef void (*image_fn)(void *ctx, int img, int tid);

typedef struct {
  image_fn fn; void *ctx; int first, last, tid;
} work_t;

static void *worker(void *arg)
{
  work_t *w = (work_t *)arg;
  for (int i = w->first; i < w->last; i++) w->fn(w->ctx, i, w->tid);
  return NULL;
}

static double run_batch(image_fn fn, void *ctx, int batch, int threads)
{
  if (threads < 1) threads = 1;
  if (threads > batch) threads = batch;
  if (threads > 256) threads = 256;
  pthread_t th[256];
  work_t wk[256];
  double t0 = now_s();
  int per = (batch + threads - 1) / threads;
  for (int t = 0; t < threads; t++) {
    wk[t].fn = fn; wk[t].ctx = ctx; wk[t].tid = t;
    wk[t].first = t * per;
    wk[t].last = (t + 1) * per < batch ? (t + 1) * per : batch;
    if (threads == 1) worker(&wk[t]);
    else pthread_create(&th[t], NULL, worker, &wk[t]);
  }
  if (threads > 1) for (int t = 0; t < threads; t++) pthread_join(th[t], NULL);
  return now_s() - t0;
}

static int clamp_threads(int threads, int batch)
{
  if (threads < 1) threads = 1;
  if (threads > batch) threads = batch;
  if (threads > 256) threads = 256;
  return threads;
}

/* ======================= conv / pointwise ================================ */
typedef struct {
  int which;
  const uint8_t *in; const int8_t *bias; uint8_t *out; const int8_t *w;
  bn_t *k; bn_t *lambda;
  uint16_t out_mult, out_shift, dim_in_x, dim_in_y, ch_in, dim_out_x, dim_out_y, ch_out,
           kx, ky, pt, pb, pl, pr, sx, sy;
  int relu, bn;
  size_t in_sz, out_sz, col_sz;
  uint8_t **s_in, **s_out, **s_col;
} conv_ctx;

static void conv_image(void *vctx, int img, int tid)
{
  conv_ctx *c = (conv_ctx *)vctx;
  memcpy(c->s_in[tid], c->in + (size_t)img * c->in_sz, c->in_sz);
  void (*fn)(const uint8_t *, uint8_t *, const int8_t *, uint8_t *, const int8_t *, bn_t *, bn_t *,
             const uint16_t, const uint16_t, const uint16_t, const uint16_t, const uint16_t,
             const uint16_t, const uint16_t, const uint16_t, const uint16_t, const uint16_t,
             const uint16_t, const uint16_t, const uint16_t, const uint16_t, const uint16_t,
             const uint16_t, int, int);
  switch (c->which) {
    case 0:  fn = pulp_nn_conv_Ho_parallel; break;
    case 1:  fn = pulp_nn_conv_HoWo_parallel; break;
    case 2:  fn = pulp_nn_pointwise_HoWo_parallel; break;
    case 3:  fn = pulp_nn_pointwise_Ho_parallel; break;
    case 4:  fn = pulp_nn_conv_Co_parallel; break;
    default: fn = pulp_nn_pointwise_Co_parallel; break;
  }
  fn(c->s_in[tid], c->s_col[tid], c->bias, c->s_out[tid], c->w, c->k, c->lambda,
     c->out_mult, c->out_shift, c->dim_in_x, c->dim_in_y, c->ch_in, c->dim_out_x, c->dim_out_y,
     c->ch_out, c->kx, c->ky, c->pt, c->pb, c->pl, c->pr, c->sx, c->sy, c->relu, c->bn);
  memcpy(c->out + (size_t)img * c->out_sz, c->s_out[tid], c->out_sz);
}

double refdrv_conv(int which, const uint8_t *in, const int8_t *bias, uint8_t *out, const int8_t *w,
                   void *k, void *lambda, int out_mult, int out_shift,
                   int dim_in_x, int dim_in_y, int ch_in, int dim_out_x, int dim_out_y, int ch_out,
                   int kx, int ky, int pt, int pb, int pl, int pr, int sx, int sy,
                   int relu, int bn, int batch, int threads)
{
  conv_ctx c;
  memset(&c, 0, sizeof c);
  c.which = which; c.in = in; c.bias = bias; c.out = out; c.w = w;
  c.k = (bn_t *)k; c.lambda = (bn_t *)lambda;
  c.out_mult = out_mult; c.out_shift = out_shift; c.dim_in_x = dim_in_x; c.dim_in_y = dim_in_y;
  c.ch_in = ch_in; c.dim_out_x = dim_out_x; c.dim_out_y = dim_out_y; c.ch_out = ch_out;
  c.kx = kx; c.ky = ky; c.pt = pt; c.pb = pb; c.pl = pl; c.pr = pr; c.sx = sx; c.sy = sy;
  c.relu = relu; c.bn = bn;
  c.in_sz = (size_t)dim_in_x * dim_in_y * ch_in;
  c.out_sz = (size_t)dim_out_x * dim_out_y * ch_out;
  c.col_sz = (size_t)2 * NUM_CORES * ch_in * kx * ky;
  threads = clamp_threads(threads, batch);
  uint8_t *s_in[256], *s_out[256], *s_col[256];
  bump_t b = { 0 };
  for (int t = 0; t < threads; t++) {
    s_in[t] = bump(&b, c.in_sz); s_out[t] = bump(&b, c.out_sz); s_col[t] = bump(&b, c.col_sz);
    if (!s_in[t] || !s_out[t] || !s_col[t]) return -1.0;
  }
  c.s_in = s_in; c.s_out = s_out; c.s_col = s_col;
  return run_batch(conv_image, &c, batch, threads);
}

/* ============================ depthwise =================================== */
typedef struct {
  const uint8_t *in; const int8_t *bias; uint8_t *out; const int8_t *w;
  bn_t *k; bn_t *lambda;
  uint16_t out_mult, out_shift, dim_in_x, dim_in_y, ch, dim_out_x, dim_out_y,
           kx, ky, pt, pb, pl, pr, sx, sy;
  int relu, bn, in_is_hwc, variant;
  size_t in_sz, out_sz, buf_sz;
  uint8_t **s_in, **s_out, **s_buf;
  double *glue;
} dw_ctx;

static void dw_image(void *vctx, int img, int tid)
{
  dw_ctx *c = (dw_ctx *)vctx;
  const uint8_t *src = c->in + (size_t)img * c->in_sz;
  if (c->in_is_hwc) {
    /* layout glue that is NOT reference code: HWC -> CHW, timed separately */
    double t0 = now_s();
    const size_t hw = (size_t)c->dim_in_x * c->dim_in_y, C = c->ch;
    uint8_t *dst = c->s_in[tid];
    for (size_t p = 0; p < hw; p++)
      for (size_t ch = 0; ch < C; ch++) dst[ch * hw + p] = src[p * C + ch];
    c->glue[tid] += now_s() - t0;
  } else {
    memcpy(c->s_in[tid], src, c->in_sz);
  }
  /* bn_t k/lambda are advanced through by-value copies inside the callee */
  if (c->variant == 0)
    pulp_nn_depthwise_generic(c->s_in[tid], c->s_buf[tid], c->bias, c->s_out[tid], c->w, NULL,
                              c->k, c->lambda, c->out_mult, c->out_shift, c->dim_in_x, c->dim_in_y,
                              c->ch, c->dim_out_x, c->dim_out_y, c->ch, c->kx, c->ky, c->pt, c->pb,
                              c->pl, c->pr, c->sx, c->sy, (int8_t)c->relu, (int8_t)c->bn);
  else
    pulp_nn_depthwise_generic_less_4_weights(c->s_in[tid], c->s_buf[tid], c->bias, c->s_out[tid],
                              c->w, NULL, c->k, c->lambda, c->out_mult, c->out_shift, c->dim_in_x,
                              c->dim_in_y, c->ch, c->dim_out_x, c->dim_out_y, c->ch, c->kx, c->ky,
                              c->pt, c->pb, c->pl, c->pr, c->sx, c->sy, (int8_t)c->relu,
                              (int8_t)c->bn);
  memcpy(c->out + (size_t)img * c->out_sz, c->s_out[tid], c->out_sz);
}

double refdrv_depthwise(int variant, const uint8_t *in, const int8_t *bias, uint8_t *out,
                        const int8_t *w, void *k, void *lambda, int out_mult, int out_shift,
                        int dim_in_x, int dim_in_y, int ch, int dim_out_x, int dim_out_y,
                        int kx, int ky, int pt, int pb, int pl, int pr, int sx, int sy,
                        int relu, int bn, int in_is_hwc, int batch, int threads,
                        double *glue_seconds)
{
  dw_ctx c;
  memset(&c, 0, sizeof c);
  c.variant = variant; c.in = in; c.bias = bias; c.out = out; c.w = w;
  c.k = (bn_t *)k; c.lambda = (bn_t *)lambda;
  c.out_mult = out_mult; c.out_shift = out_shift; c.dim_in_x = dim_in_x; c.dim_in_y = dim_in_y;
  c.ch = ch; c.dim_out_x = dim_out_x; c.dim_out_y = dim_out_y;
  c.kx = kx; c.ky = ky; c.pt = pt; c.pb = pb; c.pl = pl; c.pr = pr; c.sx = sx; c.sy = sy;
  c.relu = relu; c.bn = bn; c.in_is_hwc = in_is_hwc;
  c.in_sz = (size_t)dim_in_x * dim_in_y * ch;
  c.out_sz = (size_t)dim_out_x * dim_out_y * ch;
  c.buf_sz = (size_t)NUM_CORES * ((size_t)kx * (dim_in_y + pt + pb) + kx) + 16;
  threads = clamp_threads(threads, batch);
  uint8_t *s_in[256], *s_out[256], *s_buf[256];
  double glue[256];
  bump_t b = { 0 };
  for (int t = 0; t < threads; t++) {
    s_in[t] = bump(&b, c.in_sz); s_out[t] = bump(&b, c.out_sz); s_buf[t] = bump(&b, c.buf_sz);
    glue[t] = 0.0;
    if (!s_in[t] || !s_out[t] || !s_buf[t]) return -1.0;
  }
  c.s_in = s_in; c.s_out = s_out; c.s_buf = s_buf; c.glue = glue;
  double dt = run_batch(dw_image, &c, batch, threads);
  if (glue_seconds) {
    double g = 0.0;
    for (int t = 0; t < threads; t++) if (glue[t] > g) g = glue[t];
    *glue_seconds = g;   /* slowest worker's share, comparable with the wall time */
  }
  return dt;
}

/* ================= depthwise 3x3 stride 1, matmul ========================== */
typedef struct {
  const uint8_t *in; uint8_t *out; const int8_t *w; bn_t *k; bn_t *lambda;
  int R, C, CH, p_l, p_r, out_shift, out_mult, relu, bn;
  size_t in_sz, out_sz;
  uint8_t **s_in, **s_out;
} dw3_ctx;

static void dw3_image(void *vctx, int img, int tid)
{
  dw3_ctx *c = (dw3_ctx *)vctx;
  memcpy(c->s_in[tid], c->in + (size_t)img * c->in_sz, c->in_sz);
  pulp_nn_depthwise_3x3_s1(c->s_in[tid], c->s_out[tid], c->R, c->C, c->CH, c->p_l, c->p_r,
                           (int8_t *)c->w, (int8_t)c->out_shift, (uint16_t)c->out_mult, c->k,
                           c->lambda, c->relu, c->bn, NULL);
  memcpy(c->out + (size_t)img * c->out_sz, c->s_out[tid], c->out_sz);
}

/* in: [batch][CH][R][C]; out: [batch][R-2][C][CH] */
double refdrv_depthwise_3x3_s1(const uint8_t *in, uint8_t *out, int R, int C, int CH, int p_l,
                               int p_r, const int8_t *w, int out_shift, int out_mult, void *k,
                               void *lambda, int relu, int bn, int batch, int threads)
{
  dw3_ctx c;
  memset(&c, 0, sizeof c);
  c.in = in; c.out = out; c.w = w; c.k = (bn_t *)k; c.lambda = (bn_t *)lambda;
  c.R = R; c.C = C; c.CH = CH; c.p_l = p_l; c.p_r = p_r; c.out_shift = out_shift;
  c.out_mult = out_mult; c.relu = relu; c.bn = bn;
  c.in_sz = (size_t)R * C * CH;
  c.out_sz = (size_t)(R - 2) * C * CH;
  threads = clamp_threads(threads, batch);
  uint8_t *s_in[256], *s_out[256];
  bump_t b = { 0 };
  for (int t = 0; t < threads; t++) {
    s_in[t] = bump(&b, c.in_sz); s_out[t] = bump(&b, c.out_sz);
    if (!s_in[t] || !s_out[t]) return -1.0;
  }
  c.s_in = s_in; c.s_out = s_out;
  return run_batch(dw3_image, &c, batch, threads);
}

/* in2: the two im2col columns [2][K]; out: [2][ch_out] (pOut, pOut2 = pOut + ch_out).
 * *ret_offset receives (returned pointer - pOut). */
double refdrv_matmul(const int8_t *w, const uint8_t *in2, int ch_out, int K, int out_shift,
                     int out_mult, void *k, void *lambda, const int8_t *bias, uint8_t *out,
                     int relu, int bn, long *ret_offset)
{
  bump_t b = { 0 };
  uint8_t *s_in = bump(&b, 2 * (size_t)K), *s_out = bump(&b, 2 * (size_t)ch_out);
  if (!s_in || !s_out) return -1.0;
  memcpy(s_in, in2, 2 * (size_t)K);
  double t0 = now_s();
  uint8_t *r = pulp_nn_matmul(w, s_in, (uint16_t)ch_out, (uint16_t)K, (uint16_t)out_shift,
                              (uint16_t)out_mult, (bn_t *)k, (bn_t *)lambda, bias, s_out,
                              s_out + ch_out, relu, bn);
  double dt = now_s() - t0;
  memcpy(out, s_out, 2 * (size_t)ch_out);
  if (ret_offset) *ret_offset = (long)(r - s_out);
  return dt;
}

/* ====================== sub-byte unpack helpers ============================ */
/* the helpers live in pulp_nn_utils.c and are declared in pulp_nn_utils.h, which cannot be included
 * here (it pulls in pmsis.h a second time through a different path); same signatures */
void pulp_nn_im2col_u4_to_u8(uint8_t *pInput, uint8_t *pOutput, unsigned int blockSize);
void pulp_nn_im2col_u2_to_u8(uint8_t *pInput, uint8_t *pOutput, unsigned int blockSize);
void pulp_nn_i4_to_i8(int8_t *pSrc, int8_t *pDst);
void pulp_nn_i2_to_i8(int8_t *pSrc, int8_t *pDst);

/* kind: 0 u4, 1 u2, 2 i4, 3 i2. n_out = number of 8-bit results. The signed helpers widen one
 * 32-bit word per call, so n_out must then be a multiple of 8 (i4) or 16 (i2). The helpers load
 * whole words: the input copy is padded. */
double refdrv_unpack(int kind, const uint8_t *in, uint8_t *out, unsigned int n_out)
{
  const unsigned per_byte = (kind == 0 || kind == 2) ? 2u : 4u;
  const size_t n_in = n_out / per_byte;
  bump_t b = { 0 };
  uint8_t *s_in = bump(&b, n_in + 8), *s_out = bump(&b, (size_t)n_out + 16);
  if (!s_in || !s_out) return -1.0;
  memset(s_in, 0, n_in + 8);
  memcpy(s_in, in, n_in);
  double t0 = now_s();
  if (kind == 0) pulp_nn_im2col_u4_to_u8(s_in, s_out, n_out);
  else if (kind == 1) pulp_nn_im2col_u2_to_u8(s_in, s_out, n_out);
  else if (kind == 2) for (size_t i = 0; i < n_in; i += 4) pulp_nn_i4_to_i8((int8_t *)s_in + i, (int8_t *)s_out + 2 * i);
  else for (size_t i = 0; i < n_in; i += 4) pulp_nn_i2_to_i8((int8_t *)s_in + i, (int8_t *)s_out + 4 * i);
  double dt = now_s() - t0;
  memcpy(out, s_out, n_out);
  return dt;
}

/* ============================== linear ==================================== */
typedef struct {
  const uint8_t *in; const int8_t *bias; uint8_t *out8; int32_t *out32; const int8_t *w;
  bn_t *k; bn_t *lambda; uint16_t out_mult; int8_t out_shift; uint16_t dim_vec, num_o;
  int relu, bn, raw32;
  uint8_t **s_in, **s_out;
} lin_ctx;

static void lin_image(void *vctx, int img, int tid)
{
  lin_ctx *c = (lin_ctx *)vctx;
  memcpy(c->s_in[tid], c->in + (size_t)img * c->dim_vec, c->dim_vec);
  if (c->raw32) {
    pulp_nn_linear_out_32(c->s_in[tid], (int8_t *)c->bias, (int32_t *)c->s_out[tid],
                          (int8_t *)c->w, c->dim_vec, c->num_o);
    memcpy(c->out32 + (size_t)img * c->num_o, c->s_out[tid], (size_t)4 * c->num_o);
  } else {
    pulp_nn_linear(c->s_in[tid], (int8_t *)c->bias, c->s_out[tid], (int8_t *)c->w, c->k, c->lambda,
                   c->out_mult, c->out_shift, c->dim_vec, c->num_o, c->relu, c->bn);
    memcpy(c->out8 + (size_t)img * c->num_o, c->s_out[tid], c->num_o);
  }
}

double refdrv_linear(int raw32, const uint8_t *in, const int8_t *bias, void *out, const int8_t *w,
                     void *k, void *lambda, int out_mult, int out_shift, int dim_vec, int num_o,
                     int relu, int bn, int batch, int threads)
{
  lin_ctx c;
  memset(&c, 0, sizeof c);
  c.in = in; c.bias = bias; c.w = w; c.k = (bn_t *)k; c.lambda = (bn_t *)lambda;
  c.out8 = (uint8_t *)out; c.out32 = (int32_t *)out;
  c.out_mult = out_mult; c.out_shift = (int8_t)out_shift; c.dim_vec = dim_vec; c.num_o = num_o;
  c.relu = relu; c.bn = bn; c.raw32 = raw32;
  threads = clamp_threads(threads, batch);
  uint8_t *s_in[256], *s_out[256];
  bump_t b = { 0 };
  for (int t = 0; t < threads; t++) {
    s_in[t] = bump(&b, dim_vec); s_out[t] = bump(&b, (size_t)4 * num_o);
    if (!s_in[t] || !s_out[t]) return -1.0;
  }
  c.s_in = s_in; c.s_out = s_out;
  return run_batch(lin_image, &c, batch, threads);
}

/* =========================== pooling / add ================================ */
typedef struct {
  int op;   /* 0 maxpool, 1 avgpool, 2 add */
  const uint8_t *in, *in2; uint8_t *out; uint8_t *in_after;
  bn_t lambda, out_add; uint16_t out_shift, m1, m2;
  uint16_t dim_in_x, dim_in_y, ch, dim_out_x, dim_out_y, kx, ky, pt, pb, pl, pr, sx, sy;
  int requant;
  size_t in_sz, out_sz;
  uint8_t **s_in, **s_in2, **s_out;
} pool_ctx;

static void pool_image(void *vctx, int img, int tid)
{
  pool_ctx *c = (pool_ctx *)vctx;
  memcpy(c->s_in[tid], c->in + (size_t)img * c->in_sz, c->in_sz);
  if (c->op == 0) {
    pulp_nn_maxpool(c->s_in[tid], c->s_out[tid], c->dim_in_x, c->dim_in_y, c->ch, c->dim_out_x,
                    c->dim_out_y, c->kx, c->ky, c->pt, c->pb, c->pl, c->pr, c->sx, c->sy);
    if (c->in_after) memcpy(c->in_after + (size_t)img * c->in_sz, c->s_in[tid], c->in_sz);
  } else if (c->op == 1) {
    pulp_nn_avgpool(c->s_in[tid], c->s_out[tid], c->lambda, c->out_shift, c->out_add, c->dim_in_x,
                    c->dim_in_y, c->ch, c->dim_out_x, c->dim_out_y, c->kx, c->ky, c->pt, c->pb,
                    c->pl, c->pr, c->sx, c->sy, c->requant);
  } else {
    memcpy(c->s_in2[tid], c->in2 + (size_t)img * c->in_sz, c->in_sz);
    pulp_nn_add(c->s_in[tid], c->s_in2[tid], c->s_out[tid], c->m1, c->m2, c->out_shift,
                c->dim_in_y, c->dim_in_x, c->ch);
  }
  memcpy(c->out + (size_t)img * c->out_sz, c->s_out[tid], c->out_sz);
}

static double pool_common(pool_ctx *c, int batch, int threads)
{
  threads = clamp_threads(threads, batch);
  uint8_t *s_in[256], *s_in2[256], *s_out[256];
  bump_t b = { 0 };
  for (int t = 0; t < threads; t++) {
    s_in[t] = bump(&b, c->in_sz); s_in2[t] = bump(&b, c->in_sz); s_out[t] = bump(&b, c->out_sz);
    if (!s_in[t] || !s_in2[t] || !s_out[t]) return -1.0;
  }
  c->s_in = s_in; c->s_in2 = s_in2; c->s_out = s_out;
  return run_batch(pool_image, c, batch, threads);
}

double refdrv_maxpool(const uint8_t *in, uint8_t *out, uint8_t *in_after,
                      int dim_in_x, int dim_in_y, int ch, int dim_out_x, int dim_out_y,
                      int kx, int ky, int pt, int pb, int pl, int pr, int sx, int sy,
                      int batch, int threads)
{
  pool_ctx c;
  memset(&c, 0, sizeof c);
  c.op = 0; c.in = in; c.out = out; c.in_after = in_after;
  c.dim_in_x = dim_in_x; c.dim_in_y = dim_in_y; c.ch = ch; c.dim_out_x = dim_out_x;
  c.dim_out_y = dim_out_y; c.kx = kx; c.ky = ky; c.pt = pt; c.pb = pb; c.pl = pl; c.pr = pr;
  c.sx = sx; c.sy = sy;
  c.in_sz = (size_t)dim_in_x * dim_in_y * ch; c.out_sz = (size_t)dim_out_x * dim_out_y * ch;
  return pool_common(&c, batch, threads);
}

double refdrv_avgpool(const uint8_t *in, uint8_t *out, int64_t lambda, int out_shift,
                      int64_t out_add, int dim_in_x, int dim_in_y, int ch, int dim_out_x,
                      int dim_out_y, int kx, int ky, int pt, int pb, int pl, int pr, int sx, int sy,
                      int requant, int batch, int threads)
{
  pool_ctx c;
  memset(&c, 0, sizeof c);
  c.op = 1; c.in = in; c.out = out; c.lambda = (bn_t)lambda; c.out_add = (bn_t)out_add;
  c.out_shift = out_shift; c.requant = requant;
  c.dim_in_x = dim_in_x; c.dim_in_y = dim_in_y; c.ch = ch; c.dim_out_x = dim_out_x;
  c.dim_out_y = dim_out_y; c.kx = kx; c.ky = ky; c.pt = pt; c.pb = pb; c.pl = pl; c.pr = pr;
  c.sx = sx; c.sy = sy;
  c.in_sz = (size_t)dim_in_x * dim_in_y * ch; c.out_sz = (size_t)dim_out_x * dim_out_y * ch;
  return pool_common(&c, batch, threads);
}

double refdrv_add(const uint8_t *in1, const uint8_t *in2, uint8_t *out, int m1, int m2,
                  int out_shift, int dim_h, int dim_w, int ch, int batch, int threads)
{
  pool_ctx c;
  memset(&c, 0, sizeof c);
  c.op = 2; c.in = in1; c.in2 = in2; c.out = out; c.m1 = m1; c.m2 = m2; c.out_shift = out_shift;
  c.dim_in_x = dim_w; c.dim_in_y = dim_h; c.ch = ch;
  c.in_sz = (size_t)dim_h * dim_w * ch; c.out_sz = c.in_sz;
  return pool_common(&c, batch, threads);
}
