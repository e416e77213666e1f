// entry_points.cu -- the extern "C" kernel entry points: argument validation, host-buffer
// staging and dispatch to the launchers. One template per reference function, instantiated for
// the 32-bit and the 64-bit batch-norm tree.
#include <type_traits>

#include "internal.cuh"

namespace pulpnn {

namespace {

template <typename BN_T> constexpr int bn_mode() { return sizeof(BN_T) == 4 ? EPI_BN32 : EPI_BN64; }

// (flag_relu, flag_batch_norm) -> epilogue, 32bit/src/pulp_nn_matmul.c:144-216.
template <typename BN_T>
int conv_mode(int flag_relu, int flag_bn)
{
  if (flag_bn && flag_relu) return bn_mode<BN_T>();
  if (flag_relu == 1) return EPI_MULT;
  return EPI_NONE;
}
// 32bit/src/pulp_nn_depthwise_generic.c:167-178: the multiplier path tests truthiness.
template <typename BN_T>
int dw_mode(int8_t flag_relu, int8_t flag_bn)
{
  if (flag_bn && flag_relu) return bn_mode<BN_T>();
  if (flag_relu) return EPI_MULT;
  return EPI_NONE;
}

bool check_shift(int mode, int out_shift, const char *who)
{
  // the helpers take the shift as int8_t (32bit/src/pulp_nn_utils.c:39,151)
  const int d = (int)(int8_t)out_shift;
  const int hi = mode == EPI_BN64 ? 63 : 31;
  if (out_shift != d || d < 0 || d > hi) {
    set_error(PULPNN_ERR_INVALID_ARG, "%s: out_shift %d outside 0..%d", who, out_shift, hi);
    return false;
  }
  return true;
}

bool begin(Context &c, const char *who)
{
  (void)who;
  return ensure_device(c);
}

#define REQUIRE(cond, code, ...)            \
  do {                                      \
    if (!(cond)) {                          \
      set_error(code, __VA_ARGS__);         \
      return;                               \
    }                                       \
  } while (0)

// ---- convolution ---------------------------------------------------------------------------
template <typename BN_T>
void conv_entry(const char *who, bool pointwise, const uint8_t *in, const int8_t *bias, uint8_t *out,
                const int8_t *w, BN_T *k, BN_T *lambda, int out_mult, int out_shift, int dim_in_x,
                int dim_in_y, int ch_in, int dim_out_x, int dim_out_y, int ch_out, int kx, int ky,
                int pt, int pb, int pl, int pr, int sx, int sy, int flag_relu, int flag_bn)
{
  Context &c = ctx();
  if (!begin(c, who)) return;
  REQUIRE(in && out && w, PULPNN_ERR_INVALID_ARG, "%s: NULL input, output or weight pointer", who);
  REQUIRE(dim_in_x > 0 && dim_in_y > 0 && ch_in > 0 && dim_out_x > 0 && dim_out_y > 0 && ch_out > 0,
          PULPNN_ERR_INVALID_ARG, "%s: zero dimension", who);
  const int mode = conv_mode<BN_T>(flag_relu, flag_bn);
  if (!check_shift(mode, out_shift, who)) return;
  REQUIRE(mode < EPI_BN32 || (k && lambda), PULPNN_ERR_INVALID_ARG, "%s: batch-norm mode needs k and lambda", who);
  if (pointwise) {
    // 32bit/src/pulp_nn_pointwise_HoWo_parallel.c:103 indexes the input with dim_in_x and walks
    // dim_out pixels: only equal sizes are a well-defined 1x1 convolution.
    REQUIRE(dim_in_x == dim_out_x && dim_in_y == dim_out_y, PULPNN_ERR_UNSUPPORTED,
            "%s: pointwise needs dim_in == dim_out (got %dx%d -> %dx%d)", who, dim_in_x, dim_in_y,
            dim_out_x, dim_out_y);
    kx = ky = 1; pt = pb = pl = pr = 0; sx = sy = 1;
  } else {
    REQUIRE(kx > 0 && ky > 0 && sx > 0 && sy > 0, PULPNN_ERR_INVALID_ARG, "%s: zero kernel size or stride", who);
    // outside this the reference reads past its input (interior pixels are not bounds-checked,
    // 32bit/src/pulp_nn_conv_Ho_parallel.c:119-126)
    REQUIRE((dim_out_x - 1) * sx + kx <= dim_in_x + pl + pr && (dim_out_y - 1) * sy + ky <= dim_in_y + pt + pb,
            PULPNN_ERR_UNSUPPORTED, "%s: output size larger than floor((in + pads - kernel)/stride) + 1", who);
  }
  const long long K = (long long)kx * ky * ch_in;
  // num_col_im2col is a uint16_t in the reference matmul (32bit/src/pulp_nn_matmul.c:31)
  REQUIRE(K <= 65535, PULPNN_ERR_UNSUPPORTED, "%s: reduction length %lld exceeds 65535", who, K);

  const size_t in_b = (size_t)c.batch * dim_in_x * dim_in_y * ch_in;
  const size_t out_b = (size_t)c.batch * dim_out_x * dim_out_y * ch_out;
  Stager st(c);
  ConvProblem p;
  p.in = static_cast<const uint8_t *>(st.in(in, in_b));
  p.w = static_cast<const int8_t *>(st.in(w, (size_t)ch_out * K));
  p.out = st.out(out, out_b);
  p.epi.bias = st.in(bias, ch_out);
  p.epi.k = mode >= EPI_BN32 ? st.in(k, sizeof(BN_T) * ch_out) : nullptr;
  p.epi.lambda = mode >= EPI_BN32 ? st.in(lambda, sizeof(BN_T) * ch_out) : nullptr;
  if (!st.ok()) return;
  p.epi.mode = mode;
  p.epi.out_mult = (int)(int16_t)(uint16_t)out_mult;
  p.epi.shift = out_shift;
  p.B = c.batch; p.H = dim_in_y; p.W = dim_in_x; p.Cin = ch_in; p.Ho = dim_out_y; p.Wo = dim_out_x;
  p.Cout = ch_out; p.ky = ky; p.kx = kx; p.pt = pt; p.pl = pl; p.sy = sy; p.sx = sx;
  if (!launch_conv(c, p)) return;
  st.finish();
}

// ---- depthwise -----------------------------------------------------------------------------
// The reference equals a zero-padded depthwise convolution only inside this domain; outside it
// its strip builder reads neighbouring bytes, so such calls are rejected rather than imitated.
bool depthwise_domain(const char *who, int W, int H, int Wo, int Ho, int kx, int ky, int pt, int pb,
                      int pl, int pr, int sx, int sy, bool need_four_taps)
{
  if (!(kx & 1) || pl != kx / 2) {
    // right-hand zero padding is derived from kx/2 (32bit/src/pulp_nn_depthwise_generic.c:316)
    set_error(PULPNN_ERR_UNSUPPORTED, "%s: needs odd dim_kernel_x and padding_x_left == dim_kernel_x/2", who);
    return false;
  }
  if (need_four_taps && kx * ky < 4) {
    // the tap loop is a do-while over groups of four (ibid. :157-166); the _less_4_weights variant
    // tests before the first group (pulp_nn_depthwise_generic_less_4_weights.c:156) and takes any count
    set_error(PULPNN_ERR_UNSUPPORTED, "%s: needs at least 4 taps", who);
    return false;
  }
  if ((Ho - 1) * sy + ky > H + pt + pb || (Wo - 1) * sx + kx > W + pl + pr) {
    set_error(PULPNN_ERR_UNSUPPORTED, "%s: output size larger than floor((in + pads - kernel)/stride) + 1", who);
    return false;
  }
  // columns: [0, n_left) are built with left zeros only, then at least one column and every
  // column below Wo - padding_x_right is copied without any check (ibid. :185-280); only the
  // last padding_x_right columns get right-hand zeros.
  const int n_left = pl > 0 ? (pl + sx - 1) / sx : 0;
  const int mid_end = (Wo - pr) > (n_left + 1) ? (Wo - pr) : (n_left + 1);
  if (mid_end > Wo) {
    set_error(PULPNN_ERR_UNSUPPORTED, "%s: output too narrow for the reference's column zones", who);
    return false;
  }
  const int last_unpadded = mid_end - 1;     // also covers the left-zone columns
  if (last_unpadded * sx - pl + kx > W) {
    set_error(PULPNN_ERR_UNSUPPORTED, "%s: a window needs right-hand zeros outside the last padding_x_right columns", who);
    return false;
  }
  return true;
}

template <typename BN_T>
void depthwise_entry(const char *who, bool in_is_hwc, bool need_four_taps, const uint8_t *in, const int8_t *bias, uint8_t *out,
                     const int8_t *w, BN_T *k, BN_T *lambda, int out_mult, int out_shift, int W, int H,
                     int ch_in, int Wo, int Ho, int ch_out, int kx, int ky, int pt, int pb, int pl,
                     int pr, int sx, int sy, int8_t flag_relu, int8_t flag_bn)
{
  Context &c = ctx();
  if (!begin(c, who)) return;
  REQUIRE(in && out && w, PULPNN_ERR_INVALID_ARG, "%s: NULL input, output or weight pointer", who);
  REQUIRE(W > 0 && H > 0 && ch_in > 0 && Wo > 0 && Ho > 0 && kx > 0 && ky > 0 && sx > 0 && sy > 0,
          PULPNN_ERR_INVALID_ARG, "%s: zero dimension", who);
  REQUIRE(ch_in == ch_out, PULPNN_ERR_UNSUPPORTED, "%s: channel multiplier other than 1", who);
  const int mode = dw_mode<BN_T>(flag_relu, flag_bn);
  if (!check_shift(mode, out_shift, who)) return;
  REQUIRE(mode < EPI_BN32 || (k && lambda), PULPNN_ERR_INVALID_ARG, "%s: batch-norm mode needs k and lambda", who);
  if (!depthwise_domain(who, W, H, Wo, Ho, kx, ky, pt, pb, pl, pr, sx, sy, need_four_taps)) return;

  Stager st(c);
  DepthwiseProblem p;
  p.in = static_cast<const uint8_t *>(st.in(in, (size_t)c.batch * W * H * ch_in));
  p.w = static_cast<const int8_t *>(st.in(w, (size_t)ch_in * kx * ky));
  p.out = static_cast<uint8_t *>(st.out(out, (size_t)c.batch * Wo * Ho * ch_in));
  p.epi.bias = st.in(bias, ch_in);
  p.epi.k = mode >= EPI_BN32 ? st.in(k, sizeof(BN_T) * ch_in) : nullptr;
  p.epi.lambda = mode >= EPI_BN32 ? st.in(lambda, sizeof(BN_T) * ch_in) : nullptr;
  if (!st.ok()) return;
  p.epi.mode = mode;
  p.epi.out_mult = (int)(int16_t)(uint16_t)out_mult;
  p.epi.shift = out_shift;
  p.B = c.batch; p.H = H; p.W = W; p.C = ch_in; p.Ho = Ho; p.Wo = Wo; p.ky = ky; p.kx = kx;
  p.pt = pt; p.pl = pl; p.sy = sy; p.sx = sx; p.in_is_hwc = in_is_hwc;
  if (!launch_depthwise(c, p)) return;
  st.finish();
}

// ---- pulp_nn_depthwise_3x3_s1 ------------------------------------------------------------------
// 32bit/src/pulp_nn_depthwise_3x3_s1.c:28-210: CHW input of R rows x C columns, 3x3 filter, stride
// 1, NO vertical padding (rows 0 .. R-3 are produced, :103), HWC output of R-2 rows x C columns,
// no bias. Left and right columns are padded only when p_l / p_r are set (:105,196). The function
// equals a zero-padded convolution only for p_l = p_r = 1 and even C: without p_l the row loop
// starts at column 0 with the window of column 1 and runs two columns into the next row, and an
// odd C makes the two-column loop (:140) write one pixel past the row. Such calls are rejected.
template <typename BN_T>
void depthwise_3x3_s1_entry(const uint8_t *in, uint8_t *out, int R, int C, int CH, int p_l, int p_r,
                            const int8_t *w, int out_shift, int out_mult, BN_T *k, BN_T *lambda,
                            int flag_relu, int flag_bn)
{
  const char *who = "pulp_nn_depthwise_3x3_s1";
  Context &c = ctx();
  if (!begin(c, who)) return;
  REQUIRE(in && out && w, PULPNN_ERR_INVALID_ARG, "%s: NULL input, output or weight pointer", who);
  REQUIRE(R >= 3 && C >= 2 && CH > 0 && R <= 65535 && C <= 65535 && CH <= 65535, PULPNN_ERR_INVALID_ARG,
          "%s: needs 3 <= R, 2 <= C, 1 <= CH, all at most 65535", who);
  REQUIRE(p_l == 1 && p_r == 1 && (C & 1) == 0, PULPNN_ERR_UNSUPPORTED,
          "%s: only p_l = p_r = 1 with an even C is a zero-padded convolution in the reference", who);
  const int mode = conv_mode<BN_T>(flag_relu, flag_bn);
  if (!check_shift(mode, out_shift, who)) return;
  REQUIRE(mode < EPI_BN32 || (k && lambda), PULPNN_ERR_INVALID_ARG, "%s: batch-norm mode needs kappa and lambda", who);
  Stager st(c);
  DepthwiseProblem p;
  p.in = static_cast<const uint8_t *>(st.in(in, (size_t)c.batch * R * C * CH));
  p.w = static_cast<const int8_t *>(st.in(w, (size_t)CH * 9));
  p.out = static_cast<uint8_t *>(st.out(out, (size_t)c.batch * (R - 2) * C * CH));
  p.epi.bias = nullptr;
  p.epi.k = mode >= EPI_BN32 ? st.in(k, sizeof(BN_T) * CH) : nullptr;
  p.epi.lambda = mode >= EPI_BN32 ? st.in(lambda, sizeof(BN_T) * CH) : nullptr;
  if (!st.ok()) return;
  p.epi.mode = mode;
  p.epi.out_mult = (int)(int16_t)(uint16_t)out_mult;
  p.epi.shift = out_shift;
  p.B = c.batch; p.H = R; p.W = C; p.C = CH; p.Ho = R - 2; p.Wo = C; p.ky = 3; p.kx = 3;
  p.pt = 0; p.pl = 1; p.sy = 1; p.sx = 1; p.in_is_hwc = false;
  if (!launch_depthwise(c, p)) return;
  st.finish();
}

// ---- pulp_nn_matmul --------------------------------------------------------------------------
// The inner kernel of the reference's convolutions (32bit/src/pulp_nn_matmul.c:27-298): the two
// im2col columns pInBuffer[0 .. K) and pInBuffer[K .. 2K) (:55-56) against all ch_out filters,
// results to pOut and pOut2, the same three requantisation modes (:144-216). Two rows of the GEMM
// that serves the convolutions; the batch setting does not apply.
template <typename BN_T>
void matmul_entry(const int8_t *w, const uint8_t *in, int ch_out, int K, int out_shift, int out_mult,
                  BN_T *k, BN_T *lambda, const int8_t *bias, uint8_t *out, uint8_t *out2, int flag_relu,
                  int flag_bn)
{
  const char *who = "pulp_nn_matmul";
  Context &c = ctx();
  if (!begin(c, who)) return;
  REQUIRE(in && out && out2 && w, PULPNN_ERR_INVALID_ARG, "%s: NULL input, output or weight pointer", who);
  REQUIRE(ch_out > 0 && K > 0, PULPNN_ERR_INVALID_ARG, "%s: zero dimension", who);
  const int mode = conv_mode<BN_T>(flag_relu, flag_bn);
  if (!check_shift(mode, out_shift, who)) return;
  REQUIRE(mode < EPI_BN32 || (k && lambda), PULPNN_ERR_INVALID_ARG, "%s: batch-norm mode needs k and lambda", who);
  Stager st(c);
  ConvProblem p;
  const uint8_t *din = static_cast<const uint8_t *>(st.in(in, 2 * (size_t)K));
  p.w = static_cast<const int8_t *>(st.in(w, (size_t)ch_out * K));
  uint8_t *dout[2];
  const bool adjacent = out2 == out + ch_out;          // the usual call: one [2][ch_out] block
  if (adjacent) {
    dout[0] = static_cast<uint8_t *>(st.out(out, 2 * (size_t)ch_out));
    dout[1] = dout[0] ? dout[0] + ch_out : nullptr;
  } else {
    dout[0] = static_cast<uint8_t *>(st.out(out, (size_t)ch_out));
    dout[1] = static_cast<uint8_t *>(st.out(out2, (size_t)ch_out));
  }
  p.epi.bias = st.in(bias, ch_out);
  p.epi.k = mode >= EPI_BN32 ? st.in(k, sizeof(BN_T) * ch_out) : nullptr;
  p.epi.lambda = mode >= EPI_BN32 ? st.in(lambda, sizeof(BN_T) * ch_out) : nullptr;
  if (!st.ok()) return;
  p.epi.mode = mode;
  p.epi.out_mult = (int)(int16_t)(uint16_t)out_mult;
  p.epi.shift = out_shift;
  p.B = 1; p.H = p.Ho = 1; p.Cin = K; p.Cout = ch_out; p.ky = p.kx = 1; p.pt = p.pl = 0; p.sy = p.sx = 1;
  if (adjacent) {
    p.W = p.Wo = 2; p.in = din; p.out = dout[0];
    if (!launch_conv(c, p)) return;
  } else {
    p.W = p.Wo = 1;
    for (int r = 0; r < 2; r++) {
      p.in = din + (size_t)r * K; p.out = dout[r];
      if (!launch_conv(c, p)) return;
    }
  }
  st.finish();
}

// ---- linear --------------------------------------------------------------------------------
template <typename BN_T>
void linear_entry(const uint8_t *in, const int8_t *bias, uint8_t *out, const int8_t *w, BN_T *k,
                  BN_T *lambda, int out_mult, int out_shift, int dim_vec, int num_o, int flag_relu,
                  int flag_bn)
{
  const char *who = "pulp_nn_linear";
  Context &c = ctx();
  if (!begin(c, who)) return;
  REQUIRE(in && out && w, PULPNN_ERR_INVALID_ARG, "%s: NULL input, output or weight pointer", who);
  REQUIRE(dim_vec > 0 && num_o > 0, PULPNN_ERR_INVALID_ARG, "%s: zero dimension", who);
  const int mode = conv_mode<BN_T>(flag_relu, flag_bn);
  if (!check_shift(mode, out_shift, who)) return;
  REQUIRE(mode < EPI_BN32 || (k && lambda), PULPNN_ERR_INVALID_ARG, "%s: batch-norm mode needs k and lambda", who);
  Stager st(c);
  ConvProblem p;
  p.in = static_cast<const uint8_t *>(st.in(in, (size_t)c.batch * dim_vec));
  p.w = static_cast<const int8_t *>(st.in(w, (size_t)num_o * dim_vec));
  p.out = st.out(out, (size_t)c.batch * num_o);
  p.epi.bias = st.in(bias, num_o);
  p.epi.k = mode >= EPI_BN32 ? st.in(k, sizeof(BN_T) * num_o) : nullptr;
  p.epi.lambda = mode >= EPI_BN32 ? st.in(lambda, sizeof(BN_T) * num_o) : nullptr;
  if (!st.ok()) return;
  p.epi.mode = mode;
  p.epi.out_mult = (int)(int16_t)(uint16_t)out_mult;
  p.epi.shift = out_shift;
  p.B = c.batch; p.H = 1; p.W = 1; p.Cin = dim_vec; p.Ho = 1; p.Wo = 1; p.Cout = num_o;
  p.ky = p.kx = 1; p.pt = p.pl = 0; p.sy = p.sx = 1;
  if (!launch_conv(c, p)) return;
  st.finish();
}

void linear_out_32_entry(const uint8_t *in, const int8_t *bias, int32_t *out, const int8_t *w,
                         int dim_vec, int num_o)
{
  const char *who = "pulp_nn_linear_out_32";
  Context &c = ctx();
  if (!begin(c, who)) return;
  REQUIRE(in && out && w, PULPNN_ERR_INVALID_ARG, "%s: NULL input, output or weight pointer", who);
  REQUIRE(dim_vec > 0 && num_o > 0, PULPNN_ERR_INVALID_ARG, "%s: zero dimension", who);
  Stager st(c);
  ConvProblem p;
  p.in = static_cast<const uint8_t *>(st.in(in, (size_t)c.batch * dim_vec));
  p.w = static_cast<const int8_t *>(st.in(w, (size_t)num_o * dim_vec));
  p.out = st.out(out, (size_t)4 * c.batch * num_o);
  // read as int32 words (32bit/src/pulp_nn_linear_out_32.c:54)
  p.epi.bias = st.in(bias, (size_t)4 * num_o);
  if (!st.ok()) return;
  REQUIRE((reinterpret_cast<uintptr_t>(p.epi.bias) & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 3) == 0,
          PULPNN_ERR_INVALID_ARG, "%s: int32 bias/output must be 4-byte aligned", who);
  p.epi.k = p.epi.lambda = nullptr;
  p.epi.mode = EPI_RAW32; p.epi.out_mult = 0; p.epi.shift = 0;
  p.B = c.batch; p.H = 1; p.W = 1; p.Cin = dim_vec; p.Ho = 1; p.Wo = 1; p.Cout = num_o;
  p.ky = p.kx = 1; p.pt = p.pl = 0; p.sy = p.sx = 1;
  if (!launch_conv(c, p)) return;
  st.finish();
}

// ---- pooling -------------------------------------------------------------------------------
bool pool_geometry(const char *who, PoolProblem &p, Context &c, int W, int H, int C, int Wo, int Ho,
                   int kx, int ky, int pt, int pb, int pl, int pr, int sx, int sy)
{
  if (!(W > 0 && H > 0 && C > 0 && Wo > 0 && Ho > 0 && kx > 0 && ky > 0 && sx > 0 && sy > 0)) {
    set_error(PULPNN_ERR_INVALID_ARG, "%s: zero dimension", who);
    return false;
  }
  p.B = c.batch; p.H = H; p.W = W; p.C = C; p.Ho = Ho; p.Wo = Wo; p.ky = ky; p.kx = kx;
  p.pt = pt; p.pb = pb; p.pl = pl; p.pr = pr; p.sy = sy; p.sx = sx;
  return true;
}

void maxpool_entry(uint8_t *in, uint8_t *out, int W, int H, int C, int Wo, int Ho, int kx, int ky,
                   int pt, int pb, int pl, int pr, int sx, int sy)
{
  const char *who = "pulp_nn_maxpool";
  Context &c = ctx();
  if (!begin(c, who)) return;
  REQUIRE(in && out, PULPNN_ERR_INVALID_ARG, "%s: NULL pointer", who);
  PoolProblem p{};
  if (!pool_geometry(who, p, c, W, H, C, Wo, Ho, kx, ky, pt, pb, pl, pr, sx, sy)) return;
  // The reference pools along x in place in Im_in (32bit/src/pulp_nn_maxpool.c:63,85-92); a
  // window that starts at or left of a column already overwritten would read pooled values.
  REQUIRE(sx > pl, PULPNN_ERR_UNSUPPORTED, "%s: needs stride_x > padding_l (the reference pools in place)", who);
  REQUIRE(Wo <= W, PULPNN_ERR_UNSUPPORTED, "%s: dim_im_out_x exceeds dim_im_in_x", who);
  REQUIRE((Wo - 1) * sx - pl < W && (Ho - 1) * sy - pt < H, PULPNN_ERR_UNSUPPORTED,
          "%s: an output window lies entirely outside the image", who);
  Stager st(c);
  const size_t in_b = (size_t)c.batch * W * H * C;
  uint8_t *din = static_cast<uint8_t *>(c.opt_maxpool_clobber ? st.inout(in, in_b)
                                                              : const_cast<void *>(st.in(in, in_b)));
  p.in = din;
  p.out = static_cast<uint8_t *>(st.out(out, (size_t)c.batch * Wo * Ho * C));
  if (!st.ok()) return;
  if (!launch_maxpool(c, p, c.opt_maxpool_clobber ? din : nullptr)) return;
  st.finish();
}

template <typename BN_T>
void avgpool_entry(uint8_t *in, uint8_t *out, BN_T lambda, int out_shift, BN_T out_add, int W, int H,
                   int C, int Wo, int Ho, int kx, int ky, int pt, int pb, int pl, int pr, int sx,
                   int sy, int flag_requant)
{
  const char *who = "pulp_nn_avgpool";
  Context &c = ctx();
  if (!begin(c, who)) return;
  REQUIRE(in && out, PULPNN_ERR_INVALID_ARG, "%s: NULL pointer", who);
  PoolProblem p{};
  if (!pool_geometry(who, p, c, W, H, C, Wo, Ho, kx, ky, pt, pb, pl, pr, sx, sy)) return;
  const int hi = sizeof(BN_T) == 4 ? 31 : 63;
  REQUIRE(!flag_requant || (out_shift >= 0 && out_shift <= hi), PULPNN_ERR_INVALID_ARG,
          "%s: out_shift %d outside 0..%d", who, out_shift, hi);
  p.bn_bits = 8 * (int)sizeof(BN_T); p.requant = flag_requant != 0; p.shift = out_shift;
  p.lambda = (long long)lambda; p.out_add = (long long)out_add;
  Stager st(c);
  p.in = static_cast<const uint8_t *>(st.in(in, (size_t)c.batch * W * H * C));
  p.out = static_cast<uint8_t *>(st.out(out, (size_t)c.batch * Wo * Ho * C));
  if (!st.ok()) return;
  if (!launch_avgpool(c, p)) return;
  st.finish();
}

void add_entry(uint8_t *a, uint8_t *b, uint8_t *out, int m1, int m2, int out_shift, int H, int W, int C)
{
  const char *who = "pulp_nn_add";
  Context &c = ctx();
  if (!begin(c, who)) return;
  REQUIRE(a && b && out, PULPNN_ERR_INVALID_ARG, "%s: NULL pointer", who);
  REQUIRE(H > 0 && W > 0 && C > 0, PULPNN_ERR_INVALID_ARG, "%s: zero dimension", who);
  const int d = (int)(int8_t)out_shift;
  REQUIRE(d == out_shift && d >= 0 && d <= 31, PULPNN_ERR_INVALID_ARG, "%s: out_shift %d outside 0..31", who, out_shift);
  const size_t n = (size_t)c.batch * H * W * C;
  Stager st(c);
  const uint8_t *da = static_cast<const uint8_t *>(st.in(a, n));
  const uint8_t *db = static_cast<const uint8_t *>(st.in(b, n));
  uint8_t *dout = static_cast<uint8_t *>(st.out(out, n));
  if (!st.ok()) return;
  // the multipliers reach the helper as int16_t (32bit/src/pulp_nn_utils.c:50-51)
  if (!launch_add(c, da, db, dout, n, (int)(int16_t)(uint16_t)m1, (int)(int16_t)(uint16_t)m2, d)) return;
  st.finish();
}

}  // namespace

// contraction dispatch: tensor cores where the shape allows, CUDA cores otherwise
bool launch_conv(Context &c, const ConvProblem &p)
{
  if (!c.opt_force_generic && c.opt_split_k == 0 && !(c.opt_tune & 16) && gemm_fewrows_supported(p)) return launch_gemm_fewrows(c, p);
  // The SM-pair kernel: measured equal to the one-CTA kernel for K = 512 (0.054 against 0.053 ms on
  // 14x14x512 -> 512 at batch 1024) and 3-5 % faster for K = 1024 (0.047 against 0.049 ms on 7x7x1024 ->
  // 1024), slower below a few hundred rows per SM pair: taken for K >= 1024 and large M, or on request.
  if (!c.opt_force_generic && c.opt_split_k == 0 && igemm_tc2_supported(c, p) &&
      ((c.opt_tune & 8) || (p.Cin >= 1024 && ((long long)p.B * p.Ho * p.Wo / 256) * (p.Cout / 256) >= 4LL * 74)))
    return launch_igemm_tc2(c, p);
  if (!c.opt_force_generic && igemm_tc_supported(c, p)) return launch_igemm_tc(c, p);
  if (!c.opt_force_generic && conv_smallcin_tc_supported(p)) return launch_conv_smallcin_tc(c, p);
  if (!c.opt_force_generic && conv_smallcin_supported(p)) return launch_conv_smallcin(c, p);
  return launch_conv_generic(c, p);
}

}  // namespace pulpnn

using namespace pulpnn;

#define PULPNN_DEFINE_TREE(SFX, BN_T)                                                                   \
  extern "C" void pulp_nn_conv_Ho_parallel##SFX(PULPNN_CONV_PARAMS(BN_T))                               \
  {                                                                                                     \
    (void)pIm2ColBuffer;                                                                                \
    conv_entry<BN_T>("pulp_nn_conv_Ho_parallel", false, pInBuffer, bias, pOutBuffer, pWeight, k, lambda, \
                     out_mult, out_shift, dim_in_x, dim_in_y, ch_in, dim_out_x, dim_out_y, ch_out,      \
                     dim_kernel_x, dim_kernel_y, padding_y_top, padding_y_bottom, padding_x_left,       \
                     padding_x_right, stride_x, stride_y, flag_relu, flag_batch_norm);                  \
  }                                                                                                     \
  extern "C" void pulp_nn_conv_HoWo_parallel##SFX(PULPNN_CONV_PARAMS(BN_T))                             \
  {                                                                                                     \
    (void)pIm2ColBuffer;                                                                                \
    conv_entry<BN_T>("pulp_nn_conv_HoWo_parallel", false, pInBuffer, bias, pOutBuffer, pWeight, k,      \
                     lambda, out_mult, out_shift, dim_in_x, dim_in_y, ch_in, dim_out_x, dim_out_y,      \
                     ch_out, dim_kernel_x, dim_kernel_y, padding_y_top, padding_y_bottom,               \
                     padding_x_left, padding_x_right, stride_x, stride_y, flag_relu, flag_batch_norm);  \
  }                                                                                                     \
  extern "C" void pulp_nn_pointwise_HoWo_parallel##SFX(PULPNN_CONV_PARAMS(BN_T))                        \
  {                                                                                                     \
    (void)pIm2ColBuffer;                                                                                \
    conv_entry<BN_T>("pulp_nn_pointwise_HoWo_parallel", true, pInBuffer, bias, pOutBuffer, pWeight, k,  \
                     lambda, out_mult, out_shift, dim_in_x, dim_in_y, ch_in, dim_out_x, dim_out_y,      \
                     ch_out, dim_kernel_x, dim_kernel_y, padding_y_top, padding_y_bottom,               \
                     padding_x_left, padding_x_right, stride_x, stride_y, flag_relu, flag_batch_norm);  \
  }                                                                                                     \
  /* the other core-slicing variants of the reference compute the same function */                      \
  extern "C" void pulp_nn_conv_Co_parallel##SFX(PULPNN_CONV_PARAMS(BN_T))                               \
  {                                                                                                     \
    (void)pIm2ColBuffer;                                                                                \
    conv_entry<BN_T>("pulp_nn_conv_Co_parallel", false, pInBuffer, bias, pOutBuffer, pWeight, k, lambda, \
                     out_mult, out_shift, dim_in_x, dim_in_y, ch_in, dim_out_x, dim_out_y, ch_out,      \
                     dim_kernel_x, dim_kernel_y, padding_y_top, padding_y_bottom, padding_x_left,       \
                     padding_x_right, stride_x, stride_y, flag_relu, flag_batch_norm);                  \
  }                                                                                                     \
  extern "C" void pulp_nn_pointwise_Ho_parallel##SFX(PULPNN_CONV_PARAMS(BN_T))                          \
  {                                                                                                     \
    (void)pIm2ColBuffer;                                                                                \
    conv_entry<BN_T>("pulp_nn_pointwise_Ho_parallel", true, pInBuffer, bias, pOutBuffer, pWeight, k,    \
                     lambda, out_mult, out_shift, dim_in_x, dim_in_y, ch_in, dim_out_x, dim_out_y,      \
                     ch_out, dim_kernel_x, dim_kernel_y, padding_y_top, padding_y_bottom,               \
                     padding_x_left, padding_x_right, stride_x, stride_y, flag_relu, flag_batch_norm);  \
  }                                                                                                     \
  extern "C" void pulp_nn_pointwise_Co_parallel##SFX(PULPNN_CONV_PARAMS(BN_T))                          \
  {                                                                                                     \
    (void)pIm2ColBuffer;                                                                                \
    conv_entry<BN_T>("pulp_nn_pointwise_Co_parallel", true, pInBuffer, bias, pOutBuffer, pWeight, k,    \
                     lambda, out_mult, out_shift, dim_in_x, dim_in_y, ch_in, dim_out_x, dim_out_y,      \
                     ch_out, dim_kernel_x, dim_kernel_y, padding_y_top, padding_y_bottom,               \
                     padding_x_left, padding_x_right, stride_x, stride_y, flag_relu, flag_batch_norm);  \
  }                                                                                                     \
  extern "C" void pulp_nn_depthwise_generic_less_4_weights##SFX(PULPNN_DW_PARAMS(BN_T))                 \
  {                                                                                                     \
    (void)bufferC; (void)bufferB;                                                                       \
    depthwise_entry<BN_T>("pulp_nn_depthwise_generic_less_4_weights", false, false, Im_in, bias, Im_out, \
                          wt, k, lambda, out_mult, out_shift, dim_im_in_x, dim_im_in_y, ch_im_in,       \
                          dim_im_out_x, dim_im_out_y, ch_im_out, dim_kernel_x, dim_kernel_y,            \
                          padding_y_top, padding_y_bottom, padding_x_left, padding_x_right, stride_x,   \
                          stride_y, FLAG_RELU, FLAG_BATCH_NORM);                                        \
  }                                                                                                     \
  extern "C" void pulp_nn_depthwise_generic##SFX(PULPNN_DW_PARAMS(BN_T))                                \
  {                                                                                                     \
    (void)bufferC; (void)bufferB;                                                                       \
    depthwise_entry<BN_T>("pulp_nn_depthwise_generic", false, true, Im_in, bias, Im_out, wt, k, lambda, \
                          out_mult, out_shift, dim_im_in_x, dim_im_in_y, ch_im_in, dim_im_out_x,        \
                          dim_im_out_y, ch_im_out, dim_kernel_x, dim_kernel_y, padding_y_top,           \
                          padding_y_bottom, padding_x_left, padding_x_right, stride_x, stride_y,        \
                          FLAG_RELU, FLAG_BATCH_NORM);                                                  \
  }                                                                                                     \
  extern "C" void pulpnn_depthwise_hwc##SFX(PULPNN_DW_PARAMS(BN_T))                                     \
  {                                                                                                     \
    (void)bufferC; (void)bufferB;                                                                       \
    depthwise_entry<BN_T>("pulpnn_depthwise_hwc", true, true, Im_in, bias, Im_out, wt, k, lambda, out_mult, \
                          out_shift, dim_im_in_x, dim_im_in_y, ch_im_in, dim_im_out_x, dim_im_out_y,    \
                          ch_im_out, dim_kernel_x, dim_kernel_y, padding_y_top, padding_y_bottom,       \
                          padding_x_left, padding_x_right, stride_x, stride_y, FLAG_RELU,               \
                          FLAG_BATCH_NORM);                                                             \
  }                                                                                                     \
  extern "C" void pulp_nn_depthwise_3x3_s1##SFX(uint8_t *In_Img, uint8_t *Out_Img, int R, int C, int CH, \
                                                int p_l, int p_r, int8_t *Kernel, int8_t out_shift,     \
                                                uint16_t out_mult, BN_T *kappa, BN_T *lambda,           \
                                                int flag_relu, int flag_batch_norm,                     \
                                                unsigned int *memory_chan)                              \
  {                                                                                                     \
    (void)memory_chan;                                                                                  \
    depthwise_3x3_s1_entry<BN_T>(In_Img, Out_Img, R, C, CH, p_l, p_r, Kernel, out_shift, out_mult,      \
                                 kappa, lambda, flag_relu, flag_batch_norm);                            \
  }                                                                                                     \
  extern "C" uint8_t *pulp_nn_matmul##SFX(const int8_t *pWeight, uint8_t *pInBuffer, uint16_t ch_out,   \
                                          uint16_t num_col_im2col, uint16_t out_shift,                  \
                                          uint16_t out_mult, BN_T *k, BN_T *lambda, const int8_t *bias, \
                                          uint8_t *pOut, uint8_t *pOut2, int flag_relu,                 \
                                          int flag_batch_norm)                                          \
  {                                                                                                     \
    matmul_entry<BN_T>(pWeight, pInBuffer, ch_out, num_col_im2col, out_shift, out_mult, k, lambda,      \
                       bias, pOut, pOut2, flag_relu, flag_batch_norm);                                  \
    return pOut ? pOut + 2 * (size_t)ch_out : pOut;      /* 32bit/src/pulp_nn_matmul.c:296-297 */       \
  }                                                                                                     \
  extern "C" void pulp_nn_linear##SFX(uint8_t *pInBuffer, int8_t *bias, uint8_t *pOutBuffer,            \
                                      int8_t *pWeights, BN_T *k, BN_T *lambda, uint16_t out_mult,       \
                                      int8_t out_shift, uint16_t dim_vec, uint16_t num_o_neurons,       \
                                      int flag_relu, int flag_batch_norm)                               \
  {                                                                                                     \
    linear_entry<BN_T>(pInBuffer, bias, pOutBuffer, pWeights, k, lambda, out_mult, out_shift, dim_vec,  \
                       num_o_neurons, flag_relu, flag_batch_norm);                                      \
  }                                                                                                     \
  extern "C" void pulp_nn_linear_out_32##SFX(uint8_t *pInBuffer, int8_t *bias, int32_t *pOutBuffer,     \
                                             int8_t *pWeights, uint16_t dim_vec, uint16_t num_o_neurons)\
  {                                                                                                     \
    linear_out_32_entry(pInBuffer, bias, pOutBuffer, pWeights, dim_vec, num_o_neurons);                 \
  }                                                                                                     \
  extern "C" void pulp_nn_maxpool##SFX(uint8_t *Im_in, uint8_t *Im_out, PULPNN_POOL_GEOMETRY)           \
  {                                                                                                     \
    maxpool_entry(Im_in, Im_out, dim_im_in_x, dim_im_in_y, ch_im_in, dim_im_out_x, dim_im_out_y,        \
                  dim_kernel_x, dim_kernel_y, padding_t, padding_b, padding_l, padding_r, stride_x,     \
                  stride_y);                                                                            \
  }                                                                                                     \
  extern "C" void pulp_nn_avgpool##SFX(uint8_t *Im_in, uint8_t *Im_out, BN_T lambda, uint16_t out_shift,\
                                       BN_T out_add, PULPNN_POOL_GEOMETRY, int flag_requant)            \
  {                                                                                                     \
    avgpool_entry<BN_T>(Im_in, Im_out, lambda, out_shift, out_add, dim_im_in_x, dim_im_in_y, ch_im_in,  \
                        dim_im_out_x, dim_im_out_y, dim_kernel_x, dim_kernel_y, padding_t, padding_b,   \
                        padding_l, padding_r, stride_x, stride_y, flag_requant);                        \
  }                                                                                                     \
  extern "C" void pulp_nn_add##SFX(uint8_t *Im_in_1, uint8_t *Im_in_2, uint8_t *Im_out,                 \
                                   uint16_t out_mult1, uint16_t out_mult2, uint16_t out_shift,          \
                                   uint16_t dim_im_in_h, uint16_t dim_im_in_w, uint16_t ch_im_in)       \
  {                                                                                                     \
    add_entry(Im_in_1, Im_in_2, Im_out, out_mult1, out_mult2, out_shift, dim_im_in_h, dim_im_in_w,      \
              ch_im_in);                                                                                \
  }

PULPNN_DEFINE_TREE(_bn32, int32_t)
PULPNN_DEFINE_TREE(_bn64, int64_t)
