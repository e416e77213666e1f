/*
 * pulpnn_b200.h -- C ABI of the B200 (sm_100a) implementation of the PULP-NN
 * 8-bit HWC inference kernels.
 *
 * Every kernel entry point keeps the name, the parameter list and the
 * arithmetic of the reference prototype it replaces; the citation beside each
 * one is the line of 32bit/include/pulp_nn_kernels.h (the 64bit/ header is
 * identical except that k/lambda are int64_t). The reference ships two source
 * trees that export the same names with different batch-norm widths; here one
 * library exports both, suffixed _bn32 / _bn64 (libpulpnn_b200.so), and two
 * thin libraries (libpulpnn_b200_32.so, libpulpnn_b200_64.so, see
 * pulpnn_b200_dropin.h) export the unsuffixed reference names.
 *
 * Calling convention on the GPU
 *  - ONE host thread makes the call once; the grid plays the role of the
 *    reference's cluster of cores. Work is enqueued on the calling thread's
 *    current stream (pulpnn_set_stream) and the call returns without waiting,
 *    unless a buffer is in host memory (see below).
 *  - Pointers may be device pointers (the fast path) or ordinary host
 *    pointers. Host buffers are staged through device memory owned by the
 *    library and the call then returns only after the results are back in the
 *    caller's buffers.
 *  - The reference processes one image per call. pulpnn_set_batch(n) makes
 *    every activation pointer address n images stored back to back; weights
 *    and batch-norm parameters are shared by the batch.
 *  - Scratch arguments of the reference (pIm2ColBuffer, bufferC, bufferB) are
 *    accepted and ignored; they may be NULL.
 *  - The entry points return void like the reference. A call whose arguments
 *    are invalid or outside the supported domain enqueues nothing and records
 *    an error for the calling thread (pulpnn_last_error). There is no CPU
 *    fallback of any kind.
 */
#ifndef PULPNN_B200_H
#define PULPNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status ------------------------------------------------------------- */
enum {
  PULPNN_OK = 0,
  PULPNN_ERR_INVALID_ARG = 1,   /* NULL pointer, zero dimension, shift out of range ...     */
  PULPNN_ERR_UNSUPPORTED = 2,   /* outside the domain where the reference is well defined   */
  PULPNN_ERR_CUDA = 3,          /* a CUDA runtime/driver call failed                        */
  PULPNN_ERR_NO_DEVICE = 4,     /* no usable GPU: the library never computes on the CPU     */
  PULPNN_ERR_DEVICE_WAIT = 5    /* a bounded wait inside a kernel ran out (see status word) */
};

/* ---- per-thread context -------------------------------------------------- */
int  pulpnn_set_device(int device);          /* also creates the context; returns a status   */
int  pulpnn_set_stream(void *cuda_stream);   /* cudaStream_t; NULL = the default stream       */
int  pulpnn_set_batch(int n_images);         /* n >= 1; sticky until changed                  */
int  pulpnn_get_batch(void);
int  pulpnn_synchronize(void);               /* waits for the stream; returns a status        */
int  pulpnn_last_error(void);
const char *pulpnn_last_error_message(void);
void pulpnn_clear_error(void);
/* kernels launched by this library since it was loaded (all threads) */
unsigned long long pulpnn_launch_count(void);
/* Reads and clears the device-side status word: 0 = every bounded wait in the
 * tensor-core kernels completed. Synchronises the stream first. */
int  pulpnn_device_status(void);

/* Tuning / test switches (value 0 or 1 unless stated). */
enum {
  PULPNN_OPT_FORCE_GENERIC = 1,   /* route contractions to the generic CUDA-core kernel      */
  PULPNN_OPT_MAXPOOL_CLOBBER = 2, /* also reproduce the reference's overwrite of Im_in       */
  PULPNN_OPT_SPLIT_K = 3,         /* 0 = choose automatically, n > 0 = force n K-slices      */
  PULPNN_OPT_FUSE_DWPW = 4,       /* network runner: run a 3x3 stride-1 depthwise layer and   */
                                  /* the pointwise layer behind it as ONE kernel where a      */
                                  /* fused kernel exists (default 1); results are identical   */
  PULPNN_OPT_TUNE = 5             /* measurement switch, a bit mask (0 = the defaults). Bits 3-5 */
                                  /* select alternative launch configurations (8: SM-pair GEMM   */
                                  /* from K = 512 on, 16: no few-rows GEMM, 32: the 32-channel   */
                                  /* fused pair with its depthwise sums on the tensor cores);    */
                                  /* results identical.                                          */
                                  /* Bits 8-11 switch PARTS of the tensor-core kernels off to    */
                                  /* time the rest (epilogue, loads, MMAs, stores): the output   */
                                  /* is then wrong by design. Never set them outside a timing run */
};
int  pulpnn_set_option(int option, int value);
int  pulpnn_get_option(int option);

/* ---- kernel entry points -------------------------------------------------- */
/* shared parameter list of the convolution family (pulp_nn_kernels.h:56-82) */
#define PULPNN_CONV_PARAMS(BN_T)                                                              \
  const uint8_t *pInBuffer, uint8_t *pIm2ColBuffer, const int8_t *bias, uint8_t *pOutBuffer,  \
  const int8_t *pWeight, BN_T *k, BN_T *lambda, const uint16_t out_mult,                      \
  const uint16_t out_shift, const uint16_t dim_in_x, const uint16_t dim_in_y,                 \
  const uint16_t ch_in, const uint16_t dim_out_x, const uint16_t dim_out_y,                   \
  const uint16_t ch_out, const uint16_t dim_kernel_x, const uint16_t dim_kernel_y,            \
  const uint16_t padding_y_top, const uint16_t padding_y_bottom,                              \
  const uint16_t padding_x_left, const uint16_t padding_x_right, const uint16_t stride_x,     \
  const uint16_t stride_y, int flag_relu, int flag_batch_norm

/* parameter list of the depthwise family (pulp_nn_kernels.h:282-309) */
#define PULPNN_DW_PARAMS(BN_T)                                                                \
  const uint8_t *Im_in, uint8_t *bufferC, const int8_t *bias, uint8_t *Im_out,                \
  const int8_t *wt, uint8_t *bufferB, BN_T *k, BN_T *lambda, uint16_t out_mult,               \
  uint16_t out_shift, const uint16_t dim_im_in_x, const uint16_t dim_im_in_y,                 \
  const uint16_t ch_im_in, const uint16_t dim_im_out_x, const uint16_t dim_im_out_y,          \
  const uint16_t ch_im_out, const uint16_t dim_kernel_x, const uint16_t dim_kernel_y,         \
  const uint16_t padding_y_top, const uint16_t padding_y_bottom,                              \
  const uint16_t padding_x_left, const uint16_t padding_x_right, const uint16_t stride_x,     \
  const uint16_t stride_y, int8_t FLAG_RELU, int8_t FLAG_BATCH_NORM

/* parameter list of the pooling pair (pulp_nn_kernels.h:264-280 and :33-53) */
#define PULPNN_POOL_GEOMETRY                                                                  \
  uint16_t dim_im_in_x, uint16_t dim_im_in_y, uint16_t ch_im_in, uint16_t dim_im_out_x,       \
  uint16_t dim_im_out_y, uint16_t dim_kernel_x, uint16_t dim_kernel_y, uint16_t padding_t,    \
  uint16_t padding_b, uint16_t padding_l, uint16_t padding_r, uint16_t stride_x,              \
  uint16_t stride_y

/*
 * One tree of entry points. SFX is appended to every reference name, BN_T is
 * the batch-norm parameter type of that tree.
 *
 *  pulp_nn_conv_Ho_parallel         pulp_nn_kernels.h:56    zero-padded convolution, HWC in/out,
 *  pulp_nn_conv_HoWo_parallel       pulp_nn_kernels.h:112   weights [ch_out][ky][kx][ch_in]; the two
 *                                                           differ in the reference only in how cores
 *                                                           split the rows, so they share one kernel
 *  pulp_nn_pointwise_HoWo_parallel  pulp_nn_kernels.h:140   1x1 convolution; kernel/pad/stride
 *                                                           arguments are ignored as in the reference
 *  pulp_nn_conv_Co_parallel         pulp_nn_kernels.h:84    the remaining core-slicing variants: the
 *  pulp_nn_pointwise_Ho_parallel    pulp_nn_kernels.h:168   same function of the same arguments as
 *  pulp_nn_pointwise_Co_parallel    pulp_nn_kernels.h:196   the two above (a grid has no cores to
 *                                                           slice over), so they share their kernels.
 *                                                           Defined as the convolution itself: the
 *                                                           reference's Co-parallel files mis-step
 *                                                           their bias and weight pointers between
 *                                                           channel chunks, which is not imitated
 *  pulp_nn_depthwise_generic        pulp_nn_kernels.h:282   CHW in, HWC out
 *  pulp_nn_depthwise_generic_less_4_weights  :311           same, for kernels of fewer than 4 taps
 *                                                           (accepts any number of taps)
 *  pulp_nn_depthwise_3x3_s1         pulp_nn_kernels.h:340   CHW in (R x C), HWC out (R-2 x C): 3x3,
 *                                                           stride 1, no vertical padding, no bias.
 *                                                           Accepted for p_l = p_r = 1 and even C,
 *                                                           where the reference is a zero-padded
 *                                                           convolution; memory_chan is ignored
 *  pulp_nn_matmul                   pulp_nn_kernels.h:248   the convolutions' inner kernel: two
 *                                                           im2col columns (pInBuffer, pInBuffer +
 *                                                           num_col_im2col) x ch_out filters into
 *                                                           pOut and pOut2; returns pOut + 2*ch_out.
 *                                                           The batch setting does not apply
 *  pulp_nn_linear                   pulp_nn_kernels.h:224   uint8 output, requantised
 *  pulp_nn_linear_out_32            pulp_nn_kernels.h:239   raw int32 output; bias is read as int32[]
 *  pulp_nn_maxpool                  pulp_nn_kernels.h:264   Im_in is left intact unless
 *                                                           PULPNN_OPT_MAXPOOL_CLOBBER is set
 *  pulp_nn_avgpool                  pulp_nn_kernels.h:33    lambda/out_add have the tree's width
 *  pulp_nn_add                      pulp_nn_kernels.h:21
 *
 *  pulpnn_depthwise_hwc             extension: pulp_nn_depthwise_generic arithmetic on HWC input
 *                                   (what every producer in this API emits); no reference counterpart
 */
#define PULPNN_DECLARE_TREE(SFX, BN_T)                                                        \
  void pulp_nn_conv_Ho_parallel##SFX(PULPNN_CONV_PARAMS(BN_T));                               \
  void pulp_nn_conv_HoWo_parallel##SFX(PULPNN_CONV_PARAMS(BN_T));                             \
  void pulp_nn_pointwise_HoWo_parallel##SFX(PULPNN_CONV_PARAMS(BN_T));                        \
  void pulp_nn_conv_Co_parallel##SFX(PULPNN_CONV_PARAMS(BN_T));                               \
  void pulp_nn_pointwise_Ho_parallel##SFX(PULPNN_CONV_PARAMS(BN_T));                          \
  void pulp_nn_pointwise_Co_parallel##SFX(PULPNN_CONV_PARAMS(BN_T));                          \
  void pulp_nn_depthwise_generic##SFX(PULPNN_DW_PARAMS(BN_T));                                \
  void pulp_nn_depthwise_generic_less_4_weights##SFX(PULPNN_DW_PARAMS(BN_T));                 \
  void pulpnn_depthwise_hwc##SFX(PULPNN_DW_PARAMS(BN_T));                                     \
  void pulp_nn_depthwise_3x3_s1##SFX(uint8_t *In_Img, uint8_t *Out_Img, int R, int C, int CH,  \
                                     int p_l, int p_r, int8_t *Kernel, int8_t out_shift,      \
                                     uint16_t out_mult, BN_T *kappa, BN_T *lambda,            \
                                     int flag_relu, int flag_batch_norm,                      \
                                     unsigned int *memory_chan);                              \
  uint8_t *pulp_nn_matmul##SFX(const int8_t *pWeight, uint8_t *pInBuffer, uint16_t ch_out,    \
                               uint16_t num_col_im2col, uint16_t out_shift, uint16_t out_mult,\
                               BN_T *k, BN_T *lambda, const int8_t *bias, uint8_t *pOut,      \
                               uint8_t *pOut2, int flag_relu, int flag_batch_norm);           \
  void pulp_nn_linear##SFX(uint8_t *pInBuffer, int8_t *bias, uint8_t *pOutBuffer,             \
                           int8_t *pWeights, BN_T *k, BN_T *lambda, uint16_t out_mult,        \
                           int8_t out_shift, uint16_t dim_vec, uint16_t num_o_neurons,        \
                           int flag_relu, int flag_batch_norm);                               \
  void pulp_nn_linear_out_32##SFX(uint8_t *pInBuffer, int8_t *bias, int32_t *pOutBuffer,      \
                                  int8_t *pWeights, uint16_t dim_vec, uint16_t num_o_neurons);\
  void pulp_nn_maxpool##SFX(uint8_t *Im_in, uint8_t *Im_out, PULPNN_POOL_GEOMETRY);           \
  void pulp_nn_avgpool##SFX(uint8_t *Im_in, uint8_t *Im_out, BN_T lambda, uint16_t out_shift, \
                            BN_T out_add, PULPNN_POOL_GEOMETRY, int flag_requant);            \
  void pulp_nn_add##SFX(uint8_t *Im_in_1, uint8_t *Im_in_2, uint8_t *Im_out,                  \
                        uint16_t out_mult1, uint16_t out_mult2, uint16_t out_shift,           \
                        uint16_t dim_im_in_h, uint16_t dim_im_in_w, uint16_t ch_im_in);

PULPNN_DECLARE_TREE(_bn32, int32_t)
PULPNN_DECLARE_TREE(_bn64, int64_t)

/*
 * Layout change of uint8 activations, CHW <-> HWC, for the images of the current batch. No
 * counterpart in the reference, which needs one all the same: pulp_nn_depthwise_generic reads CHW
 * (32bit/src/pulp_nn_depthwise_generic.c:74) while every kernel of the library, the depthwise one
 * included, writes HWC (ibid. :81,179). In and out must not overlap.
 */
void pulpnn_chw_to_hwc(const uint8_t *Im_in, uint8_t *Im_out, uint16_t dim_im_x, uint16_t dim_im_y, uint16_t ch_im);
void pulpnn_hwc_to_chw(const uint8_t *Im_in, uint8_t *Im_out, uint16_t dim_im_x, uint16_t dim_im_y, uint16_t ch_im);

/*
 * Sub-byte unpack helpers of the reference as bulk device operations. Packed values sit
 * little-endian in their bytes (element i of a byte = bits [w*i, w*i+w)).
 *   pulp_nn_im2col_u4_to_u8, pulp_nn_im2col_u2_to_u8   32bit/include/pulp_nn_utils.h:65,67
 *       (32bit/src/pulp_nn_utils.c:396-438): blockSize = number of uint8 results; it must be a
 *       multiple of 2 (4): the reference's tail loops never end otherwise.
 *   pulpnn_i4_to_i8, pulpnn_i2_to_i8                    the sign-extending counterparts, bulk forms of
 *       pulp_nn_i4_to_i8 / pulp_nn_i2_to_i8 (pulp_nn_utils.c:255,289); n = number of int8 results.
 * Device or host buffers; the batch setting does not apply.
 */
void pulp_nn_im2col_u4_to_u8(uint8_t *pInput, uint8_t *pOutput, unsigned int blockSize);
void pulp_nn_im2col_u2_to_u8(uint8_t *pInput, uint8_t *pOutput, unsigned int blockSize);
void pulpnn_i4_to_i8(const int8_t *pSrc, int8_t *pDst, unsigned int n);
void pulpnn_i2_to_i8(const int8_t *pSrc, int8_t *pDst, unsigned int n);

/*
 * The scalar requantisers of pulp_nn_utils.h as element-wise bulk device operations: n int32
 * accumulators in, one result byte each out (not packed); element i takes the parameters of channel
 * i % channels; bits = 8, 4 or 2 selects the clip range 255 / 15 / 3. Device or host buffers.
 *   pulpnn_bn_quant_bulk     pulp_nn_bn_quant_u8 / _u4 / _u2   32bit/include/pulp_nn_utils.h:23,29,41
 *                            (32bit/src/pulp_nn_utils.c:35-45,158-167,180-189): clip((k*phi + lambda) >> d),
 *                            int32 wrap-around in the 32-bit tree, int64 in the 64-bit tree
 *   pulpnn_quant_bulk        pulp_nn_quant_u8 / _u4 / _u2      pulp_nn_utils.h:25,31,43
 *                            (pulp_nn_utils.c:148-156,169-178,191-199): clip((m*phi) >> d); the shifted
 *                            value is cut to int16 for 8 bits in both trees and for 4 / 2 bits in the
 *                            64-bit tree only (64bit/src/pulp_nn_utils.c:153,175,197)
 *   pulpnn_threshold_quant_bulk   pulp_nn_i4_quant / pulp_nn_i2_quant   pulp_nn_utils.h:69,71
 *                            (pulp_nn_utils.c:438-540): the signed 4- or 2-bit level of each input among a
 *                            channel's thresholds (int16; 16 per channel of which 15 are read for 4
 *                            bits, 4 per channel of which 3 are read for 2 bits), one int8 out
 *   pulp_nn_avg_and_replace_int8   pulp_nn_utils.h:39 (pulp_nn_utils.c:95-115), the reference's own
 *                            signature: base[i] = (base[i] + target[i]) >> 1 on signed bytes, for
 *                            length >> 2 whole words; the batch setting does not apply
 */
void pulpnn_bn_quant_bulk_bn32(const int32_t *phi, const int32_t *k, const int32_t *lambda, int8_t d, uint8_t *out,
                               unsigned int n, unsigned int channels, int bits);
void pulpnn_bn_quant_bulk_bn64(const int32_t *phi, const int64_t *k, const int64_t *lambda, int8_t d, uint8_t *out,
                               unsigned int n, unsigned int channels, int bits);
void pulpnn_quant_bulk_bn32(const int32_t *phi, int16_t m, int8_t d, uint8_t *out, unsigned int n, int bits);
void pulpnn_quant_bulk_bn64(const int32_t *phi, int16_t m, int8_t d, uint8_t *out, unsigned int n, int bits);
void pulpnn_threshold_quant_bulk(const int32_t *in, const int16_t *thr, int8_t *out, unsigned int n,
                                 unsigned int channels, int bits);
void pulp_nn_avg_and_replace_int8(int8_t *base, int8_t *target, uint16_t length);

/*
 * pulpnn_linear_out_32_static_scratch -- no counterpart in the reference.
 *
 * The arithmetic of pulp_nn_linear_out_32 (int32 accumulators, bias read as int32 words, no
 * requantisation) for n_vectors input vectors, computed with K split over k_slices groups of
 * CTAs, for callers that must not allocate: a service that has given all free device memory to
 * its own pool, or a deployment with a fixed, audited memory budget, cannot have a library call
 * cudaMalloc behind its back (the ordinary split-K path does, the first time and whenever a
 * larger problem arrives). Here the partial sums live in a 4 MiB array that is part of the
 * library image (every GPU that loads the library holds it until the process exits), and the
 * call uses no cudaMalloc, cudaFree or any other allocating routine.
 *
 *  - All four buffers must be device (or managed) memory of the context's GPU -- host buffers
 *    would need staging memory; pInBuffer and pWeights 16-byte aligned, pOutBuffer and bias
 *    4-byte aligned; bias may be NULL; dim_vec must be a multiple of 16.
 *  - Limit: k_slices * n_vectors * num_o_neurons <= 1048576 partial sums (k_slices >= 2, and
 *    dim_vec long enough to split); anything larger is refused with PULPNN_ERR_UNSUPPORTED.
 *  - The first call on a device looks up the array's device address; make that first call
 *    before any stream capture is begun.
 *  - Every call shares the one array, which keeps the previous call's contents. Nothing in it
 *    has to start at zero (each call writes every partial sum it later reads), but two calls
 *    whose kernels overlap on the GPU -- different streams, different host threads -- race.
 *  - Enqueues on the calling thread's stream and returns a status (PULPNN_OK or an error code).
 *  - A bounded wait that runs out inside its kernel is recorded in a status word that is built
 *    into the library as well, and shows up in pulpnn_device_status() like any other.
 */
int pulpnn_linear_out_32_static_scratch(const uint8_t *pInBuffer, const int32_t *bias,
                                        int32_t *pOutBuffer, const int8_t *pWeights, int dim_vec,
                                        int num_o_neurons, int n_vectors, int k_slices);

/*
 * pulpnn_selftest_wait_timeout -- diagnostic, no counterpart in the reference.
 *
 * Every wait inside the TMA / tensor-core kernels is bounded: when it runs out the kernel leaves
 * through its ordinary exit and records a code in the device status word. This call exercises
 * exactly that path without disturbing anything: a one-warp kernel waits, with the given limit
 * (microseconds, clamped to 1..100000), on a barrier that nothing will ever complete. After it,
 * pulpnn_device_status() returns a non-zero code (and clears it) and pulpnn_last_error() is
 * PULPNN_ERR_DEVICE_WAIT; the GPU and the context stay usable. Returns PULPNN_OK when the
 * kernel was enqueued.
 */
int pulpnn_selftest_wait_timeout(unsigned int limit_us);

/* ---- sequential network runner --------------------------------------------
 * The reference is a kernel library; its user chains the calls. This runner is
 * that chain for one GPU: layers are appended in order, parameters are copied
 * to the device once, and run() pushes a batch through every layer with
 * activations ping-ponging between two device buffers owned by the network.
 * Depthwise layers use the HWC-input kernel, so no layout change is needed
 * between layers. Different GPUs run different slices of the batch; nothing is
 * exchanged between them.
 */
typedef struct pulpnn_net pulpnn_net_t;

enum {
  PULPNN_LAYER_CONV = 0,        /* pulp_nn_conv_Ho_parallel                       */
  PULPNN_LAYER_POINTWISE = 1,   /* pulp_nn_pointwise_HoWo_parallel                */
  PULPNN_LAYER_DEPTHWISE = 2,   /* pulpnn_depthwise_hwc                            */
  PULPNN_LAYER_AVGPOOL = 3,     /* pulp_nn_avgpool, flag_requant = 0              */
  PULPNN_LAYER_MAXPOOL = 4,     /* pulp_nn_maxpool                                */
  PULPNN_LAYER_LINEAR_OUT_32 = 5/* pulp_nn_linear_out_32 (must be the last layer) */
};

typedef struct {
  int type;                       /* PULPNN_LAYER_*                                     */
  int dim_in_x, dim_in_y, ch_in;
  int dim_out_x, dim_out_y, ch_out;
  int dim_kernel_x, dim_kernel_y;
  int padding_y_top, padding_y_bottom, padding_x_left, padding_x_right;
  int stride_x, stride_y;
  int out_mult, out_shift, flag_relu, flag_batch_norm;
  const int8_t *weights;          /* host or device memory; copied at add time          */
  const int8_t *bias;             /* may be NULL (int32 words for LINEAR_OUT_32)        */
  const void *k, *lambda;         /* ch_out values of the network's batch-norm width    */
} pulpnn_layer_desc_t;

pulpnn_net_t *pulpnn_net_create(int bn_bits, int max_batch);
int  pulpnn_net_add_layer(pulpnn_net_t *net, const pulpnn_layer_desc_t *desc);
/* Freezes the layer list and allocates the activation buffers. micro_batch = 0
 * lets the library choose how many images travel through the stack together. */
int  pulpnn_net_finalize(pulpnn_net_t *net, int micro_batch);
/* input: n_images x (first layer's input) bytes; output: n_images x (last
 * layer's output). Either may be host or device memory. Enqueues on the calling
 * thread's stream; synchronises only if a host buffer is involved. */
int  pulpnn_net_run(pulpnn_net_t *net, const uint8_t *input, void *output, int n_images);
/* The same with HOST buffers (pinned memory for real overlap), without waiting: the copies and the
 * kernels of this batch are enqueued and the call returns a ticket (0 or 1; a negative value is
 * minus an error code). pulpnn_net_wait(net, ticket) returns once the batch's results are in
 * `output`. Two batches can be in flight, so in a loop that submits batch i+1 before it waits for
 * batch i the input copy of one batch runs under the compute of the other and the step time is the
 * longer of the two instead of their sum. `input` must stay valid and `output` untouched until the
 * wait; submitting a third batch waits for the first by itself. */
int  pulpnn_net_submit(pulpnn_net_t *net, const uint8_t *input, void *output, int n_images);
int  pulpnn_net_wait(pulpnn_net_t *net, int ticket);
/* Test hook: run the first n_layers layers only and copy that layer's output. */
int  pulpnn_net_run_prefix(pulpnn_net_t *net, const uint8_t *input, void *output, int n_images,
                           int n_layers);
/* Measurement hook: like pulpnn_net_run on device buffers, with a CUDA event recorded on the
 * stream between consecutive layer calls; layer_ms[l] receives the milliseconds layer l took
 * (summed over micro-batches). Synchronises. */
int  pulpnn_net_run_timed(pulpnn_net_t *net, const uint8_t *input, void *output, int n_images,
                          float *layer_ms);
int  pulpnn_net_num_layers(const pulpnn_net_t *net);
size_t pulpnn_net_layer_output_bytes(const pulpnn_net_t *net, int layer);   /* per image */
/* How layer `layer` ran in the most recent run: 0 = a kernel of its own, 1 / 2 = the first /
 * second layer of a pair executed as one fused kernel (PULPNN_OPT_FUSE_DWPW); -1 = no such layer. */
int  pulpnn_net_layer_role(const pulpnn_net_t *net, int layer);
/* The kernel family that ran layer `layer` in the most recent run ("igemm_tc_kernel", ...), for
 * measurement tables; "" before the first run. */
const char *pulpnn_net_layer_kernel(const pulpnn_net_t *net, int layer);
/* Kernel launches the most recent pulpnn_net_run / _run_prefix / _run_timed of this network made
 * (0 before the first run). n_images is ignored. */
unsigned long long pulpnn_net_launches_per_run(const pulpnn_net_t *net, int n_images);
void pulpnn_net_destroy(pulpnn_net_t *net);

#ifdef __cplusplus
}
#endif
#endif /* PULPNN_B200_H */
