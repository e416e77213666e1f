/* dropin.c -- unsuffixed reference names forwarding to one tree of libpulpnn_b200.so.
 * Compiled twice: -DPULPNN_BN_BITS=32 -> libpulpnn_b200_32.so, =64 -> libpulpnn_b200_64.so. */
#include "../../include/pulpnn_b200_dropin.h"

#if PULPNN_BN_BITS == 32
#define BN_T int32_t
#define SFX(name) name##_bn32
#else
#define BN_T int64_t
#define SFX(name) name##_bn64
#endif

#define CONV_ARGS                                                                              \
  pInBuffer, pIm2ColBuffer, bias, pOutBuffer, pWeight, k, lambda, out_mult, out_shift,         \
  dim_in_x, dim_in_y, ch_in, dim_out_x, dim_out_y, ch_out, dim_kernel_x, dim_kernel_y,         \
  padding_y_top, padding_y_bottom, padding_x_left, padding_x_right, stride_x, stride_y,        \
  flag_relu, flag_batch_norm
#define DW_ARGS                                                                                \
  Im_in, bufferC, bias, Im_out, wt, bufferB, k, lambda, out_mult, out_shift, dim_im_in_x,      \
  dim_im_in_y, ch_im_in, dim_im_out_x, dim_im_out_y, ch_im_out, dim_kernel_x, dim_kernel_y,    \
  padding_y_top, padding_y_bottom, padding_x_left, padding_x_right, stride_x, stride_y,        \
  FLAG_RELU, FLAG_BATCH_NORM
#define POOL_ARGS                                                                              \
  dim_im_in_x, dim_im_in_y, ch_im_in, dim_im_out_x, dim_im_out_y, dim_kernel_x, dim_kernel_y,  \
  padding_t, padding_b, padding_l, padding_r, stride_x, stride_y

void pulp_nn_conv_Ho_parallel(PULPNN_CONV_PARAMS(BN_T)) { SFX(pulp_nn_conv_Ho_parallel)(CONV_ARGS); }
void pulp_nn_conv_HoWo_parallel(PULPNN_CONV_PARAMS(BN_T)) { SFX(pulp_nn_conv_HoWo_parallel)(CONV_ARGS); }
void pulp_nn_pointwise_HoWo_parallel(PULPNN_CONV_PARAMS(BN_T)) { SFX(pulp_nn_pointwise_HoWo_parallel)(CONV_ARGS); }
void pulp_nn_conv_Co_parallel(PULPNN_CONV_PARAMS(BN_T)) { SFX(pulp_nn_conv_Co_parallel)(CONV_ARGS); }
void pulp_nn_pointwise_Ho_parallel(PULPNN_CONV_PARAMS(BN_T)) { SFX(pulp_nn_pointwise_Ho_parallel)(CONV_ARGS); }
void pulp_nn_pointwise_Co_parallel(PULPNN_CONV_PARAMS(BN_T)) { SFX(pulp_nn_pointwise_Co_parallel)(CONV_ARGS); }
void pulp_nn_depthwise_generic(PULPNN_DW_PARAMS(BN_T)) { SFX(pulp_nn_depthwise_generic)(DW_ARGS); }
void pulp_nn_depthwise_generic_less_4_weights(PULPNN_DW_PARAMS(BN_T)) { SFX(pulp_nn_depthwise_generic_less_4_weights)(DW_ARGS); }
void pulpnn_depthwise_hwc(PULPNN_DW_PARAMS(BN_T)) { SFX(pulpnn_depthwise_hwc)(DW_ARGS); }
void pulp_nn_depthwise_3x3_s1(uint8_t *In_Img, uint8_t *Out_Img, int R, int C, int CH, int p_l, int p_r,
                              int8_t *Kernel, int8_t out_shift, uint16_t out_mult, BN_T *kappa, BN_T *lambda,
                              int flag_relu, int flag_batch_norm, unsigned int *memory_chan)
{
  SFX(pulp_nn_depthwise_3x3_s1)(In_Img, Out_Img, R, C, CH, p_l, p_r, Kernel, out_shift, out_mult, kappa, lambda,
                                flag_relu, flag_batch_norm, memory_chan);
}
uint8_t *pulp_nn_matmul(const int8_t *pWeight, uint8_t *pInBuffer, uint16_t ch_out, uint16_t num_col_im2col,
                        uint16_t out_shift, uint16_t out_mult, BN_T *k, BN_T *lambda, const int8_t *bias,
                        uint8_t *pOut, uint8_t *pOut2, int flag_relu, int flag_batch_norm)
{
  return SFX(pulp_nn_matmul)(pWeight, pInBuffer, ch_out, num_col_im2col, out_shift, out_mult, k, lambda, bias,
                             pOut, pOut2, flag_relu, flag_batch_norm);
}
void pulp_nn_linear(uint8_t *pInBuffer, int8_t *bias, uint8_t *pOutBuffer, int8_t *pWeights, BN_T *k,
                    BN_T *lambda, uint16_t out_mult, int8_t out_shift, uint16_t dim_vec,
                    uint16_t num_o_neurons, int flag_relu, int flag_batch_norm)
{
  SFX(pulp_nn_linear)(pInBuffer, bias, pOutBuffer, pWeights, k, lambda, out_mult, out_shift, dim_vec,
                      num_o_neurons, flag_relu, flag_batch_norm);
}
void pulp_nn_linear_out_32(uint8_t *pInBuffer, int8_t *bias, int32_t *pOutBuffer, int8_t *pWeights,
                           uint16_t dim_vec, uint16_t num_o_neurons)
{
  SFX(pulp_nn_linear_out_32)(pInBuffer, bias, pOutBuffer, pWeights, dim_vec, num_o_neurons);
}
void pulp_nn_maxpool(uint8_t *Im_in, uint8_t *Im_out, PULPNN_POOL_GEOMETRY)
{
  SFX(pulp_nn_maxpool)(Im_in, Im_out, POOL_ARGS);
}
void pulp_nn_avgpool(uint8_t *Im_in, uint8_t *Im_out, BN_T lambda, uint16_t out_shift, BN_T out_add,
                     PULPNN_POOL_GEOMETRY, int flag_requant)
{
  SFX(pulp_nn_avgpool)(Im_in, Im_out, lambda, out_shift, out_add, POOL_ARGS, flag_requant);
}
void pulp_nn_add(uint8_t *Im_in_1, uint8_t *Im_in_2, uint8_t *Im_out, uint16_t out_mult1,
                 uint16_t out_mult2, uint16_t out_shift, uint16_t dim_im_in_h, uint16_t dim_im_in_w,
                 uint16_t ch_im_in)
{
  SFX(pulp_nn_add)(Im_in_1, Im_in_2, Im_out, out_mult1, out_mult2, out_shift, dim_im_in_h, dim_im_in_w,
                   ch_im_in);
}
