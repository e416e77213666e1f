/*
 * pulpnn_b200_dropin.h -- the reference's own function names.
 *
 * The PULP-NN tree a program is built against fixes the width of the batch-norm
 * parameters (32bit/ or 64bit/, same function names in both). A program written
 * against 32bit/include/pulp_nn_kernels.h or 64bit/include/pulp_nn_kernels.h
 * switches to this library by including this header instead, with
 * PULPNN_BN_BITS defined as 32 or 64, and linking libpulpnn_b200_32.so or
 * libpulpnn_b200_64.so: the unsuffixed names below have the reference's exact
 * parameter lists (citations in pulpnn_b200.h) and forward to the suffixed entry
 * points of libpulpnn_b200.so.
 */
#ifndef PULPNN_B200_DROPIN_H
#define PULPNN_B200_DROPIN_H

#include "pulpnn_b200.h"

#ifndef PULPNN_BN_BITS
#error "define PULPNN_BN_BITS as 32 or 64 (the reference tree being replaced)"
#endif

#ifdef __cplusplus
extern "C" {
#endif

#if PULPNN_BN_BITS == 32
PULPNN_DECLARE_TREE(, int32_t)
#elif PULPNN_BN_BITS == 64
PULPNN_DECLARE_TREE(, int64_t)
#else
#error "PULPNN_BN_BITS must be 32 or 64"
#endif

#ifdef __cplusplus
}
#endif
#endif /* PULPNN_B200_DROPIN_H */
