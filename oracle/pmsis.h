/*
 * pmsis.h -- host stand-in for the PULP platform header, TEST INFRASTRUCTURE ONLY.
 *
 * The PULP-NN sources include "pmsis.h" for three things: the 4x8-bit vector
 * types, the cluster calls (core id, team barrier) and the Xpulp compiler
 * builtins. This file supplies portable definitions of exactly those so the
 * unmodified reference sources compile with a stock x86-64 gcc. It is used
 * only to build the checker under oracle/_ref/ ; nothing that ships links it.
 *
 * Semantics of each builtin are the ones the reference relies on at its call
 * sites (file:line are paths inside the PULP-NN tree):
 *   sdotusp4   32bit/src/pulp_nn_matmul.c:105-113   c + sum_i u8[i]*s8[i]
 *   clipu_r    32bit/src/pulp_nn_utils.c:43         clamp a 32-bit int to [0,hi]
 *   fl1        32bit/src/pulp_nn_conv_Ho_parallel.c:63  index of the top set bit
 *   bextract/u 32bit/src/pulp_nn_utils.c:208,222    bit-field extract (signed/unsigned)
 *   pack4      32bit/src/pulp_nn_utils.c:212,226    build a v4s or v4u from 4 scalars
 *   maxu4/avg4 32bit/src/pulp_nn_utils.c:80,108     per-byte unsigned max / signed mean
 *   minsi/maxsi 32bit/src/pulp_nn_avgpool.c:26-27   signed min / max
 *   shuffleb   32bit/src/pulp_nn_depthwise_3x3_s1.c:89  byte permute r[i]=v[m[i]&3]
 *   clipu      32bit/src/pulp_nn_depthwise_3x3_s1.c:26  clamp to [lo,hi]
 *
 * Build flags this shim expects (see oracle/Makefile): -std=gnu11 -fwrapv
 * -fno-strict-aliasing -fno-semantic-interposition -DNUM_CORES=<power of two>.
 */
#ifndef PULPNN_HOST_PMSIS_H
#define PULPNN_HOST_PMSIS_H

#include <stdint.h>
#include <stddef.h>

#ifndef NUM_CORES
#define NUM_CORES 1
#endif

typedef int8_t  v4s __attribute__((vector_size(4)));
typedef uint8_t v4u __attribute__((vector_size(4)));

/* ---- cluster calls ------------------------------------------------------
 * With NUM_CORES == 1 the single "core" has id 0 and the barrier is a no-op.
 * A threaded build (NUM_CORES > 1) gets both from the driver translation unit.
 */
#if NUM_CORES == 1
static inline int  pi_core_id(void) { return 0; }
static inline void pi_cl_team_barrier(int unused) { (void)unused; }
#else
extern __thread int pulpnn_host_core_id;
extern void pulpnn_host_team_barrier(void);
static inline int  pi_core_id(void) { return pulpnn_host_core_id; }
static inline void pi_cl_team_barrier(int unused) { (void)unused; pulpnn_host_team_barrier(); }
#endif

/* ---- builtins ----------------------------------------------------------- */
static inline int pulpnn_host_sdotusp4(v4u a, v4s b, int c)
{
  return c + (int)a[0] * (int)b[0] + (int)a[1] * (int)b[1]
           + (int)a[2] * (int)b[2] + (int)a[3] * (int)b[3];
}
/* The hardware instruction works on a 32-bit register: a wider argument is
 * truncated by the parameter conversion before it is clamped. */
static inline int pulpnn_host_clipu_r(int x, int hi)
{
  return x < 0 ? 0 : (x > hi ? hi : x);
}
static inline int pulpnn_host_clipu(int x, int lo, int hi)
{
  return x < lo ? lo : (x > hi ? hi : x);
}
static inline int pulpnn_host_fl1(unsigned int x)
{
  return x ? 31 - __builtin_clz(x) : -1;
}
static inline unsigned int pulpnn_host_bextractu(unsigned int x, int size, int off)
{
  unsigned int m = size >= 32 ? 0xffffffffu : ((1u << size) - 1u);
  return (x >> off) & m;
}
static inline int pulpnn_host_bextract(int x, int size, int off)
{
  unsigned int f = pulpnn_host_bextractu((unsigned int)x, size, off);
  unsigned int s = 1u << (size - 1);
  return (int)((f ^ s) - s);
}
static inline v4u pulpnn_host_maxu4(v4u a, v4u b)
{
  v4u r;
  for (int i = 0; i < 4; i++) r[i] = a[i] > b[i] ? a[i] : b[i];
  return r;
}
static inline v4s pulpnn_host_avg4(v4s a, v4s b)
{
  v4s r;
  for (int i = 0; i < 4; i++) r[i] = (int8_t)(((int)a[i] + (int)b[i]) >> 1);
  return r;
}
static inline int pulpnn_host_minsi(int a, int b) { return a < b ? a : b; }
static inline int pulpnn_host_maxsi(int a, int b) { return a > b ? a : b; }

#define __builtin_pulp_sdotusp4(a, b, c)      pulpnn_host_sdotusp4((a), (b), (c))
#define __builtin_pulp_clipu_r(x, hi)         pulpnn_host_clipu_r((x), (hi))
#define __builtin_pulp_clipu(x, lo, hi)       pulpnn_host_clipu((x), (lo), (hi))
#define __builtin_pulp_fl1(x)                 pulpnn_host_fl1((unsigned int)(x))
#define __builtin_pulp_bextractu(x, s, o)     pulpnn_host_bextractu((x), (s), (o))
#define __builtin_pulp_bextract(x, s, o)      pulpnn_host_bextract((x), (s), (o))
#define __builtin_pulp_maxu4(a, b)            pulpnn_host_maxu4((a), (b))
#define __builtin_pulp_avg4(a, b)             pulpnn_host_avg4((a), (b))
#define __builtin_pulp_minsi(a, b)            pulpnn_host_minsi((a), (b))
#define __builtin_pulp_maxsi(a, b)            pulpnn_host_maxsi((a), (b))
/* the element type of the result follows the (cast) type of the arguments */
#define __builtin_pulp_pack4(a, b, c, d) \
  ((__typeof__(a) __attribute__((vector_size(4)))){ (a), (b), (c), (d) })
#define __builtin_pulp_shuffleb(v, m) \
  __builtin_shuffle((v), (__typeof__(v))((m) & 3))

#endif /* PULPNN_HOST_PMSIS_H */
