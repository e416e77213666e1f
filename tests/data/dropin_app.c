/* A program written the way a PULP-NN application is -- reference names, reference parameter
 * lists, host buffers -- compiled against pulpnn_b200_dropin.h and linked with the line
 * INTEGRATION.md gives. Prints "status <code>" and, when a GPU computed the result,
 * "sum <checksum>" of the residual add it ran. */
#include <stdio.h>
#include <string.h>

#define PULPNN_BN_BITS 32
#include "pulpnn_b200_dropin.h"

int main(void)
{
  static uint8_t a[4 * 4 * 16], b[4 * 4 * 16], out[4 * 4 * 16];
  for (int i = 0; i < (int)sizeof(a); i++) { a[i] = (uint8_t)(i * 7); b[i] = (uint8_t)(255 - i); }
  memset(out, 0x55, sizeof(out));
  pulp_nn_add(a, b, out, 3, 5, 2, 4, 4, 16);
  const int st = pulpnn_last_error();
  printf("status %d\n", st);
  if (st == PULPNN_OK) {
    unsigned sum = 0;
    for (int i = 0; i < (int)sizeof(out); i++) sum += out[i];
    printf("sum %u\n", sum);
  }
  return 0;
}
