/* The C ABI seen from plain C: the header must compile as C, the library must link without any
 * C++ or CUDA header, and argument checking must answer before any device is touched. */
#include <stdio.h>
#include <string.h>

#include "warpir_b200.h"

int main(void) {
  int bad = 0;
  if (warpir_abi_version() != WARPIR_ABI_VERSION) { printf("abi version mismatch\n"); bad = 1; }
  if (strcmp(warpir_strerror(WARPIR_OK), "ok") != 0) { printf("strerror(OK)\n"); bad = 1; }
  /* rejected before any CUDA call: negative size, bad layout flag, bad tile width */
  if (warpir_gemm_bf16(0, 0, 0, -1, 8, 8, 1, 0, 0) != WARPIR_EINVAL) { printf("negative M accepted\n"); bad = 1; }
  if (warpir_gemm_bf16(0, 0, 0, 8, 8, 8, 7, 0, 0) != WARPIR_EINVAL) { printf("bad b_layout accepted\n"); bad = 1; }
  if (warpir_gemm_bf16_ex(0, 0, 0, 8, 8, 8, 1, 96, 0, 0, 0) != WARPIR_EINVAL) { printf("bad block_n accepted\n"); bad = 1; }
  if (warpir_attn_fwd_bf16(0, 0, 0, 0, 0, 1, 1, 1, 64, 96, 0.1f, 0, 0, 0) != WARPIR_ESHAPE) { printf("D = 96 accepted\n"); bad = 1; }
  if (warpir_attn_bwd_bf16(0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 1, 1, 1, 64, 80, 0.1f, 0, 0, 0) != WARPIR_ESHAPE) { printf("bwd D = 80 accepted\n"); bad = 1; }
  if (warpir_gemm_bf16_allgather(0, 0, 0, 0, 8, 8, 8, 1, 0, 0) != WARPIR_EINVAL) { printf("n_dst = 0 accepted\n"); bad = 1; }
  if (warpir_launch_generated(0, "x", 0, 0, 0, 0, 0, 0, 0) != WARPIR_EINVAL) { printf("NULL module accepted\n"); bad = 1; }
  if (strlen(warpir_last_error()) == 0) { printf("no error text after a failure\n"); bad = 1; }
  /* empty problems succeed without touching a device */
  if (warpir_gemm_bf16(0, 0, 0, 0, 8, 8, 1, 0, 0) != WARPIR_OK) { printf("empty GEMM rejected\n"); bad = 1; }
  if (warpir_attn_fwd_bf16(0, 0, 0, 0, 0, 0, 1, 1, 64, 64, 0.1f, 0, 0, 0) != WARPIR_OK) { printf("empty attention rejected\n"); bad = 1; }
  printf(bad ? "FAILED\n" : "ok\n");
  return bad;
}
