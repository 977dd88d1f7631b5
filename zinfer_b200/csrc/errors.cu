// The error channel of the C entry points: a per-thread message for refusals.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"

static thread_local char g_last_error[512] = "";

extern "C" const char* zi_last_error() { return g_last_error; }

int zi_refuse(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return ZI_REFUSED;
}

int zi_check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

// Programmatic dependent launch is on unless ZINFER_B200_PDL=0 (or zi_set_pdl(0)).
int g_zi_pdl_enabled = [] {
  const char* v = getenv("ZINFER_B200_PDL");
  return (v && v[0] == '0') ? 0 : 1;
}();

extern "C" void zi_set_pdl(int enabled) { g_zi_pdl_enabled = enabled ? 1 : 0; }
extern "C" int zi_get_pdl() { return g_zi_pdl_enabled; }
