// Last-error storage shared by every launcher (thread-local, host side).
#include <stdarg.h>
#include <stdio.h>

#include "api.h"
#include "common.cuh"

static thread_local char g_last_error[512] = "";

void hb_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

extern "C" const char* hb_last_error(void) { return g_last_error; }
extern "C" int hb_abi_version(void) { return 1; }

// Programmatic dependent launch between consecutive kernels of a stream (see common.cuh).
static int g_pdl = 0;   // measured slower than plain stream order inside captured decode graphs: off unless asked for
int hb_pdl_enabled(void) { return g_pdl; }
extern "C" void hb_set_pdl(int mode) { g_pdl = (mode >= 0 && mode <= 2) ? mode : 0; }
extern "C" int hb_get_pdl(void) { return g_pdl; }
