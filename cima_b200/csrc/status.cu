// Error text of the kernel library (see common.cuh).
#include "common.cuh"
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static thread_local char g_err[512] = "";

extern "C" const char* cima_last_error() { return g_err; }

int cima_fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// Version of the entry points' signatures; the Python side refuses a library that answers otherwise.
extern "C" int cima_abi_version() { return 20; }

bool cima_pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* v = getenv("CIMA_NO_PDL");
    on = (v && strcmp(v, "1") == 0) ? 0 : 1;
  }
  return on == 1;
}
