// Error reporting of the `fast` library (the tensor-core and small-batch bf16 kernels).
#include "common.cuh"

#include <stdarg.h>

static thread_local char g_err[512];
void hb_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof g_err, fmt, ap);
  va_end(ap);
}
HB_EXPORT const char* hb_last_error() { return g_err; }
HB_EXPORT int hb_fast_abi_version() { return 1; }
int g_hb_pdl = 1;
HB_EXPORT void hb_set_pdl(int on) { g_hb_pdl = on; }
