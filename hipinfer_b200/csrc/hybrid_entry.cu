// Error reporting of the `hybrid` library: residual streams with learned mixing (hyper-connections), the state-space
// recurrence with a scalar decay per head and its short convolution, the selective recurrence with a decay per (channel,
// state) pair, the residual row after a sublayer with the norm after the sum, routed feed-forward layers, and a gated
// activation with biases and limits.
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
HB_EXPORT int hb_hybrid_abi_version() { return 1; }
int g_hb_pdl = 1;
HB_EXPORT void hb_set_pdl(int on) { g_hb_pdl = on; }
