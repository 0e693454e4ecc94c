// Error plumbing and version of the C-ABI library.
#include <stdarg.h>
#include <stdio.h>
#include "common.cuh"

static thread_local char g_err[512] = "";
bool g_wb_pdl = true;
bool g_wb_pdl_gemm = true;

void wb_set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

const char *wein_b200_last_error_buf() { return g_err; }

extern "C" {
const char *wein_b200_last_error(void) { return g_err; }
uint32_t wein_b200_abi_version(void) { return 1; }
// 0 launches every kernel fully serialised (no programmatic dependent launch); default 1
void wein_b200_set_pdl(uint32_t on) { g_wb_pdl = (on & 1u) != 0; g_wb_pdl_gemm = on == 1u; }
}
