// Error plumbing and version of the C-ABI library.
#include <stdarg.h>
#include <stdio.h>
#include "common.cuh"

static thread_local char g_err[512] = "";

void wb_set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

const char *wein_b200_last_error_buf() { return g_err; }

extern "C" {
const char *wein_b200_last_error(void) { return g_err; }
uint32_t wein_b200_abi_version(void) { return 2; }
}
