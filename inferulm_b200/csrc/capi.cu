// Error plumbing and version of the C-ABI library.
#include <stdarg.h>
#include <stdio.h>
#include <mutex>
#include <unordered_set>
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

// Shared-memory carve-out.  An SM splits one 256 KB array between L1 and shared memory, and the split is a mode of the SM:
// CTAs of two kernels that ask for different splits cannot be resident together, and the SM drains before it switches.  A
// round is a chain of ~300 short kernels that overlap head to tail, so every kernel of the library asks for the same split
// (percent of the array as shared memory; -1 leaves the driver's per-kernel default).
static int g_carveout = -1;
static std::mutex g_prep_mu;
static std::unordered_set<const void *> g_prepared;
void wb_prepare_kernel(const void *kern) {
    if (g_carveout < 0) return;
    std::lock_guard<std::mutex> lk(g_prep_mu);
    if (g_prepared.count(kern)) return;
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, g_carveout);
    cudaGetLastError();   // a hint only: never an error of the launch that follows
    g_prepared.insert(kern);
}

extern "C" {
const char *wein_b200_last_error(void) { return g_err; }
uint32_t wein_b200_abi_version(void) { return 1; }
// 0 launches every kernel fully serialised (no programmatic dependent launch); default 1
void wein_b200_set_pdl(uint32_t on) { g_wb_pdl = (on & 1u) != 0; g_wb_pdl_gemm = on == 1u; }
// A/B switch, to be called before the first launch: shared-memory carve-out preference of every kernel, -1 = driver default
void wein_b200_set_carveout(int32_t percent) { g_carveout = percent; }
}

WB_TRACE_SETTER(capi)   // diagnostic builds only (see common.cuh); expands to nothing otherwise
