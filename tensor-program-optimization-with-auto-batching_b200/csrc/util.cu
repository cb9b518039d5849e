// Error reporting and launch counter shared by all entry points.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace mlora {

static thread_local char g_err[512] = "";
std::atomic<uint64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// Programmatic dependent launch policy.  Which kernels are launched programmatically dependent (may become
// resident, and run whatever does not depend on earlier kernels, while the kernel before them still runs) is a
// bit mask: bit 0 projection (its weight producer streams ahead), 1 LoRA shrink, 2 attention, 3 RMSNorm, 4 the
// rest.  Measured on the benchmark's decode step (ms per step): none (0) 5.9, projection only (1) 4.98-5.60,
// projection + RMSNorm (9) 5.00-5.53 -- the default --, + shrink (11) 5.01-5.57, + attention (13, 15, 31) 5.25-5.8
// (its early-resident CTAs take registers and issue slots from the kernel before them).
// The one documented switch: MLORA_PDL_MASK=<mask>.
static int pdl_mask() {
  static const int mask = [] {
    const char* e = getenv("MLORA_PDL_MASK");
    return e ? atoi(e) : 9;
  }();
  return mask;
}
bool pdl_enabled() { return (pdl_mask() & 16) != 0; }
bool pdl_enabled_gemm() { return (pdl_mask() & 1) != 0; }
bool pdl_enabled_shrink() { return (pdl_mask() & 2) != 0; }
bool pdl_enabled_attn() { return (pdl_mask() & 4) != 0; }
bool pdl_enabled_norm() { return (pdl_mask() & 8) != 0; }

void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

}  // namespace mlora

extern "C" {
int mlora_version(void) { return 100; }
const char* mlora_last_error(void) { return mlora::g_err; }
uint64_t mlora_launch_count(void) { return mlora::g_launches.load(std::memory_order_relaxed); }
}
