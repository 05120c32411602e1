// Process-wide state every other translation unit of libasd_b200.so links against: the thread-local error
// message, the launch counter and the per-thread tuning pointer.  Kept apart from the entry points of the individual
// components so that a library holding only some of them (one model family) still links.
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>

#include <atomic>

#include "../../include/asd_b200.h"
#include "asd_internal.h"

namespace asd {

static thread_local char g_err[512] = "";
thread_local const Tuning* g_tuning = nullptr;
static std::atomic<long long> g_launches{0};

int set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return -1;
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

}  // namespace asd

using namespace asd;

extern "C" {

int asd_abi_version(void) { return ASD_B200_ABI_VERSION; }
const char* asd_last_error(void) { return g_err; }
long long asd_launch_count(void) { return g_launches.load(); }
void asd_reset_launch_count(void) { g_launches.store(0); }

}  // extern "C"
