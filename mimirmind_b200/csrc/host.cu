// Host-side state of the kernel library: the last error message.
#include <string.h>

static thread_local char g_last_error[512] = "";

void mm_set_last_error(const char* msg) {
    strncpy(g_last_error, msg ? msg : "", sizeof(g_last_error) - 1);
    g_last_error[sizeof(g_last_error) - 1] = 0;
}

extern "C" __attribute__((visibility("default"))) const char* mm_last_error() { return g_last_error; }

// Programmatic dependent launch for the decode-path kernels.  Off by default: on B200 the captured decode step
// measured slower with it (3.8 ms -> 6.4 ms at batch 8 with one kernel of look-ahead, 9.6 ms with an unbounded
// chain), so it stays an option for experiments.
int g_mm_pdl = 0;
extern "C" __attribute__((visibility("default"))) void mm_set_pdl(int on) { g_mm_pdl = on ? 1 : 0; }
extern "C" __attribute__((visibility("default"))) int mm_get_pdl() { return g_mm_pdl; }

// Every kernel launch of this library counts itself here (MM_CHECK_LAUNCH).
long long g_mm_launch_count = 0;
extern "C" __attribute__((visibility("default"))) long long mm_launch_count() { return g_mm_launch_count; }
