// Host-side state of the kernel library: the last error message.
#include <stdlib.h>
#include <string.h>

static thread_local char g_last_error[512] = "";

void mm_set_last_error(const char* msg) {
    strncpy(g_last_error, msg ? msg : "", sizeof(g_last_error) - 1);
    g_last_error[sizeof(g_last_error) - 1] = 0;
}

extern "C" __attribute__((visibility("default"))) const char* mm_last_error() { return g_last_error; }

// Dependent launches of the weight-streaming kernels (common.cuh says when they pay).  On unless the environment says
// MIMIRMIND_B200_DEPENDENT_LAUNCH=0 (or mm_set_pdl(0) is called): a way out on a driver where they misbehave.
static int dependent_launch_default() {
    const char* v = getenv("MIMIRMIND_B200_DEPENDENT_LAUNCH");
    return (v != nullptr && v[0] == '0') ? 0 : 1;
}
int g_mm_pdl = dependent_launch_default();
long long g_mm_dep_count = -1;     // the launch count right after the last launch that a dependent launch may follow
void* g_mm_dep_stream = nullptr;
extern "C" __attribute__((visibility("default"))) void mm_set_pdl(int on) { g_mm_pdl = on ? 1 : 0; }
extern "C" __attribute__((visibility("default"))) int mm_get_pdl() { return g_mm_pdl; }

// Every kernel launch of this library counts itself here (MM_CHECK_LAUNCH).
long long g_mm_launch_count = 0;
extern "C" __attribute__((visibility("default"))) long long mm_launch_count() { return g_mm_launch_count; }
