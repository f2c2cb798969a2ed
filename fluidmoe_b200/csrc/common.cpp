// Last-error string shared by every entry point of the native library.
#include <stdio.h>
#include <string.h>

static thread_local char g_err[512] = {0};

extern "C" __attribute__((visibility("default"))) void fm_set_error(const char* msg) {
  snprintf(g_err, sizeof(g_err), "%s", msg ? msg : "");
}
extern "C" __attribute__((visibility("default"))) const char* fm_last_error(void) { return g_err; }
