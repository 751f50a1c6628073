// Per-thread error message behind mggb_last_error(), and the version query.
#include "common.h"

namespace {
thread_local char g_msg[512] = "";
}

namespace mggb {

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_msg, sizeof(g_msg), fmt, ap);
    va_end(ap);
    return code;
}

void clear_error() { g_msg[0] = '\0'; }

}  // namespace mggb

extern "C" int mggb_version(void) { return 100; }
extern "C" const char* mggb_last_error(void) { return g_msg; }
