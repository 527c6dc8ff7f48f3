// Error reporting of the `fast` module (each module is a library of its own).
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"

static thread_local char g_error[512];

void x0ne_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
}

X0NE_API const char* x0ne_last_error() { return g_error; }

bool x0ne_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("X0NE_PDL");
        on = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

