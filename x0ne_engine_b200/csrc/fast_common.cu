// Error reporting of the `fast` module (each module is a library of its own).
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

static thread_local char g_error[512];

void x0ne_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
}

X0NE_API const char* x0ne_last_error() { return g_error; }
