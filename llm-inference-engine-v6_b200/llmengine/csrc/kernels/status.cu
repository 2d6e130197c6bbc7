// The last error text of a kernel library (each library carries its own copy of this file).
#include <cstdarg>
#include <cstring>

#include "common.cuh"

static thread_local char g_last_error[512] = "";

extern "C" const char* llm_last_error() { return g_last_error; }

void llm_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

static bool g_dependent_launch = true;

extern "C" void llm_set_dependent_launch(int on) { g_dependent_launch = on != 0; }
bool llm_dependent_launch() { return g_dependent_launch; }
