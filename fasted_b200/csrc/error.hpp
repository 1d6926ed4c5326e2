#pragma once
#include <string>

namespace fasted {
// Records the message returned by fasted_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);
}  // namespace fasted
