// Leveled log lines on standard error: "[inferllm_b200] warning: ...".  The level comes from the
// environment variable ILLM_LOG (error, warning, info, debug; default warning) or set_log_level().
// The reference prints through INFER_LOG unconditionally (src/utils.h:108-118).
#pragma once
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace illm {

enum class LogLevel : int { Error = 0, Warning = 1, Info = 2, Debug = 3 };

inline int& log_level_ref() {
    static int level = [] {
        const char* e = getenv("ILLM_LOG");
        if (!e) return 1;
        if (!strcmp(e, "error")) return 0;
        if (!strcmp(e, "info")) return 2;
        if (!strcmp(e, "debug")) return 3;
        return 1;
    }();
    return level;
}
inline void set_log_level(LogLevel l) { log_level_ref() = (int)l; }

inline void log_line(LogLevel l, const char* fmt, ...) {
    if ((int)l > log_level_ref()) return;
    static const char* names[] = {"error: ", "warning: ", "", ""};
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    fprintf(stderr, "[inferllm_b200] %s%s\n", names[(int)l], buf);
    fflush(stderr);
}

}  // namespace illm
