// Shared pieces of the C binding: the thread's last error and the guard that turns exceptions into
// status codes.  Every entry point of binding/*.cpp returns 0 or the code of the error class
// (util/error.h); the message is read with illm_last_error().
#pragma once
#include <cstdlib>
#include <cstring>
#include <string>

#include "util/error.h"
#include "util/json.h"

namespace illm {
namespace binding {

void set_last_error(int code, const std::string& message);
char* dup_string(const std::string& s);      // malloc'd; the caller frees it with illm_free
Json parse_json_arg(const char* text, const char* what);

template <typename F> int guard(F&& f) {
    try {
        f();
        return 0;
    } catch (const Error& e) {
        set_last_error(e.code, e.what());
        return e.code;
    } catch (const std::exception& e) {
        set_last_error(99, e.what());
        return 99;
    } catch (...) {
        set_last_error(99, "unknown error");
        return 99;
    }
}

}  // namespace binding
}  // namespace illm

#define ILLM_API extern "C" __attribute__((visibility("default")))
