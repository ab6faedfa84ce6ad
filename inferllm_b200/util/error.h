// Errors of the library.  Every failure that a caller can cause or has to handle is one of these
// exceptions; the C binding turns them into a status code and a message, the command-line programs
// into one line on standard error and exit code 1.  Nothing aborts the process: the reference stops
// on INFER_ASSERT (src/utils.h:120-130), a library that serves many requests must not.
#pragma once
#include <stdexcept>
#include <string>

namespace illm {

struct Error : std::runtime_error {
    explicit Error(const std::string& what, int code) : std::runtime_error(what), code(code) {}
    int code;   // which class the Python binding raises (see binding.py)
};
// A config.json that cannot be used: a missing key, a wrong type, an unsupported value.
struct ConfigError : Error { explicit ConfigError(const std::string& w) : Error(w, 1) {} };
// Weight files that do not fit the model (one message lists everything) or cannot be read.
struct WeightError : Error { explicit WeightError(const std::string& w) : Error(w, 2) {} };
// Misuse of the cache: a slot that is not live, a page freed twice, a sequence beyond its longest length.
struct CacheError : Error { explicit CacheError(const std::string& w, int code = 3) : Error(w, code) {} };
// No free slot, or not enough free pages for the step.
struct CacheFull : CacheError { explicit CacheFull(const std::string& w) : CacheError(w, 4) {} };
// A step or an engine option that cannot be carried out, or an error word raised by a kernel.
struct EngineError : Error { explicit EngineError(const std::string& w) : Error(w, 5) {} };
// A size that a kernel does not take, or a CUDA error of a launch.
struct KernelError : Error { explicit KernelError(const std::string& w) : Error(w, 6) {} };
// A request that can never fit the cache (the generation loop).
struct RequestTooLong : Error { explicit RequestTooLong(const std::string& w) : Error(w, 7) {} };
// A sampling parameter outside its range.
struct ValueError : Error { explicit ValueError(const std::string& w) : Error(w, 8) {} };

}  // namespace illm
