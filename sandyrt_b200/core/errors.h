// Error types of the engine's host side.  Every failure is a sandy::Error that carries the
// name of its kind; the C interface hands both to the caller, and the Python binding raises the
// exception class of that name.
#pragma once

#include <stdexcept>
#include <string>
#include <utility>

namespace sandy {

class Error : public std::runtime_error {
public:
    Error(std::string kind, const std::string& message, std::string details = "")
        : std::runtime_error(message), kind_(std::move(kind)), details_(std::move(details)) {}
    const std::string& kind() const { return kind_; }
    // Optional structured form of the message (JSON text), for callers that want the parts.
    const std::string& details() const { return details_; }

private:
    std::string kind_;
    std::string details_;
};

#define SANDY_ERROR_KIND(Name)                                              \
    class Name : public Error {                                             \
    public:                                                                 \
        explicit Name(const std::string& message) : Error(#Name, message) {} \
    }

SANDY_ERROR_KIND(ConfigError);         // config.json missing, malformed or naming impossible sizes
SANDY_ERROR_KIND(WeightFileError);     // the weight file is missing, truncated or malformed
SANDY_ERROR_KIND(CacheError);          // misuse of the cache: unknown request, page freed twice, ...
SANDY_ERROR_KIND(OutOfPages);          // a pool cannot supply a reservation; nothing was taken
SANDY_ERROR_KIND(NoFreeSlot);          // every state slot is held
SANDY_ERROR_KIND(RequestRefused);      // the request can never be served
SANDY_ERROR_KIND(StepError);           // a step that cannot run as given
SANDY_ERROR_KIND(KernelError);         // a kernel launch failed or a kernel reported a fault
SANDY_ERROR_KIND(UnsupportedShape);    // sizes or dtypes a kernel refuses
SANDY_ERROR_KIND(KernelBuildError);    // a kernel library is missing and cannot be made
SANDY_ERROR_KIND(ValueError);          // a bad argument

// The weight file does not hold exactly the tensors the model needs.  The message lists
// everything that is wrong; `details()` holds the same as JSON
// {"path", "missing": [...], "unexpected": [...], "wrong_shape": [[name, got, want]...], "wrong_kind": [[name, dtype]...]}.
class WeightBindingError : public Error {
public:
    WeightBindingError(const std::string& message, std::string details)
        : Error("WeightBindingError", message, std::move(details)) {}
};

#undef SANDY_ERROR_KIND

}  // namespace sandy
