// The kernel libraries of csrc/, loaded on demand.
//
// Each `<name>.cu` of csrc/ is its own shared library (`<name>.so`), built at first use, so that
// a run compiles only what its model and dtype need.  `kernel("gemm_tc", "sandy_gemm_tc")` opens
// the library if it is not open yet and returns the symbol.  Where the libraries are: the folder
// set by `set_kernel_dir`, else $SANDYRT_KERNEL_DIR, else the folder this library itself was
// loaded from.  A library that is missing or stale is first offered to the *provider*, a callback
// that may build it (the Python binding installs one that runs nvcc); without a provider, or if
// it fails, loading throws KernelBuildError.  There is no other implementation behind any kernel.
#pragma once

#include <string>

#include "../csrc/sandy_kernels.h"

namespace sandy {

// Returns 0 when `<dir>/<name>.so` is present and current after the call; `dir` may be rewritten
// (at most `dir_capacity` bytes) if the provider keeps its libraries elsewhere.
using KernelProvider = int (*)(const char* name, char* dir, int dir_capacity);

void set_kernel_dir(const std::string& dir);
void set_kernel_provider(KernelProvider provider);
void* kernel_symbol(const char* library, const char* symbol);

// Number of kernel launches issued through this library so far (benchmarks report it).
extern long long g_launches;

// Typed access: KERNEL(gemm_tc, sandy_gemm_tc)(args...)
#define SANDY_KERNEL(lib, fn) (reinterpret_cast<decltype(&fn)>(::sandy::kernel_symbol(#lib, #fn)))

}  // namespace sandy
