#include "kernels.h"

#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>

#include "errors.h"

namespace sandy {

long long g_launches = 0;

namespace {
std::mutex g_lock;
std::string g_dir;
KernelProvider g_provider = nullptr;
std::map<std::string, void*> g_libs;
std::map<std::string, void*> g_symbols;

std::string own_dir() {
    Dl_info info;
    if (dladdr((void*)&own_dir, &info) && info.dli_fname) {
        std::string p = info.dli_fname;
        const size_t slash = p.rfind('/');
        if (slash != std::string::npos) return p.substr(0, slash);
    }
    return ".";
}
}  // namespace

void set_kernel_dir(const std::string& dir) {
    std::lock_guard<std::mutex> g(g_lock);
    g_dir = dir;
}
void set_kernel_provider(KernelProvider provider) {
    std::lock_guard<std::mutex> g(g_lock);
    g_provider = provider;
}

void* kernel_symbol(const char* library, const char* symbol) {
    std::lock_guard<std::mutex> g(g_lock);
    const std::string key = std::string(library) + ":" + symbol;
    auto hit = g_symbols.find(key);
    if (hit != g_symbols.end()) return hit->second;
    void* lib = nullptr;
    auto lit = g_libs.find(library);
    if (lit != g_libs.end()) lib = lit->second;
    if (!lib) {
        std::string dir = g_dir;
        if (dir.empty())
            if (const char* e = std::getenv("SANDYRT_KERNEL_DIR")) dir = e;
        if (dir.empty()) dir = own_dir();
        if (g_provider) {
            char buf[4096];
            std::strncpy(buf, dir.c_str(), sizeof buf - 1);
            buf[sizeof buf - 1] = 0;
            if (g_provider(library, buf, (int)sizeof buf) != 0)
                throw KernelBuildError(std::string("the kernel library '") + library + "' could not be built; there is no other path");
            dir = buf;
        }
        const std::string path = dir + "/" + library + ".so";
        lib = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
        if (!lib) {
            const char* why = dlerror();
            throw KernelBuildError("cannot load " + path + ": " + (why ? why : "unknown error") +
                                   " (build the kernel libraries first: python -m sandyrt_b200.csrc.build)");
        }
        g_libs[library] = lib;
    }
    void* sym = dlsym(lib, symbol);
    if (!sym) throw KernelBuildError(std::string("kernel library '") + library + "' has no symbol " + symbol);
    g_symbols[key] = sym;
    return sym;
}

}  // namespace sandy
