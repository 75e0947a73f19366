#include "driver_api.hpp"

#include <dlfcn.h>
#include <mutex>

namespace driver {

// cuda.h renames several entry points to versioned symbols (cuMemAlloc -> cuMemAlloc_v2, ...); the
// two-step stringification below yields the versioned name that libcuda actually exports.
#define GPURS_STRINGIFY(x) #x
#define GPURS_SYMBOL(x) GPURS_STRINGIFY(x)

const Api *api() {
    static Api table;
    static bool ready = false;
    static std::once_flag once;
    std::call_once(once, [] {
        void *library = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
        if (!library) library = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
        if (!library) return;
        bool complete = true;
#define GPURS_RESOLVE(name)                                                                  \
    table.name = reinterpret_cast<decltype(&::name)>(dlsym(library, GPURS_SYMBOL(name)));    \
    complete = complete && table.name != nullptr;
        GPURS_DRIVER_FUNCTIONS(GPURS_RESOLVE)
#undef GPURS_RESOLVE
        ready = complete;
    });
    return ready ? &table : nullptr;
}

}  // namespace driver
