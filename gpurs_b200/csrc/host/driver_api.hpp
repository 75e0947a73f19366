// The CUDA driver entry points this library uses, resolved from libcuda.so.1 at first use so that the
// library itself loads (and its exported symbols can be inspected) on a machine without a GPU driver.
// The reference binds the same functions statically: crates/driver/src/ffi.rs:47-214.
#pragma once
#include <cuda.h>

namespace driver {

#define GPURS_DRIVER_FUNCTIONS(X) \
    X(cuInit)                     \
    X(cuGetErrorName)             \
    X(cuGetErrorString)           \
    X(cuDeviceGet)                \
    X(cuDeviceGetAttribute)       \
    X(cuDeviceTotalMem)           \
    X(cuDevicePrimaryCtxRetain)   \
    X(cuDevicePrimaryCtxRelease)  \
    X(cuCtxPushCurrent)           \
    X(cuCtxPopCurrent)            \
    X(cuCtxSynchronize)           \
    X(cuStreamCreate)             \
    X(cuStreamDestroy)            \
    X(cuStreamSynchronize)        \
    X(cuStreamWaitEvent)          \
    X(cuStreamIsCapturing)        \
    X(cuStreamBeginCapture)       \
    X(cuStreamEndCapture)         \
    X(cuGraphInstantiate)         \
    X(cuGraphLaunch)              \
    X(cuGraphExecDestroy)         \
    X(cuGraphDestroy)             \
    X(cuGraphGetNodes)            \
    X(cuEventCreate)              \
    X(cuEventRecord)              \
    X(cuEventSynchronize)         \
    X(cuEventElapsedTime)         \
    X(cuEventDestroy)             \
    X(cuMemAlloc)                 \
    X(cuMemFree)                  \
    X(cuMemGetInfo)               \
    X(cuMemcpyHtoDAsync)          \
    X(cuMemcpyDtoHAsync)          \
    X(cuMemsetD8Async)            \
    X(cuMemHostAlloc)             \
    X(cuMemFreeHost)              \
    X(cuMemcpy2DAsync)            \
    X(cuMemcpyDtoDAsync)          \
    X(cuIpcGetMemHandle)          \
    X(cuIpcOpenMemHandle)         \
    X(cuIpcCloseMemHandle)        \
    X(cuTensorMapEncodeTiled)     \
    X(cuModuleLoadData)           \
    X(cuModuleUnload)             \
    X(cuModuleGetFunction)        \
    X(cuFuncSetAttribute)         \
    X(cuFuncGetAttribute)         \
    X(cuLaunchKernelEx)

struct Api {
#define GPURS_DECLARE(name) decltype(&::name) name = nullptr;
    GPURS_DRIVER_FUNCTIONS(GPURS_DECLARE)
#undef GPURS_DECLARE
};

// Returns the resolved table, or nullptr when libcuda.so.1 or one of its symbols is missing.
const Api *api();

}  // namespace driver
