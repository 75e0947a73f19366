// Internal definitions of the opaque handles behind include/gpurs_b200.h.
#pragma once
#include "../../../include/gpurs_b200.h"
#include "driver_api.hpp"

#include <map>
#include <string>
#include <vector>

struct gpurs_module {
    gpurs_gpu *gpu;
    CUmodule handle;
};

struct gpurs_kernel {
    gpurs_module *module;
    CUfunction function;
    std::string name;
    uint32_t reserved_shared = 0;
};

struct gpurs_gpu {
    const driver::Api *api;
    CUdevice device;
    CUcontext context;
    int major, minor, multiprocessors;
    size_t total_bytes;
    CUstream transfer;                 // internal stream for upload / zeros / download
    CUdeviceptr status;                // 4 x u32 written by bounded device waits that give up
    gpurs_module *builtin = nullptr;   // the embedded sm_100a image, loaded on first use
    std::map<std::string, gpurs_kernel *> kernels;
    uint64_t launches = 0;
    // One allocation of scratch memory.  A recorded graph keeps the address it was recorded with, so a block stays
    // allocated while any live graph borrows it (`graphs`), even after the handle has moved on to a larger block.
    struct Block {
        CUdeviceptr pointer = 0;
        size_t bytes = 0;
        int graphs = 0;          // live gpurs_graph objects whose recording holds this block's address
        bool current = true;     // false once the handle has replaced it: freed when the last graph lets go
    };
    // Scratch owned by the handle.  Each scratch has one user at a time: `event` marks the end of the previous
    // user's work and the next user's stream waits on it.
    struct Scratch {
        Block *block = nullptr;
        CUevent event = nullptr;
        bool used = false;
        bool captured = false;   // borrowed by work recorded into the capture now in progress
    };
    // Helper streams and events of the host-buffer product (created on first use): copies in and out run beside the
    // caller's stream and are tied to it by events.
    CUstream copy_in = nullptr, copy_out = nullptr;
    std::vector<CUevent> events;
    // One stream per peer for the copies of gpurs_matmul_allgather's copy-engine form (created on first use).
    std::vector<CUstream> peer_streams;
    Scratch workspace;   // grow-only: the hi/lo split copies of fp32 operands
    Scratch turns;       // fixed: the turn counters of split-K products, zero between launches
};

struct gpurs_stream {
    gpurs_gpu *gpu;
    CUstream handle;
    bool owned;
};

// A captured and instantiated sequence of operations.
struct gpurs_graph {
    gpurs_gpu *gpu;
    CUgraph graph;
    CUgraphExec executable;
    size_t nodes;                // operations recorded: what one replay adds to the launch count
    // The scratch blocks whose addresses the recording holds (null = none): kept allocated until the graph is freed.
    gpurs_gpu::Block *workspace_block, *turns_block;
};

struct gpurs_event {
    gpurs_gpu *gpu;
    CUevent handle;
};

namespace runtime {

// Makes a gpu's context current for the lifetime of the guard and restores the previous one after,
// like `Context::enter` in the reference (crates/driver/src/context.rs:117-129).
class Enter {
  public:
    explicit Enter(gpurs_gpu *gpu) : gpu_(gpu) { pushed_ = gpu_->api->cuCtxPushCurrent(gpu_->context) == CUDA_SUCCESS; }
    ~Enter() {
        CUcontext previous;
        if (pushed_) gpu_->api->cuCtxPopCurrent(&previous);
    }
    Enter(const Enter &) = delete;
    Enter &operator=(const Enter &) = delete;

  private:
    gpurs_gpu *gpu_;
    bool pushed_;
};

// Records the failure detail for gpurs_last_error and returns `code` unchanged.
int fail_driver(const driver::Api *api, const char *operation, CUresult code);
int fail(const char *operation, int code, const char *description);

// The built-in kernel with the given entry name, with `shared_bytes` of dynamic shared memory reserved.
int builtin_kernel(gpurs_gpu *gpu, const char *name, uint32_t shared_bytes, gpurs_kernel **out);

// `programmatic`: launch with the programmatic-stream-serialization attribute (the kernel must execute
// griddepcontrol.wait before it touches global memory; the built-in GEMMs do).
int launch(gpurs_kernel *kernel, gpurs_stream *stream, const gpurs_launch_config *config, void **params, bool programmatic = false);

// Borrows at least `bytes` of the gpu's scratch for work about to be enqueued on `stream`; the work of
// the previous borrower is ordered before it.  Call workspace_release once that work is enqueued.
int workspace_acquire(gpurs_stream *stream, size_t bytes, CUdeviceptr *out);
int workspace_release(gpurs_stream *stream);
// The same for the block of zero-initialised turn counters (`bytes` is fixed after the first call).
int turns_acquire(gpurs_stream *stream, size_t bytes, CUdeviceptr *out);
int turns_release(gpurs_stream *stream);
// At least `count` reusable events (no timing) in gpu->events, and the two helper streams.
int copy_pipeline(gpurs_gpu *gpu, size_t count);
// At least `count` streams in gpu->peer_streams.
int peer_pipeline(gpurs_gpu *gpu, size_t count);

}  // namespace runtime

#define GPURS_TRY(api, call)                                                     \
    do {                                                                         \
        CUresult gpurs_result_ = (api)->call;                                    \
        if (gpurs_result_ != CUDA_SUCCESS) return runtime::fail_driver((api), #call, gpurs_result_); \
    } while (0)
