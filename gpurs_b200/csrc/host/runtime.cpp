// Context, stream, event, memory, TMA-descriptor and module entry points of the C ABI: the part of the
// boundary that stands where the reference's `crates/driver` stands (context.rs, stream.rs, memory.rs,
// module.rs, launch.rs), written against the CUDA driver API only.
#include "runtime.hpp"

#include <cstring>
#include <new>

extern "C" const unsigned char gpurs_embedded_image[];
extern "C" const unsigned long long gpurs_embedded_image_size;

namespace {

struct LastError {
    std::string operation, name, description;
    int code = 0;
};
thread_local LastError last_error;

}  // namespace

namespace runtime {

int fail_driver(const driver::Api *api, const char *operation, CUresult code) {
    std::string op(operation);
    size_t paren = op.find('(');
    if (paren != std::string::npos) op.resize(paren);
    const char *name = nullptr, *description = nullptr;
    if (api) {
        api->cuGetErrorName(code, &name);
        api->cuGetErrorString(code, &description);
    }
    last_error.operation = op;
    last_error.name = name ? name : "CUDA_ERROR_UNKNOWN";
    last_error.description = description ? description : "";
    last_error.code = int(code);
    return int(code);
}

int fail(const char *operation, int code, const char *description) {
    last_error.operation = operation;
    last_error.name = "GPURS_ERROR";
    last_error.description = description;
    last_error.code = code;
    return code;
}

int builtin_kernel(gpurs_gpu *gpu, const char *name, uint32_t shared_bytes, gpurs_kernel **out) {
    auto found = gpu->kernels.find(name);
    if (found == gpu->kernels.end()) {
        if (!gpu->builtin) {
            int result = gpurs_module_load(gpu, gpurs_embedded_image, size_t(gpurs_embedded_image_size), &gpu->builtin);
            if (result != GPURS_OK) return result;
        }
        gpurs_kernel *kernel = nullptr;
        int result = gpurs_module_kernel(gpu->builtin, name, &kernel);
        if (result != GPURS_OK) return result;
        found = gpu->kernels.emplace(name, kernel).first;
    }
    if (found->second->reserved_shared < shared_bytes) {
        int result = gpurs_kernel_reserve_shared(found->second, shared_bytes);
        if (result != GPURS_OK) return result;
    }
    *out = found->second;
    return GPURS_OK;
}

int launch(gpurs_kernel *kernel, gpurs_stream *stream, const gpurs_launch_config *config, void **params, bool programmatic) {
    gpurs_gpu *gpu = stream->gpu;
    CUlaunchConfig launch_config;
    std::memset(&launch_config, 0, sizeof launch_config);
    launch_config.gridDimX = config->grid[0];
    launch_config.gridDimY = config->grid[1] ? config->grid[1] : 1;
    launch_config.gridDimZ = config->grid[2] ? config->grid[2] : 1;
    launch_config.blockDimX = config->block[0];
    launch_config.blockDimY = config->block[1] ? config->block[1] : 1;
    launch_config.blockDimZ = config->block[2] ? config->block[2] : 1;
    launch_config.sharedMemBytes = config->shared_bytes;
    launch_config.hStream = stream->handle;
    CUlaunchAttribute attributes[2];
    std::memset(attributes, 0, sizeof attributes);
    CUlaunchAttribute &attribute = attributes[0];
    const uint32_t cluster_size = (config->cluster[0] ? config->cluster[0] : 1) * (config->cluster[1] ? config->cluster[1] : 1) *
                                  (config->cluster[2] ? config->cluster[2] : 1);
    if (cluster_size > 1) {
        attribute.id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
        attribute.value.clusterDim.x = config->cluster[0] ? config->cluster[0] : 1;
        attribute.value.clusterDim.y = config->cluster[1] ? config->cluster[1] : 1;
        attribute.value.clusterDim.z = config->cluster[2] ? config->cluster[2] : 1;
        launch_config.numAttrs = 1;
    }
    if (programmatic) {
        // As the reference launches its kernels (crates/gpurs/src/host/context.rs:270-281): the kernel may begin its
        // set-up before the previous kernel of the stream has finished.
        CUlaunchAttribute &serialization = attributes[launch_config.numAttrs++];
        serialization.id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
        serialization.value.programmaticStreamSerializationAllowed = 1;
    }
    launch_config.attrs = launch_config.numAttrs ? attributes : nullptr;
    GPURS_TRY(gpu->api, cuLaunchKernelEx(&launch_config, kernel->function, params, nullptr));
    gpu->launches++;
    return GPURS_OK;
}

// Lets go of one graph's hold on a block; a block the handle has already replaced is freed with its last holder.
void block_unborrow(gpurs_gpu *gpu, gpurs_gpu::Block *block) {
    if (!block) return;
    if (--block->graphs == 0 && !block->current) {
        gpu->api->cuMemFree(block->pointer);
        delete block;
    }
}

static int scratch_acquire(gpurs_stream *stream, gpurs_gpu::Scratch &scratch, size_t bytes, bool zeroed, CUdeviceptr *out) {
    gpurs_gpu *gpu = stream->gpu;
    const driver::Api *api = gpu->api;
    // Work recorded into a graph runs later, perhaps many times: it cannot be ordered by an event recorded now, and the
    // block must not move under it.  The graph remembers that it borrows the block and orders itself at every replay.
    CUstreamCaptureStatus capture = CU_STREAM_CAPTURE_STATUS_NONE;
    GPURS_TRY(api, cuStreamIsCapturing(stream->handle, &capture));
    const size_t held = scratch.block ? scratch.block->bytes : 0;
    if (capture == CU_STREAM_CAPTURE_STATUS_ACTIVE) {
        if (held < bytes)
            return fail("capture", GPURS_E_INVALID_ARGUMENT, "scratch memory cannot grow during a capture: run the same product once before capturing it");
        scratch.captured = true;
        *out = scratch.block->pointer;
        return GPURS_OK;
    }
    if (held < bytes) {
        // Nobody may still be using the old block when it is replaced.  A block whose address a live graph holds is not
        // freed here: it stays allocated, for that graph's replays alone, until the graph is freed.
        GPURS_TRY(api, cuCtxSynchronize());
        const size_t rounded = (bytes + (size_t(2) << 20) - 1) & ~((size_t(2) << 20) - 1);
        gpurs_gpu::Block *fresh = new (std::nothrow) gpurs_gpu::Block{};
        if (!fresh) return fail("scratch", GPURS_E_SIZE_OVERFLOW, "out of host memory");
        const CUresult allocated = api->cuMemAlloc(&fresh->pointer, rounded);
        if (allocated != CUDA_SUCCESS) {
            delete fresh;
            return fail_driver(api, "cuMemAlloc", allocated);
        }
        fresh->bytes = rounded;
        if (gpurs_gpu::Block *old = scratch.block) {
            old->current = false;
            if (old->graphs == 0) {
                api->cuMemFree(old->pointer);
                delete old;
            }
        }
        scratch.block = fresh;
        scratch.used = false;
        if (zeroed) {
            GPURS_TRY(api, cuMemsetD8Async(fresh->pointer, 0, rounded, gpu->transfer));
            GPURS_TRY(api, cuStreamSynchronize(gpu->transfer));
        }
    }
    if (!scratch.event) GPURS_TRY(api, cuEventCreate(&scratch.event, CU_EVENT_DISABLE_TIMING));
    if (scratch.used) GPURS_TRY(api, cuStreamWaitEvent(stream->handle, scratch.event, 0));
    *out = scratch.block->pointer;
    return GPURS_OK;
}

static int scratch_release(gpurs_stream *stream, gpurs_gpu::Scratch &scratch) {
    CUstreamCaptureStatus capture = CU_STREAM_CAPTURE_STATUS_NONE;
    GPURS_TRY(stream->gpu->api, cuStreamIsCapturing(stream->handle, &capture));
    if (capture == CU_STREAM_CAPTURE_STATUS_ACTIVE) return GPURS_OK;
    GPURS_TRY(stream->gpu->api, cuEventRecord(scratch.event, stream->handle));
    scratch.used = true;
    return GPURS_OK;
}

int workspace_acquire(gpurs_stream *stream, size_t bytes, CUdeviceptr *out) { return scratch_acquire(stream, stream->gpu->workspace, bytes, false, out); }
int workspace_release(gpurs_stream *stream) { return scratch_release(stream, stream->gpu->workspace); }
int turns_acquire(gpurs_stream *stream, size_t bytes, CUdeviceptr *out) { return scratch_acquire(stream, stream->gpu->turns, bytes, true, out); }
int turns_release(gpurs_stream *stream) { return scratch_release(stream, stream->gpu->turns); }

int copy_pipeline(gpurs_gpu *gpu, size_t count) {
    if (!gpu->copy_in) GPURS_TRY(gpu->api, cuStreamCreate(&gpu->copy_in, CU_STREAM_NON_BLOCKING));
    if (!gpu->copy_out) GPURS_TRY(gpu->api, cuStreamCreate(&gpu->copy_out, CU_STREAM_NON_BLOCKING));
    while (gpu->events.size() < count) {
        CUevent event = nullptr;
        GPURS_TRY(gpu->api, cuEventCreate(&event, CU_EVENT_DISABLE_TIMING));
        gpu->events.push_back(event);
    }
    return GPURS_OK;
}

int peer_pipeline(gpurs_gpu *gpu, size_t count) {
    while (gpu->peer_streams.size() < count) {
        CUstream stream = nullptr;
        GPURS_TRY(gpu->api, cuStreamCreate(&stream, CU_STREAM_NON_BLOCKING));
        gpu->peer_streams.push_back(stream);
    }
    return GPURS_OK;
}

}  // namespace runtime

using runtime::Enter;
using runtime::fail;

extern "C" {

int gpurs_last_error(const char **operation, const char **name, const char **description) {
    if (operation) *operation = last_error.operation.c_str();
    if (name) *name = last_error.name.c_str();
    if (description) *description = last_error.description.c_str();
    return last_error.code;
}

// ---- context ------------------------------------------------------------------------------------

int gpurs_gpu_new(int ordinal, gpurs_gpu **out) {
    if (!out) return fail("gpurs_gpu_new", GPURS_E_INVALID_ARGUMENT, "null output pointer");
    *out = nullptr;
    const driver::Api *api = driver::api();
    if (!api) return fail("gpurs_gpu_new", GPURS_E_DRIVER_UNAVAILABLE, "libcuda.so.1 could not be loaded");
    GPURS_TRY(api, cuInit(0));
    CUdevice device;
    GPURS_TRY(api, cuDeviceGet(&device, ordinal));
    int major = 0, minor = 0, multiprocessors = 0;
    GPURS_TRY(api, cuDeviceGetAttribute(&major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, device));
    GPURS_TRY(api, cuDeviceGetAttribute(&minor, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR, device));
    GPURS_TRY(api, cuDeviceGetAttribute(&multiprocessors, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, device));
    // An sm_100a image runs on compute capability 10.0 and nothing else, the same rule as
    // `Target::supports` for architecture-specific targets (crates/artifact/src/target.rs:68-72).
    if (major != 10 || minor != 0)
        return fail("gpurs_gpu_new", GPURS_E_INCOMPATIBLE_DEVICE, "the embedded sm_100a image needs a compute capability 10.0 device");
    size_t total = 0;
    GPURS_TRY(api, cuDeviceTotalMem(&total, device));
    CUcontext context;
    GPURS_TRY(api, cuDevicePrimaryCtxRetain(&context, device));
    gpurs_gpu *gpu = new (std::nothrow) gpurs_gpu{};
    if (!gpu) {
        api->cuDevicePrimaryCtxRelease(device);
        return fail("gpurs_gpu_new", GPURS_E_SIZE_OVERFLOW, "out of host memory");
    }
    gpu->api = api;
    gpu->device = device;
    gpu->context = context;
    gpu->major = major;
    gpu->minor = minor;
    gpu->multiprocessors = multiprocessors;
    gpu->total_bytes = total;
    int result = GPURS_OK;
    {
        Enter enter(gpu);
        CUresult r = api->cuStreamCreate(&gpu->transfer, CU_STREAM_NON_BLOCKING);
        if (r == CUDA_SUCCESS) r = api->cuMemAlloc(&gpu->status, 16);
        if (r == CUDA_SUCCESS) r = api->cuMemsetD8Async(gpu->status, 0, 16, gpu->transfer);
        if (r == CUDA_SUCCESS) r = api->cuStreamSynchronize(gpu->transfer);
        if (r != CUDA_SUCCESS) result = runtime::fail_driver(api, "gpurs_gpu_new", r);
    }
    if (result != GPURS_OK) {
        api->cuDevicePrimaryCtxRelease(device);
        delete gpu;
        return result;
    }
    *out = gpu;
    return GPURS_OK;
}

void gpurs_gpu_free(gpurs_gpu *gpu) {
    if (!gpu) return;
    {
        Enter enter(gpu);
        for (auto &entry : gpu->kernels) delete entry.second;
        if (gpu->builtin) {
            gpu->api->cuModuleUnload(gpu->builtin->handle);
            delete gpu->builtin;
        }
        gpu->api->cuMemFree(gpu->status);
        for (gpurs_gpu::Scratch *scratch : {&gpu->workspace, &gpu->turns}) {
            // a block that a graph still holds is left to that graph (graphs are to be freed before their gpu)
            if (gpurs_gpu::Block *block = scratch->block) {
                block->current = false;
                if (block->graphs == 0) {
                    gpu->api->cuMemFree(block->pointer);
                    delete block;
                }
            }
            if (scratch->event) gpu->api->cuEventDestroy(scratch->event);
        }
        gpu->api->cuStreamDestroy(gpu->transfer);
        if (gpu->copy_in) gpu->api->cuStreamDestroy(gpu->copy_in);
        if (gpu->copy_out) gpu->api->cuStreamDestroy(gpu->copy_out);
        for (CUevent event : gpu->events) gpu->api->cuEventDestroy(event);
        for (CUstream stream : gpu->peer_streams) gpu->api->cuStreamDestroy(stream);
    }
    gpu->api->cuDevicePrimaryCtxRelease(gpu->device);
    delete gpu;
}

int gpurs_gpu_properties(gpurs_gpu *gpu, int *major, int *minor, int *multiprocessors, size_t *total_bytes) {
    if (!gpu) return fail("gpurs_gpu_properties", GPURS_E_INVALID_ARGUMENT, "null gpu");
    if (major) *major = gpu->major;
    if (minor) *minor = gpu->minor;
    if (multiprocessors) *multiprocessors = gpu->multiprocessors;
    if (total_bytes) *total_bytes = gpu->total_bytes;
    return GPURS_OK;
}

uint64_t gpurs_launch_count(gpurs_gpu *gpu) { return gpu ? gpu->launches : 0; }

// ---- streams and events -------------------------------------------------------------------------

int gpurs_stream_new(gpurs_gpu *gpu, gpurs_stream **out) {
    if (!gpu || !out) return fail("gpurs_stream_new", GPURS_E_INVALID_ARGUMENT, "null argument");
    Enter enter(gpu);
    CUstream handle;
    GPURS_TRY(gpu->api, cuStreamCreate(&handle, CU_STREAM_NON_BLOCKING));
    *out = new gpurs_stream{gpu, handle, true};
    return GPURS_OK;
}

int gpurs_stream_borrow(gpurs_gpu *gpu, void *raw, gpurs_stream **out) {
    if (!gpu || !out) return fail("gpurs_stream_borrow", GPURS_E_INVALID_ARGUMENT, "null argument");
    *out = new gpurs_stream{gpu, static_cast<CUstream>(raw), false};
    return GPURS_OK;
}

void gpurs_stream_free(gpurs_stream *stream) {
    if (!stream) return;
    if (stream->owned) {
        Enter enter(stream->gpu);
        stream->gpu->api->cuStreamDestroy(stream->handle);
    }
    delete stream;
}

void *gpurs_stream_raw(gpurs_stream *stream) { return stream ? stream->handle : nullptr; }

static int collect_status(gpurs_gpu *gpu, uint32_t status[4]) {
    const driver::Api *api = gpu->api;
    GPURS_TRY(api, cuMemcpyDtoHAsync(status, gpu->status, 16, gpu->transfer));
    GPURS_TRY(api, cuStreamSynchronize(gpu->transfer));
    if (status[0] != 0) {
        GPURS_TRY(api, cuMemsetD8Async(gpu->status, 0, 16, gpu->transfer));
        GPURS_TRY(api, cuStreamSynchronize(gpu->transfer));
    }
    return GPURS_OK;
}

int gpurs_stream_synchronize(gpurs_stream *stream) {
    if (!stream) return fail("gpurs_stream_synchronize", GPURS_E_INVALID_ARGUMENT, "null stream");
    gpurs_gpu *gpu = stream->gpu;
    Enter enter(gpu);
    GPURS_TRY(gpu->api, cuStreamSynchronize(stream->handle));
    uint32_t status[4];
    int result = collect_status(gpu, status);
    if (result != GPURS_OK) return result;
    if (status[0] != 0) return fail("gpurs_stream_synchronize", GPURS_E_DEVICE_TIMEOUT, "a bounded wait inside a kernel gave up");
    return GPURS_OK;
}

// ---- graphs ---------------------------------------------------------------------------------------

int gpurs_stream_capture_begin(gpurs_stream *stream) {
    if (!stream) return fail("gpurs_stream_capture_begin", GPURS_E_INVALID_ARGUMENT, "null stream");
    gpurs_gpu *gpu = stream->gpu;
    Enter enter(gpu);
    gpu->workspace.captured = gpu->turns.captured = false;
    // Relaxed mode: this library looks kernels up and sets their attributes lazily, which stricter modes forbid
    // while any capture is in progress.
    GPURS_TRY(gpu->api, cuStreamBeginCapture(stream->handle, CU_STREAM_CAPTURE_MODE_RELAXED));
    return GPURS_OK;
}

int gpurs_stream_capture_end(gpurs_stream *stream, gpurs_graph **out) {
    if (!stream || !out) return fail("gpurs_stream_capture_end", GPURS_E_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    gpurs_gpu *gpu = stream->gpu;
    Enter enter(gpu);
    CUgraph graph = nullptr;
    GPURS_TRY(gpu->api, cuStreamEndCapture(stream->handle, &graph));
    if (!graph) return fail("gpurs_stream_capture_end", GPURS_E_INVALID_ARGUMENT, "the capture was invalidated");
    size_t nodes = 0;
    CUresult code = gpu->api->cuGraphGetNodes(graph, nullptr, &nodes);
    CUgraphExec executable = nullptr;
    if (code == CUDA_SUCCESS) code = gpu->api->cuGraphInstantiate(&executable, graph, 0);
    if (code != CUDA_SUCCESS) {
        gpu->api->cuGraphDestroy(graph);
        return runtime::fail_driver(gpu->api, "cuGraphInstantiate", code);
    }
    gpurs_graph *result = new (std::nothrow) gpurs_graph{gpu, graph, executable, nodes, gpu->workspace.captured ? gpu->workspace.block : nullptr,
                                                         gpu->turns.captured ? gpu->turns.block : nullptr};
    gpu->workspace.captured = gpu->turns.captured = false;
    if (result) {
        // the recording holds these addresses: the blocks must outlive it, wherever the handle's scratch moves meanwhile
        if (result->workspace_block) result->workspace_block->graphs++;
        if (result->turns_block) result->turns_block->graphs++;
    }
    if (!result) {
        gpu->api->cuGraphExecDestroy(executable);
        gpu->api->cuGraphDestroy(graph);
        return fail("gpurs_stream_capture_end", GPURS_E_INVALID_ARGUMENT, "out of host memory");
    }
    *out = result;
    return GPURS_OK;
}

int gpurs_graph_launch(gpurs_graph *graph, gpurs_stream *stream) {
    if (!graph || !stream) return fail("gpurs_graph_launch", GPURS_E_INVALID_ARGUMENT, "null argument");
    if (graph->gpu != stream->gpu) return fail("gpurs_graph_launch", GPURS_E_CONTEXT_MISMATCH, "graph and stream belong to different gpu handles");
    gpurs_gpu *gpu = graph->gpu;
    Enter enter(gpu);
    // A graph that borrows the handle's scratch takes its turn like any other borrower.
    gpurs_gpu::Scratch *borrowed[2] = {graph->workspace_block ? &gpu->workspace : nullptr, graph->turns_block ? &gpu->turns : nullptr};
    for (gpurs_gpu::Scratch *scratch : borrowed)
        if (scratch && scratch->used) GPURS_TRY(gpu->api, cuStreamWaitEvent(stream->handle, scratch->event, 0));
    GPURS_TRY(gpu->api, cuGraphLaunch(graph->executable, stream->handle));
    for (gpurs_gpu::Scratch *scratch : borrowed)
        if (scratch) {
            if (!scratch->event) GPURS_TRY(gpu->api, cuEventCreate(&scratch->event, CU_EVENT_DISABLE_TIMING));
            GPURS_TRY(gpu->api, cuEventRecord(scratch->event, stream->handle));
            scratch->used = true;
        }
    gpu->launches += graph->nodes;
    return GPURS_OK;
}

void gpurs_graph_free(gpurs_graph *graph) {
    if (!graph) return;
    Enter enter(graph->gpu);
    graph->gpu->api->cuGraphExecDestroy(graph->executable);
    graph->gpu->api->cuGraphDestroy(graph->graph);
    // Replays still in flight may be using the blocks: wait for them before a replaced block is freed.
    if ((graph->workspace_block && !graph->workspace_block->current) || (graph->turns_block && !graph->turns_block->current))
        graph->gpu->api->cuCtxSynchronize();
    runtime::block_unborrow(graph->gpu, graph->workspace_block);
    runtime::block_unborrow(graph->gpu, graph->turns_block);
    delete graph;
}

int gpurs_status_read(gpurs_gpu *gpu, uint32_t status[4]) {
    if (!gpu || !status) return fail("gpurs_status_read", GPURS_E_INVALID_ARGUMENT, "null argument");
    Enter enter(gpu);
    GPURS_TRY(gpu->api, cuCtxSynchronize());
    return collect_status(gpu, status);
}

int gpurs_event_record_timed(gpurs_stream *stream, gpurs_event **out) {
    if (!stream || !out) return fail("gpurs_event_record_timed", GPURS_E_INVALID_ARGUMENT, "null argument");
    gpurs_gpu *gpu = stream->gpu;
    Enter enter(gpu);
    CUevent handle;
    GPURS_TRY(gpu->api, cuEventCreate(&handle, CU_EVENT_DEFAULT));
    CUresult r = gpu->api->cuEventRecord(handle, stream->handle);
    if (r != CUDA_SUCCESS) {
        gpu->api->cuEventDestroy(handle);
        return runtime::fail_driver(gpu->api, "cuEventRecord", r);
    }
    *out = new gpurs_event{gpu, handle};
    return GPURS_OK;
}

int gpurs_event_synchronize(gpurs_event *event) {
    if (!event) return fail("gpurs_event_synchronize", GPURS_E_INVALID_ARGUMENT, "null event");
    Enter enter(event->gpu);
    GPURS_TRY(event->gpu->api, cuEventSynchronize(event->handle));
    return GPURS_OK;
}

int gpurs_event_elapsed_ms(gpurs_event *start, gpurs_event *end, float *milliseconds) {
    if (!start || !end || !milliseconds) return fail("gpurs_event_elapsed_ms", GPURS_E_INVALID_ARGUMENT, "null argument");
    if (start->gpu->context != end->gpu->context)
        return fail("gpurs_event_elapsed_ms", GPURS_E_CONTEXT_MISMATCH, "events of different contexts");
    Enter enter(start->gpu);
    GPURS_TRY(start->gpu->api, cuEventSynchronize(end->handle));
    GPURS_TRY(start->gpu->api, cuEventElapsedTime(milliseconds, start->handle, end->handle));
    return GPURS_OK;
}

void gpurs_event_free(gpurs_event *event) {
    if (!event) return;
    Enter enter(event->gpu);
    event->gpu->api->cuEventDestroy(event->handle);
    delete event;
}

// ---- memory -------------------------------------------------------------------------------------

int gpurs_alloc(gpurs_gpu *gpu, size_t bytes, gpurs_device_ptr *out) {
    if (!gpu || !out) return fail("gpurs_alloc", GPURS_E_INVALID_ARGUMENT, "null argument");
    *out = 0;
    if (bytes == 0) return GPURS_OK;
    Enter enter(gpu);
    CUdeviceptr pointer;
    GPURS_TRY(gpu->api, cuMemAlloc(&pointer, bytes));
    *out = pointer;
    return GPURS_OK;
}

int gpurs_free(gpurs_gpu *gpu, gpurs_device_ptr pointer) {
    if (!gpu) return fail("gpurs_free", GPURS_E_INVALID_ARGUMENT, "null gpu");
    if (pointer == 0) return GPURS_OK;
    Enter enter(gpu);
    GPURS_TRY(gpu->api, cuMemFree(pointer));
    return GPURS_OK;
}

int gpurs_upload(gpurs_gpu *gpu, const void *host, size_t bytes, gpurs_device_ptr *out) {
    if (!gpu || !out || (!host && bytes)) return fail("gpurs_upload", GPURS_E_INVALID_ARGUMENT, "null argument");
    int result = gpurs_alloc(gpu, bytes, out);
    if (result != GPURS_OK || bytes == 0) return result;
    Enter enter(gpu);
    CUresult r = gpu->api->cuMemcpyHtoDAsync(*out, host, bytes, gpu->transfer);
    if (r == CUDA_SUCCESS) r = gpu->api->cuStreamSynchronize(gpu->transfer);
    if (r != CUDA_SUCCESS) {
        gpu->api->cuMemFree(*out);
        *out = 0;
        return runtime::fail_driver(gpu->api, "cuMemcpyHtoDAsync", r);
    }
    return GPURS_OK;
}

int gpurs_zeros(gpurs_gpu *gpu, size_t bytes, gpurs_device_ptr *out) {
    if (!gpu || !out) return fail("gpurs_zeros", GPURS_E_INVALID_ARGUMENT, "null argument");
    int result = gpurs_alloc(gpu, bytes, out);
    if (result != GPURS_OK || bytes == 0) return result;
    Enter enter(gpu);
    // The reference leaves the clear asynchronous and orders later users through its region tracking
    // (crates/gpurs/src/host/tracking.rs:121-142); without that tracker the clear is awaited here.
    CUresult r = gpu->api->cuMemsetD8Async(*out, 0, bytes, gpu->transfer);
    if (r == CUDA_SUCCESS) r = gpu->api->cuStreamSynchronize(gpu->transfer);
    if (r != CUDA_SUCCESS) {
        gpu->api->cuMemFree(*out);
        *out = 0;
        return runtime::fail_driver(gpu->api, "cuMemsetD8Async", r);
    }
    return GPURS_OK;
}

int gpurs_download(gpurs_gpu *gpu, gpurs_device_ptr source, void *host, size_t bytes) {
    if (!gpu || (!host && bytes)) return fail("gpurs_download", GPURS_E_INVALID_ARGUMENT, "null argument");
    if (bytes == 0) return GPURS_OK;
    Enter enter(gpu);
    // Writers may be on any stream of the context: wait for all of them, as the reference orders the
    // download after every recorded writer (crates/gpurs/src/host/memory/buffer.rs:251-271).
    GPURS_TRY(gpu->api, cuCtxSynchronize());
    GPURS_TRY(gpu->api, cuMemcpyDtoHAsync(host, source, bytes, gpu->transfer));
    GPURS_TRY(gpu->api, cuStreamSynchronize(gpu->transfer));
    return GPURS_OK;
}

int gpurs_copy_to_device(gpurs_stream *stream, gpurs_device_ptr destination, const void *host, size_t bytes) {
    if (!stream || (!host && bytes)) return fail("gpurs_copy_to_device", GPURS_E_INVALID_ARGUMENT, "null argument");
    if (bytes == 0) return GPURS_OK;
    Enter enter(stream->gpu);
    GPURS_TRY(stream->gpu->api, cuMemcpyHtoDAsync(destination, host, bytes, stream->handle));
    return GPURS_OK;
}

int gpurs_copy_to_host(gpurs_stream *stream, void *host, gpurs_device_ptr source, size_t bytes) {
    if (!stream || (!host && bytes)) return fail("gpurs_copy_to_host", GPURS_E_INVALID_ARGUMENT, "null argument");
    if (bytes == 0) return GPURS_OK;
    Enter enter(stream->gpu);
    GPURS_TRY(stream->gpu->api, cuMemcpyDtoHAsync(host, source, bytes, stream->handle));
    return GPURS_OK;
}

int gpurs_fill_u8(gpurs_stream *stream, gpurs_device_ptr destination, uint8_t value, size_t bytes) {
    if (!stream) return fail("gpurs_fill_u8", GPURS_E_INVALID_ARGUMENT, "null stream");
    if (bytes == 0) return GPURS_OK;
    Enter enter(stream->gpu);
    GPURS_TRY(stream->gpu->api, cuMemsetD8Async(destination, value, bytes, stream->handle));
    return GPURS_OK;
}

int gpurs_memory_info(gpurs_gpu *gpu, size_t *free_bytes, size_t *total_bytes) {
    if (!gpu) return fail("gpurs_memory_info", GPURS_E_INVALID_ARGUMENT, "null gpu");
    Enter enter(gpu);
    size_t free_now = 0, total = 0;
    GPURS_TRY(gpu->api, cuMemGetInfo(&free_now, &total));
    if (free_bytes) *free_bytes = free_now;
    if (total_bytes) *total_bytes = total;
    return GPURS_OK;
}

int gpurs_host_alloc(gpurs_gpu *gpu, size_t bytes, void **out) {
    if (!gpu || !out) return fail("gpurs_host_alloc", GPURS_E_INVALID_ARGUMENT, "null argument");
    Enter enter(gpu);
    GPURS_TRY(gpu->api, cuMemHostAlloc(out, bytes ? bytes : 1, CU_MEMHOSTALLOC_PORTABLE));
    return GPURS_OK;
}

int gpurs_host_free(gpurs_gpu *gpu, void *pointer) {
    if (!gpu) return fail("gpurs_host_free", GPURS_E_INVALID_ARGUMENT, "null gpu");
    if (!pointer) return GPURS_OK;
    Enter enter(gpu);
    GPURS_TRY(gpu->api, cuMemFreeHost(pointer));
    return GPURS_OK;
}

// ---- inter-process memory --------------------------------------------------------------------------

int gpurs_ipc_export(gpurs_gpu *gpu, gpurs_device_ptr pointer, uint8_t handle[64]) {
    if (!gpu || !pointer || !handle) return fail("gpurs_ipc_export", GPURS_E_INVALID_ARGUMENT, "null argument");
    static_assert(sizeof(CUipcMemHandle) == 64, "the handle is 64 bytes");
    Enter enter(gpu);
    CUipcMemHandle raw;
    GPURS_TRY(gpu->api, cuIpcGetMemHandle(&raw, pointer));
    std::memcpy(handle, &raw, sizeof raw);
    return GPURS_OK;
}

int gpurs_ipc_open(gpurs_gpu *gpu, const uint8_t handle[64], gpurs_device_ptr *out) {
    if (!gpu || !handle || !out) return fail("gpurs_ipc_open", GPURS_E_INVALID_ARGUMENT, "null argument");
    Enter enter(gpu);
    CUipcMemHandle raw;
    std::memcpy(&raw, handle, sizeof raw);
    CUdeviceptr pointer = 0;
    GPURS_TRY(gpu->api, cuIpcOpenMemHandle(&pointer, raw, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS));
    *out = pointer;
    return GPURS_OK;
}

int gpurs_ipc_close(gpurs_gpu *gpu, gpurs_device_ptr pointer) {
    if (!gpu) return fail("gpurs_ipc_close", GPURS_E_INVALID_ARGUMENT, "null gpu");
    if (!pointer) return GPURS_OK;
    Enter enter(gpu);
    GPURS_TRY(gpu->api, cuIpcCloseMemHandle(pointer));
    return GPURS_OK;
}

// ---- TMA descriptors ----------------------------------------------------------------------------

int gpurs_tensor_map_encode(gpurs_gpu *gpu, void *descriptor, int element_type, uint32_t rank, gpurs_device_ptr address,
                            const uint64_t *dims, const uint64_t *strides_bytes, const uint32_t *box, int swizzle,
                            int l2_promotion) {
    if (!gpu || !descriptor || !dims || !box || (rank > 1 && !strides_bytes))
        return fail("gpurs_tensor_map_encode", GPURS_E_INVALID_ARGUMENT, "null argument");
    if (rank < 1 || rank > 5) return fail("gpurs_tensor_map_encode", GPURS_E_INVALID_VIEW, "rank must be 1..5");
    if (reinterpret_cast<uintptr_t>(descriptor) % 64 != 0)
        return fail("gpurs_tensor_map_encode", GPURS_E_INVALID_VIEW, "the descriptor must be 64-byte aligned");
    CUtensorMapDataType type;
    uint64_t element_bytes;
    switch (element_type) {
    case GPURS_F16: type = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; element_bytes = 2; break;
    case GPURS_BF16: type = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; element_bytes = 2; break;
    case GPURS_F32: type = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; element_bytes = 4; break;
    case GPURS_I32: type = CU_TENSOR_MAP_DATA_TYPE_INT32; element_bytes = 4; break;
    case GPURS_I8:
    case GPURS_E4M3: type = CU_TENSOR_MAP_DATA_TYPE_UINT8; element_bytes = 1; break;
    default: return fail("gpurs_tensor_map_encode", GPURS_E_INVALID_ARGUMENT, "unknown element type");
    }
    if (swizzle < 0 || swizzle > 3 || l2_promotion < 0 || l2_promotion > 3)
        return fail("gpurs_tensor_map_encode", GPURS_E_INVALID_ARGUMENT, "unknown swizzle or L2 promotion");
    // The rules `validate` enforces in the reference (crates/gpurs/src/gpu/tensor/hopper/cursor.rs:110-116)
    // and the ones cuTensorMapEncodeTiled states: 16-byte base and strides, box of 1..256 per dimension,
    // inner box extent a multiple of 16 bytes and within the swizzle span.
    if (address % 16 != 0) return fail("gpurs_tensor_map_encode", GPURS_E_INVALID_VIEW, "the base address must be 16-byte aligned");
    static const uint32_t span[4] = {0, 32, 64, 128};
    if ((box[0] * element_bytes) % 16 != 0 || (swizzle && box[0] * element_bytes > span[swizzle]))
        return fail("gpurs_tensor_map_encode", GPURS_E_INVALID_VIEW, "inner box extent must be a multiple of 16 bytes within the swizzle span");
    cuuint64_t global_dims[5], global_strides[4];
    cuuint32_t box_dims[5], element_strides[5];
    for (uint32_t i = 0; i < rank; i++) {
        if (dims[i] == 0 || dims[i] > (1ull << 32)) return fail("gpurs_tensor_map_encode", GPURS_E_SIZE_OVERFLOW, "dimension out of range");
        if (box[i] == 0 || box[i] > 256) return fail("gpurs_tensor_map_encode", GPURS_E_INVALID_VIEW, "box extent must be 1..256");
        global_dims[i] = dims[i];
        box_dims[i] = box[i];
        element_strides[i] = 1;
        if (i + 1 < rank) {
            if (strides_bytes[i] % 16 != 0 || strides_bytes[i] >= (1ull << 40))
                return fail("gpurs_tensor_map_encode", GPURS_E_INVALID_VIEW, "strides must be multiples of 16 bytes below 2^40");
            global_strides[i] = strides_bytes[i];
        }
    }
    Enter enter(gpu);
    GPURS_TRY(gpu->api, cuTensorMapEncodeTiled(static_cast<CUtensorMap *>(descriptor), type, rank, reinterpret_cast<void *>(address),
                                               global_dims, global_strides, box_dims, element_strides,
                                               CU_TENSOR_MAP_INTERLEAVE_NONE, static_cast<CUtensorMapSwizzle>(swizzle),
                                               static_cast<CUtensorMapL2promotion>(l2_promotion),
                                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
    return GPURS_OK;
}

// ---- modules ------------------------------------------------------------------------------------

const void *gpurs_kernel_image(size_t *bytes) {
    if (bytes) *bytes = size_t(gpurs_embedded_image_size);
    return gpurs_embedded_image;
}

int gpurs_module_load(gpurs_gpu *gpu, const void *image, size_t bytes, gpurs_module **out) {
    if (!gpu || !image || !out || bytes == 0) return fail("gpurs_module_load", GPURS_E_INVALID_ARGUMENT, "null argument");
    Enter enter(gpu);
    CUmodule handle;
    GPURS_TRY(gpu->api, cuModuleLoadData(&handle, image));
    *out = new gpurs_module{gpu, handle};
    return GPURS_OK;
}

void gpurs_module_free(gpurs_module *module) {
    if (!module) return;
    Enter enter(module->gpu);
    module->gpu->api->cuModuleUnload(module->handle);
    delete module;
}

int gpurs_module_kernel(gpurs_module *module, const char *name, gpurs_kernel **out) {
    if (!module || !name || !out) return fail("gpurs_module_kernel", GPURS_E_INVALID_ARGUMENT, "null argument");
    Enter enter(module->gpu);
    CUfunction function;
    CUresult r = module->gpu->api->cuModuleGetFunction(&function, module->handle, name);
    if (r == CUDA_ERROR_NOT_FOUND) return fail("gpurs_module_kernel", GPURS_E_UNKNOWN_KERNEL, name);
    if (r != CUDA_SUCCESS) return runtime::fail_driver(module->gpu->api, "cuModuleGetFunction", r);
    *out = new gpurs_kernel{module, function, name, 0};
    return GPURS_OK;
}

int gpurs_kernel_reserve_shared(gpurs_kernel *kernel, uint32_t bytes) {
    if (!kernel) return fail("gpurs_kernel_reserve_shared", GPURS_E_INVALID_ARGUMENT, "null kernel");
    gpurs_gpu *gpu = kernel->module->gpu;
    Enter enter(gpu);
    GPURS_TRY(gpu->api, cuFuncSetAttribute(kernel->function, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, int(bytes)));
    kernel->reserved_shared = bytes;
    return GPURS_OK;
}

int gpurs_kernel_registers(gpurs_kernel *kernel, int *registers) {
    if (!kernel || !registers) return fail("gpurs_kernel_registers", GPURS_E_INVALID_ARGUMENT, "null argument");
    gpurs_gpu *gpu = kernel->module->gpu;
    Enter enter(gpu);
    GPURS_TRY(gpu->api, cuFuncGetAttribute(registers, CU_FUNC_ATTRIBUTE_NUM_REGS, kernel->function));
    return GPURS_OK;
}

int gpurs_kernel_launch(gpurs_kernel *kernel, gpurs_stream *stream, const gpurs_launch_config *config, void **params) {
    if (!kernel || !stream || !config) return fail("gpurs_kernel_launch", GPURS_E_INVALID_ARGUMENT, "null argument");
    if (kernel->module->gpu->context != stream->gpu->context)
        return fail("gpurs_kernel_launch", GPURS_E_CONTEXT_MISMATCH, "kernel and stream belong to different contexts");
    if (config->block[0] == 0 || config->grid[0] == 0)
        return fail("gpurs_kernel_launch", GPURS_E_INVALID_VIEW, "empty launch geometry");
    Enter enter(stream->gpu);
    return runtime::launch(kernel, stream, config, params);
}

}  // extern "C"
