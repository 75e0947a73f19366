// gpurs_comm_*: the one collective of the sharded matrix-multiply path, the optional all-gather of C after an
// M-sharded product, as a plain NCCL call behind the C ABI.  The reference drives a single device and has no
// collective (crates/gpurs/src/lib.rs:7-9); a multi-GPU host binds these next to gpurs_matmul, one process (or thread)
// and one communicator per GPU.  The fused form, gpurs_matmul_allgather, needs no communicator at all; this is the
// baseline it is measured against, reachable through the same boundary.
//
// NCCL is resolved from libnccl.so.2 at first use (the copy already loaded into the process, if any, else the
// system's), so the library loads, and everything else in it works, on a machine without NCCL.
#include "runtime.hpp"

#include <dlfcn.h>
#include <cstring>
#include <mutex>
#include <new>

namespace {

// The part of NCCL's C interface used here, declared locally: ncclResult_t is an int (0 = success), ncclComm_t an opaque
// pointer, ncclUniqueId 128 opaque bytes passed by value, ncclInt8 = 0.
struct UniqueId {
    char internal[128];
};
struct Nccl {
    int (*ncclGetUniqueId)(UniqueId *) = nullptr;
    int (*ncclCommInitRank)(void **, int, UniqueId, int) = nullptr;
    int (*ncclCommDestroy)(void *) = nullptr;
    int (*ncclAllGather)(const void *, void *, size_t, int, void *, void *) = nullptr;
    const char *(*ncclGetErrorString)(int) = nullptr;
    int (*ncclGetVersion)(int *) = nullptr;
};

const Nccl *nccl() {
    static Nccl table;
    static bool ready = false;
    static std::once_flag once;
    std::call_once(once, [] {
        void *library = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!library) library = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!library) return;
#define GPURS_RESOLVE(name) table.name = reinterpret_cast<decltype(table.name)>(dlsym(library, #name))
        GPURS_RESOLVE(ncclGetUniqueId);
        GPURS_RESOLVE(ncclCommInitRank);
        GPURS_RESOLVE(ncclCommDestroy);
        GPURS_RESOLVE(ncclAllGather);
        GPURS_RESOLVE(ncclGetErrorString);
        GPURS_RESOLVE(ncclGetVersion);
#undef GPURS_RESOLVE
        ready = table.ncclGetUniqueId && table.ncclCommInitRank && table.ncclCommDestroy && table.ncclAllGather && table.ncclGetErrorString;
    });
    return ready ? &table : nullptr;
}

int fail_nccl(const Nccl *api, const char *operation, int code) {
    return runtime::fail(operation, GPURS_E_COLLECTIVE, api->ncclGetErrorString(code));
}

}  // namespace

struct gpurs_comm {
    gpurs_gpu *gpu;
    void *handle;
    uint32_t world, rank;
};

extern "C" int gpurs_comm_unique_id(uint8_t id[GPURS_COMM_ID_BYTES]) {
    if (!id) return runtime::fail("gpurs_comm_unique_id", GPURS_E_INVALID_ARGUMENT, "null argument");
    const Nccl *api = nccl();
    if (!api) return runtime::fail("gpurs_comm_unique_id", GPURS_E_COLLECTIVE, "libnccl.so.2 could not be loaded");
    static_assert(sizeof(UniqueId) == GPURS_COMM_ID_BYTES, "an NCCL unique id is 128 bytes");
    UniqueId unique;
    const int code = api->ncclGetUniqueId(&unique);
    if (code != 0) return fail_nccl(api, "ncclGetUniqueId", code);
    std::memcpy(id, &unique, sizeof unique);
    return GPURS_OK;
}

extern "C" int gpurs_comm_init(gpurs_gpu *gpu, const uint8_t id[GPURS_COMM_ID_BYTES], uint32_t world, uint32_t rank, gpurs_comm **out) {
    const char *const op = "gpurs_comm_init";
    if (!gpu || !id || !out) return runtime::fail(op, GPURS_E_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    if (world < 1 || rank >= world) return runtime::fail(op, GPURS_E_INVALID_ARGUMENT, "world must be at least 1 and rank below it");
    const Nccl *api = nccl();
    if (!api) return runtime::fail(op, GPURS_E_COLLECTIVE, "libnccl.so.2 could not be loaded");
    UniqueId unique;
    std::memcpy(&unique, id, sizeof unique);
    runtime::Enter enter(gpu);     // NCCL binds the communicator to the device that is current now
    void *handle = nullptr;
    const int code = api->ncclCommInitRank(&handle, int(world), unique, int(rank));
    if (code != 0) return fail_nccl(api, "ncclCommInitRank", code);
    gpurs_comm *comm = new (std::nothrow) gpurs_comm{gpu, handle, world, rank};
    if (!comm) {
        api->ncclCommDestroy(handle);
        return runtime::fail(op, GPURS_E_SIZE_OVERFLOW, "out of host memory");
    }
    *out = comm;
    return GPURS_OK;
}

extern "C" int gpurs_comm_allgather(gpurs_comm *comm, gpurs_stream *stream, gpurs_device_ptr full, uint64_t block_bytes) {
    const char *const op = "gpurs_comm_allgather";
    if (!comm || !stream) return runtime::fail(op, GPURS_E_INVALID_ARGUMENT, "null argument");
    if (comm->gpu->context != stream->gpu->context) return runtime::fail(op, GPURS_E_CONTEXT_MISMATCH, "communicator and stream belong to different contexts");
    if (block_bytes == 0) return GPURS_OK;
    if (!full) return runtime::fail(op, GPURS_E_INVALID_ARGUMENT, "null buffer");
    if (block_bytes > (~uint64_t(0)) / comm->world) return runtime::fail(op, GPURS_E_SIZE_OVERFLOW, "the gathered size overflows");
    const Nccl *api = nccl();
    runtime::Enter enter(comm->gpu);
    // In place: this rank's block already lies at its position in the gathered buffer.
    const void *mine = reinterpret_cast<const void *>(full + uint64_t(comm->rank) * block_bytes);
    const int code = api->ncclAllGather(mine, reinterpret_cast<void *>(full), size_t(block_bytes), /* ncclInt8 */ 0, comm->handle, stream->handle);
    if (code != 0) return fail_nccl(api, "ncclAllGather", code);
    return GPURS_OK;
}

extern "C" void gpurs_comm_free(gpurs_comm *comm) {
    if (!comm) return;
    if (const Nccl *api = nccl()) {
        runtime::Enter enter(comm->gpu);
        api->ncclCommDestroy(comm->handle);
    }
    delete comm;
}
