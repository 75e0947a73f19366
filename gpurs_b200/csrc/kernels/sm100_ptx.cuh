// Thin inline-PTX wrappers for the sm_100a features the GEMM kernels are built from: mbarrier,
// TMA tile loads, tensor memory (TMEM) management, tcgen05.mma / commit / ld and cluster helpers.
//
// Every wait in this file is bounded: a wait that does not complete within WAIT_LIMIT_NS returns
// false instead of spinning for ever, so a kernel can record the failure and leave the GPU usable.
// (The reference's equivalent, `barrier_wait` in crates/gpurs/src/gpu/tensor/hopper/intrinsics.rs:15-16,
// spins without a limit.)
#pragma once
#include <cstdint>
#include <cuda.h>

namespace ptx {

constexpr unsigned long long WAIT_LIMIT_NS = 1500ull * 1000ull * 1000ull;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t lane_id() {
    uint32_t l;
    asm volatile("mov.u32 %0, %laneid;" : "=r"(l));
    return l;
}

// ---- cluster ---------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %cluster_ctarank;" : "=r"(r));
    return r;
}

// Programmatic dependent launch, as the reference's compiled kernels use it (crates/codegen/src/kernel.rs:161-171): a kernel
// launched with the programmatic-serialization attribute may start while the previous kernel of the stream is still
// running; `wait` blocks until that kernel has completed and its memory is visible, `launch` lets the NEXT kernel of the
// stream start its own set-up.  Both are no-ops in a kernel launched without the attribute.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// The address, in the cluster's shared window, of `local` in the CTA with rank `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}

// ---- mbarrier --------------------------------------------------------------------------------

__device__ __forceinline__ void mbarrier_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbarrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbarrier_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrive on a barrier anywhere in the cluster (address from map_to_cta).
__device__ __forceinline__ void mbarrier_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// The same arrive without release semantics.  A release at cluster scope makes the arriving thread wait for every
// memory operation it still has in flight (global loads included) before the arrive is performed, which costs about a
// thousand cycles per hand-off; a thread that hands back TENSOR memory it has finished reading (tcgen05.wait::ld has
// returned, tcgen05.fence::before_thread_sync executed) publishes nothing through ordinary memory and needs no release.
__device__ __forceinline__ void mbarrier_arrive_cluster_relaxed(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

__device__ __forceinline__ void mbarrier_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbarrier_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

__device__ __forceinline__ bool mbarrier_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Waits for the phase with the given parity to complete.  Returns false when the wait ran out of
// time or when another role of the block raised `*abort_flag` (a shared-memory word).
template <bool CLUSTER_SCOPE = false>
__device__ __forceinline__ bool mbarrier_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag) {
    unsigned long long start = 0;
    for (uint32_t spin = 1;; ++spin) {
        bool done = CLUSTER_SCOPE ? mbarrier_try_wait_cluster(bar, parity) : mbarrier_try_wait(bar, parity);
        if (done) return true;
        if ((spin & 0xff) == 0) {
            if (*abort_flag != 0) return false;
            unsigned long long now = global_timer();
            if (start == 0) start = now;
            else if (now - start > WAIT_LIMIT_NS) return false;
        }
    }
}

// ---- TMA ------------------------------------------------------------------------------------

__device__ __forceinline__ void prefetch_tensor_map(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 2-D tile load into this CTA's shared memory, completing on a barrier of this CTA.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int32_t x, int32_t y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// 2-D tile load into this CTA's shared memory whose completion may be counted on a barrier of the
// other CTA of a CTA pair (`cluster_bar` comes from map_to_cta).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int32_t x, int32_t y, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y)
        : "memory");
}

// The same two loads for rank-3 tensors (x, y, z = innermost to outermost), used for batches of matrices: z is the batch.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int32_t x, int32_t y, int32_t z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, int32_t x, int32_t y, int32_t z, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// ---- tensor memory --------------------------------------------------------------------------

template <int CTA_GROUP>
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t columns) {
    if constexpr (CTA_GROUP == 1)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(columns) : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(columns) : "memory");
}

template <int CTA_GROUP>
__device__ __forceinline__ void tmem_relinquish() {
    if constexpr (CTA_GROUP == 1) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    else asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

template <int CTA_GROUP>
__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
    if constexpr (CTA_GROUP == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
    else
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Arrive once on `bar` when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// CTA-pair form: arrives on the barrier at the same offset in every CTA named by `cta_mask`.
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(cta_mask) : "memory");
}

// Operand kinds of tcgen05.mma.
enum : int { KIND_F16 = 0, KIND_TF32 = 1, KIND_I8 = 2, KIND_F8F6F4 = 3 };

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.  `accumulate` = 0 overwrites D.
template <int KIND, int CTA_GROUP>
__device__ __forceinline__ void tcgen05_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
#define GPURS_MMA(KINDSTR, GROUPSTR)                                                                      \
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"                                         \
                 "tcgen05.mma.cta_group::" GROUPSTR ".kind::" KINDSTR " [%0], %1, %2, %3, p;\n\t}"          \
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory")
    if constexpr (CTA_GROUP == 1) {
        if constexpr (KIND == KIND_F16) GPURS_MMA("f16", "1");
        else if constexpr (KIND == KIND_TF32) GPURS_MMA("tf32", "1");
        else if constexpr (KIND == KIND_I8) GPURS_MMA("i8", "1");
        else GPURS_MMA("f8f6f4", "1");
    } else {
        if constexpr (KIND == KIND_F16) GPURS_MMA("f16", "2");
        else if constexpr (KIND == KIND_TF32) GPURS_MMA("tf32", "2");
        else if constexpr (KIND == KIND_I8) GPURS_MMA("i8", "2");
        else GPURS_MMA("f8f6f4", "2");
    }
#undef GPURS_MMA
}

// D[tmem] += A[smem] * B[smem]: the accumulating form with its predicate fixed, so that the issuing thread spends no
// instruction on it.
template <int KIND, int CTA_GROUP>
__device__ __forceinline__ void tcgen05_mma_accumulate(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
#define GPURS_MMA(KINDSTR, GROUPSTR)                                                                      \
    asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 0, 0;\n\t"                                        \
                 "tcgen05.mma.cta_group::" GROUPSTR ".kind::" KINDSTR " [%0], %1, %2, %3, p;\n\t}"          \
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc) : "memory")
    if constexpr (CTA_GROUP == 1) {
        if constexpr (KIND == KIND_F16) GPURS_MMA("f16", "1");
        else if constexpr (KIND == KIND_TF32) GPURS_MMA("tf32", "1");
        else if constexpr (KIND == KIND_I8) GPURS_MMA("i8", "1");
        else GPURS_MMA("f8f6f4", "1");
    } else {
        if constexpr (KIND == KIND_F16) GPURS_MMA("f16", "2");
        else if constexpr (KIND == KIND_TF32) GPURS_MMA("tf32", "2");
        else if constexpr (KIND == KIND_I8) GPURS_MMA("i8", "2");
        else GPURS_MMA("f8f6f4", "2");
    }
#undef GPURS_MMA
}

// 32 lanes x 32 consecutive 32-bit columns: lane i of the warp receives columns [c, c+32) of
// TMEM lane (base lane + i).
__device__ __forceinline__ void tmem_load_32x32(uint32_t address, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(address)
        : "memory");
}

__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes wide and stored with
// the 128-byte swizzle in groups of eight rows (1024 bytes apart): start address, leading offset
// 16 B (unused by this layout), stride offset 1024 B, descriptor version 1, layout SWIZZLE_128B.
// The same fields are built by the reference in shared/tile.rs:81-84 and blackwell/tensor_memory.rs:20.
__device__ __forceinline__ uint64_t smem_descriptor_k_major_sw128(uint32_t address) {
    return static_cast<uint64_t>((address & 0x3ffffu) >> 4) | (1ull << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}

}  // namespace ptx

namespace ptx {

// ---- 2:4 structured sparsity ----------------------------------------------------------------------

// Copies 128 rows x 128 bits from shared memory into 4 columns of tensor memory (one row per TMEM lane):
// the sparsity metadata of four tcgen05.mma.sp instructions.  Ordered with the tcgen05.mma that the same
// thread issues afterwards.
template <int CTA_GROUP>
__device__ __forceinline__ void tcgen05_copy_128x128b(uint32_t tmem_address, uint64_t smem_descriptor) {
    if constexpr (CTA_GROUP == 1) asm volatile("tcgen05.cp.cta_group::1.128x128b [%0], %1;" ::"r"(tmem_address), "l"(smem_descriptor) : "memory");
    else asm volatile("tcgen05.cp.cta_group::2.128x128b [%0], %1;" ::"r"(tmem_address), "l"(smem_descriptor) : "memory");
}

// Descriptor of 128 rows of 16 bytes stored back to back (no swizzle): groups of eight rows are 128 bytes apart.
__device__ __forceinline__ uint64_t smem_descriptor_rows16(uint32_t address) {
    return static_cast<uint64_t>((address & 0x3ffffu) >> 4) | (1ull << 16) | (static_cast<uint64_t>(128 >> 4) << 32) | (1ull << 46);
}

// D[tmem] (+)= A[smem, 2:4 compressed] * B[smem], metadata in tensor memory at `metadata_tmem`.  16-bit kinds.
template <int CTA_GROUP>
__device__ __forceinline__ void tcgen05_mma_sparse_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t metadata_tmem,
                                                       uint32_t idesc, uint32_t accumulate) {
    if constexpr (CTA_GROUP == 1)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t"
                     "tcgen05.mma.sp.cta_group::1.kind::f16 [%0], %1, %2, [%3], %4, p;\n\t}"
                     ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(metadata_tmem), "r"(idesc), "r"(accumulate) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t"
                     "tcgen05.mma.sp.cta_group::2.kind::f16 [%0], %1, %2, [%3], %4, p;\n\t}"
                     ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(metadata_tmem), "r"(idesc), "r"(accumulate) : "memory");
}

}  // namespace ptx

namespace ptx {

// 32 lanes x 64 consecutive 32-bit columns in one instruction (see tmem_load_32x32).
__device__ __forceinline__ void tmem_load_32x64(uint32_t address, uint32_t (&r)[64]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
                 : "r"(address)
                 : "memory");
}

// Per-warpgroup register budget (all four warps of the warpgroup execute it together).
template <int REGISTERS>
__device__ __forceinline__ void registers_increase() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGISTERS)); }
template <int REGISTERS>
__device__ __forceinline__ void registers_decrease() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGISTERS)); }

}  // namespace ptx

namespace ptx {

// (sum0, sum1) += (value0, value1) * scale, both lanes in one packed instruction.
__device__ __forceinline__ void fma2(float &sum0, float &sum1, uint32_t value0, uint32_t value1, float scale) {
    asm("{\n\t.reg .b64 v, s, d;\n\t"
        "mov.b64 v, {%2, %3};\n\t"
        "mov.b64 s, {%4, %4};\n\t"
        "mov.b64 d, {%0, %1};\n\t"
        "fma.rn.f32x2 d, v, s, d;\n\t"
        "mov.b64 {%0, %1}, d;\n\t}"
        : "+f"(sum0), "+f"(sum1)
        : "r"(value0), "r"(value1), "f"(scale));
}

}  // namespace ptx

namespace ptx {

// ---- L2 residency hints for TMA loads --------------------------------------------------------------

__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

// tma_load_2d / tma_load_2d_pair with an L2 cache policy attached to the lines the load touches.
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap *map, int32_t x, int32_t y, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t dst, const CUtensorMap *map, int32_t x, int32_t y, uint32_t cluster_bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y), "l"(policy)
        : "memory");
}

}  // namespace ptx

namespace ptx {

// 32 lanes x 16 consecutive 32-bit columns (see tmem_load_32x32).
__device__ __forceinline__ void tmem_load_32x16(uint32_t address, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(address)
                 : "memory");
}

__device__ __forceinline__ uint32_t load_acquire(const unsigned int *address) {
    uint32_t value;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(value) : "l"(address) : "memory");
    return value;
}

}  // namespace ptx

namespace ptx {

// Shared-memory matrix descriptor of an MN-major operand stored as blocks of `rows` K-rows x 128 bytes (128 bytes of
// consecutive M/N elements per K index, 128-byte swizzle in groups of eight rows): the leading offset is the distance
// between consecutive 128-byte-wide blocks along M/N (one TMA box), the stride offset the 1024 bytes between groups
// of eight K-rows.
__device__ __forceinline__ uint64_t smem_descriptor_mn_major_sw128(uint32_t address, uint32_t block_bytes) {
    return static_cast<uint64_t>((address & 0x3ffffu) >> 4) | (static_cast<uint64_t>(block_bytes >> 4) << 16) |
           (static_cast<uint64_t>(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

}  // namespace ptx

namespace ptx {

// ---- TMA stores (shared -> global), tracked in bulk groups of the issuing thread ------------------------

// Makes this thread's earlier writes to shared memory visible to the TMA unit.
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Stores one box from shared memory to the tensor at (x, y); parts of the box outside the tensor are dropped.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int32_t x, int32_t y, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y)
                 : "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, int32_t x, int32_t y, int32_t z, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y), "r"(z)
                 : "memory");
}

// The same box added element-wise into the tensor (fp32 tensors: atomic adds performed by the TMA unit).  Like the store
// it must not start at a negative coordinate.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap *map, int32_t x, int32_t y, uint32_t src) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y)
                 : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// Waits until at most PENDING of this thread's store groups still read their shared-memory source.
template <int PENDING>
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(PENDING) : "memory"); }

// Waits until at most PENDING of this thread's store groups are incomplete (their writes performed).
template <int PENDING>
__device__ __forceinline__ void tma_store_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(PENDING) : "memory"); }

__device__ __forceinline__ void store_shared_v4(uint32_t address, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(address), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

}  // namespace ptx

namespace ptx {

// ---- per-thread asynchronous copies (global -> shared, 16 bytes), for gathered rows --------------------

// Copies `valid` (0 or 16) bytes from `source` and fills the rest of the 16 with zeros; does not block.
__device__ __forceinline__ void copy_async_16(uint32_t dst, const void *source, uint32_t valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(source), "r"(valid) : "memory");
}

// Arrives on `bar` once every copy_async_16 this thread has issued so far has landed.  Counts as one of the
// arrivals the barrier was initialised to expect.
__device__ __forceinline__ void copy_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

}  // namespace ptx
