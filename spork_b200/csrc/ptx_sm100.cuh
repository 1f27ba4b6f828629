// Inline-PTX building blocks for sm_100a kernels: mbarrier, TMA (bulk tensor
// copies), tcgen05 (tensor memory + 5th generation tensor-core MMA) and the
// cluster primitives a CTA pair needs.  Every spin-wait here is bounded: after
// a wall-clock limit it reports failure instead of hanging the GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace spork {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%laneid;" : "=r"(r));
    return r;
}

__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------- cluster ---

// One lane of a converged warp (the same one every time).
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// Address of the same shared-memory location in another CTA of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta_rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta_rank));
    return r;
}

__device__ __forceinline__ void cluster_arrive_release()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}

__device__ __forceinline__ void cluster_wait_acquire()
{
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ------------------------------------------------- programmatic dependent launch ---

// Blocks until every kernel this launch depends on in its stream has completed and its memory
// operations are visible.  A kernel launched with the "programmatic stream serialization" attribute may
// begin before its predecessor has finished; everything it does before this instruction must be
// independent of the predecessor (barrier set-up, tensor-memory allocation, descriptor prefetch).
// Without that attribute the instruction returns at once.
__device__ __forceinline__ void grid_dependency_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Tells the runtime that the next kernel in the stream, if it was launched with that attribute, may be
// scheduled as soon as every CTA of this grid has executed this instruction or exited.
__device__ __forceinline__ void grid_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// --------------------------------------------------------------- mbarrier ---

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrive on a barrier that may live in another CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Same, with cluster-scope acquire: pairs with arrivals made by the peer CTA.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wall-clock limit of one wait.  Far above any legitimate wait (the longest is
// one output tile's main loop, well under a millisecond) and short enough that
// a protocol bug ends the kernel instead of hanging the device.
constexpr uint64_t kWaitLimitNs = 2000000000ull;

// Bounded wait.  `abort_flag` is a CTA-shared word: once any role of the CTA
// has given up, the others stop waiting at their next slow-path check.
// Returns false if the wait was abandoned.
// `backoff_ns` > 0 puts the thread to sleep between polls (for waits that are long
// and not latency critical: fewer issued instructions, less power).
template <bool kClusterScope = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t backoff_ns = 0, uint64_t limit_ns = kWaitLimitNs)
{
    for (uint32_t fast = 0; fast < 64; ++fast) {
        if (kClusterScope ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity)) {
            return true;
        }
        if (backoff_ns != 0u) {
            __nanosleep(backoff_ns);
        }
    }
    const uint64_t deadline = global_timer_ns() + limit_ns;
    for (uint32_t spin = 0;; ++spin) {
        if (kClusterScope ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity)) {
            return true;
        }
        if (backoff_ns != 0u) {
            __nanosleep(backoff_ns);
        }
        if ((spin & 63u) == 63u) {
            if (*abort_flag != 0u || global_timer_ns() > deadline) {
                return false;
            }
        }
    }
}

// -------------------------------------------------------------------- TMA ---

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// Make generic-proxy writes to shared memory visible to the async proxy (TMA).
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Order generic-proxy accesses (of any state space, here: other CTAs' plain stores to global memory that an
// acquire has made visible) before later async-proxy accesses (TMA reduce-adds) of this thread.
__device__ __forceinline__ void fence_proxy_async_all()
{
    asm volatile("fence.proxy.async;" ::: "memory");
}

// Counter in global memory that CTAs of one grid signal each other through.
__device__ __forceinline__ void red_release_gpu_add(uint32_t* addr, uint32_t v)
{
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* addr)
{
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
    return v;
}

// Bounded wait until the counter has reached `target` (modulo 2^32).  Returns false if abandoned.
__device__ __forceinline__ bool counter_wait(const uint32_t* addr, uint32_t target, volatile uint32_t* abort_flag,
                                             uint64_t limit_ns = kWaitLimitNs)
{
    if ((int32_t)(ld_acquire_gpu(addr) - target) >= 0) {
        return true;
    }
    const uint64_t deadline = global_timer_ns() + limit_ns;
    for (uint32_t spin = 0;; ++spin) {
        if ((int32_t)(ld_acquire_gpu(addr) - target) >= 0) {
            return true;
        }
        __nanosleep(200);
        if ((spin & 63u) == 63u) {
            if (*abort_flag != 0u || global_timer_ns() > deadline) {
                return false;
            }
        }
    }
}

// L2 eviction-priority policies for loads that carry a cache hint.
__device__ __forceinline__ uint64_t l2_policy_evict_last()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ uint64_t l2_policy_evict_first()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ uint64_t l2_policy_evict_normal()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ void tma_load_2d_hint(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int32_t x,
                                                 int32_t y, uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t smem_dst, const CUtensorMap* map, uint32_t cluster_bar,
                                                      int32_t x, int32_t y, uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4}], [%2], %5;"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y), "l"(policy)
        : "memory");
}

// 2-D tile load, global -> this CTA's shared memory; completion bytes are
// credited to `bar` (an address in this CTA's shared window).
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int32_t x,
                                            int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// Same for a CTA pair: the data lands in this CTA's shared memory, the
// completion bytes are credited to `cluster_bar`, which may be the pair
// leader's barrier (a shared::cluster address obtained with map_to_cta).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* map, uint32_t cluster_bar,
                                                 int32_t x, int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int32_t x,
                                            int32_t y, int32_t z)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// 3-D forms of the hinted loads: z selects the matrix of a batch.
__device__ __forceinline__ void tma_load_3d_hint(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int32_t x,
                                                 int32_t y, int32_t z, uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4, %5}], [%2], %6;"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair_hint(uint32_t smem_dst, const CUtensorMap* map, uint32_t cluster_bar,
                                                      int32_t x, int32_t y, int32_t z, uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4, %5}], [%2], %6;"
        :
        : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y), "r"(z), "l"(policy)
        : "memory");
}

// 2-D tile store, shared -> global (elements outside the tensor are clipped).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t smem_src, int32_t x, int32_t y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 :
                 : "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_src), "r"(x), "r"(y)
                 : "memory");
}

// 2-D tile reduce-add, shared -> global (fp32 add into the destination).
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t smem_src, int32_t x, int32_t y)
{
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 :
                 : "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_src), "r"(x), "r"(y)
                 : "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t smem_src, int32_t x, int32_t y,
                                             int32_t z)
{
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 :
                 : "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_src), "r"(x), "r"(y), "r"(z)
                 : "memory");
}

__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* map, uint32_t smem_src, int32_t x, int32_t y,
                                                  int32_t z)
{
    asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
                 :
                 : "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_src), "r"(x), "r"(y), "r"(z)
                 : "memory");
}

__device__ __forceinline__ void bulk_commit_group()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Wait until at most N of this thread's bulk groups still READ shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Wait until at most N of this thread's bulk groups are incomplete.
template <int N>
__device__ __forceinline__ void bulk_wait_group()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------- tcgen05 ---

template <int CG>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result_addr, uint32_t columns)
{
    if (CG == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result_addr),
                     "r"(columns)
                     : "memory");
    } else {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result_addr),
                     "r"(columns)
                     : "memory");
    }
}

template <int CG>
__device__ __forceinline__ void tmem_relinquish()
{
    if (CG == 1) {
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
}

template <int CG>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns)
{
    if (CG == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
    } else {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
    }
}

__device__ __forceinline__ void tcgen05_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile whose rows are
// 128 bytes (one 128B-swizzle atom wide) and packed at a 128-byte pitch, so
// that 8-row groups are 1024 bytes apart.  The tile base must be 1024-byte
// aligned; stepping along K inside the atom adds the byte offset >> 4 to the
// low word.
__device__ __forceinline__ uint64_t umma_desc_kmajor_sw128(uint32_t smem_addr)
{
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address, bits [0,14)
    desc |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (unused when swizzled)
    desc |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset: 8 rows * 128 B
    desc |= static_cast<uint64_t>(1) << 46;                      // descriptor version for sm_100
    desc |= static_cast<uint64_t>(2) << 61;                      // layout type: 128-byte swizzle
    return desc;
}

// Shared-memory matrix descriptor for an MN-major operand (the contiguous
// direction is M or N, not K) stored as 128B-swizzle atoms of 64 fp16 along MN
// by 8 along K (1024 bytes each).  `mn_atom_stride` is the byte distance
// between atoms that are neighbours along MN, `k_atom_stride` between
// neighbours along K.
__device__ __forceinline__ uint64_t umma_desc_mnmajor_sw128(uint32_t smem_addr, uint32_t mn_atom_stride,
                                                            uint32_t k_atom_stride)
{
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    desc |= static_cast<uint64_t>((mn_atom_stride >> 4) & 0x3FFFu) << 16;  // leading byte offset
    desc |= static_cast<uint64_t>((k_atom_stride >> 4) & 0x3FFFu) << 32;   // stride byte offset
    desc |= static_cast<uint64_t>(1) << 46;
    desc |= static_cast<uint64_t>(2) << 61;
    return desc;
}

// Instruction descriptor for kind::f16: fp16 A and B, fp32 accumulator.
// a_mn_major / b_mn_major select the operand's contiguous direction.
// `bf16` selects bfloat16 operands instead of fp16 (same instruction kind).
__host__ __device__ constexpr uint32_t umma_idesc_f16_f32(uint32_t m, uint32_t n, bool a_mn_major = false,
                                                          bool b_mn_major = false, bool bf16 = false)
{
    return (1u << 4)                          // accumulator format: fp32
           | ((bf16 ? 1u : 0u) << 7)          // A format: 0 = fp16, 1 = bf16
           | ((bf16 ? 1u : 0u) << 10)         // B format
           | (a_mn_major ? (1u << 15) : 0u)   //
           | (b_mn_major ? (1u << 16) : 0u)   //
           | ((n >> 3) << 17)                 // N / 8
           | ((m >> 4) << 24);                // M / 16
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
template <int CG>
__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate)
{
    if (CG == 1) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
            "}"
            :
            : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
            "}"
            :
            : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// Same with fp32 operands in shared memory read as tf32 (kind::tf32, K = 8 per instruction).
template <int CG>
__device__ __forceinline__ void umma_tf32_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate)
{
    if (CG == 1) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
            "}"
            :
            : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t"
            "}"
            :
            : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// Instruction descriptor for kind::tf32: tf32 A and B (K-major), fp32 accumulator.
__host__ __device__ constexpr uint32_t umma_idesc_tf32_f32(uint32_t m, uint32_t n)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// The same two MMAs taking each 64-bit shared-memory descriptor as its two 32-bit halves: the high half
// (strides, version, swizzle mode) is a constant and the low half (start address >> 4, leading offset)
// advances by small constants, so the issuing thread spends one integer add per operand instead of
// rebuilding the descriptor.
__device__ __forceinline__ void umma_f16_ss_cta1(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                 uint32_t b_hi, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_f16_ts_cta1(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi,
                                                 uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .b64 db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t"
        "}"
        :
        : "r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}

// High halves of the two descriptor kinds used with 128-byte swizzle, and the low half for an address.
constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);  // 8-row groups 1024 B apart
__device__ __forceinline__ uint32_t desc_lo_kmajor(uint32_t smem_addr)
{
    return ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16);
}
__device__ __forceinline__ uint32_t desc_lo_mnmajor(uint32_t smem_addr, uint32_t mn_atom_stride)
{
    return ((smem_addr & 0x3FFFFu) >> 4) | (((mn_atom_stride >> 4) & 0x3FFFu) << 16);
}

// D[tmem] (+)= A[tmem] * B[smem]; issued by ONE thread.
template <int CG>
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate)
{
    if (CG == 1) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
            "}"
            :
            : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t"
            "}"
            :
            : "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// Make `cluster_bar` (a shared::cluster address: this CTA's or the peer's
// barrier) receive one arrival when every tcgen05 operation this thread has
// issued so far has completed.
template <int CG>
__device__ __forceinline__ void umma_commit(uint32_t cluster_bar)
{
    if (CG == 1) {
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar)
                     : "memory");
    } else {
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar)
                     : "memory");
    }
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives the 32
// columns of TMEM lane (lane base of taddr + i).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns, registers -> TMEM.
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns, registers -> TMEM.
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
          "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),
          "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_st_wait()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ void st_global_v4(void* ptr, uint4 v)
{
    asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(ptr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ----------------------------------------------------------- checked build ---

// Range checks of a debug build (-DSPORK_CHECKED): every shared-memory address handed to TMA, to an MMA
// descriptor or to a staging store, every tensor-memory address and every TMA coordinate is tested
// against what the kernel allocated before it is used.  A failed check records a code in the device
// status word (first failure wins, never a trap) and the caller skips the access; the kernel then ends
// through its bounded waits.  In a normal build every method is the constant `true` and costs nothing.
// Status word of a failed check: 0xC0000000 | code << 16 | block index (low 16 bits).
struct Checker {
    uint32_t* status;
    uint32_t smem_lo, smem_hi;    // shared window of the CTA's dynamic allocation
    uint32_t tmem_lo, tmem_cols;  // tensor-memory allocation (column base and width)

#ifdef SPORK_CHECKED
    __device__ __forceinline__ bool fail(uint32_t code) const
    {
        atomicCAS(status, 0u, 0xC0000000u | ((code & 0xFFFu) << 16) | (blockIdx.x & 0xFFFFu));
        return false;
    }
    // [addr, addr + bytes) inside the allocation, addr aligned to `align`
    __device__ __forceinline__ bool smem(uint32_t addr, uint32_t bytes, uint32_t align, uint32_t code) const
    {
        return (addr >= smem_lo && addr + bytes <= smem_hi && (addr & (align - 1u)) == 0u) ? true : fail(code);
    }
    // columns [col, col + cols) of lanes [lane, lane + 32) inside the allocation (lane = bits 16.. of taddr)
    __device__ __forceinline__ bool tmem(uint32_t taddr, uint32_t cols, uint32_t code) const
    {
        const uint32_t col = taddr & 0xFFFFu, lane = taddr >> 16;
        const uint32_t lo = tmem_lo & 0xFFFFu;
        return (col >= lo && col + cols <= lo + tmem_cols && lane < 128u) ? true : fail(code);
    }
    // innermost TMA coordinate: not negative and on a 16-byte boundary; the others: not negative
    __device__ __forceinline__ bool tma_coords(int32_t x, uint32_t elem_bytes, int32_t y, int32_t z, uint32_t code) const
    {
        return (x >= 0 && (((uint32_t)x * elem_bytes) & 15u) == 0u && y >= 0 && z >= 0) ? true : fail(code);
    }
#else
    __device__ __forceinline__ bool smem(uint32_t, uint32_t, uint32_t, uint32_t) const { return true; }
    __device__ __forceinline__ bool tmem(uint32_t, uint32_t, uint32_t) const { return true; }
    __device__ __forceinline__ bool tma_coords(int32_t, uint32_t, int32_t, int32_t, uint32_t) const { return true; }
#endif
};

}  // namespace ptx
}  // namespace spork
