// Thin inline-PTX wrappers for the sm_100a features the kernels use: mbarrier, TMA
// (cp.async.bulk.tensor), tcgen05 (TMEM allocation, UMMA, TMEM loads) and proxy fences.
// Every TMA load here is a plain single-destination copy.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace sdxlq::ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* pointer) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

// ---- mbarrier ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done = 0;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait: polls the barrier and gives up after `limit_cycles` SM clocks or as soon as
// the CTA-wide abort word is set. Returns false when it gave up.
__device__ __forceinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile uint32_t* abort_word,
                                            long long limit_cycles) {
    const long long start = clock64();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 0x3FFu) == 0) {
            if (*abort_word != 0) return false;
            if (clock64() - start > limit_cycles) return false;
        }
    }
}

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  volatile uint32_t* abort_word,
                                                  long long limit_cycles) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_word, limit_cycles);
}

// ---- TMA ---------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const void* tensor_map, uint32_t bar,
                                            int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// Orders a tensor map that was written to global memory by the host (cudaMemcpy) before its
// first use by this CTA's TMA unit.
__device__ __forceinline__ void fence_tensormap_acquire(const void* tensor_map) {
    asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;"
                 ::"l"(reinterpret_cast<uint64_t>(tensor_map))
                 : "memory");
}

// ---- tcgen05 -----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_result), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t tmem_address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_address), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; `accumulate` == 0 overwrites D.
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                        uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The four MMAs of one pipeline stage in a single statement. A stage holds 128 bytes of K per row
// (one swizzle span) and every MMA consumes 32 of them, so the operand start addresses advance by
// 32 B >> 4 = 2 descriptor units per MMA. The 64-bit shared-memory descriptors are passed as their
// low words (start address, leading offset) plus the common high word (stride, version, swizzle)
// so that the issuing thread does 32-bit arithmetic only. `accumulate_first` == 0 makes the first
// MMA overwrite the accumulator; the other three always accumulate.
#define SDXLQ_UMMA_STAGE(NAME, GROUP, KIND)                                                              \
    __device__ __forceinline__ void NAME(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, \
                                         uint32_t idesc, uint32_t accumulate_first) {                    \
        asm volatile(                                                                                    \
            "{\n\t"                                                                                      \
            ".reg .pred p, q;\n\t"                                                                       \
            ".reg .b64 da, db;\n\t"                                                                      \
            ".reg .b32 a, b;\n\t"                                                                        \
            "setp.ne.b32 p, %5, 0;\n\t"                                                                  \
            "setp.ne.b32 q, %6, 0;\n\t"                                                                  \
            "mov.b64 da, {%1, %3};\n\t"                                                                  \
            "mov.b64 db, {%2, %3};\n\t"                                                                  \
            "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], da, db, %4, p;\n\t"                   \
            "add.u32 a, %1, 2;\n\t"                                                                      \
            "add.u32 b, %2, 2;\n\t"                                                                      \
            "mov.b64 da, {a, %3};\n\t"                                                                   \
            "mov.b64 db, {b, %3};\n\t"                                                                   \
            "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], da, db, %4, q;\n\t"                   \
            "add.u32 a, %1, 4;\n\t"                                                                      \
            "add.u32 b, %2, 4;\n\t"                                                                      \
            "mov.b64 da, {a, %3};\n\t"                                                                   \
            "mov.b64 db, {b, %3};\n\t"                                                                   \
            "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], da, db, %4, q;\n\t"                   \
            "add.u32 a, %1, 6;\n\t"                                                                      \
            "add.u32 b, %2, 6;\n\t"                                                                      \
            "mov.b64 da, {a, %3};\n\t"                                                                   \
            "mov.b64 db, {b, %3};\n\t"                                                                   \
            "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], da, db, %4, q;\n\t"                   \
            "}\n"                                                                                        \
            ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate_first), "r"(1u) \
            : "memory");                                                                                 \
    }
SDXLQ_UMMA_STAGE(umma_stage_i8, "1", "i8")
SDXLQ_UMMA_STAGE(umma_stage_f8f6f4, "1", "f8f6f4")
SDXLQ_UMMA_STAGE(umma_stage_f16, "1", "f16")
SDXLQ_UMMA_STAGE(umma_stage_i8_pair, "2", "i8")
SDXLQ_UMMA_STAGE(umma_stage_f8f6f4_pair, "2", "f8f6f4")
SDXLQ_UMMA_STAGE(umma_stage_f16_pair, "2", "f16")
#undef SDXLQ_UMMA_STAGE

// Operand kind tag of the stage-wide MMA: 0 kind::i8, 1 kind::f8f6f4, 2 kind::f16.
template <int KindTag, bool kPair>
__device__ __forceinline__ void umma_stage(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                           uint32_t idesc, uint32_t accumulate_first) {
    if constexpr (kPair) {
        if constexpr (KindTag == 0) umma_stage_i8_pair(tmem_d, a_lo, b_lo, desc_hi, idesc, accumulate_first);
        else if constexpr (KindTag == 1) umma_stage_f8f6f4_pair(tmem_d, a_lo, b_lo, desc_hi, idesc, accumulate_first);
        else umma_stage_f16_pair(tmem_d, a_lo, b_lo, desc_hi, idesc, accumulate_first);
    } else {
        if constexpr (KindTag == 0) umma_stage_i8(tmem_d, a_lo, b_lo, desc_hi, idesc, accumulate_first);
        else if constexpr (KindTag == 1) umma_stage_f8f6f4(tmem_d, a_lo, b_lo, desc_hi, idesc, accumulate_first);
        else umma_stage_f16(tmem_d, a_lo, b_lo, desc_hi, idesc, accumulate_first);
    }
}

// Low word of the SWIZZLE_128B K-major operand descriptor for the tile at `smem_address`, and the
// high word every such descriptor shares (see umma_smem_desc_sw128 for the fields).
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t smem_address) {
    return ((smem_address & 0x3FFFFu) >> 4) | (1u << 16);
}
constexpr uint32_t kUmmaDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);

// Makes `bar` (a CTA-local mbarrier) track completion of all tcgen05 operations issued so far
// by this thread; one arrival is delivered when they finish.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns: thread t of the warp receives lane (base + t).
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t tmem_address, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(tmem_address)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x8(uint32_t tmem_address, uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(tmem_address)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// The wait with the loaded registers named as in/out operands: every use of them is ordered after
// the wait by a data dependency, also when other loads were issued in between (software
// pipelining, where a later load is in flight while these values are consumed).
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[8]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])
                 :
                 : "memory");
}

__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :
                 : "memory");
}

__device__ __forceinline__ void tmem_ld_wait(uint32_t (&a)[8], uint32_t (&b)[8]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]),
                   "+r"(b[0]), "+r"(b[1]), "+r"(b[2]), "+r"(b[3]), "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7])
                 :
                 : "memory");
}

// Register reallocation between warpgroups (four consecutive warps): every warp of the warpgroup
// executes the same instruction. `dec` returns registers to the SM's pool, `inc` waits until the
// pool holds enough and takes them. The count is a multiple of 8 in [24, 256].
template <uint32_t Registers>
__device__ __forceinline__ void setmaxnreg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Registers));
}
template <uint32_t Registers>
__device__ __forceinline__ void setmaxnreg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Registers));
}

// Programmatic dependent launch. `grid_dependency_wait` blocks until the grids this one depends on
// have completed and their memory is visible; `grid_launch_dependents` lets a dependent grid that
// was launched with the programmatic attribute start being scheduled. Both do nothing in a grid
// launched without such a dependency.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- CTA pairs (cta_group::2) ----------------------------------------------------------------
// Two CTAs of a cluster work on one 256-row tile: each loads its 128 rows of A and half of the B
// rows into its own shared memory, the even-ranked CTA (the leader) issues the MMAs, and each
// CTA's tensor memory receives its 128 rows of the accumulator.
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;     // clears the CTA-rank bit of a shared::cluster address

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}

__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_address, uint32_t rank) {
    uint32_t mapped;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(mapped) : "r"(smem_address), "r"(rank));
    return mapped;
}

// Arrive on a barrier given by its shared::cluster address (possibly in the peer CTA).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_address) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_address) : "memory");
}

// TMA load issued by either CTA of a pair: the data lands in the issuing CTA's shared memory,
// the transaction bytes are counted on the LEADER's barrier (same offset, rank bit cleared).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const void* tensor_map, uint32_t bar,
                                                 int32_t x, int32_t y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(bar & kPeerBitMask), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_result), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t tmem_address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_address), "r"(columns)
                 : "memory");
}

#define SDXLQ_UMMA_PAIR(NAME, KIND)                                                                     \
    __device__ __forceinline__ void NAME(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,            \
                                         uint32_t idesc, uint32_t accumulate) {                         \
        asm volatile(                                                                                   \
            "{\n\t"                                                                                     \
            ".reg .pred p;\n\t"                                                                         \
            "setp.ne.b32 p, %4, 0;\n\t"                                                                 \
            "tcgen05.mma.cta_group::2.kind::" KIND " [%0], %1, %2, %3, p;\n\t"                          \
            "}\n"                                                                                       \
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)                        \
            : "memory");                                                                                \
    }
SDXLQ_UMMA_PAIR(umma_i8_pair, "i8")
SDXLQ_UMMA_PAIR(umma_f8f6f4_pair, "f8f6f4")
SDXLQ_UMMA_PAIR(umma_f16_pair, "f16")
#undef SDXLQ_UMMA_PAIR

// Completion of the pair's MMAs -> one arrival on the barrier at `cluster_address` (own or peer CTA).
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_address) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_address)
                 : "memory");
}

// Instruction descriptor for kind::i8 / kind::f8f6f4 / kind::f16, both operands K-major.
// c_format: 1 = F32, 2 = S32. a/b format: i8 -> 1 (signed); f8f6f4 -> 0 E4M3, 1 E5M2; f16 -> 0.
__host__ __device__ constexpr uint32_t umma_instr_desc(uint32_t c_format, uint32_t a_format,
                                                       uint32_t b_format, uint32_t m, uint32_t n) {
    return (c_format << 4) | (a_format << 7) | (b_format << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

}  // namespace sdxlq::ptx
