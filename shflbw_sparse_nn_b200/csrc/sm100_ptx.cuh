// Thin inline-PTX wrappers for the sm_100a features the kernels use: mbarrier, cp.async,
// proxy fences, tcgen05 (TMEM alloc / mma / commit / ld) and the shared-memory matrix
// descriptors that tcgen05.mma consumes.  No library code; each wrapper is one instruction
// or one documented bit layout.
#pragma once

#include <cstdint>
#include <cuda_fp16.h>

namespace sm100 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// ------------------------------------------------------------------ mbarrier ----
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    // Make barrier initialisation visible to the async proxy (tcgen05.commit arrives on it).
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar))
                 : "memory");
}
// Non-blocking phase test.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns when the phase with the given parity completes, the CTA-wide abort
// flag is raised, or `limit_cycles` SM clocks pass.  On timeout it raises the abort flag and
// records `code` in the global status word; the caller carries on (results are then garbage,
// but every later wait returns at once and the kernel drains and exits).
//
// The already-complete case is one inlined test; the polling loop lives in a function that is
// NOT inlined, so the hot loops of the kernel stay short and straight (the kernels proved
// sensitive to instruction fetch: a taken branch to a cold line cost ~150 clk).  Between
// polls the thread sleeps `backoff_ns` so waiting warps leave the issue slots to the others.
// `heed_abort = false` is for the clean-up wait of the abort path itself (the flag is already up
// there); `code` 0 records nothing.
__device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, volatile int* cta_abort,
                                            int* status_word, int code, long long limit_cycles,
                                            uint32_t backoff_ns, bool heed_abort) {
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (true) {
        if (backoff_ns) __nanosleep(backoff_ns);
        if (mbar_test(bar, parity)) return true;
        if ((++spins & 0xf) == 0) {
            if (heed_abort && *cta_abort) return false;
            if (clock64() - t0 > limit_cycles) {
                *cta_abort = 1;
                if (code) atomicCAS(status_word, 0, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* cta_abort,
                                                  int* status_word, int code, long long limit_cycles,
                                                  uint32_t backoff_ns = 40, bool heed_abort = true) {
    // Most waits in the kernels are short (a few hundred clocks): poll a handful of times in
    // line before paying for the call and the first sleep of the slow path.
#pragma unroll 1
    for (int i = 0; i < 12; ++i)
        if (mbar_test(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, cta_abort, status_word, code, limit_cycles, backoff_ns, heed_abort);
}

// ----------------------------------------------------------------- bulk copy ----
// Adds `bytes` to the barrier's pending transaction count (no arrival).
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Contiguous global -> shared copy by the copy engine; completes `bytes` on the barrier.
// Both addresses 16-byte aligned, bytes a multiple of 16.  The source is this GPU's memory.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// One arrival plus `bytes` added to the pending transaction count, in one operation.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Subtracts `bytes` from the pending transaction count by hand (tuning builds that skip a copy).
__device__ __forceinline__ void mbar_complete_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.complete_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// TMA tile::gather4: rows r0..r3 of a 2-D tensor (tensor map box = W columns x 1 row), columns
// [col, col + W), land as 4 consecutive rows of W elements at dst (swizzled as the map says) and
// complete 4*W*elemsize bytes on the barrier.  Columns or rows outside the tensor read as zero.
// The map must describe memory of THIS GPU; this is the plain .shared::cta form, no multicast.
__device__ __forceinline__ void tma_gather4(uint32_t dst_smem, const void* tmap, int col, int r0, int r1, int r2, int r3,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
        ::"r"(dst_smem), "l"(tmap), "r"(col), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(smem_u32(bar))
        : "memory");
}

// 32-byte global store (one whole L2 sector) from two 16-byte registers sets; dst 32-byte aligned.
__device__ __forceinline__ void st_global_32B(void* dst, const uint4& a, const uint4& b) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w),
                 "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w) : "memory");
}

// ------------------------------------------------------------------ cp.async ----
// 16-byte global->shared copy through L2 only; src_bytes = 0 zero-fills the destination.
__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes)
                 : "memory");
}
// 4-byte global->shared copy (used to prefetch row ids); src_bytes = 0 stores zero.
__device__ __forceinline__ void cp_async_4(uint32_t dst_smem, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// Deferred arrival: the mbarrier receives one arrival (already counted in its expected
// count, hence .noinc) once all cp.async copies this thread has issued so far have landed.
// The issuing thread does not wait.
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Generic-proxy writes (cp.async, st.shared) -> visible to the async proxy (tcgen05.mma reads).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------- programmatic dependent launch ----
// A kernel launched with the programmatic-stream-serialization attribute may start while the
// kernel before it in the stream is still running.  grid_dependency_wait() blocks until that
// kernel has completed and its writes are visible (no-op without the attribute);
// grid_dependency_launch() lets the NEXT kernel of the stream start early (no-op when that one
// was launched without the attribute).  Everything a kernel does before its wait must not touch
// data the previous kernel writes -- or buffers it still reads.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ------------------------------------------------------- register budgets ----
// Change the per-thread register budget of the executing warpgroup (4 consecutive warps, all
// of which must execute the same instruction).  The count is a multiple of 8 in [24, 256].
// .dec returns registers to the SM's pool at once; .inc waits until the pool holds enough.
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// ------------------------------------------------------------------- tcgen05 ----
// TMEM allocation: one full warp; ncols a power of two in [32, 512].  The base address
// (lane 0, first column) is written to *slot in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], kind::f16 (fp16/bf16 in, fp32 or fp16 out),
// issued by ONE thread.  accumulate = 0 overwrites D.
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                            uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive once on an mbarrier when all tcgen05.mma issued so far by this thread complete.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}

// TMEM -> registers: the warp's 32 lanes x 32 consecutive fp32 columns (thread = lane).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
          "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
          "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
          "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// TMEM -> registers: the warp's 32 lanes x 16 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// TMEM -> registers: the warp's 32 lanes x 8 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld_32x32b_x8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------- descriptors ----
// Shared-memory matrix descriptor (64 bit):
//   [ 0,14) start address >> 4      [16,30) leading-dimension byte offset >> 4
//   [32,46) stride byte offset >> 4 [46,48) version = 1 (Blackwell)
//   [49,52) base offset = 0         [61,64) swizzle: 0 none, 2 = 128 B, 4 = 64 B, 6 = 32 B
// For an MN-major operand with 128-byte swizzle the canonical layout is, in 16-byte units,
//   ((8, n), (8, k)) : ((1, LBO), (8, SBO))
// i.e. one K row is a 128-byte line (64 fp16 along MN), eight K rows form a 1024-byte atom,
// atoms repeat along MN every LBO bytes and along K every SBO bytes, and the 16-byte chunk
// index inside a line is XORed with (row % 8).  With 64-byte swizzle the line is 64 bytes
// (32 fp16), the atom 512 bytes, and the chunk index is XORed with ((row / 2) % 4); with 32-byte
// swizzle the line is 32 bytes (16 fp16), the atom 256 bytes, and the XOR term is ((row / 4) % 2).
constexpr uint64_t kSwizzle128B = 2, kSwizzle64B = 4, kSwizzle32B = 6;
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes, uint64_t swizzle) {
    return (uint64_t)((smem_addr & 0x3ffffu) >> 4) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (swizzle << 61);
}

// Instruction descriptor (32 bit) for kind::f16 with fp16 A/B, fp32 D, both operands
// MN-major:  [4,6) D format 1 = f32, [7,10) A format 0 = f16, [10,13) B format 0 = f16,
// bit 15 A MN-major, bit 16 B MN-major, [17,23) N >> 3, [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc_f16_mnmajor(int M, int N) {
    return (1u << 4) | (1u << 15) | (1u << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

}  // namespace sm100
