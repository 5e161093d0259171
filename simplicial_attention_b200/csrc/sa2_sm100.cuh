// Thin inline-PTX wrappers for the sm_100a features the tensor-core kernels
// use: mbarriers, TMA tiled loads, tcgen05 MMA / TMEM load-store / commit, and
// the shared-memory and instruction descriptors that tcgen05.mma takes.
//
// Every wait is bounded: a barrier that does not complete within
// WAIT_LIMIT_CYCLES makes the waiter record an error word and return false,
// so a logic error ends the kernel with a status instead of hanging the GPU.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sa2 {
namespace sm100 {

constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;   // about one second

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Optional wait accounting (compile with -DSA2_PROF=<CTA>): lane 0 of every warp of one CTA adds the cycles
// it spends in a wait to slot 8 * warp + slot of a table; sa2_prof_read() copies the table to the host.
#ifdef SA2_PROF
__device__ unsigned long long g_prof[512];
// the cycles are summed in shared memory (a read-modify-write of global memory after every wait would itself
// cost more than most waits) and copied out once, when the warp is done
__device__ __forceinline__ unsigned long long *prof_slots() {
    __shared__ unsigned long long s[8 * 24];          // up to 24 warps
    return s;
}
__device__ __forceinline__ bool prof_lane() {
    return blockIdx.x == SA2_PROF && blockIdx.y == 0 && blockIdx.z == 0 && (threadIdx.x & 31) == 0;
}
__device__ __forceinline__ void prof_begin() {
    if (prof_lane())
        for (int k = 0; k < 8; ++k) prof_slots()[(threadIdx.x >> 5) * 8 + k] = 0;
}
__device__ __forceinline__ void prof_add(int slot, long long cycles) {
    if (slot >= 0 && prof_lane()) prof_slots()[(threadIdx.x >> 5) * 8 + slot] += (unsigned long long)cycles;
}
__device__ __forceinline__ void prof_end() {
    if (prof_lane())
        for (int k = 0; k < 8; ++k) g_prof[(threadIdx.x >> 5) * 8 + k] += prof_slots()[(threadIdx.x >> 5) * 8 + k];
}
#define SA2_PROF_ADD(slot, cycles) sa2::sm100::prof_add(slot, cycles)
#define SA2_PROF_END() sa2::sm100::prof_end()
// segment timing: SA2_PROF_MARK(t) starts a segment, SA2_PROF_LAP(slot, t) books the time since and restarts
#define SA2_PROF_MARK(t) long long t = clock64()
#define SA2_PROF_LAP(slot, t) do { const long long _n = clock64(); sa2::sm100::prof_add(slot, _n - t); t = _n; } while (0)
#else
#define SA2_PROF_ADD(slot, cycles) do { } while (0)
#define SA2_PROF_END() do { } while (0)
#define SA2_PROF_MARK(t) do { } while (0)
#define SA2_PROF_LAP(slot, t) do { } while (0)
#endif

// Bounded wait.  `abort_flag` is a CTA-wide shared word: once any thread gives
// up, every later wait in the CTA returns false at once.  `prof` names the accounting slot (see above).
// `sleep_ns` > 0 makes the poller yield its issue slots between tries (used by
// whole warps that wait; the single MMA-issuing lanes poll without sleeping).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, unsigned sleep_ns = 0,
                                          int prof = -1, long long limit_cycles = WAIT_LIMIT_CYCLES) {
#ifdef SA2_PROF
    const long long t0 = clock64();       // a try_wait may suspend the thread: the first try counts as waiting too
    if (mbar_try_wait(bar, parity)) { SA2_PROF_ADD(prof, clock64() - t0); return true; }
#else
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
#endif
    int spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if (sleep_ns) __nanosleep(sleep_ns);
        if ((++spins & 255) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit_cycles) {
                *abort_flag = 1;
                return false;
            }
        }
    }
    SA2_PROF_ADD(prof, clock64() - t0);
    return true;
}

// make generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma)
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// --------------------------------------------------------------------- TMA
// 4-D tiled load: coordinates are (channel, head, row, batch), innermost first.
__device__ __forceinline__ void tma_load_4d(void *smem_dst, const void *tmap, uint64_t *bar,
                                            int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void *tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ----------------------------------------------------------------- tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_holder, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(smem_holder)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrive on `bar` once every tcgen05 operation this thread issued so far has completed
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}

// 32 lanes x 32 columns of 32-bit: thread t of the warp gets columns [col, col+32) of TMEM lane (lane_base + t)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// Per-warpgroup register budget (all four warps of an aligned warpgroup must execute it).
template <int N> __device__ __forceinline__ void reg_alloc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_dealloc() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// ------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor for tiles stored as rows of 128 bytes with the
// 128-byte swizzle (16-byte chunk index XOR (row & 7)); 8 rows form a 1024-byte
// group and groups follow each other at `group_stride_bytes`.
//   K-major operand  (rows = M or N, 64 bf16 of K per row): advance K by 16 elements = +32 bytes
//   MN-major operand (rows = K, 64 bf16 of M/N per row):    advance K by 16 rows     = +2048 bytes
// `block_stride_bytes` is the distance between 64-element blocks along M/N for
// MN-major operands wider than 64 (unused otherwise).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr, uint32_t group_stride_bytes = 1024,
                                                    uint32_t block_stride_bytes = 16) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);                   // start address
    d |= (uint64_t)((block_stride_bytes >> 4) & 0x3FFF) << 16;    // leading byte offset
    d |= (uint64_t)((group_stride_bytes >> 4) & 0x3FFF) << 32;    // stride byte offset
    d |= (uint64_t)1 << 46;                                       // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                                       // SWIZZLE_128B
    return d;
}

// Instruction descriptor for kind::f16 with bf16 operands and fp32 accumulation.
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, bool a_mn_major, bool b_mn_major) {
    return (1u << 4)                          // D format: f32
         | (1u << 7)                          // A format: bf16
         | (1u << 10)                         // B format: bf16
         | ((a_mn_major ? 1u : 0u) << 15)
         | ((b_mn_major ? 1u : 0u) << 16)
         | ((uint32_t)(N >> 3) << 17)
         | ((uint32_t)(M >> 4) << 24);
}

// byte offset of 16-byte chunk `chunk` (0..7) of row `row` in a 128-byte-swizzled tile
__device__ __forceinline__ uint32_t sw128_offset(int row, int chunk) {
    return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4));
}

}  // namespace sm100
}  // namespace sa2
