// Forward kernel on the 5th-generation tensor cores (tcgen05 + TMEM + TMA),
// bf16 operands, fp32 accumulation, head dim 64.
//
// One CTA owns 128 query rows of one (batch, query head).  For every offset
// e = i - k of the second key ("sweep") it forms A_e[i,:] = q_i * k2_{i-e}
// (bf16, CUDA cores, 128-byte-swizzled shared memory), multiplies it against
// the TMA-staged K1 tiles of the window (S = A_e K1^T, 128x128x64 per tile,
// accumulator in TMEM), turns S into P = exp2(c*S - ref) in registers, writes
// P to TMEM as bf16 and feeds it as the A operand of W_e += P V1 (128x64x128,
// V1 tile as an MN-major B operand).  At the end of a sweep the row owner adds
// v2_{i-e} * W_e to its output registers.  The softmax is joint over all
// (j, e): one denominator per row.
//
// Warp roles (512 threads, four aligned warpgroups):
//   warp 0        TMA producer: the K1/V1 window and the 127 + 32 second-key rows
//                 the tile can pair with, loaded once and resident in shared memory;
//                 then issues the tcgen05.mma stream of group 1 (one lane)
//   warp 1        owns the TMEM allocation, issues the tcgen05.mma stream of group 0
//   warps 2-3     idle (they fill the issuers' warpgroup)
//   warps 4-7     output group, one thread per query row: builds the A tile of each
//                 group's next sweep as soon as the last S product of its current sweep
//                 has completed, and at the end of a sweep adds v2_{i-e} * W_e to the
//                 row's output registers (one accumulator per softmax group)
//   warps 8-11    softmax group 0: even sweeps, one thread per query row
//   warps 12-15   softmax group 1: odd sweeps, one thread per query row
// An even and an odd sweep are in flight together, so while one group runs the
// exponentials of its tile the tensor cores work for the other and each SM
// sub-partition has two softmax warps to hide latencies.  A softmax thread keeps
// only (reference, denominator) per row; the output thread keeps the two groups'
// accumulators, each against the reference its group last reported, and merges
// them at the end.  Registers move between the warpgroups with setmaxnreg.
//
// The unit of the pipeline is half a key tile (64 keys): S = A_e K1[64 rows]^T is
// 128x64, and every group has two S and two P buffers, so its next unit is
// ready in TMEM while it works on the current one.
//
// TMEM columns, group g, buffer s: S [128g + 64s, +64), P (bf16) [384 + 64g + 32s, +32);
// W of group g [256 + 64g, +64).
//
// Reference handling: probabilities are computed against a per-row reference
// that only moves when it must, so the W accumulator in TMEM normally never
// needs a rescale; bf16 has fp32's exponent range, so P may exceed 1 by many
// orders of magnitude without loss.  When the probabilities of a tile sum to
// more than 2^64 (always true for a row's very first tile, whose reference is
// -inf) the warp takes a slow path: exact tile maximum, rescale of the row's
// partial sums (including W in TMEM), recomputation of P.
#pragma once
#include "sa2_common.cuh"
#include "sa2_sm100.cuh"
#include <cuda.h>
#include <math_constants.h>

namespace sa2 {
namespace tc {

using namespace sa2::sm100;

constexpr int TQ = 128;          // query rows per CTA
constexpr int TJ = 128;          // first-key rows per tile
constexpr int FWD_THREADS = 512;
// Register hand-over between warpgroups (launch: 128 per thread; the budgets must add up to 4 * 128, or
// the growing group never returns from its setmaxnreg).
constexpr int FWD_REGS_LAUNCH = 128, FWD_REGS_ISSUE = 56, FWD_REGS_SOFTMAX = 112, FWD_REGS_OUT = 232;
static_assert(FWD_REGS_ISSUE + 2 * FWD_REGS_SOFTMAX + FWD_REGS_OUT == 4 * FWD_REGS_LAUNCH, "register pool must balance");
static_assert(FWD_REGS_SOFTMAX < FWD_REGS_LAUNCH, "the softmax groups release registers");
constexpr int MAX_NT = 5;        // K1/V1 tiles resident in shared memory (head dim 64)
constexpr uint32_t TILE_BYTES = TJ * 64 * 2;
constexpr int K2_ROWS = 160;     // second-key rows kept in shared memory: positions i0 - 32 ... i0 + 127

enum FwdBar {
    BAR_KV_FULL = 0,                     // [MAX_NT]
    BAR_A_FULL = BAR_KV_FULL + MAX_NT,   // [2] per group
    BAR_K2_FULL = BAR_A_FULL + 2,
    BAR_W_FULL = BAR_K2_FULL + 2,        // [2] per group
    BAR_W_EMPTY = BAR_W_FULL + 2,        // [2] per group
    BAR_S_FULL = BAR_W_EMPTY + 2,        // [4] group * 2 + buffer
    BAR_P_FULL = BAR_S_FULL + 4,         // [4]
    BAR_PV_DONE = BAR_P_FULL + 4,        // [4]
    BAR_A_FREE = BAR_PV_DONE + 4,        // [2] per group: every S product of the sweep has completed
    BAR_REF_FULL = BAR_A_FREE + 2,       // [2] per group: the sweep's final reference is in shared memory
    BAR_COUNT = BAR_REF_FULL + 2
};

// error bits reported through the device status word
enum { ERR_FWD_PRODUCER = 1, ERR_FWD_MMA = 2, ERR_FWD_SOFTMAX = 4, ERR_FWD_OUTPUT = 8 };

struct FwdParams {
    KernelParams kp;
    int nt;          // tiles per query tile: ceil((w1 + 127) / 128), <= MAX_NT
    float c;         // scale * log2(e)
    int *status;     // device status word
};

// per-row hand-over between a softmax thread and the output thread of its row:
// [group][sweep parity][128] final reference of the sweep, then [group][128] denominator and
// [group][128] the reference it is expressed against
constexpr int FWD_STATS_FLOATS = 2 * 2 * 128 + 2 * 128 + 2 * 128;
// at least 120 KB: one CTA per SM, so the 512-column TMEM allocation never waits for a co-resident CTA
inline size_t fwd_smem_bytes(int nt) {
    const size_t need = 1024 + (size_t)nt * 2 * TILE_BYTES + 2 * TILE_BYTES + K2_ROWS * 128 + FWD_STATS_FLOATS * 4 + 256 + 1024;
    return need > 120 * 1024 ? need : 120 * 1024;
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float lg2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162 *>(&a), *reinterpret_cast<__nv_bfloat162 *>(&b));
    return *reinterpret_cast<uint32_t *>(&r);
}

#ifndef SA2_WARP_WAIT_SLEEP
#define SA2_WARP_WAIT_SLEEP 64
#endif
// every lane of the warp waits; the result is uniform so that the .sync.aligned
// tcgen05 instructions that follow are never reached by a partial warp
__device__ __forceinline__ bool warp_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int prof = -1) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, SA2_WARP_WAIT_SLEEP, prof));
}

struct FwdGeom {
    int i0, i_last, jbase, t_first, ntiles, nsweeps;
    int upe;          // units (half tiles) per sweep
    int units[2];     // units each group processes: its sweeps x upe
};

__device__ __forceinline__ FwdGeom fwd_geom(const FwdParams &P) {
    FwdGeom g;
    g.i0 = blockIdx.x * TQ;
    g.i_last = min(g.i0 + TQ - 1, P.kp.n - 1);
    g.jbase = g.i0 + P.kp.off1 + TJ - TJ * P.nt;      // tile t covers rows jbase + 128 t ... + 127
    g.t_first = g.jbase >= 0 ? 0 : min(P.nt - 1, (-g.jbase) / TJ);
    g.ntiles = P.nt - g.t_first;
    g.nsweeps = min(P.kp.w2, g.i_last + P.kp.off2 + 1);
    g.upe = 2 * g.ntiles;
    g.units[0] = ((g.nsweeps + 1) / 2) * g.upe;
    g.units[1] = (g.nsweeps / 2) * g.upe;
    return g;
}

// ------------------------------------------------------------------ warp 0 (one lane)
__device__ __forceinline__ void fwd_producer(const FwdParams &P, const FwdGeom &g, const CUtensorMap *mapK, const CUtensorMap *mapV,
                                             const CUtensorMap *mapK2, uint8_t *sK, uint8_t *sV, uint8_t *sK2, uint64_t *bars) {
    const KernelParams &kp = P.kp;
    const int h = blockIdx.y, b = blockIdx.z, hk = h / kp.g;
    prefetch_tmap(mapK);
    prefetch_tmap(mapV);
    prefetch_tmap(mapK2);
    if (kp.w2 <= 32) {
        mbar_arrive_expect_tx(&bars[BAR_K2_FULL], K2_ROWS * 128);
        for (int bx = 0; bx < K2_ROWS / 32; ++bx)
            tma_load_4d(sK2 + bx * 4096, mapK2, &bars[BAR_K2_FULL], 0, hk, g.i0 + kp.off2 - 32 + 32 * bx, b);
    } else {
        mbar_arrive(&bars[BAR_K2_FULL]);
    }
    for (int t = P.nt - 1; t >= g.t_first; --t) {      // the diagonal tile first
        mbar_arrive_expect_tx(&bars[BAR_KV_FULL + t], 2 * TILE_BYTES);
        tma_load_4d(sK + (size_t)t * TILE_BYTES, mapK, &bars[BAR_KV_FULL + t], 0, hk, g.jbase + TJ * t, b);
        tma_load_4d(sV + (size_t)t * TILE_BYTES, mapV, &bars[BAR_KV_FULL + t], 0, hk, g.jbase + TJ * t, b);
    }
}

// ------------------------------------------------------------------ MMA issuers (one lane each)
// Lane 0 of warp 1 issues for group 0 and lane 0 of warp 0 for group 1: the two groups touch disjoint
// TMEM columns and only read shared memory, so their MMA streams need no ordering between them, and
// two issuing threads double the rate at which instructions reach the tensor cores.
// Group g's stream: unit r is half tile r % upe of the group's (r / upe)-th sweep, e = 2 (r / upe) + g.
__device__ __forceinline__ int fwd_mma(const FwdGeom &g, int grp, uint32_t tmem, uint8_t *sK, uint8_t *sV, uint8_t *sA,
                                       uint64_t *bars, volatile int *abort_flag) {
    constexpr uint32_t IDESC_S = idesc_bf16(128, 64, false, false);
    constexpr uint32_t IDESC_PV = idesc_bf16(128, 64, false, true);
    // descriptors differ only in their start-address field (units of 16 bytes): build them once
    const uint64_t dA = smem_desc_sw128(smem_u32(sA) + grp * TILE_BYTES);
    const uint64_t dK = smem_desc_sw128(smem_u32(sK));
    const uint64_t dV = smem_desc_sw128(smem_u32(sV));
    const uint32_t tS = tmem + grp * 128, tW = tmem + 256 + grp * 64, tP = tmem + 384 + grp * 64;
    const int n = g.units[grp];

    // running position of the unit whose S is issued next (s_*) and whose PV is issued next (p_*)
    int s_k = 0, s_w = 0, p_k = 0, p_w = 0;

    auto issue_s = [&](int r) -> bool {
        const int tile = g.t_first + (s_w >> 1), half = s_w & 1, sb = r & 1;
        if (s_w == 0 && !mbar_wait(&bars[BAR_A_FULL + grp], s_k & 1, abort_flag, 0, 1)) return false;
        if (s_k == 0 && half == 0 && !mbar_wait(&bars[BAR_KV_FULL + tile], 0, abort_flag)) return false;
        tc_fence_after();
        const uint64_t kt = dK + (uint64_t)((tile * TILE_BYTES + half * 8192) >> 4);
        const uint32_t d = tS + sb * 64;
        mma_ss(d, dA, kt, IDESC_S, 0u);
        mma_ss(d, dA + 2, kt + 2, IDESC_S, 1u);
        mma_ss(d, dA + 4, kt + 4, IDESC_S, 1u);
        mma_ss(d, dA + 6, kt + 6, IDESC_S, 1u);
        tc_commit(&bars[BAR_S_FULL + grp * 2 + sb]);
        if (s_w == g.upe - 1) tc_commit(&bars[BAR_A_FREE + grp]);      // the A stage may be rebuilt
        if (++s_w == g.upe) { s_w = 0; ++s_k; }
        return true;
    };
    auto issue_pv = [&](int r) -> bool {
        const int tile = g.t_first + (p_w >> 1), half = p_w & 1, sb = r & 1;
        if (!mbar_wait(&bars[BAR_P_FULL + grp * 2 + sb], (r >> 1) & 1, abort_flag, 0, 2)) return false;
        if (p_w == 0 && p_k >= 1 && !mbar_wait(&bars[BAR_W_EMPTY + grp], (p_k - 1) & 1, abort_flag, 0, 3)) return false;
        tc_fence_after();
        const uint64_t vt = dV + (uint64_t)((tile * TILE_BYTES + half * 8192) >> 4);
        const uint32_t a = tP + sb * 32;
        mma_ts(tW, a, vt, IDESC_PV, p_w > 0 ? 1u : 0u);
        mma_ts(tW, a + 8, vt + 128, IDESC_PV, 1u);
        mma_ts(tW, a + 16, vt + 256, IDESC_PV, 1u);
        mma_ts(tW, a + 24, vt + 384, IDESC_PV, 1u);
        tc_commit(&bars[BAR_PV_DONE + grp * 2 + sb]);
        if (p_w == g.upe - 1) tc_commit(&bars[BAR_W_FULL + grp]);
        if (++p_w == g.upe) { p_w = 0; ++p_k; }
        return true;
    };

    for (int r = 0; r < 2 && r < n; ++r)
        if (!issue_s(r)) return ERR_FWD_MMA;
    for (int r = 0; r < n; ++r) {
        if (!issue_pv(r)) return ERR_FWD_MMA;
        if (r + 2 < n && !issue_s(r + 2)) return ERR_FWD_MMA;
    }
    return 0;
}

// ------------------------------------------------------------------ softmax groups (warps 8-11, 12-15)
// exp2(c * s - ref) for 32 logits of one row -> 16 packed bf16 pairs; returns their sum.
// Columns outside (lo, hi] are masked (window / causality / sequence start).
__device__ __forceinline__ float fwd_probs32(const uint32_t (&s)[32], uint32_t (&pk)[16], float c, float ref,
                                             bool full, int col0, int lo, int hi) {
    float sum0 = 0.f, sum1 = 0.f;
    if (full) {
#pragma unroll
        for (int x = 0; x < 32; x += 2) {
            const float p0 = ex2(fmaf(__uint_as_float(s[x]), c, -ref));
            const float p1 = ex2(fmaf(__uint_as_float(s[x + 1]), c, -ref));
            sum0 += p0; sum1 += p1;
            pk[x >> 1] = pack_bf16(p0, p1);
        }
    } else {
        // Valid columns are the integers in (lo, hi]: |col - mid| <= half, and an invalid column is at least
        // half + 1 away, so saturate(half + 1 - |col - mid|) is exactly 1 or 0: two FADDs and an FMUL on the
        // FMA pipe instead of two compares and a select on the (half as wide) ALU pipe.  The exponent is
        // clamped so that a masked-out logit far above the reference cannot produce inf * 0; a clamped
        // valid logit still trips the slow path.
        const float mid = 0.5f * (float)(lo + 1 + hi), hwp = 0.5f * (float)(hi - lo - 1) + 1.f;
#pragma unroll
        for (int x = 0; x < 32; x += 2) {
            const float v0 = __saturatef(hwp - fabsf((float)(col0 + x) - mid));
            const float v1 = __saturatef(hwp - fabsf((float)(col0 + x + 1) - mid));
            const float p0 = ex2(fminf(fmaf(__uint_as_float(s[x]), c, -ref), 100.f)) * v0;
            const float p1 = ex2(fminf(fmaf(__uint_as_float(s[x + 1]), c, -ref), 100.f)) * v1;
            sum0 += p0; sum1 += p1;
            pk[x >> 1] = pack_bf16(p0, p1);
        }
    }
    return sum0 + sum1;
}

__device__ __forceinline__ int fwd_softmax(const FwdParams &P, const FwdGeom &g, int grp, uint32_t tmem, float *stats,
                                           uint64_t *bars, volatile int *abort_flag) {
    const KernelParams &kp = P.kp;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = (warp & 3) * 32 + lane;            // query row within the tile = TMEM lane
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t s_addr = lane_addr + grp * 128, p_addr = lane_addr + 384 + grp * 64, w_addr = lane_addr + 256 + grp * 64;
    const int i = g.i0 + r;
    const bool row_ok = i < kp.n;
    const float c = P.c;
    const int nsw = grp == 0 ? (g.nsweeps + 1) / 2 : g.nsweeps / 2;
    float *ref_slot = stats + grp * 256 + r;          // + 128 * (sweep parity)

    float ref = -CUDART_INF_F, l = 0.f;

    for (int k = 0; k < nsw; ++k) {
        const int e = 2 * k + grp;
        const bool sweep_ok = row_ok && (i + kp.off2 - e >= 0);
#pragma unroll 1
        for (int w = 0; w < g.upe; ++w) {
            const int u = k * g.upe + w, sb = u & 1;
            const int j0 = g.jbase + TJ * (g.t_first + (w >> 1)) + 64 * (w & 1);
            // valid columns of this row: lo < col <= hi
            const int d1 = i + kp.off1 - j0;
            const int hi = sweep_ok ? min(d1, 63) : -1;
            const int lo = max(d1 - kp.w1, -j0 - 1);
            if (!warp_wait(&bars[BAR_S_FULL + grp * 2 + sb], (u >> 1) & 1, abort_flag, 1)) return ERR_FWD_SOFTMAX;
            tc_fence_after();
            const bool full = __all_sync(0xffffffffu, lo < 0 && hi >= 63);

            float tile_sum = 0.f;
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
                uint32_t s[32], pk[16];
                tmem_ld32(s_addr + sb * 64 + ch * 32, s);
                tmem_wait_ld();
                tile_sum += fwd_probs32(s, pk, c, ref, full, ch * 32, lo, hi);
                tmem_st16(p_addr + sb * 32 + ch * 16, pk);
            }
            const bool exceed = !(tile_sum <= 1.8446744e19f);       // above 2^64, inf or NaN
            if (__any_sync(0xffffffffu, exceed)) {
                // ---- slow path (whole warp): exact maximum of this unit, rescale, recompute
                float mx = -CUDART_INF_F;
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    uint32_t s[32];
                    tmem_ld32(s_addr + sb * 64 + ch * 32, s);
                    tmem_wait_ld();
#pragma unroll
                    for (int x = 0; x < 32; ++x) {
                        const int col = ch * 32 + x;
                        if (col > lo && col <= hi) mx = fmaxf(mx, __uint_as_float(s[x]));
                    }
                }
                float f = 1.f;
                if (exceed) {
                    const float nref = mx * c;
                    f = ex2(ref - nref);                       // 0 when ref was -inf
                    l *= f;
                    ref = nref;     // the output thread rescales its accumulator when it sees the new reference
                }
                if (w > 0) {
                    // W of this sweep already holds partial sums against the old reference
                    const int up = u - 1;
                    if (!warp_wait(&bars[BAR_PV_DONE + grp * 2 + (up & 1)], (up >> 1) & 1, abort_flag)) return ERR_FWD_SOFTMAX;
                    tc_fence_after();
#pragma unroll 1
                    for (int half = 0; half < 2; ++half) {
                        uint32_t wv[32];
                        tmem_ld32(w_addr + half * 32, wv);
                        tmem_wait_ld();
#pragma unroll
                        for (int x = 0; x < 32; ++x) wv[x] = __float_as_uint(__uint_as_float(wv[x]) * f);
                        tmem_st32(w_addr + half * 32, wv);
                    }
                }
                tile_sum = 0.f;
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    uint32_t s[32], pk[16];
                    tmem_ld32(s_addr + sb * 64 + ch * 32, s);
                    tmem_wait_ld();
                    tile_sum += fwd_probs32(s, pk, c, ref, false, ch * 32, lo, hi);
                    tmem_st16(p_addr + sb * 32 + ch * 16, pk);
                }
            }
            l += tile_sum;
            tmem_wait_st();
            if (w == g.upe - 1) {
                // W_e is expressed against the reference the row has now.  The output thread has read the
                // slot of sweep k - 2 before it released that sweep's W; waiting for the release of sweep
                // k - 1 also keeps this barrier from running two phases ahead of its reader.
                if (k >= 1 && !warp_wait(&bars[BAR_W_EMPTY + grp], (k - 1) & 1, abort_flag)) return ERR_FWD_SOFTMAX;
                ref_slot[(k & 1) * 128] = ref;
                mbar_arrive(&bars[BAR_REF_FULL + grp]);
            }
            tc_fence_before();
            mbar_arrive(&bars[BAR_P_FULL + grp * 2 + sb]);
        }
    }
    stats[512 + grp * 128 + r] = l;
    stats[768 + grp * 128 + r] = ref;
    return 0;
}

// ------------------------------------------------------------------ output group (warps 4-7)
// Thread r owns query row r: it builds row r of every A tile and accumulates the row's output, one
// accumulator per softmax group, each against the reference that group reported with its last sweep.
__device__ __forceinline__ int fwd_output(const FwdParams &P, const FwdGeom &g, uint32_t tmem, float (&o0)[64], float (&o1)[64],
                                          float &ref0, float &ref1, uint8_t *sA, const uint8_t *sK2, const float *stats,
                                          uint64_t *bars, volatile int *abort_flag) {
    const KernelParams &kp = P.kp;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const int h = blockIdx.y, b = blockIdx.z, hk = h / kp.g;
    const int i = g.i0 + r;
    const bool row_ok = i < kp.n;
    const __nv_bfloat16 *k2 = reinterpret_cast<const __nv_bfloat16 *>(kp.k2.p);
    const __nv_bfloat16 *v2 = reinterpret_cast<const __nv_bfloat16 *>(kp.v2.p);
    const bool k2_in_smem = kp.w2 <= 32;
    const int nsw0 = (g.nsweeps + 1) / 2, nsw1 = g.nsweeps / 2;

    uint4 qv[8];
#pragma unroll
    for (int cc = 0; cc < 8; ++cc) qv[cc] = make_uint4(0u, 0u, 0u, 0u);
    if (row_ok) {
        const __nv_bfloat16 *qrow = reinterpret_cast<const __nv_bfloat16 *>(kp.q.p) + elem_off(kp.q, b, i, h);
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) qv[cc] = __ldg(reinterpret_cast<const uint4 *>(qrow + cc * 8));
    }

    // row r of A_e = q_i * k2_{i-e} for sweep e = 2 k + grp, into the group's A stage
    auto build_a = [&](int grp, int k) {
        const int e = 2 * k + grp;
        uint8_t *dst = sA + (size_t)grp * TILE_BYTES;
        const int kk = i + kp.off2 - e;
        const bool ok = row_ok && kk >= 0;
        const __nv_bfloat16 *krow = k2 + elem_off(kp.k2, b, ok ? kk : 0, hk);
        // all eight loads first, then the products and stores
        uint4 kv[8];
#pragma unroll
        for (int cc = 0; cc < 8; ++cc)
            kv[cc] = !ok ? make_uint4(0u, 0u, 0u, 0u)
                         : k2_in_smem ? *reinterpret_cast<const uint4 *>(sK2 + sw128_offset(r + 32 - e, cc))
                                      : __ldg(reinterpret_cast<const uint4 *>(krow + cc * 8));
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
            uint4 v;
            v.x = mul_bf16x2(qv[cc].x, kv[cc].x); v.y = mul_bf16x2(qv[cc].y, kv[cc].y);
            v.z = mul_bf16x2(qv[cc].z, kv[cc].z); v.w = mul_bf16x2(qv[cc].w, kv[cc].w);
            *reinterpret_cast<uint4 *>(dst + sw128_offset(r, cc)) = v;
        }
        fence_proxy_async_smem();
        mbar_arrive(&bars[BAR_A_FULL + grp]);
    };

    // o += v2_{i-e} * W_e (TMEM), after moving o to the reference W_e was built against
    auto drain = [&](int grp, int k, float (&o)[64], float &ref_o) -> bool {
        if (!warp_wait(&bars[BAR_REF_FULL + grp], k & 1, abort_flag, 2)) return false;
        const float ref_w = stats[grp * 256 + (k & 1) * 128 + r];
        if (!warp_wait(&bars[BAR_W_FULL + grp], k & 1, abort_flag, 3)) return false;
        tc_fence_after();
        const int kk = i + kp.off2 - (2 * k + grp);
        const bool ok = row_ok && kk >= 0 && ref_w > -CUDART_INF_F;
        if (ok && ref_w > ref_o) {
            const float f = ex2(ref_o - ref_w);              // 0 while the accumulator is still empty
#pragma unroll
            for (int x = 0; x < 64; ++x) o[x] *= f;
            ref_o = ref_w;
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            uint32_t w[32];
            tmem_ld32(lane_addr + 256 + grp * 64 + half * 32, w);
            tmem_wait_ld();
            if (ok) {
                const __nv_bfloat16 *vp = v2 + elem_off(kp.v2, b, kk, hk) + half * 32;
                uint4 raw[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) raw[u] = __ldg(reinterpret_cast<const uint4 *>(vp + u * 8));
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t rr[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
                    for (int z = 0; z < 4; ++z) {
                        const __nv_bfloat162 vv = *reinterpret_cast<const __nv_bfloat162 *>(&rr[z]);
                        const int x = half * 32 + u * 8 + z * 2;
                        o[x] = fmaf(__uint_as_float(w[u * 8 + z * 2]), __low2float(vv), o[x]);
                        o[x + 1] = fmaf(__uint_as_float(w[u * 8 + z * 2 + 1]), __high2float(vv), o[x + 1]);
                    }
                }
            }
        }
        tc_fence_before();
        mbar_arrive(&bars[BAR_W_EMPTY + grp]);
        return true;
    };

    if (!warp_wait(&bars[BAR_K2_FULL], 0, abort_flag)) return ERR_FWD_OUTPUT;
    if (nsw0 > 0) build_a(0, 0);
    if (nsw1 > 0) build_a(1, 0);
    for (int k = 0; k < nsw0; ++k) {
        // the A stages first: the tensor cores wait for them, the W accumulators have a unit's slack
        if (k + 1 < nsw0) {
            if (!warp_wait(&bars[BAR_A_FREE + 0], k & 1, abort_flag, 1)) return ERR_FWD_OUTPUT;
            build_a(0, k + 1);
        }
        if (k + 1 < nsw1) {
            if (!warp_wait(&bars[BAR_A_FREE + 1], k & 1, abort_flag, 1)) return ERR_FWD_OUTPUT;
            build_a(1, k + 1);
        }
        if (!drain(0, k, o0, ref0)) return ERR_FWD_OUTPUT;
        if (k < nsw1 && !drain(1, k, o1, ref1)) return ERR_FWD_OUTPUT;
    }
    return 0;
}

__device__ __forceinline__ void fwd_rows_sync() { asm volatile("bar.sync 2, 384;" ::: "memory"); }

__global__ void __launch_bounds__(FWD_THREADS, 1)
fwd_kernel(const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
           const __grid_constant__ CUtensorMap mapK2, const FwdParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sK = smem;
    uint8_t *sV = sK + (size_t)P.nt * TILE_BYTES;
    uint8_t *sA = sV + (size_t)P.nt * TILE_BYTES;
    uint8_t *sK2 = sA + 2 * TILE_BYTES;
    float *stats = reinterpret_cast<float *>(sK2 + K2_ROWS * 128);
    uint64_t *bars = reinterpret_cast<uint64_t *>(stats + FWD_STATS_FLOATS);
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + BAR_COUNT);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        for (int x = 0; x < BAR_COUNT; ++x) {
            const bool many = (x >= BAR_P_FULL && x < BAR_P_FULL + 4) || (x >= BAR_W_EMPTY && x < BAR_W_EMPTY + 2) ||
                              (x >= BAR_A_FULL && x < BAR_A_FULL + 2) || (x >= BAR_REF_FULL && x < BAR_REF_FULL + 2);
            mbar_init(&bars[x], many ? 128u : 1u);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_holder, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_holder;
    const FwdGeom g = fwd_geom(P);

    int err = 0;
#ifdef SA2_PROF
    const long long prof_t0 = clock64();
    sa2::sm100::prof_begin();
#endif
    if (warp < 4) {
        reg_dealloc<FWD_REGS_ISSUE>();                // one instruction for the whole warpgroup
        if ((threadIdx.x & 31) == 0) {
            if (warp == 0) {
                fwd_producer(P, g, &mapK, &mapV, &mapK2, sK, sV, sK2, bars);
                err = fwd_mma(g, 1, tmem, sK, sV, sA, bars, abort_flag);
            } else if (warp == 1) {
                err = fwd_mma(g, 0, tmem, sK, sV, sA, bars, abort_flag);
            }
        }
        __syncwarp();
    } else if (warp >= 8) {
        reg_dealloc<FWD_REGS_SOFTMAX>();
        err = fwd_softmax(P, g, (warp - 8) >> 2, tmem, stats, bars, abort_flag);
        // the barrier sits outside fwd_softmax so that a group that gave up still reaches it
        fwd_rows_sync();
    } else {
        reg_alloc<FWD_REGS_OUT>();
        float o0[64], o1[64];
#pragma unroll
        for (int x = 0; x < 64; ++x) { o0[x] = 0.f; o1[x] = 0.f; }
        float ref0 = -CUDART_INF_F, ref1 = -CUDART_INF_F;
        err = fwd_output(P, g, tmem, o0, o1, ref0, ref1, sA, sK2, stats, bars, abort_flag);
        fwd_rows_sync();                              // both groups' denominators are in shared memory

        // merge the two groups' states: each accumulator is expressed against its group's last reference
        const KernelParams &kp = P.kp;
        const int r = ((warp & 3) * 32) + (threadIdx.x & 31);
        const int i = g.i0 + r;
        const float l0 = stats[512 + r], l1 = stats[640 + r];
        const float lref0 = stats[768 + r], lref1 = stats[896 + r];
        const float rmax = fmaxf(lref0, lref1);
        const float f0 = lref0 > -CUDART_INF_F ? ex2(lref0 - rmax) : 0.f;
        const float f1 = lref1 > -CUDART_INF_F ? ex2(lref1 - rmax) : 0.f;
        const float l = l0 * f0 + l1 * f1;
        if (i < kp.n) {
            // a CTA in which any wait ran out reports NaN instead of leaving its rows unwritten
            const bool bad = err != 0 || *abort_flag != 0;
            // an accumulator that last saw an older reference than its group's final one is moved to it
            const float inv = bad ? CUDART_NAN_F : 1.f / l;
            const float s0 = ref0 > -CUDART_INF_F ? ex2(ref0 - rmax) * inv : (bad ? inv : 0.f);
            const float s1 = ref1 > -CUDART_INF_F ? ex2(ref1 - rmax) * inv : (bad ? inv : 0.f);
            __nv_bfloat16 *op = reinterpret_cast<__nv_bfloat16 *>(kp.out.p) + elem_off(kp.out, blockIdx.z, i, blockIdx.y);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                uint4 v;
                v.x = pack_bf16(o0[u * 8 + 0] * s0 + o1[u * 8 + 0] * s1, o0[u * 8 + 1] * s0 + o1[u * 8 + 1] * s1);
                v.y = pack_bf16(o0[u * 8 + 2] * s0 + o1[u * 8 + 2] * s1, o0[u * 8 + 3] * s0 + o1[u * 8 + 3] * s1);
                v.z = pack_bf16(o0[u * 8 + 4] * s0 + o1[u * 8 + 4] * s1, o0[u * 8 + 5] * s0 + o1[u * 8 + 5] * s1);
                v.w = pack_bf16(o0[u * 8 + 6] * s0 + o1[u * 8 + 6] * s1, o0[u * 8 + 7] * s0 + o1[u * 8 + 7] * s1);
                *reinterpret_cast<uint4 *>(op + u * 8) = v;
            }
            kp.lse[((int64_t)blockIdx.z * kp.hq + blockIdx.y) * kp.n + i] = bad ? CUDART_NAN_F : (rmax + lg2(l)) * 0.6931471805599453f;
        }
    }
    if (err) atomicOr(P.status, err);
    SA2_PROF_ADD(0, clock64() - prof_t0);
    SA2_PROF_END();

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace tc
}  // namespace sa2
