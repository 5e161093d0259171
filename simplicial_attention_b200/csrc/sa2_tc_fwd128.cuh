// Forward kernel on the 5th-generation tensor cores (tcgen05 + TMEM + TMA),
// bf16 operands, fp32 accumulation, head dim 128.
//
// Same formulation as the head-dim-64 kernel (sa2_tc_fwd.cuh): a CTA owns 128
// query rows of one (batch, query head); per offset e = i - k ("sweep") it forms
// A_e[i,:] = q_i * k2_{i-e}, S = A_e K1^T per 64-key unit, P = exp2(c S - ref),
// W_e += P V1, and at the end of the sweep the row owner adds v2_{i-e} * W_e to
// its output registers.  Two softmax groups own the even and the odd sweeps.
//
// What head dim 128 changes:
//   * A K1/V1 window of 640 rows is 320 KB and does not fit in shared memory,
//     so its 64-row units stream through two TMA rings (four K1 units, four V1
//     units) once per pair of sweeps: the two softmax groups walk the window in
//     the same order, and a ring slot is refilled when both groups' products on
//     it have completed.  The units come from L2 (the windows of the query tiles
//     in flight overlap almost entirely); A_e is built and W_e folded once per
//     sweep, as in the head-dim-64 kernel.
//   * Every operand row is 256 bytes: tiles are stored as two 64-channel blocks
//     of 128-byte swizzled rows.  S runs eight K=16 steps over the two blocks;
//     W_e += P V1 uses the V1 unit as one MN-major B operand of N = 128 (the
//     two channel blocks are the descriptor's leading-dimension blocks).
//   * W_e is 128 TMEM columns per group, so P (bf16) is written over the S
//     columns it was computed from: S/P 4 x 64 columns, W 2 x 128 = 512.  A
//     unit's S is read completely before its P is stored, and the next S into
//     a buffer is issued only after the product that read P from it has
//     completed.
//   * The output accumulator of a row is 128 fp32 values: two threads per row
//     (one per 64-channel block, in two warpgroups) keep ONE accumulator each,
//     held against the larger of the references the two softmax groups have
//     reported; a sweep whose reference is lower is scaled down while it is
//     folded in.
//
// Warps (768 threads, six aligned warpgroups):
//   0, 1   lane 0 issues the S products of group 0 / group 1 (warp 1 owns the TMEM allocation)
//   2, 3   lane 0 issues the P V1 products of group 0 / group 1.  A thread issues one tcgen05
//          instruction per 60-130 cycles and a unit takes 12 products and 6 commits, so with one
//          issuing thread per group the issue itself (~3900 cycles per unit) paced the kernel.
//   4-7    output threads of channel block 0, one per query row
//   8-11   output threads of channel block 1
//   12-15  softmax group 0 (even sweeps), 16-19 softmax group 1 (odd sweeps)
//   20, 21 lane 0 is the TMA producer of the K1 ring / of the V1 ring; 22-23 idle
#pragma once
#include "sa2_tc_fwd.cuh"

namespace sa2 {
namespace tc {
namespace f128 {

constexpr int THREADS = 768;
// 768 threads start with 80 registers each; every warpgroup executes one setmaxnreg, and the budgets must add
// up to at most 6 * 80 or the growing groups never return from theirs.
constexpr int REGS_LAUNCH = 80, REGS_ISSUE = 56, REGS_OUT = 128, REGS_SOFTMAX = 72, REGS_PRODUCE = 24;
static_assert(REGS_ISSUE + 2 * REGS_OUT + 2 * REGS_SOFTMAX + REGS_PRODUCE <= 6 * REGS_LAUNCH, "register pool must balance");
static_assert(REGS_ISSUE <= REGS_LAUNCH && REGS_SOFTMAX <= REGS_LAUNCH && REGS_PRODUCE <= REGS_LAUNCH && REGS_OUT >= REGS_LAUNCH,
              "issuers, softmax groups and producers release registers, the output groups take them");

constexpr int UNIT = 64;                          // first-key rows per unit
constexpr int SLOTS = 4;                          // slots of the K1 ring and of the V1 ring
constexpr uint32_t BLK_BYTES = UNIT * 128;        // one [64 rows][64 channels] swizzled block
constexpr uint32_t UNIT_BYTES = 2 * BLK_BYTES;    // a unit of K1 or V1: channel block 0, channel block 1
constexpr uint32_t ABLK_BYTES = TQ * 128;         // one [128 rows][64 channels] block of an A tile
constexpr uint32_t A_BYTES = 2 * ABLK_BYTES;

enum Bar {
    B_K_FULL = 0,                   // [SLOTS]
    B_K_EMPTY = B_K_FULL + SLOTS,   // [SLOTS] both groups' S products on the slot have completed
    B_V_FULL = B_K_EMPTY + SLOTS,   // [SLOTS]
    B_V_EMPTY = B_V_FULL + SLOTS,   // [SLOTS] both groups' P V1 products on the slot have completed
    B_A_FULL = B_V_EMPTY + SLOTS,   // [2] per group
    B_A_FREE = B_A_FULL + 2,        // [2]
    B_W_FULL = B_A_FREE + 2,        // [2]
    B_W_EMPTY = B_W_FULL + 2,       // [2]
    B_REF_FULL = B_W_EMPTY + 2,     // [2]
    B_S_FULL = B_REF_FULL + 2,      // [4] group * 2 + buffer
    B_P_FULL = B_S_FULL + 4,        // [4]
    B_PV_DONE = B_P_FULL + 4,       // [4]
    B_COUNT = B_PV_DONE + 4
};

struct Params {
    KernelParams kp;
    int nh;          // 64-row units per query tile: ceil((w1 + 127) / 64)
    float c;         // scale * log2(e)
    int pv_split;    // diagnostic: issue W += P V1 as two N = 64 products instead of one N = 128
    int *status;
};

inline size_t smem_bytes() {
    return 1024 + (size_t)2 * SLOTS * UNIT_BYTES + 2 * A_BYTES + FWD_STATS_FLOATS * 4 + B_COUNT * 8 + 64;
}

struct Geom {
    int i0, i_last, hbase, h_first, nunits, nsweeps;
    int nsw[2];       // sweeps of each softmax group
};

__device__ __forceinline__ Geom geom(const Params &P) {
    Geom g;
    g.i0 = blockIdx.x * TQ;
    g.i_last = min(g.i0 + TQ - 1, P.kp.n - 1);
    g.hbase = g.i0 + P.kp.off1 + TQ - UNIT * P.nh;        // unit x covers rows hbase + 64 x ... + 63
    g.h_first = g.hbase >= 0 ? 0 : min(P.nh - 1, (-g.hbase) / UNIT);
    g.nunits = P.nh - g.h_first;
    g.nsweeps = min(P.kp.w2, g.i_last + P.kp.off2 + 1);
    g.nsw[0] = (g.nsweeps + 1) / 2;
    g.nsw[1] = g.nsweeps / 2;
    return g;
}

// ------------------------------------------------------------------ TMA producers (warps 2 and 3, one lane each)
// Item x = (pair of sweeps x / nunits, unit x % nunits) goes to slot x % SLOTS; the walk is the one of
// group 0, which has at least as many sweeps as group 1.
__device__ __forceinline__ int producer(const Params &P, const Geom &g, const CUtensorMap *map, uint8_t *ring, int full0, int empty0,
                                        uint64_t *bars, volatile int *abort_flag) {
    const int hk = blockIdx.y / P.kp.g, b = blockIdx.z;
    prefetch_tmap(map);
    const int items = g.nsw[0] * g.nunits;
    int w = 0;
    for (int x = 0; x < items; ++x) {
        const int slot = x % SLOTS;
        if (x >= SLOTS && !mbar_wait(&bars[empty0 + slot], (x / SLOTS - 1) & 1, abort_flag, 32, 1)) return ERR_FWD_PRODUCER;
        const int row = g.hbase + UNIT * (g.h_first + w);
        mbar_arrive_expect_tx(&bars[full0 + slot], UNIT_BYTES);
        tma_load_4d(ring + slot * UNIT_BYTES, map, &bars[full0 + slot], 0, hk, row, b);
        tma_load_4d(ring + slot * UNIT_BYTES + BLK_BYTES, map, &bars[full0 + slot], 64, hk, row, b);
        if (++w == g.nunits) w = 0;
    }
    // every load must have landed before the CTA may exit, even if the consumers gave up
    for (int x = max(0, items - SLOTS); x < items; ++x)
        if (!mbar_wait(&bars[full0 + x % SLOTS], (x / SLOTS) & 1, abort_flag, 32)) return ERR_FWD_PRODUCER;
    return 0;
}

// ------------------------------------------------------------------ MMA issuers (two lanes per group)
// Group g's units: unit r is unit r % nunits of the group's (r / nunits)-th sweep, e = 2 (r / nunits) + g,
// in ring slot r % SLOTS.  Buffer r & 1 of the group holds S, then P, of unit r.  The S products and the
// P V1 products of a group are issued by two threads; everything that orders them goes through barriers.
__device__ __forceinline__ int issue_s(const Params &P, const Geom &g, int grp, uint32_t tmem, uint8_t *sK, uint8_t *sA,
                                       uint64_t *bars, volatile int *abort_flag) {
    constexpr uint32_t IDESC_S = idesc_bf16(128, 64, false, false);
    const uint64_t dA = smem_desc_sw128(smem_u32(sA) + grp * A_BYTES);
    const uint64_t dK = smem_desc_sw128(smem_u32(sK));
    const uint32_t tS = tmem + grp * 128;
    const int nu = g.nunits;
    const int n = g.nsw[grp] * nu;
    int w = 0, ks = 0;
    for (int u = 0; u < n; ++u) {
        const int sb = u & 1, slot = u % SLOTS;
        if (w == 0 && !mbar_wait(&bars[B_A_FULL + grp], ks & 1, abort_flag, 0, 1)) return ERR_FWD_MMA;
        if (!mbar_wait(&bars[B_K_FULL + slot], (u / SLOTS) & 1, abort_flag, 0, 2)) return ERR_FWD_MMA;
        // P of the unit that used this buffer last must have been consumed: S overwrites it
        if (u >= 2 && !mbar_wait(&bars[B_PV_DONE + grp * 2 + sb], ((u - 2) >> 1) & 1, abort_flag, 0, 3)) return ERR_FWD_MMA;
        tc_fence_after();
        const uint64_t kt = dK + (uint64_t)((slot * UNIT_BYTES) >> 4);
        const uint32_t d = tS + sb * 64;
#pragma unroll
        for (int st = 0; st < 8; ++st) {
            const uint64_t a = dA + (uint64_t)(((st >> 2) * ABLK_BYTES) >> 4) + (uint64_t)((st & 3) * 2);
            const uint64_t k = kt + (uint64_t)(((st >> 2) * BLK_BYTES) >> 4) + (uint64_t)((st & 3) * 2);
            mma_ss(d, a, k, IDESC_S, st > 0 ? 1u : 0u);
        }
        tc_commit(&bars[B_S_FULL + grp * 2 + sb]);
        tc_commit(&bars[B_K_EMPTY + slot]);
        if (w == nu - 1) tc_commit(&bars[B_A_FREE + grp]);      // the A stage may be rebuilt
        if (++w == nu) { w = 0; ++ks; }
    }
    // The rings follow group 0's walk.  With an odd number of sweeps group 1 has one sweep less: it lets the
    // units of that last sweep pass, so that every slot still collects two releases.
    for (int x = n; x < g.nsw[0] * nu; ++x) {
        const int slot = x % SLOTS;
        if (!mbar_wait(&bars[B_K_FULL + slot], (x / SLOTS) & 1, abort_flag, 32)) return ERR_FWD_MMA;
        mbar_arrive(&bars[B_K_EMPTY + slot]);
    }
    return 0;
}

__device__ __forceinline__ int issue_pv(const Params &P, const Geom &g, int grp, uint32_t tmem, uint8_t *sV,
                                        uint64_t *bars, volatile int *abort_flag) {
    constexpr uint32_t IDESC_PV = idesc_bf16(128, 128, false, true);
    constexpr uint32_t IDESC_PV64 = idesc_bf16(128, 64, false, true);
    const uint64_t dV = smem_desc_sw128(smem_u32(sV), 1024, BLK_BYTES);     // N = 128: channel blocks 8 KB apart
    const uint32_t tS = tmem + grp * 128, tW = tmem + 256 + grp * 128;
    const int nu = g.nunits;
    const int n = g.nsw[grp] * nu;
    int w = 0, ks = 0;
    for (int u = 0; u < n; ++u) {
        const int sb = u & 1, slot = u % SLOTS;
        if (!mbar_wait(&bars[B_V_FULL + slot], (u / SLOTS) & 1, abort_flag, 0, 4)) return ERR_FWD_MMA;
        if (!mbar_wait(&bars[B_P_FULL + grp * 2 + sb], (u >> 1) & 1, abort_flag, 0, 5)) return ERR_FWD_MMA;
        if (w == 0 && ks >= 1 && !mbar_wait(&bars[B_W_EMPTY + grp], (ks - 1) & 1, abort_flag, 0, 6)) return ERR_FWD_MMA;
        tc_fence_after();
        const uint32_t a = tS + sb * 64;                 // P lies over the first 32 columns of its S
        const uint64_t vt = dV + (uint64_t)((slot * UNIT_BYTES) >> 4);
        if (!P.pv_split) {
#pragma unroll
            for (int st = 0; st < 4; ++st) mma_ts(tW, a + st * 8, vt + st * 128, IDESC_PV, (w > 0 || st > 0) ? 1u : 0u);
        } else {
#pragma unroll
            for (int st = 0; st < 4; ++st) {
                mma_ts(tW, a + st * 8, vt + st * 128, IDESC_PV64, (w > 0 || st > 0) ? 1u : 0u);
                mma_ts(tW + 64, a + st * 8, vt + (BLK_BYTES >> 4) + st * 128, IDESC_PV64, (w > 0 || st > 0) ? 1u : 0u);
            }
        }
        tc_commit(&bars[B_PV_DONE + grp * 2 + sb]);
        tc_commit(&bars[B_V_EMPTY + slot]);
        if (w == nu - 1) tc_commit(&bars[B_W_FULL + grp]);
        if (++w == nu) { w = 0; ++ks; }
    }
    for (int x = n; x < g.nsw[0] * nu; ++x) {
        const int slot = x % SLOTS;
        if (!mbar_wait(&bars[B_V_FULL + slot], (x / SLOTS) & 1, abort_flag, 32)) return ERR_FWD_MMA;
        mbar_arrive(&bars[B_V_EMPTY + slot]);
    }
    return 0;
}

// ------------------------------------------------------------------ softmax groups (warps 12-15, 16-19)
__device__ __forceinline__ int softmax(const Params &P, const Geom &g, int grp, uint32_t tmem, float *stats,
                                       uint64_t *bars, volatile int *abort_flag) {
    const KernelParams &kp = P.kp;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = (warp & 3) * 32 + lane;            // query row within the tile = TMEM lane
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t s_addr = lane_addr + grp * 128, w_addr = lane_addr + 256 + grp * 128;
    const int i = g.i0 + r;
    const bool row_ok = i < kp.n;
    const float c = P.c;
    const int nsw = g.nsw[grp];
    float *ref_slot = stats + grp * 256 + r;          // + 128 * (parity of the group's sweep counter)

    float ref = -CUDART_INF_F, l = 0.f;
    int u = 0;
    const int nu = g.nunits;
    // The hand-over of a unit's P (wait for the TMEM stores, then arrive) is deferred until the first load of
    // the next unit has been issued, so that the store latency passes under that load.
    int pending = -1;
    {
        for (int ks = 0; ks < nsw; ++ks) {
            const int e = 2 * ks + grp;
            const bool sweep_ok = row_ok && (i + kp.off2 - e >= 0);
#pragma unroll 1
            for (int w = 0; w < nu; ++w, ++u) {
                const int sb = u & 1;
                const int j0 = g.hbase + UNIT * (g.h_first + w);
                // valid columns of this row: lo < col <= hi
                const int d1 = i + kp.off1 - j0;
                const int hi = sweep_ok ? min(d1, 63) : -1;
                const int lo = max(d1 - kp.w1, -j0 - 1);
                if (!warp_wait(&bars[B_S_FULL + grp * 2 + sb], (u >> 1) & 1, abort_flag, 1)) return ERR_FWD_SOFTMAX;
                tc_fence_after();
                const bool full = __all_sync(0xffffffffu, lo < 0 && hi >= 63);
                const uint32_t buf = s_addr + sb * 64;

                // the whole unit is read before any P is stored: P lies over the S columns
                uint32_t s[32], pk0[16], pk1[16];
                tmem_ld32(buf, s);
                if (pending >= 0) {
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(&bars[B_P_FULL + grp * 2 + pending]);
                    pending = -1;
                }
                tmem_wait_ld();
                float tile_sum = fwd_probs32(s, pk0, c, ref, full, 0, lo, hi);
                tmem_ld32(buf + 32, s);
                tmem_wait_ld();
                tile_sum += fwd_probs32(s, pk1, c, ref, full, 32, lo, hi);
                const bool exceed = !(tile_sum <= 1.8446744e19f);       // above 2^64, inf or NaN
                if (__any_sync(0xffffffffu, exceed)) {
                    // ---- slow path (whole warp): exact maximum of this unit, rescale, recompute
                    float mx = -CUDART_INF_F;
#pragma unroll 1
                    for (int ch = 0; ch < 2; ++ch) {
                        tmem_ld32(buf + ch * 32, s);
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
                        ref = nref;
                    }
                    if (w > 0) {
                        // W of this sweep already holds partial sums against the old reference
                        const int up = u - 1;
                        if (!warp_wait(&bars[B_PV_DONE + grp * 2 + (up & 1)], (up >> 1) & 1, abort_flag)) return ERR_FWD_SOFTMAX;
                        tc_fence_after();
#pragma unroll 1
                        for (int q4 = 0; q4 < 4; ++q4) {
                            tmem_ld32(w_addr + q4 * 32, s);
                            tmem_wait_ld();
#pragma unroll
                            for (int x = 0; x < 32; ++x) s[x] = __float_as_uint(__uint_as_float(s[x]) * f);
                            tmem_st32(w_addr + q4 * 32, s);
                        }
                    }
                    tmem_ld32(buf, s);
                    tmem_wait_ld();
                    tile_sum = fwd_probs32(s, pk0, c, ref, false, 0, lo, hi);
                    tmem_ld32(buf + 32, s);
                    tmem_wait_ld();
                    tile_sum += fwd_probs32(s, pk1, c, ref, false, 32, lo, hi);
                }
                l += tile_sum;
                tmem_st16(buf, pk0);
                tmem_st16(buf + 16, pk1);
                pending = sb;
                if (w == nu - 1) {
                    // W of this sweep is expressed against the reference the row has now.  The output
                    // threads have read the slot of two sweeps ago before they released that sweep's W;
                    // waiting for the release of the previous one also keeps this barrier from running two
                    // phases ahead of its readers.
                    if (ks >= 1 && !warp_wait(&bars[B_W_EMPTY + grp], (ks - 1) & 1, abort_flag, 2)) return ERR_FWD_SOFTMAX;
                    ref_slot[(ks & 1) * 128] = ref;
                    mbar_arrive(&bars[B_REF_FULL + grp]);
                }
            }
        }
    }
    if (pending >= 0) {
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&bars[B_P_FULL + grp * 2 + pending]);
    }
    stats[512 + grp * 128 + r] = l;
    stats[768 + grp * 128 + r] = ref;
    return 0;
}

// ------------------------------------------------------------------ output threads (warps 4-7: channels 0-63, 8-11: 64-127)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}

__device__ __forceinline__ int output(const Params &P, const Geom &g, int cb, uint32_t tmem, float (&o)[64], float &ref_o,
                                      uint8_t *sA, const float *stats, uint64_t *bars, volatile int *abort_flag) {
    const KernelParams &kp = P.kp;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const int h = blockIdx.y, b = blockIdx.z, hk = h / kp.g;
    const int i = g.i0 + r;
    const bool row_ok = i < kp.n;
    const __nv_bfloat16 *k2 = reinterpret_cast<const __nv_bfloat16 *>(kp.k2.p);
    const __nv_bfloat16 *v2 = reinterpret_cast<const __nv_bfloat16 *>(kp.v2.p);
    const __nv_bfloat16 *qrow = reinterpret_cast<const __nv_bfloat16 *>(kp.q.p) + elem_off(kp.q, b, row_ok ? i : 0, h) + cb * 64;
    const int T0 = g.nsw[0], T1 = g.nsw[1];

    // This thread's half of row r of A_e = q_i * k2_{i-e}, e = 2 t + grp, into the group's A stage.  The
    // loads of the first 32 channels are issued before the wait for the stage (`bar`, unless null), so
    // that their latency passes while the tensor cores still read the previous A_e.
    auto build_a = [&](int grp, int t, uint64_t *bar, uint32_t parity) -> bool {
        const int e = 2 * t + grp;
        uint8_t *dst = sA + (size_t)grp * A_BYTES + (size_t)cb * ABLK_BYTES;
        const int kk = i + kp.off2 - e;
        const bool ok = row_ok && kk >= 0;
        const __nv_bfloat16 *krow = k2 + elem_off(kp.k2, b, ok ? kk : 0, hk) + cb * 64;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            uint4 qv[4], kv[4];
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                qv[cc] = ok ? __ldg(reinterpret_cast<const uint4 *>(qrow + (half * 4 + cc) * 8)) : make_uint4(0u, 0u, 0u, 0u);
                kv[cc] = ok ? __ldg(reinterpret_cast<const uint4 *>(krow + (half * 4 + cc) * 8)) : make_uint4(0u, 0u, 0u, 0u);
            }
            if (half == 0 && bar && !warp_wait(bar, parity, abort_flag, 1)) return false;
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                uint4 v;
                v.x = mul_bf16x2(qv[cc].x, kv[cc].x); v.y = mul_bf16x2(qv[cc].y, kv[cc].y);
                v.z = mul_bf16x2(qv[cc].z, kv[cc].z); v.w = mul_bf16x2(qv[cc].w, kv[cc].w);
                *reinterpret_cast<uint4 *>(dst + sw128_offset(r, half * 4 + cc)) = v;
            }
        }
        fence_proxy_async_smem();
        mbar_arrive(&bars[B_A_FULL + grp]);
        return true;
    };

    // o += v2_{i-e} * W (TMEM), with o held against the larger reference seen so far; the v2 row is
    // fetched before the waits
    auto drain = [&](int grp, int t) -> bool {
        const int kk = i + kp.off2 - (2 * t + grp);
        const bool row = row_ok && kk >= 0;
        const __nv_bfloat16 *vp = v2 + elem_off(kp.v2, b, row ? kk : 0, hk) + cb * 64;
        uint4 raw[8];
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) raw[cc] = row ? __ldg(reinterpret_cast<const uint4 *>(vp + cc * 8)) : make_uint4(0u, 0u, 0u, 0u);
        if (!warp_wait(&bars[B_REF_FULL + grp], t & 1, abort_flag, 2)) return false;
        const float ref_w = stats[grp * 256 + (t & 1) * 128 + r];
        if (!warp_wait(&bars[B_W_FULL + grp], t & 1, abort_flag, 3)) return false;
        tc_fence_after();
        const bool ok = row && ref_w > -CUDART_INF_F;
        float fw = 1.f;
        if (ok) {
            if (ref_w > ref_o) {
                const float f = ex2(ref_o - ref_w);              // 0 while the accumulator is still empty
#pragma unroll
                for (int x = 0; x < 64; ++x) o[x] *= f;
                ref_o = ref_w;
            } else {
                fw = ex2(ref_w - ref_o);
            }
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t w[16];
            tmem_ld16(lane_addr + 256 + grp * 128 + cb * 64 + q4 * 16, w);
            tmem_wait_ld();
            if (ok) {
#pragma unroll
                for (int u8 = 0; u8 < 2; ++u8) {
                    const uint4 rv = raw[q4 * 2 + u8];
                    const uint32_t rr[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                    for (int z = 0; z < 4; ++z) {
                        const __nv_bfloat162 vv = *reinterpret_cast<const __nv_bfloat162 *>(&rr[z]);
                        const int x = q4 * 16 + u8 * 8 + z * 2;
                        o[x] = fmaf(__uint_as_float(w[u8 * 8 + z * 2]), __low2float(vv) * fw, o[x]);
                        o[x + 1] = fmaf(__uint_as_float(w[u8 * 8 + z * 2 + 1]), __high2float(vv) * fw, o[x + 1]);
                    }
                }
            }
        }
        tc_fence_before();
        mbar_arrive(&bars[B_W_EMPTY + grp]);
        return true;
    };

    if (T0 > 0) build_a(0, 0, nullptr, 0);
    if (T1 > 0) build_a(1, 0, nullptr, 0);
    for (int t = 0; t < T0; ++t) {
        // the A stages first: the tensor cores wait for them, the W accumulators have a unit's slack
        if (t + 1 < T0 && !build_a(0, t + 1, &bars[B_A_FREE + 0], t & 1)) return ERR_FWD_OUTPUT;
        if (t + 1 < T1 && !build_a(1, t + 1, &bars[B_A_FREE + 1], t & 1)) return ERR_FWD_OUTPUT;
        if (!drain(0, t)) return ERR_FWD_OUTPUT;
        if (t < T1 && !drain(1, t)) return ERR_FWD_OUTPUT;
    }
    return 0;
}

__device__ __forceinline__ void rows_sync() { asm volatile("bar.sync 2, 512;" ::: "memory"); }

__global__ void __launch_bounds__(THREADS, 1)
fwd128_kernel(const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV, const Params P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sK = smem;                               // K1 ring
    uint8_t *sV = sK + SLOTS * UNIT_BYTES;            // V1 ring
    uint8_t *sA = sV + SLOTS * UNIT_BYTES;
    float *stats = reinterpret_cast<float *>(sA + 2 * A_BYTES);
    uint64_t *bars = reinterpret_cast<uint64_t *>(stats + FWD_STATS_FLOATS);
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + B_COUNT);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5;
    const Geom g = geom(P);
    if (threadIdx.x == 0) {
        for (int x = 0; x < B_COUNT; ++x) {
            uint32_t count = 1;
            if ((x >= B_K_EMPTY && x < B_K_EMPTY + SLOTS) || (x >= B_V_EMPTY && x < B_V_EMPTY + SLOTS)) count = 2;   // both groups
            else if (x >= B_A_FULL && x < B_A_FULL + 2) count = 256;        // both output threads of every row
            else if (x >= B_W_EMPTY && x < B_W_EMPTY + 2) count = 256;
            else if (x >= B_REF_FULL && x < B_REF_FULL + 2) count = 128;
            else if (x >= B_P_FULL && x < B_P_FULL + 4) count = 128;
            mbar_init(&bars[x], count);
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

    int err = 0;
#ifdef SA2_PROF
    const long long prof_t0 = clock64();
    sa2::sm100::prof_begin();
#endif
    if (warp < 4) {
        reg_dealloc<REGS_ISSUE>();                    // one instruction for the whole warpgroup
        if ((threadIdx.x & 31) == 0) {
            if (warp < 2) err = issue_s(P, g, warp, tmem, sK, sA, bars, abort_flag);
            else err = issue_pv(P, g, warp - 2, tmem, sV, bars, abort_flag);
        }
        __syncwarp();
    } else if (warp >= 20) {
        reg_dealloc<REGS_PRODUCE>();
        if ((threadIdx.x & 31) == 0) {
            if (warp == 20) err = producer(P, g, &mapK, sK, B_K_FULL, B_K_EMPTY, bars, abort_flag);
            else if (warp == 21) err = producer(P, g, &mapV, sV, B_V_FULL, B_V_EMPTY, bars, abort_flag);
        }
        __syncwarp();
    } else if (warp >= 12) {
        reg_dealloc<REGS_SOFTMAX>();
        err = softmax(P, g, (warp - 12) >> 2, tmem, stats, bars, abort_flag);
        // the barrier sits outside softmax() so that a group that gave up still reaches it
        rows_sync();
    } else {
        reg_alloc<REGS_OUT>();
        const int cb = (warp - 4) >> 2;
        float o[64];
#pragma unroll
        for (int x = 0; x < 64; ++x) o[x] = 0.f;
        float ref_o = -CUDART_INF_F;
        err = output(P, g, cb, tmem, o, ref_o, sA, stats, bars, abort_flag);
        rows_sync();                                  // both groups' denominators are in shared memory

        // merge: each denominator is expressed against its group's last reference, o against ref_o
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
            const float sc = bad ? CUDART_NAN_F : (ref_o > -CUDART_INF_F ? ex2(ref_o - rmax) / l : 0.f);
            __nv_bfloat16 *op = reinterpret_cast<__nv_bfloat16 *>(kp.out.p) + elem_off(kp.out, blockIdx.z, i, blockIdx.y) + cb * 64;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                uint4 v;
                v.x = pack_bf16(o[u * 8 + 0] * sc, o[u * 8 + 1] * sc);
                v.y = pack_bf16(o[u * 8 + 2] * sc, o[u * 8 + 3] * sc);
                v.z = pack_bf16(o[u * 8 + 4] * sc, o[u * 8 + 5] * sc);
                v.w = pack_bf16(o[u * 8 + 6] * sc, o[u * 8 + 7] * sc);
                *reinterpret_cast<uint4 *>(op + u * 8) = v;
            }
            if (cb == 0)
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

}  // namespace f128
}  // namespace tc
}  // namespace sa2
