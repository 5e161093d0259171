// Backward kernel for dK1 / dV1 on tcgen05 tensor cores, head dim 128 (bf16
// operands, fp32 accumulation in TMEM).
//
// Same scheme as the head-dim-64 kernel (sa2_tc_bwd_k1.cuh): a CTA owns 128 rows
// j of K1/V1 of one (batch, kv head), resident in shared memory, and walks over
// every (query head of the group, query block, offset e) that can see them:
//     S^T = K1 A_e^T - lse2/c     dP^T = V1 B_e^T - D        (rows j, columns i)
//     P^T = exp2(c S^T)           G^T = P^T * dP^T
//     dV1 += P^T B_e              dK1 += G^T A_e
// with A_e[i,:] = q_i * k2_{i-e}, B_e[i,:] = dO_i * v2_{i-e} built by the builder
// warps and the per-query statistics added by one extra K=16 product.
//
// What head dim 128 changes:
//   * rows are 256 bytes: every tile is two 64-channel blocks of 128-byte
//     swizzled rows; the first products run eight K=16 steps over the two
//     blocks, the second products take B_e / A_e as MN-major B operands of
//     N = 128 (channel blocks = leading-dimension blocks of the descriptor);
//   * dK1 and dV1 take 2 x 128 TMEM columns, so P^T / G^T (bf16) are written
//     over the S^T / dP^T columns they were computed from, and the next first
//     products into a TMEM half wait until the second products that read it
//     are done;
//   * a step covers a block of 64 query rows (not 128), so that an (A_e, B_e)
//     stage is 32 KB and three stages, the resident K1/V1 tile (64 KB) and the
//     staged second-key window fit together (a stage is held from its build
//     through both products and the exponent pass between them, ~4800 cycles,
//     so two stages paced a step at ~2900 cycles); consecutive steps alternate
//     between the two TMEM halves and their compute groups; the constant tile
//     of ones and three slots of per-query statistics share one 16 KB tile;
//   * the k2 / v2 rows a query block pairs with over all sweeps (64 + 32 rows of
//     each) are staged once per block by TMA; four builder threads per query row
//     hold 32 channels of q_i and dO_i in registers for the whole block and form
//     each step's rows from shared memory - nothing is re-read from global
//     memory per step;
//   * 640 threads in five aligned warpgroups with register hand-over.
//
// Warps: 0 TMA producer of the K1/V1 tile, then issuer of the second products
// (dV1, dK1); 1 TMEM owner and issuer of S^T; 2 issuer of dP^T; 3 idle; 4-7
// compute group of the even steps (TMEM half 0); 8-11 compute group of the odd
// steps (half 1); 12-19 builders.
// TMEM columns: half h -> S^T / P^T [128h, +64), dP^T / G^T [128h+64, +64);
// dK1 [256, 384); dV1 [384, 512).
#pragma once
#include "sa2_tc_bwd_k1.cuh"
#include "sa2_tc_fwd128.cuh"

namespace sa2 {
namespace tc {
namespace k128 {

constexpr int THREADS = 640;
constexpr int REGS_LAUNCH = 96, REGS_ISSUE = 40, REGS_COMPUTE = 128, REGS_BUILD = 88;
static_assert(REGS_ISSUE + 2 * REGS_COMPUTE + 2 * REGS_BUILD <= 5 * REGS_LAUNCH, "register pool must balance");
constexpr int QB = 64;                            // query rows per step
constexpr int STAGES = 3;
constexpr uint32_t BLK_BYTES = TJ * 128;          // K1 / V1: one [128 rows][64 channels] swizzled block
constexpr uint32_t T_BYTES = 2 * BLK_BYTES;       // the 128-row tile of 128 channels
constexpr uint32_t QBLK_BYTES = QB * 128;         // A_e / B_e: one [64 rows][64 channels] block
constexpr uint32_t AB_BYTES = 2 * QBLK_BYTES;     // A_e (or B_e) of a step
constexpr uint32_t STAGE_BYTES = 2 * AB_BYTES;    // A_e, then B_e
constexpr int WIN_ROWS = 96;                      // staged second-key rows: positions it0 - 32 ... it0 + 63
constexpr uint32_t WBLK_BYTES = WIN_ROWS * 128;   // one [96 rows][64 channels] block of the window
constexpr uint32_t WIN_BYTES = 2 * WBLK_BYTES;    // k2 (or v2) window

enum Bar {
    B_KV_FULL = 0,
    B_AB_FULL = 1,                      // [STAGES]
    B_AB_EMPTY = B_AB_FULL + STAGES,    // [STAGES]
    B_S_FULL = B_AB_EMPTY + STAGES,     // [2] per TMEM half
    B_P_FULL = B_S_FULL + 2,            // [2]
    B_G_DONE = B_P_FULL + 2,            // [2] second products of the step have completed
    B_DONE = B_G_DONE + 2,
    B_WIN_FREE = B_DONE + 1,            // the builders have finished reading the previous block's window
    B_WIN_FULL = B_WIN_FREE + 1,
    B_COUNT = B_WIN_FULL + 1
};

// The constant tile: a [128 rows][128 bytes] swizzled tile whose 16-byte chunks 0-1 hold the key-side ones
// (rows = key rows) and whose other chunks hold three slots of query statistics (rows = query rows of a
// block): slot k < 2 has its -lse2/c slab in chunks 2-3 and its -D slab in chunks 4-5 of rows [64 k, +64);
// slot 2 has -lse2/c in chunks 6-7 of rows [0, 64) and -D in chunks 6-7 of rows [64, 128).
__device__ __forceinline__ int stat_row(int slot, int which, int r) { return slot < 2 ? 64 * slot + r : 64 * which + r; }
__device__ __forceinline__ int stat_chunk(int slot, int which) { return slot < 2 ? 2 + 2 * which : 6; }

struct Params {
    KernelParams kp;
    float c;        // scale * log2(e)
    int n_split;    // diagnostic: issue the second products as two N = 64 products instead of one N = 128
    int *status;
};

inline size_t smem_bytes() {
    return 1024 + 2 * T_BYTES + STAGES * STAGE_BYTES + TILE_BYTES + 2 * WIN_BYTES + B_COUNT * 8 + 64;
}

struct Geom {
    int j0, i_lo, i_hi, n_ib, total;
};

// sweeps of query block ib (rows i_lo + 64 ib ...)
__device__ __forceinline__ int block_sweeps(const KernelParams &kp, const Geom &g, int ib) {
    const int last = min(g.i_lo + QB * ib + QB - 1, g.i_hi);
    return min(kp.w2, last + kp.off2 + 1);
}

__device__ __forceinline__ Geom geom(const KernelParams &kp) {
    Geom g;
    g.j0 = blockIdx.x * TJ;
    g.i_lo = max(0, g.j0 - kp.off1);
    g.i_hi = min(kp.n - 1, min(g.j0 + TJ - 1, kp.nk1 - 1) + kp.w1 - 1 - kp.off1);
    g.n_ib = g.i_hi >= g.i_lo ? (g.i_hi - g.i_lo) / QB + 1 : 0;
    int per_head = 0;
    for (int ib = 0; ib < g.n_ib; ++ib) per_head += block_sweeps(kp, g, ib);
    g.total = per_head * kp.g;
    return g;
}

// ---------------------------------------------------------------- builders (warps 12-19)
// Thread (r, part): query row r of the block, channels [32 part, +32).
__device__ __forceinline__ int builder(const Params &P, const Geom &g, const CUtensorMap *mapK2, const CUtensorMap *mapV2,
                                       uint8_t *sAB, uint8_t *sConst, uint8_t *sWin,
                                       uint64_t *bars, volatile int *abort_flag) {
    const KernelParams &kp = P.kp;
    const int bt = threadIdx.x - 384;      // 0..255 among the builders
    const int r = bt & 63, part = bt >> 6;
    const int cb = part >> 1, ch0 = (part & 1) * 4;      // channel block, first 16-byte chunk within its rows
    const int hk = blockIdx.y, b = blockIdx.z;
    const __nv_bfloat16 *q = reinterpret_cast<const __nv_bfloat16 *>(kp.q.p);
    const __nv_bfloat16 *k2 = reinterpret_cast<const __nv_bfloat16 *>(kp.k2.p);
    const __nv_bfloat16 *dout = reinterpret_cast<const __nv_bfloat16 *>(kp.dout.p);
    const __nv_bfloat16 *v2 = reinterpret_cast<const __nv_bfloat16 *>(kp.v2.p);
    if (bt < 128) {
        // the key-side ones: three per row (one per term of the split statistics), then zeros up to K = 16
        *reinterpret_cast<uint4 *>(sConst + sw128_offset(bt, 0)) = make_uint4(0x3f803f80u, 0x00003f80u, 0u, 0u);
        *reinterpret_cast<uint4 *>(sConst + sw128_offset(bt, 1)) = make_uint4(0u, 0u, 0u, 0u);
    }
    const float inv_c = 1.f / P.c;
    const bool win = kp.w2 <= 32;
    int s = 0, blk = 0;
    for (int hh = 0; hh < kp.g; ++hh) {
        const int h = hk * kp.g + hh;
        for (int ib = 0; ib < g.n_ib; ++ib, ++blk) {
            const int it0 = g.i_lo + QB * ib;
            const int i = it0 + r;
            const bool iv = i <= g.i_hi;
            const int ne = block_sweeps(kp, g, ib);
            if (win) {
                // The k2 / v2 rows this query block pairs with over all sweeps (positions it0 - 32 .. it0 + 63)
                // are staged once per block by TMA; every step then reads its rows from shared memory.
                if (blk > 0) mbar_arrive(&bars[B_WIN_FREE]);
                if (bt == 0) {
                    if (blk > 0 && !mbar_wait(&bars[B_WIN_FREE], (blk - 1) & 1, abort_flag)) return ERR_BK1_BUILDER;
                    mbar_arrive_expect_tx(&bars[B_WIN_FULL], 2 * WIN_BYTES);
                    const int row0 = it0 + kp.off2 - 32;
                    for (int bx = 0; bx < WIN_ROWS / 32; ++bx)
                        for (int c2 = 0; c2 < 2; ++c2) {
                            tma_load_4d(sWin + c2 * WBLK_BYTES + bx * 4096, mapK2, &bars[B_WIN_FULL], c2 * 64, hk, row0 + 32 * bx, b);
                            tma_load_4d(sWin + WIN_BYTES + c2 * WBLK_BYTES + bx * 4096, mapV2, &bars[B_WIN_FULL], c2 * 64, hk, row0 + 32 * bx, b);
                        }
                }
            }
            uint4 qv[4], dv[4];
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) { qv[cc] = make_uint4(0, 0, 0, 0); dv[cc] = make_uint4(0, 0, 0, 0); }
            float stat = 0.f;       // part 0: -lse2 / c, part 1: -D
            if (iv) {
                const __nv_bfloat16 *qp = q + elem_off(kp.q, b, i, h) + part * 32;
                const __nv_bfloat16 *dp = dout + elem_off(kp.dout, b, i, h) + part * 32;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    qv[cc] = __ldg(reinterpret_cast<const uint4 *>(qp + cc * 8));
                    dv[cc] = __ldg(reinterpret_cast<const uint4 *>(dp + cc * 8));
                }
                const int64_t o = ((int64_t)b * kp.hq + h) * kp.n + i;
                if (part == 0) stat = -kp.lse[o] * 1.4426950408889634f * inv_c;
                else if (part == 1) stat = -kp.delta[o];
            }
            if (win && !mbar_wait(&bars[B_WIN_FULL], blk & 1, abort_flag, 64, 1)) return ERR_BK1_BUILDER;
            for (int e = 0; e < ne; ++e, ++s) {
                const int stage = s % STAGES;
                // the stage is free once the second products of three steps ago have completed
                if (s >= STAGES && !warp_wait(&bars[B_AB_EMPTY + stage], (s / STAGES - 1) & 1, abort_flag, 2)) return ERR_BK1_BUILDER;
                if (e == 0 && part < 2) {
                    // Statistics of this query block (K = 16 slabs of -lse2/c and of -D) in slot blk % 3.  Step
                    // s - 3 has completed and every block has at least one step, so the slabs of three blocks ago
                    // are no longer read.
                    const int row = stat_row(blk % 3, part, r), ch = stat_chunk(blk % 3, part);
                    *reinterpret_cast<uint4 *>(sConst + sw128_offset(row, ch)) = split3_bf16(stat);
                    *reinterpret_cast<uint4 *>(sConst + sw128_offset(row, ch + 1)) = make_uint4(0u, 0u, 0u, 0u);
                }
                uint8_t *dA = sAB + (size_t)stage * STAGE_BYTES + (size_t)cb * QBLK_BYTES;
                uint8_t *dB = dA + AB_BYTES;
                const int kk = i + kp.off2 - e;
                const bool ok = iv && kk >= 0;
                const int wr = r + 32 - e;                       // row of the staged window
                const uint8_t *wk = sWin + cb * WBLK_BYTES + wr * 128, *wv = wk + WIN_BYTES;
                const __nv_bfloat16 *kp2 = k2 + elem_off(kp.k2, b, ok ? kk : 0, hk) + part * 32;
                const __nv_bfloat16 *vp2 = v2 + elem_off(kp.v2, b, ok ? kk : 0, hk) + part * 32;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    uint4 a = make_uint4(0, 0, 0, 0), bb = make_uint4(0, 0, 0, 0);
                    if (ok) {
                        const uint4 kv = win ? *reinterpret_cast<const uint4 *>(wk + (((ch0 + cc) ^ (wr & 7)) << 4))
                                             : __ldg(reinterpret_cast<const uint4 *>(kp2 + cc * 8));
                        const uint4 vv = win ? *reinterpret_cast<const uint4 *>(wv + (((ch0 + cc) ^ (wr & 7)) << 4))
                                             : __ldg(reinterpret_cast<const uint4 *>(vp2 + cc * 8));
                        a.x = mul_bf16x2(qv[cc].x, kv.x); a.y = mul_bf16x2(qv[cc].y, kv.y);
                        a.z = mul_bf16x2(qv[cc].z, kv.z); a.w = mul_bf16x2(qv[cc].w, kv.w);
                        bb.x = mul_bf16x2(dv[cc].x, vv.x); bb.y = mul_bf16x2(dv[cc].y, vv.y);
                        bb.z = mul_bf16x2(dv[cc].z, vv.z); bb.w = mul_bf16x2(dv[cc].w, vv.w);
                    }
                    *reinterpret_cast<uint4 *>(dA + sw128_offset(r, ch0 + cc)) = a;
                    *reinterpret_cast<uint4 *>(dB + sw128_offset(r, ch0 + cc)) = bb;
                }
                fence_proxy_async_smem();
                mbar_arrive(&bars[B_AB_FULL + stage]);
            }
        }
    }
    return 0;
}

// ---------------------------------------------------------------- issuers of S^T (warp 1) and dP^T (warp 2), one lane each
// Step s uses stage s % 3 and TMEM half s % 2.
__device__ __forceinline__ int mma_first(const KernelParams &kp, const Geom &g, int which, uint32_t tmem, uint8_t *sKV,
                                         uint8_t *sAB, uint8_t *sConst, uint64_t *bars, volatile int *abort_flag) {
    constexpr uint32_t IDESC_F = idesc_bf16(128, 64, false, false);
    const uint64_t dT = smem_desc_sw128(smem_u32(sKV));
    const uint64_t dAB = smem_desc_sw128(smem_u32(sAB + which * AB_BYTES));
    const uint64_t dOnes = smem_desc_sw128(smem_u32(sConst));
    if (!mbar_wait(&bars[B_KV_FULL], 0, abort_flag)) return ERR_BK1_MMA;
    int s = 0, blk = 0;
    for (int hh = 0; hh < kp.g; ++hh) {
        for (int ib = 0; ib < g.n_ib; ++ib, ++blk) {
            const int ne = block_sweeps(kp, g, ib);
            // this block's slab of the constant tile (rows are multiples of 64: whole 8-row swizzle groups)
            const uint64_t st = dOnes + (uint64_t)((stat_row(blk % 3, which, 0) * 128) >> 4) + (uint64_t)stat_chunk(blk % 3, which);
            for (int e = 0; e < ne; ++e, ++s) {
                const int stage = s % STAGES, half = s & 1;
                if (!mbar_wait(&bars[B_AB_FULL + stage], (s / STAGES) & 1, abort_flag, 0, 1)) return ERR_BK1_MMA;
                // P^T / G^T of the step that used this half last lie over these columns until its second products are done
                if (s >= 2 && !mbar_wait(&bars[B_G_DONE + half], ((s >> 1) - 1) & 1, abort_flag, 0, 2)) return ERR_BK1_MMA;
                tc_fence_after();
                const uint64_t a = dAB + (uint64_t)((stage * STAGE_BYTES) >> 4);
                const uint32_t d = tmem + half * 128 + which * 64;
#pragma unroll
                for (int k8 = 0; k8 < 8; ++k8) {
                    const uint64_t kin = (uint64_t)((k8 & 3) * 2);
                    mma_ss(d, dT + (uint64_t)(((k8 >> 2) * BLK_BYTES) >> 4) + kin, a + (uint64_t)(((k8 >> 2) * QBLK_BYTES) >> 4) + kin,
                           IDESC_F, k8 > 0 ? 1u : 0u);
                }
                mma_ss(d, dOnes, st, IDESC_F, 1u);                // - lse2_i / c, or - D_i
                tc_commit(&bars[B_S_FULL + half]);
            }
        }
    }
    return 0;
}

// ---------------------------------------------------------------- issuer of dV1, dK1 (warp 0, one lane)
__device__ __forceinline__ int mma_second(const Params &P, const Geom &g, uint32_t tmem, uint8_t *sAB, uint64_t *bars,
                                          volatile int *abort_flag) {
    constexpr uint32_t IDESC_G = idesc_bf16(128, 128, false, true);     // B operand MN-major, N = 128
    constexpr uint32_t IDESC_G64 = idesc_bf16(128, 64, false, true);
    const uint64_t dAB = smem_desc_sw128(smem_u32(sAB), 1024, QBLK_BYTES);   // channel blocks 8 KB apart
    for (int s = 0; s < g.total; ++s) {
        const int stage = s % STAGES, half = s & 1;
        if (!mbar_wait(&bars[B_P_FULL + half], (s >> 1) & 1, abort_flag, 0, 1)) return ERR_BK1_MMA;
        tc_fence_after();
        const uint64_t a = dAB + (uint64_t)((stage * STAGE_BYTES) >> 4), bq = a + (AB_BYTES >> 4);
        const uint32_t tp = tmem + half * 128, tg = tp + 64;
        const uint32_t first = s > 0 ? 1u : 0u;
        if (!P.n_split) {
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) mma_ts(tmem + 384, tp + k4 * 8, bq + k4 * 128, IDESC_G, (first || k4 > 0) ? 1u : 0u);
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) mma_ts(tmem + 256, tg + k4 * 8, a + k4 * 128, IDESC_G, (first || k4 > 0) ? 1u : 0u);
        } else {
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
                mma_ts(tmem + 384, tp + k4 * 8, bq + k4 * 128, IDESC_G64, (first || k4 > 0) ? 1u : 0u);
                mma_ts(tmem + 448, tp + k4 * 8, bq + (QBLK_BYTES >> 4) + k4 * 128, IDESC_G64, (first || k4 > 0) ? 1u : 0u);
            }
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
                mma_ts(tmem + 256, tg + k4 * 8, a + k4 * 128, IDESC_G64, (first || k4 > 0) ? 1u : 0u);
                mma_ts(tmem + 320, tg + k4 * 8, a + (QBLK_BYTES >> 4) + k4 * 128, IDESC_G64, (first || k4 > 0) ? 1u : 0u);
            }
        }
        tc_commit(&bars[B_G_DONE + half]);
        tc_commit(&bars[B_AB_EMPTY + stage]);
    }
    tc_commit(&bars[B_DONE]);
    return 0;
}

// ---------------------------------------------------------------- compute (group h: steps s = h mod 2; warps 4-7, 8-11)
__device__ __forceinline__ int compute(const Params &P, const Geom &g, int half, uint32_t tmem,
                                       uint64_t *bars, volatile int *abort_flag) {
    const KernelParams &kp = P.kp;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = (warp & 3) * 32 + lane;          // key row within the tile = TMEM lane
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t buf = lane_addr + half * 128;
    const int hk = blockIdx.y, b = blockIdx.z;
    const int j = g.j0 + r;
    const bool jv = j < kp.nk1;
    const float c = P.c;

    // the walk over the steps; a wait that runs out ends it early, the rows are then reported as NaN below
    auto walk = [&]() -> int {
        int s = 0;
        for (int hh = 0; hh < kp.g; ++hh) {
            for (int ib = 0; ib < g.n_ib; ++ib) {
                const int it0 = g.i_lo + QB * ib;
                const int ne = block_sweeps(kp, g, ib);
                const int base = j - kp.off1 - it0;                       // column of the diagonal i + off1 == j
                const int hi = jv ? min(min(QB - 1, base + kp.w1 - 1), g.i_hi - it0) : -1;
                for (int e = 0; e < ne; ++e, ++s) {
                    if ((s & 1) != half) continue;
                    const int lo = max(max(0, base), e - kp.off2 - it0);      // valid columns: lo <= col <= hi
                    if (!warp_wait(&bars[B_S_FULL + half], (s >> 1) & 1, abort_flag, 1)) return ERR_BK1_COMPUTE;
                    tc_fence_after();
                    const bool full = __all_sync(0xffffffffu, lo <= 0 && hi >= 63);
#pragma unroll
                    for (int ch = 0; ch < 2; ++ch) {
                        uint32_t sv[32], dv[32], pk[16], gk[16];
                        tmem_ld32(buf + ch * 32, sv);
                        tmem_ld32(buf + 64 + ch * 32, dv);
                        tmem_wait_ld();
                        // the accumulators already hold S^T - lse2 / c and dP^T - D
                        if (full) {
#pragma unroll
                            for (int x = 0; x < 32; x += 2) {
                                const float p0 = ex2(__uint_as_float(sv[x]) * c);
                                const float p1 = ex2(__uint_as_float(sv[x + 1]) * c);
                                pk[x >> 1] = pack_bf16(p0, p1);
                                gk[x >> 1] = pack_bf16(p0 * __uint_as_float(dv[x]), p1 * __uint_as_float(dv[x + 1]));
                            }
                        } else {
                            // valid columns are the integers in [lo, hi]: saturate(half + 1 - |col - mid|) is exactly
                            // 1 inside and 0 outside; the exponent is clamped so that a masked-out cell cannot give inf * 0
                            const float mid = 0.5f * (float)(lo + hi), hwp = 0.5f * (float)(hi - lo) + 1.f;
#pragma unroll
                            for (int x = 0; x < 32; x += 2) {
                                const int col = ch * 32 + x;
                                const float v0 = __saturatef(hwp - fabsf((float)col - mid));
                                const float v1 = __saturatef(hwp - fabsf((float)(col + 1) - mid));
                                const float p0 = ex2(fminf(__uint_as_float(sv[x]) * c, 100.f)) * v0;
                                const float p1 = ex2(fminf(__uint_as_float(sv[x + 1]) * c, 100.f)) * v1;
                                pk[x >> 1] = pack_bf16(p0, p1);
                                gk[x >> 1] = pack_bf16(p0 * __uint_as_float(dv[x]), p1 * __uint_as_float(dv[x + 1]));
                            }
                        }
                        // over columns of S^T / dP^T that this thread has already read
                        tmem_st16(buf + ch * 16, pk);
                        tmem_st16(buf + 64 + ch * 16, gk);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(&bars[B_P_FULL + half]);
                }
            }
        }
        return 0;
    };
    int err = walk();
    // drain: group 0 writes dK1, group 1 writes dV1
    if (err == 0 && !warp_wait(&bars[B_DONE], 0, abort_flag)) err = ERR_BK1_COMPUTE;
    const bool bad = __any_sync(0xffffffffu, err != 0) || *abort_flag != 0;
    tc_fence_after();
    const bool gbf16 = kp.grad_bf16 != 0;
    const TensorRef &dst = half == 0 ? kp.dk1 : kp.dv1;
    const float mul = half == 0 ? kp.scale : 1.f;
#pragma unroll 1
    for (int q4 = 0; q4 < 4; ++q4) {
        uint32_t w[32];
        tmem_ld32(lane_addr + 256 + half * 128 + q4 * 32, w);
        tmem_wait_ld();
        if (jv) {
            const int64_t off = elem_off(dst, b, j, hk) + q4 * 32;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                float x[4];
#pragma unroll
                for (int z = 0; z < 4; ++z) x[z] = bad ? CUDART_NAN_F : (g.total > 0 ? __uint_as_float(w[u * 4 + z]) : 0.f) * mul;
                store_vec<4>(dst.p, off + u * 4, gbf16, x);
            }
        }
    }
    return err;
}

__global__ void __launch_bounds__(THREADS, 1)
bwd_k1_128_kernel(const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                  const __grid_constant__ CUtensorMap mapK2, const __grid_constant__ CUtensorMap mapV2, const Params P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sK = smem;
    uint8_t *sV = sK + T_BYTES;
    uint8_t *sAB = sV + T_BYTES;                          // STAGES x (A_e, B_e)
    uint8_t *sConst = sAB + STAGES * STAGE_BYTES;         // ones and three slots of query statistics
    uint8_t *sWin = sConst + TILE_BYTES;                  // staged k2 window, then v2 window
    uint64_t *bars = reinterpret_cast<uint64_t *>(sWin + 2 * WIN_BYTES);
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + B_COUNT);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int x = 0; x < B_COUNT; ++x) {
            uint32_t count = 1;
            if ((x >= B_AB_FULL && x < B_AB_FULL + STAGES) || x == B_WIN_FREE) count = 256;     // every builder
            else if (x >= B_P_FULL && x < B_P_FULL + 2) count = 128;
            else if (x >= B_S_FULL && x < B_S_FULL + 2) count = 2;                // one commit from each first-product issuer
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
    const Geom g = geom(P.kp);

    int err = 0;
#ifdef SA2_PROF
    const long long prof_t0 = clock64();
    sa2::sm100::prof_begin();
#endif
    if (warp < 4) {
        reg_dealloc<REGS_ISSUE>();
        if (warp == 0) {
            if (lane == 0) {
                if (g.total > 0) {
                    prefetch_tmap(&mapK);
                    prefetch_tmap(&mapV);
                    mbar_arrive_expect_tx(&bars[B_KV_FULL], 2 * T_BYTES);
                    tma_load_4d(sK, &mapK, &bars[B_KV_FULL], 0, blockIdx.y, g.j0, blockIdx.z);
                    tma_load_4d(sK + BLK_BYTES, &mapK, &bars[B_KV_FULL], 64, blockIdx.y, g.j0, blockIdx.z);
                    tma_load_4d(sV, &mapV, &bars[B_KV_FULL], 0, blockIdx.y, g.j0, blockIdx.z);
                    tma_load_4d(sV + BLK_BYTES, &mapV, &bars[B_KV_FULL], 64, blockIdx.y, g.j0, blockIdx.z);
                    err = mma_second(P, g, tmem, sAB, bars, abort_flag);
                    // the tile must have landed before the CTA may exit, even if every other role gave up
                    if (!mbar_wait(&bars[B_KV_FULL], 0, abort_flag)) err |= ERR_BK1_PRODUCER;
                } else {
                    tc_commit(&bars[B_DONE]);
                }
            }
            __syncwarp();
        } else if (warp == 1 || warp == 2) {
            if (lane == 0 && g.total > 0)
                err = mma_first(P.kp, g, warp - 1, tmem, warp == 1 ? sK : sV, sAB, sConst, bars, abort_flag);
            __syncwarp();
        }
    } else if (warp < 12) {
        reg_alloc<REGS_COMPUTE>();
        err = compute(P, g, (warp - 4) >> 2, tmem, bars, abort_flag);
    } else {
        reg_dealloc<REGS_BUILD>();
        err = builder(P, g, &mapK2, &mapV2, sAB, sConst, sWin, bars, abort_flag);
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

}  // namespace k128
}  // namespace tc
}  // namespace sa2
