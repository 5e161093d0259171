// Backward kernel for dK1 / dV1 on tcgen05 tensor cores (bf16 operands, fp32
// accumulation in TMEM, head dim 64).
//
// One CTA owns 128 rows j of K1/V1 of one (batch, kv head); the tile stays in
// shared memory and dK1/dV1 for those rows accumulate in TMEM for the whole
// kernel, so nothing is reduced across CTAs and there are no atomics.  The CTA
// walks over every (query head of the group, query tile I, offset e) that can
// see its keys.  Per step the builder warps form
//     A_e[i,:] = q_i * k2_{i-e}      B_e[i,:] = dO_i * v2_{i-e}      (bf16)
// and the tensor cores compute, in two 64-column halves that ping-pong,
//     S^T  = K1 A_e^T       dP^T = V1 B_e^T          (rows j, columns i)
// the compute warps (one thread per key row j) turn them into
//     P^T = exp2(c S^T - lse2_i)      G^T = P^T * (dP^T - D_i)
// written back to TMEM as bf16, which then feed as A operands
//     dV1 += P^T B_e        dK1 += G^T A_e           (B_e / A_e as MN-major B)
// The same shared-memory tile is the K-major B operand of the first product
// and the MN-major B operand of the second.
//
// The per-query statistics are folded into the tensor-core products: every query row carries
// -lse2_i / c and -D_i, each split into three bf16 terms, in a small extra tile, and a constant tile
// of ones on the key side adds them with one more K=16 MMA, so that the accumulators already hold
// S^T - lse2 / c and dP^T - D and the compute threads need no per-column loads.
//
// Warps (480 threads; warp 14 issues dP^T next to warp 1, which issues S^T): 0 TMA producer, then issuer of the second products (dV1, dK1);
// 1 TMEM owner and issuer of the first products (S^T, dP^T); 2-5 compute group of
// half 0; 6-9 compute group of half 1; 10-13 builders.  One thread issues about one
// tcgen05.mma per 90 cycles, so the two products have an issuing thread each; dK1/dV1
// are accumulated by one thread only, which keeps the summation order fixed.
// TMEM columns: half h -> S^T [128h, +64), dP^T [128h+64, +64), P^T (bf16) [256+64h, +32),
// G^T (bf16) [288+64h, +32); dK1 [384,448); dV1 [448,512).  P^T/G^T have their own
// columns so that the next S^T/dP^T of a half can be issued as soon as the compute
// group has read the current one.
#pragma once
#include "sa2_tc_fwd.cuh"

namespace sa2 {
namespace tc {

constexpr int BK1_THREADS = 480;
// A_e / B_e stages.  A stage is released only when the second products of its step have completed, i.e.
// after build -> first products -> P^T/G^T pass -> second products; with two stages the builders (whose
// 32 shared-memory accesses per step take ~1600 cycles next to the tensor cores' operand traffic) waited
// for that chain every step and paced the kernel at ~3000 cycles per step.
constexpr int BK1_STAGES = 3;

enum Bk1Bar {
    BK1_KV_FULL = 0,
    BK1_AB_FULL = 1,     // [BK1_STAGES]
    BK1_AB_EMPTY = 4,    // [BK1_STAGES]
    BK1_S_FULL = 7,      // [2] per half
    BK1_P_FULL = 9,      // [2] per half
    BK1_G_DONE = 11,     // [2] per half: second products of the step have completed
    BK1_DONE = 13,
    BK1_WIN_FREE = 14,   // the builders have finished reading the k2/v2 window of the previous query tile
    BK1_WIN_FULL = 15,   // the window of the current query tile has landed
    BK1_BAR_COUNT = 16
};

enum { ERR_BK1_PRODUCER = 16, ERR_BK1_MMA = 32, ERR_BK1_COMPUTE = 64, ERR_BK1_BUILDER = 128 };

struct BwdParams {
    KernelParams kp;
    float c;        // scale * log2(e)
    int *status;
};

// padded above half of the SM's shared memory: one CTA per SM, so the 512-column TMEM allocation never waits
constexpr int BK1_WIN_ROWS = 160;    // second-key / second-value rows a query tile can pair with: 32 + 128
inline size_t bk1_smem_bytes() {
    return 1024 + 2 * TILE_BYTES + BK1_STAGES * 2 * TILE_BYTES + 2 * TILE_BYTES + TILE_BYTES + 2 * BK1_WIN_ROWS * 128 + 256;
}

struct Bk1Geom {
    int j0, i_lo, i_hi, n_it, total;
};

__device__ __forceinline__ int bk1_sweeps(const KernelParams &kp, const Bk1Geom &g, int t) {
    const int last = min(g.i_lo + TQ * t + TQ - 1, g.i_hi);
    return min(kp.w2, last + kp.off2 + 1);
}

__device__ __forceinline__ Bk1Geom bk1_geom(const KernelParams &kp) {
    Bk1Geom g;
    g.j0 = blockIdx.x * TJ;
    g.i_lo = max(0, g.j0 - kp.off1);
    g.i_hi = min(kp.n - 1, min(g.j0 + TJ - 1, kp.nk1 - 1) + kp.w1 - 1 - kp.off1);
    g.n_it = g.i_hi >= g.i_lo ? (g.i_hi - g.i_lo) / TQ + 1 : 0;
    int per_head = 0;
    for (int t = 0; t < g.n_it; ++t) per_head += bk1_sweeps(kp, g, t);
    g.total = per_head * kp.g;
    return g;
}

// ---------------------------------------------------------------- builders (warps 10-13)
// three bf16 terms whose sum is x to fp32 accuracy, packed with five zeros into one 16-byte chunk
__device__ __forceinline__ uint4 split3_bf16(float x) {
    const __nv_bfloat16 h0 = __float2bfloat16_rn(x);
    const float r1 = x - __bfloat162float(h0);
    const __nv_bfloat16 h1 = __float2bfloat16_rn(r1);
    const __nv_bfloat16 h2 = __float2bfloat16_rn(r1 - __bfloat162float(h1));
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    v.x = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
    v.y = (uint32_t)__bfloat16_as_ushort(h2);
    return v;
}

__device__ __forceinline__ int bk1_builder(const BwdParams &P, const Bk1Geom &g, const CUtensorMap *mapK2, const CUtensorMap *mapV2,
                                           uint8_t *sAB, uint8_t *sStat, uint8_t *sOnes, uint8_t *sWin,
                                           uint64_t *bars, volatile int *abort_flag) {
    const KernelParams &kp = P.kp;
    const int r = threadIdx.x - 320;       // row of the query tile
    const int hk = blockIdx.y, b = blockIdx.z;
    const __nv_bfloat16 *q = reinterpret_cast<const __nv_bfloat16 *>(kp.q.p);
    const __nv_bfloat16 *k2 = reinterpret_cast<const __nv_bfloat16 *>(kp.k2.p);
    const __nv_bfloat16 *dout = reinterpret_cast<const __nv_bfloat16 *>(kp.dout.p);
    const __nv_bfloat16 *v2 = reinterpret_cast<const __nv_bfloat16 *>(kp.v2.p);
    // the constant key-side tile: three ones per row (one per term of the split statistics)
    {
        uint4 one = make_uint4(0x3f803f80u, 0x00003f80u, 0u, 0u);
#pragma unroll
        for (int cc = 0; cc < 8; ++cc)
            *reinterpret_cast<uint4 *>(sOnes + sw128_offset(r, cc)) = cc == 0 ? one : make_uint4(0u, 0u, 0u, 0u);
    }
    const float inv_c = 1.f / P.c;
    int s = 0, tile_counter = 0;
    for (int hh = 0; hh < kp.g; ++hh) {
        const int h = hk * kp.g + hh;
        for (int t = 0; t < g.n_it; ++t, ++tile_counter) {
            const int i = g.i_lo + TQ * t + r;
            const bool iv = i <= g.i_hi;
            const int ne = bk1_sweeps(kp, g, t);
            // The k2 / v2 rows this query tile pairs with over all sweeps (positions it0 - 32 .. it0 + 127)
            // are staged once per tile by TMA; every step then reads its rows from shared memory.
            const bool win = kp.w2 <= 32;
            if (win) {
                if (tile_counter > 0) mbar_arrive(&bars[BK1_WIN_FREE]);
                if (r == 0) {
                    if (tile_counter > 0 && !mbar_wait(&bars[BK1_WIN_FREE], (tile_counter - 1) & 1, abort_flag)) return ERR_BK1_BUILDER;
                    mbar_arrive_expect_tx(&bars[BK1_WIN_FULL], 2 * BK1_WIN_ROWS * 128);
                    const int row0 = g.i_lo + TQ * t + kp.off2 - 32;
                    for (int bx = 0; bx < BK1_WIN_ROWS / 32; ++bx) {
                        tma_load_4d(sWin + bx * 4096, mapK2, &bars[BK1_WIN_FULL], 0, hk, row0 + 32 * bx, b);
                        tma_load_4d(sWin + BK1_WIN_ROWS * 128 + bx * 4096, mapV2, &bars[BK1_WIN_FULL], 0, hk, row0 + 32 * bx, b);
                    }
                }
                if (!mbar_wait(&bars[BK1_WIN_FULL], tile_counter & 1, abort_flag, 64, 1)) return ERR_BK1_BUILDER;
            }
            uint4 qv[8], dv[8];
#pragma unroll
            for (int cc = 0; cc < 8; ++cc) { qv[cc] = make_uint4(0, 0, 0, 0); dv[cc] = make_uint4(0, 0, 0, 0); }
            float lse2 = 0.f, dl = 0.f;
            if (iv) {
                const __nv_bfloat16 *qp = q + elem_off(kp.q, b, i, h);
                const __nv_bfloat16 *dp = dout + elem_off(kp.dout, b, i, h);
#pragma unroll
                for (int cc = 0; cc < 8; ++cc) {
                    qv[cc] = *reinterpret_cast<const uint4 *>(qp + cc * 8);
                    dv[cc] = *reinterpret_cast<const uint4 *>(dp + cc * 8);
                }
                const int64_t o = ((int64_t)b * kp.hq + h) * kp.n + i;
                lse2 = kp.lse[o] * 1.4426950408889634f;
                dl = kp.delta[o];
            }
            for (int e = 0; e < ne; ++e, ++s) {
                const int stage = s % BK1_STAGES;
                if (s >= BK1_STAGES && !warp_wait(&bars[BK1_AB_EMPTY + stage], (s / BK1_STAGES - 1) & 1, abort_flag, 2)) return ERR_BK1_BUILDER;
                if (e == 0) {
                    // Statistics of this query tile: two K = 16 slabs (-lse2/c, -D) of a four-slab tile; two
                    // such tiles hold the last four query tiles.  Step s - 3 has completed, and every tile has
                    // at least one step, so the slabs of four tiles ago are no longer read.
                    uint8_t *st = sStat + (size_t)((tile_counter >> 1) & 1) * TILE_BYTES;
                    const int c0 = (tile_counter & 1) * 4;
                    *reinterpret_cast<uint4 *>(st + sw128_offset(r, c0)) = split3_bf16(-lse2 * inv_c);
                    *reinterpret_cast<uint4 *>(st + sw128_offset(r, c0 + 1)) = make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4 *>(st + sw128_offset(r, c0 + 2)) = split3_bf16(-dl);
                    *reinterpret_cast<uint4 *>(st + sw128_offset(r, c0 + 3)) = make_uint4(0u, 0u, 0u, 0u);
                }
                uint8_t *dA = sAB + (size_t)stage * 2 * TILE_BYTES;
                uint8_t *dB = dA + TILE_BYTES;
                const int kk = i + kp.off2 - e;
                const bool ok = iv && kk >= 0;
                const __nv_bfloat16 *kp2 = k2 + elem_off(kp.k2, b, ok ? kk : 0, hk);
                const __nv_bfloat16 *vp2 = v2 + elem_off(kp.v2, b, ok ? kk : 0, hk);
                const int wr = r + 32 - e;                       // row of the staged window
                const uint8_t *wk = sWin + wr * 128, *wv = wk + BK1_WIN_ROWS * 128;
#pragma unroll
                for (int cc = 0; cc < 8; ++cc) {
                    uint4 a = make_uint4(0, 0, 0, 0), bb = make_uint4(0, 0, 0, 0);
                    if (ok) {
                        const uint4 kv = win ? *reinterpret_cast<const uint4 *>(wk + ((cc ^ (wr & 7)) << 4))
                                             : *reinterpret_cast<const uint4 *>(kp2 + cc * 8);
                        const uint4 vv = win ? *reinterpret_cast<const uint4 *>(wv + ((cc ^ (wr & 7)) << 4))
                                             : *reinterpret_cast<const uint4 *>(vp2 + cc * 8);
                        a.x = mul_bf16x2(qv[cc].x, kv.x); a.y = mul_bf16x2(qv[cc].y, kv.y);
                        a.z = mul_bf16x2(qv[cc].z, kv.z); a.w = mul_bf16x2(qv[cc].w, kv.w);
                        bb.x = mul_bf16x2(dv[cc].x, vv.x); bb.y = mul_bf16x2(dv[cc].y, vv.y);
                        bb.z = mul_bf16x2(dv[cc].z, vv.z); bb.w = mul_bf16x2(dv[cc].w, vv.w);
                    }
                    *reinterpret_cast<uint4 *>(dA + sw128_offset(r, cc)) = a;
                    *reinterpret_cast<uint4 *>(dB + sw128_offset(r, cc)) = bb;
                }
                fence_proxy_async_smem();
                mbar_arrive(&bars[BK1_AB_FULL + stage]);
            }
        }
    }
    return 0;
}

// ---------------------------------------------------------------- issuer of S^T, dP^T (warp 1, one lane)
// which = 0: S^T = K1 A_e^T - lse2 / c into columns [128 half, +64) (warp 1);
// which = 1: dP^T = V1 B_e^T - D into columns [128 half + 64, +64) (warp 14).
// The two products have an issuing thread each: the time from "the compute group has read the buffer" to
// "the next S^T / dP^T are complete" is on the critical chain of every step, and one thread issues only
// one tcgen05.mma per 60-100 cycles.
__device__ __forceinline__ int bk1_mma_first(const KernelParams &kp, const Bk1Geom &g, int which, uint32_t tmem, uint8_t *sKV,
                                             uint8_t *sAB, uint8_t *sStat, uint8_t *sOnes, uint64_t *bars, volatile int *abort_flag) {
    constexpr uint32_t IDESC_F = idesc_bf16(128, 64, false, false);
    const uint64_t dT = smem_desc_sw128(smem_u32(sKV));
    const uint64_t dAB = smem_desc_sw128(smem_u32(sAB + which * TILE_BYTES));
    const uint64_t dSt = smem_desc_sw128(smem_u32(sStat)), dOnes = smem_desc_sw128(smem_u32(sOnes));
    if (!mbar_wait(&bars[BK1_KV_FULL], 0, abort_flag)) return ERR_BK1_MMA;
    int s = 0, tile_counter = 0;
    for (int hh = 0; hh < kp.g; ++hh) {
        for (int t = 0; t < g.n_it; ++t, ++tile_counter) {
            const int ne = bk1_sweeps(kp, g, t);
            // slab (16 channels = 32 bytes = 2 descriptor units) of the statistics tile that holds this query tile
            const uint64_t stL0 = dSt + (uint64_t)((((tile_counter >> 1) & 1) * TILE_BYTES) >> 4) + (uint64_t)((tile_counter & 1) * 4);
            for (int e = 0; e < ne; ++e, ++s) {
                const int stage = s % BK1_STAGES;
                if (!mbar_wait(&bars[BK1_AB_FULL + stage], (s / BK1_STAGES) & 1, abort_flag, 0, 1)) return ERR_BK1_MMA;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    // the compute group must have read the previous step's S^T / dP^T of this half
                    if (s >= 1 && !mbar_wait(&bars[BK1_P_FULL + half], (s - 1) & 1, abort_flag, 0, 2)) return ERR_BK1_MMA;
                    tc_fence_after();
                    const uint64_t a = dAB + (uint64_t)((stage * 2 * TILE_BYTES + half * 8192) >> 4);
                    const uint64_t st = stL0 + (uint64_t)((half * 8192) >> 4) + (uint64_t)(which * 2);
                    const uint32_t d = tmem + half * 128 + which * 64;
                    mma_ss(d, dT, a, IDESC_F, 0u);
                    mma_ss(d, dT + 2, a + 2, IDESC_F, 1u);
                    mma_ss(d, dT + 4, a + 4, IDESC_F, 1u);
                    mma_ss(d, dT + 6, a + 6, IDESC_F, 1u);
                    mma_ss(d, dOnes, st, IDESC_F, 1u);                // - lse2_i / c, or - D_i
                    tc_commit(&bars[BK1_S_FULL + half]);
                }
            }
        }
    }
    return 0;
}

// ---------------------------------------------------------------- issuer of dV1, dK1 (warp 0, one lane)
__device__ __forceinline__ int bk1_mma_second(const Bk1Geom &g, uint32_t tmem, uint8_t *sAB, uint64_t *bars, volatile int *abort_flag) {
    constexpr uint32_t IDESC_G = idesc_bf16(128, 64, false, true);    // B operand MN-major
    const uint64_t dAB = smem_desc_sw128(smem_u32(sAB));
    for (int s = 0; s < g.total; ++s) {
        const int stage = s % BK1_STAGES;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            if (!mbar_wait(&bars[BK1_P_FULL + half], s & 1, abort_flag, 0, 1)) return ERR_BK1_MMA;
            tc_fence_after();
            const uint64_t a = dAB + (uint64_t)((stage * 2 * TILE_BYTES + half * 8192) >> 4), bq = a + (TILE_BYTES >> 4);
            const uint32_t t = tmem + 256 + half * 64;
            const uint32_t first = (s > 0 || half > 0) ? 1u : 0u;
            mma_ts(tmem + 448, t, bq, IDESC_G, first);
            mma_ts(tmem + 448, t + 8, bq + 128, IDESC_G, 1u);
            mma_ts(tmem + 448, t + 16, bq + 256, IDESC_G, 1u);
            mma_ts(tmem + 448, t + 24, bq + 384, IDESC_G, 1u);
            mma_ts(tmem + 384, t + 32, a, IDESC_G, first);
            mma_ts(tmem + 384, t + 40, a + 128, IDESC_G, 1u);
            mma_ts(tmem + 384, t + 48, a + 256, IDESC_G, 1u);
            mma_ts(tmem + 384, t + 56, a + 384, IDESC_G, 1u);
            tc_commit(&bars[BK1_G_DONE + half]);
        }
        tc_commit(&bars[BK1_AB_EMPTY + stage]);
    }
    tc_commit(&bars[BK1_DONE]);
    return 0;
}

// ---------------------------------------------------------------- compute (group h = half h: warps 2-5, 6-9)
__device__ __forceinline__ int bk1_compute(const BwdParams &P, const Bk1Geom &g, int half, uint32_t tmem,
                                           uint64_t *bars, volatile int *abort_flag) {
    const KernelParams &kp = P.kp;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = (warp & 3) * 32 + lane;          // key row within the tile = TMEM lane
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t buf = lane_addr + half * 128, pg = lane_addr + 256 + half * 64;
    const int hk = blockIdx.y, b = blockIdx.z;
    const int j = g.j0 + r;
    const bool jv = j < kp.nk1;
    const float c = P.c;

    // the walk over the steps; a wait that runs out ends it early, the rows are then reported as NaN below
    auto walk = [&]() -> int {
        int s = 0, tile_counter = 0;
        for (int hh = 0; hh < kp.g; ++hh) {
            for (int t = 0; t < g.n_it; ++t, ++tile_counter) {
                const int it0 = g.i_lo + TQ * t;
                const int ne = bk1_sweeps(kp, g, t);
                const int base = j - kp.off1 - it0;                       // column of the diagonal i + off1 == j
                const int hi = (jv ? min(min(TQ - 1, base + kp.w1 - 1), g.i_hi - it0) : -1) - half * 64;
                for (int e = 0; e < ne; ++e, ++s) {
                    const int lo = max(max(0, base), e - kp.off2 - it0) - half * 64;     // valid columns: lo <= col <= hi
                    if (!warp_wait(&bars[BK1_S_FULL + half], s & 1, abort_flag, 1)) return ERR_BK1_COMPUTE;
                    tc_fence_after();
                    const bool full = __all_sync(0xffffffffu, lo <= 0 && hi >= 63);
                    // P^T / G^T of the previous step must have been consumed before they are overwritten
                    if (s >= 1 && !warp_wait(&bars[BK1_G_DONE + half], (s - 1) & 1, abort_flag, 2)) return ERR_BK1_COMPUTE;
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
                            // valid columns are the integers in [lo, hi]: saturate(half + 1 - |col - mid|) is
                            // exactly 1 inside and 0 outside (FMA pipe instead of compares and selects on the
                            // ALU pipe); the exponent is clamped so that a masked-out cell cannot give inf * 0
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
                        tmem_st16(pg + ch * 16, pk);
                        tmem_st16(pg + 32 + ch * 16, gk);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(&bars[BK1_P_FULL + half]);
                }
            }
        }
        return 0;
    };
    int err = walk();
    // drain: group 0 writes dK1, group 1 writes dV1
    if (err == 0 && !warp_wait(&bars[BK1_DONE], 0, abort_flag)) err = ERR_BK1_COMPUTE;
    const bool bad = __any_sync(0xffffffffu, err != 0) || *abort_flag != 0;
    tc_fence_after();
    const bool gbf16 = kp.grad_bf16 != 0;
    const TensorRef &dst = half == 0 ? kp.dk1 : kp.dv1;
    const float mul = half == 0 ? kp.scale : 1.f;
#pragma unroll 1
    for (int hf = 0; hf < 2; ++hf) {
        uint32_t w[32];
        tmem_ld32(lane_addr + 384 + half * 64 + hf * 32, w);
        tmem_wait_ld();
        if (jv) {
            const int64_t off = elem_off(dst, b, j, hk) + hf * 32;
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

__global__ void __launch_bounds__(BK1_THREADS, 1)
bwd_k1_kernel(const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
              const __grid_constant__ CUtensorMap mapK2, const __grid_constant__ CUtensorMap mapV2, const BwdParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sK = smem;
    uint8_t *sV = sK + TILE_BYTES;
    uint8_t *sAB = sV + TILE_BYTES;                       // BK1_STAGES x (A tile, B tile)
    uint8_t *sStat = sAB + BK1_STAGES * 2 * TILE_BYTES;   // 2 tiles x 2 query tiles x (-lse2/c slab, -D slab)
    uint8_t *sOnes = sStat + 2 * TILE_BYTES;              // constant: three ones per row
    uint8_t *sWin = sOnes + TILE_BYTES;                   // staged k2 rows, then v2 rows (160 x 128 B each)
    uint64_t *bars = reinterpret_cast<uint64_t *>(sWin + 2 * BK1_WIN_ROWS * 128);
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + BK1_BAR_COUNT);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int x = 0; x < BK1_BAR_COUNT; ++x) {
            const bool many = (x >= BK1_AB_FULL && x < BK1_AB_FULL + BK1_STAGES) || (x >= BK1_P_FULL && x < BK1_P_FULL + 2) ||
                              x == BK1_WIN_FREE;
            // S_FULL collects one commit from each of the two first-product issuers
            mbar_init(&bars[x], many ? 128u : (x >= BK1_S_FULL && x < BK1_S_FULL + 2) ? 2u : 1u);
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
    const Bk1Geom g = bk1_geom(P.kp);

    int err = 0;
#ifdef SA2_PROF
    const long long prof_t0 = clock64();
    sa2::sm100::prof_begin();
#endif
    if (warp == 0) {
        if (lane == 0) {
            if (g.total > 0) {
                prefetch_tmap(&mapK);
                prefetch_tmap(&mapV);
                mbar_arrive_expect_tx(&bars[BK1_KV_FULL], 2 * TILE_BYTES);
                tma_load_4d(sK, &mapK, &bars[BK1_KV_FULL], 0, blockIdx.y, g.j0, blockIdx.z);
                tma_load_4d(sV, &mapV, &bars[BK1_KV_FULL], 0, blockIdx.y, g.j0, blockIdx.z);
                err = bk1_mma_second(g, tmem, sAB, bars, abort_flag);
                // the tile must have landed before the CTA may exit, even if every other role gave up
                if (!mbar_wait(&bars[BK1_KV_FULL], 0, abort_flag)) err |= ERR_BK1_PRODUCER;
            } else {
                tc_commit(&bars[BK1_DONE]);
            }
        }
        __syncwarp();
    } else if (warp == 1 || warp == 14) {
        if (lane == 0 && g.total > 0)
            err = bk1_mma_first(P.kp, g, warp == 1 ? 0 : 1, tmem, warp == 1 ? sK : sV, sAB, sStat, sOnes, bars, abort_flag);
        __syncwarp();
    } else if (warp < 10) {
        err = bk1_compute(P, g, (warp - 2) >> 2, tmem, bars, abort_flag);
    } else {
        err = bk1_builder(P, g, &mapK2, &mapV2, sAB, sStat, sOnes, sWin, bars, abort_flag);
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
