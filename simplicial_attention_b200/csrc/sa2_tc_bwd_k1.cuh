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
// Warps (320 threads): 0 TMA producer, 1 MMA issuer + TMEM owner, 2-5 compute,
// 6-9 builders.  TMEM columns: half h -> [128h, 128h+64) S^T then P^T,
// [128h+64, 128h+128) dP^T then G^T; dK1 [256,320); dV1 [320,384).
#pragma once
#include "sa2_tc_fwd.cuh"

namespace sa2 {
namespace tc {

constexpr int BK1_THREADS = 320;

enum Bk1Bar {
    BK1_KV_FULL = 0,
    BK1_AB_FULL = 1,     // [2]
    BK1_AB_EMPTY = 3,    // [2]
    BK1_S_FULL = 5,      // [2] per half
    BK1_P_FULL = 7,      // [2] per half
    BK1_DONE = 9,
    BK1_BAR_COUNT = 10
};

enum { ERR_BK1_PRODUCER = 16, ERR_BK1_MMA = 32, ERR_BK1_COMPUTE = 64, ERR_BK1_BUILDER = 128 };

struct BwdParams {
    KernelParams kp;
    float c;        // scale * log2(e)
    int *status;
};

// padded above half of the SM's shared memory: one CTA per SM, so the 512-column TMEM allocation never waits
inline size_t bk1_smem_bytes() { return 120 * 1024; }

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

// ---------------------------------------------------------------- builders (warps 6-9)
__device__ __forceinline__ int bk1_builder(const BwdParams &P, const Bk1Geom &g, uint8_t *sAB, float *stats,
                                           uint64_t *bars, volatile int *abort_flag) {
    const KernelParams &kp = P.kp;
    const int r = threadIdx.x - 192;       // row of the query tile
    const int hk = blockIdx.y, b = blockIdx.z;
    const __nv_bfloat16 *q = reinterpret_cast<const __nv_bfloat16 *>(kp.q.p);
    const __nv_bfloat16 *k2 = reinterpret_cast<const __nv_bfloat16 *>(kp.k2.p);
    const __nv_bfloat16 *dout = reinterpret_cast<const __nv_bfloat16 *>(kp.dout.p);
    const __nv_bfloat16 *v2 = reinterpret_cast<const __nv_bfloat16 *>(kp.v2.p);
    int s = 0, tile_counter = 0;
    for (int hh = 0; hh < kp.g; ++hh) {
        const int h = hk * kp.g + hh;
        for (int t = 0; t < g.n_it; ++t, ++tile_counter) {
            const int i = g.i_lo + TQ * t + r;
            const bool iv = i <= g.i_hi;
            const int ne = bk1_sweeps(kp, g, t);
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
                const int stage = s & 1;
                if (s >= 2 && !warp_wait(&bars[BK1_AB_EMPTY + stage], ((s >> 1) - 1) & 1, abort_flag)) return ERR_BK1_BUILDER;
                if (e == 0) {
                    // column statistics of this query tile; the buffer of two tiles ago is no longer read
                    float *st = stats + (tile_counter & 1) * 256;
                    st[r] = lse2;
                    st[128 + r] = dl;
                }
                uint8_t *dA = sAB + (size_t)stage * 2 * TILE_BYTES;
                uint8_t *dB = dA + TILE_BYTES;
                const int kk = i + kp.off2 - e;
                const bool ok = iv && kk >= 0;
                const __nv_bfloat16 *kp2 = k2 + elem_off(kp.k2, b, ok ? kk : 0, hk);
                const __nv_bfloat16 *vp2 = v2 + elem_off(kp.v2, b, ok ? kk : 0, hk);
#pragma unroll
                for (int cc = 0; cc < 8; ++cc) {
                    uint4 a = make_uint4(0, 0, 0, 0), bb = make_uint4(0, 0, 0, 0);
                    if (ok) {
                        const uint4 kv = *reinterpret_cast<const uint4 *>(kp2 + cc * 8);
                        const uint4 vv = *reinterpret_cast<const uint4 *>(vp2 + cc * 8);
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

// ---------------------------------------------------------------- MMA issuer (warp 1, one lane)
__device__ __forceinline__ int bk1_mma(const Bk1Geom &g, uint32_t tmem, uint8_t *sK, uint8_t *sV, uint8_t *sAB,
                                       uint64_t *bars, volatile int *abort_flag) {
    constexpr uint32_t IDESC_F = idesc_bf16(128, 64, false, false);   // S^T, dP^T halves
    constexpr uint32_t IDESC_G = idesc_bf16(128, 64, false, true);    // dV, dK (B operand MN-major)
    const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aAB = smem_u32(sAB);

    auto first = [&](int s, int half) -> bool {
        const int stage = s & 1;
        if (half == 0 && !mbar_wait(&bars[BK1_AB_FULL + stage], (s >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t aA = aAB + stage * 2 * TILE_BYTES + half * 8192, aB = aA + TILE_BYTES;
        const uint32_t d = tmem + half * 128;
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_ss(d, smem_desc_sw128(aK + 32 * k), smem_desc_sw128(aA + 32 * k), IDESC_F, k > 0);
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_ss(d + 64, smem_desc_sw128(aV + 32 * k), smem_desc_sw128(aB + 32 * k), IDESC_F, k > 0);
        tc_commit(&bars[BK1_S_FULL + half]);
        return true;
    };
    auto second = [&](int s, int half) -> bool {
        const int stage = s & 1;
        if (!mbar_wait(&bars[BK1_P_FULL + half], s & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t aA = aAB + stage * 2 * TILE_BYTES + half * 8192, aB = aA + TILE_BYTES;
        const uint32_t a = tmem + half * 128;
#pragma unroll
        for (int k = 0; k < 4; ++k)
            mma_ts(tmem + 320, a + 8 * k, smem_desc_sw128(aB + 2048 * k), IDESC_G, (s > 0 || half > 0 || k > 0) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k)
            mma_ts(tmem + 256, a + 64 + 8 * k, smem_desc_sw128(aA + 2048 * k), IDESC_G, (s > 0 || half > 0 || k > 0) ? 1u : 0u);
        return true;
    };

    if (!mbar_wait(&bars[BK1_KV_FULL], 0, abort_flag)) return ERR_BK1_MMA;
    if (!first(0, 0) || !first(0, 1)) return ERR_BK1_MMA;
    for (int s = 0; s < g.total; ++s) {
        if (!second(s, 0)) return ERR_BK1_MMA;
        if (s + 1 < g.total && !first(s + 1, 0)) return ERR_BK1_MMA;
        if (!second(s, 1)) return ERR_BK1_MMA;
        tc_commit(&bars[BK1_AB_EMPTY + (s & 1)]);
        if (s + 1 < g.total && !first(s + 1, 1)) return ERR_BK1_MMA;
    }
    tc_commit(&bars[BK1_DONE]);
    return 0;
}

// ---------------------------------------------------------------- compute (warps 2-5)
__device__ __forceinline__ int bk1_compute(const BwdParams &P, const Bk1Geom &g, uint32_t tmem, const float *stats,
                                           uint64_t *bars, volatile int *abort_flag) {
    const KernelParams &kp = P.kp;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = (warp & 3) * 32 + lane;          // key row within the tile = TMEM lane
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const int hk = blockIdx.y, b = blockIdx.z;
    const int j = g.j0 + r;
    const bool jv = j < kp.nk1;
    const float c = P.c;

    int s = 0, tile_counter = 0;
    for (int hh = 0; hh < kp.g; ++hh) {
        for (int t = 0; t < g.n_it; ++t, ++tile_counter) {
            const int it0 = g.i_lo + TQ * t;
            const int ne = bk1_sweeps(kp, g, t);
            const float *st = stats + (tile_counter & 1) * 256;
            const int base = j - kp.off1 - it0;                       // column of the diagonal i + off1 == j
            const int hi_all = jv ? min(min(TQ - 1, base + kp.w1 - 1), g.i_hi - it0) : -1;
            for (int e = 0; e < ne; ++e, ++s) {
                // the builders' statistics (written before they signalled this stage) must be visible
                if (e == 0 && !warp_wait(&bars[BK1_AB_FULL + (s & 1)], (s >> 1) & 1, abort_flag)) return ERR_BK1_COMPUTE;
                const int lo_all = max(max(0, base), e - kp.off2 - it0);
#pragma unroll 1
                for (int half = 0; half < 2; ++half) {
                    if (!warp_wait(&bars[BK1_S_FULL + half], s & 1, abort_flag)) return ERR_BK1_COMPUTE;
                    tc_fence_after();
                    const int lo = lo_all - half * 64, hi = hi_all - half * 64;     // valid columns: lo <= col <= hi
                    const bool full = __all_sync(0xffffffffu, lo <= 0 && hi >= 63);
                    uint32_t pp[32], gg[32];
#pragma unroll
                    for (int ch = 0; ch < 2; ++ch) {
                        uint32_t sv[32], dv[32];
                        tmem_ld32(lane_addr + half * 128 + ch * 32, sv);
                        tmem_ld32(lane_addr + half * 128 + 64 + ch * 32, dv);
                        tmem_wait_ld();
                        const float4 *l4 = reinterpret_cast<const float4 *>(st + half * 64 + ch * 32);
                        const float4 *d4 = reinterpret_cast<const float4 *>(st + 128 + half * 64 + ch * 32);
#pragma unroll
                        for (int x4 = 0; x4 < 8; ++x4) {
                            const float4 lv = l4[x4], dl = d4[x4];
                            const float ls[4] = {lv.x, lv.y, lv.z, lv.w};
                            const float ds[4] = {dl.x, dl.y, dl.z, dl.w};
                            float p[4], gq[4];
#pragma unroll
                            for (int z = 0; z < 4; ++z) {
                                const int x = x4 * 4 + z;
                                float pv = ex2(fmaf(__uint_as_float(sv[x]), c, -ls[z]));
                                if (!full) {
                                    const int col = ch * 32 + x;
                                    pv = (col >= lo && col <= hi) ? pv : 0.f;
                                }
                                p[z] = pv;
                                gq[z] = pv * (__uint_as_float(dv[x]) - ds[z]);
                            }
                            pp[ch * 16 + x4 * 2] = pack_bf16(p[0], p[1]);
                            pp[ch * 16 + x4 * 2 + 1] = pack_bf16(p[2], p[3]);
                            gg[ch * 16 + x4 * 2] = pack_bf16(gq[0], gq[1]);
                            gg[ch * 16 + x4 * 2 + 1] = pack_bf16(gq[2], gq[3]);
                        }
                    }
                    tmem_st32(lane_addr + half * 128, pp);
                    tmem_st32(lane_addr + half * 128 + 64, gg);
                    tmem_wait_st();
                    tc_fence_before();
                    mbar_arrive(&bars[BK1_P_FULL + half]);
                }
            }
        }
    }
    // drain dK1, dV1
    if (!warp_wait(&bars[BK1_DONE], 0, abort_flag)) return ERR_BK1_COMPUTE;
    tc_fence_after();
    const bool gbf16 = kp.grad_bf16 != 0;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
        const TensorRef &dst = which == 0 ? kp.dk1 : kp.dv1;
        const float mul = which == 0 ? kp.scale : 1.f;
#pragma unroll 1
        for (int hf = 0; hf < 2; ++hf) {
            uint32_t w[32];
            tmem_ld32(lane_addr + 256 + which * 64 + hf * 32, w);
            tmem_wait_ld();
            if (jv) {
                const int64_t off = elem_off(dst, b, j, hk) + hf * 32;
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    float x[4];
#pragma unroll
                    for (int z = 0; z < 4; ++z) x[z] = (g.total > 0 ? __uint_as_float(w[u * 4 + z]) : 0.f) * mul;
                    store_vec<4>(dst.p, off + u * 4, gbf16, x);
                }
            }
        }
    }
    return 0;
}

__global__ void __launch_bounds__(BK1_THREADS, 1)
bwd_k1_kernel(const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV, const BwdParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sK = smem;
    uint8_t *sV = sK + TILE_BYTES;
    uint8_t *sAB = sV + TILE_BYTES;                       // 2 stages x (A tile, B tile)
    float *stats = reinterpret_cast<float *>(sAB + 4 * TILE_BYTES);   // 2 buffers x (lse2[128], D[128])
    uint64_t *bars = reinterpret_cast<uint64_t *>(stats + 512);
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + BK1_BAR_COUNT);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int x = 0; x < BK1_BAR_COUNT; ++x) {
            const bool many = (x >= BK1_AB_FULL && x < BK1_AB_FULL + 2) || (x >= BK1_P_FULL && x < BK1_P_FULL + 2);
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
    const Bk1Geom g = bk1_geom(P.kp);

    int err = 0;
    if (warp == 0) {
        if (lane == 0 && g.total > 0) {
            prefetch_tmap(&mapK);
            prefetch_tmap(&mapV);
            mbar_arrive_expect_tx(&bars[BK1_KV_FULL], 2 * TILE_BYTES);
            tma_load_4d(sK, &mapK, &bars[BK1_KV_FULL], 0, blockIdx.y, g.j0, blockIdx.z);
            tma_load_4d(sV, &mapV, &bars[BK1_KV_FULL], 0, blockIdx.y, g.j0, blockIdx.z);
            // the tile must have landed before the CTA may exit, even if every other role gave up
            if (!mbar_wait(&bars[BK1_KV_FULL], 0, abort_flag)) err = ERR_BK1_PRODUCER;
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            if (g.total > 0) err = bk1_mma(g, tmem, sK, sV, sAB, bars, abort_flag);
            else tc_commit(&bars[BK1_DONE]);
        }
        __syncwarp();
    } else if (warp < 6) {
        err = bk1_compute(P, g, tmem, stats, bars, abort_flag);
    } else {
        err = bk1_builder(P, g, sAB, stats, bars, abort_flag);
    }
    if (err) atomicOr(P.status, err);

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace tc
}  // namespace sa2
