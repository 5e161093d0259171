// Forward kernel on the 5th-generation tensor cores (tcgen05 + TMEM + TMA),
// bf16 operands, fp32 accumulation, head dim 64.
//
// One CTA owns 128 query rows of one (batch, query head).  For every offset
// e = i - k of the second key ("sweep") it forms A_e[i,:] = q_i * k2_{i-e}
// (bf16, CUDA cores, 128-byte-swizzled shared memory), multiplies it against
// the TMA-staged K1 tiles of the window (S = A_e K1^T, 128x128x64 per tile,
// accumulator in TMEM), turns S into P = exp2(c*S - ref) in registers, writes
// P back to TMEM as bf16 and feeds it as the A operand of W_e += P V1
// (128x64x128, V1 tile as an MN-major B operand).  At the end of a sweep the
// row owner adds v2_{i-e} * W_e to its output registers.  The softmax is
// joint over all (j, e): one reference value, one denominator per row.
//
// Warp roles (192 threads):
//   warp 0      TMA producer for the K1/V1 window (loaded once, resident in
//               shared memory) and builder of the A_e tiles (2 stages)
//   warp 1      issues every tcgen05.mma (one lane), owns the TMEM allocation
//   warps 2-5   one thread per query row: softmax, P, output accumulation
//
// TMEM columns: S/P buffer 0 [0,128), S/P buffer 1 [128,256), W buffer 0
// [256,320), W buffer 1 [320,384).  P (bf16, 64 columns) overwrites the first
// half of the S buffer it was computed from.
//
// Reference handling: probabilities are computed against a per-row reference
// that is frozen during a sweep, so the W accumulator in TMEM never needs a
// rescale in the common case; bf16 has fp32's exponent range, so P may exceed 1
// by many orders of magnitude without loss.  Only when a tile holds a logit
// more than 2^64 above the reference (always true for the very first tile,
// whose reference is -inf) does the warp take a slow path: exact tile maximum,
// rescale of the row's partial sums (including W in TMEM), recomputation of P.
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
constexpr int FWD_THREADS = 192;
constexpr int MAX_NT = 5;        // K1/V1 tiles resident in shared memory (head dim 64)
constexpr uint32_t TILE_BYTES = TJ * 64 * 2;

enum FwdBar {
    BAR_KV_FULL = 0,                 // [MAX_NT]
    BAR_A_FULL = BAR_KV_FULL + MAX_NT,   // [2]
    BAR_A_EMPTY = BAR_A_FULL + 2,
    BAR_S_FULL = BAR_A_EMPTY + 2,
    BAR_P_FULL = BAR_S_FULL + 2,
    BAR_W_FULL = BAR_P_FULL + 2,
    BAR_W_EMPTY = BAR_W_FULL + 2,
    BAR_PV_DONE = BAR_W_EMPTY + 2,
    BAR_COUNT = BAR_PV_DONE + 2
};

// error bits reported through the device status word
enum { ERR_FWD_PRODUCER = 1, ERR_FWD_MMA = 2, ERR_FWD_SOFTMAX = 4 };

struct FwdParams {
    KernelParams kp;
    int nt;          // tiles per query tile: ceil((w1 + 127) / 128), <= MAX_NT
    float c;         // scale * log2(e)
    int *status;     // device status word
};

// at least 120 KB: one CTA per SM, so the 512-column TMEM allocation never waits for a co-resident CTA
inline size_t fwd_smem_bytes(int nt) {
    const size_t need = 1024 + (size_t)nt * 2 * TILE_BYTES + 2 * TILE_BYTES + 256;
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
__device__ __forceinline__ uint32_t max_bf16x2(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hmax2(*reinterpret_cast<__nv_bfloat162 *>(&a), *reinterpret_cast<__nv_bfloat162 *>(&b));
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ float bf16x2_max_as_float(uint32_t a) {
    __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162 *>(&a);
    return fmaxf(__low2float(v), __high2float(v));
}

// every lane of the warp waits; the result is uniform so that the .sync.aligned
// tcgen05 instructions that follow are never reached by a partial warp
__device__ __forceinline__ bool warp_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag));
}

struct FwdGeom {
    int i0, i_last, jbase, t_first, ntiles, nsweeps, total;
};

__device__ __forceinline__ FwdGeom fwd_geom(const FwdParams &P) {
    FwdGeom g;
    g.i0 = blockIdx.x * TQ;
    g.i_last = min(g.i0 + TQ - 1, P.kp.n - 1);
    g.jbase = g.i0 + P.kp.off1 + TJ - TJ * P.nt;      // tile t covers rows jbase + 128 t ... + 127
    g.t_first = g.jbase >= 0 ? 0 : min(P.nt - 1, (-g.jbase) / TJ);
    g.ntiles = P.nt - g.t_first;
    g.nsweeps = min(P.kp.w2, g.i_last + P.kp.off2 + 1);
    g.total = g.ntiles * g.nsweeps;
    return g;
}

// ------------------------------------------------------------------ warp 0
__device__ __forceinline__ int fwd_producer(const FwdParams &P, const FwdGeom &g, const CUtensorMap *mapK, const CUtensorMap *mapV,
                                            uint8_t *sK, uint8_t *sV, uint8_t *sA, uint64_t *bars, volatile int *abort_flag) {
    const KernelParams &kp = P.kp;
    const int lane = threadIdx.x & 31;
    const int h = blockIdx.y, b = blockIdx.z, hk = h / kp.g;
    if (lane == 0) {
        prefetch_tmap(mapK);
        prefetch_tmap(mapV);
        for (int t = P.nt - 1; t >= g.t_first; --t) {      // the diagonal tile first
            mbar_arrive_expect_tx(&bars[BAR_KV_FULL + t], 2 * TILE_BYTES);
            tma_load_4d(sK + (size_t)t * TILE_BYTES, mapK, &bars[BAR_KV_FULL + t], 0, hk, g.jbase + TJ * t, b);
            tma_load_4d(sV + (size_t)t * TILE_BYTES, mapV, &bars[BAR_KV_FULL + t], 0, hk, g.jbase + TJ * t, b);
        }
    }
    const __nv_bfloat16 *q = reinterpret_cast<const __nv_bfloat16 *>(kp.q.p);
    const __nv_bfloat16 *k2 = reinterpret_cast<const __nv_bfloat16 *>(kp.k2.p);
    for (int e = 0; e < g.nsweeps; ++e) {
        const int stage = e & 1;
        if (e >= 2 && !warp_wait(&bars[BAR_A_EMPTY + stage], ((e >> 1) - 1) & 1, abort_flag)) return ERR_FWD_PRODUCER;
        uint8_t *dst = sA + (size_t)stage * TILE_BYTES;
#pragma unroll 4
        for (int it = 0; it < 32; ++it) {
            const int chunk = it * 32 + lane;
            const int r = chunk >> 3, c = chunk & 7;
            const int i = g.i0 + r, kk = i + kp.off2 - e;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (i < kp.n && kk >= 0) {
                const uint4 a = *reinterpret_cast<const uint4 *>(q + elem_off(kp.q, b, i, h) + c * 8);
                const uint4 k = *reinterpret_cast<const uint4 *>(k2 + elem_off(kp.k2, b, kk, hk) + c * 8);
                v.x = mul_bf16x2(a.x, k.x); v.y = mul_bf16x2(a.y, k.y);
                v.z = mul_bf16x2(a.z, k.z); v.w = mul_bf16x2(a.w, k.w);
            }
            *reinterpret_cast<uint4 *>(dst + sw128_offset(r, c)) = v;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[BAR_A_FULL + stage]);
    }
    return 0;
}

// ------------------------------------------------------------------ warp 1 (one lane)
__device__ __forceinline__ int fwd_mma(const FwdParams &P, const FwdGeom &g, uint32_t tmem, uint8_t *sK, uint8_t *sV, uint8_t *sA,
                                       uint64_t *bars, volatile int *abort_flag) {
    constexpr uint32_t IDESC_S = idesc_bf16(128, 128, false, false);
    constexpr uint32_t IDESC_PV = idesc_bf16(128, 64, false, true);
    const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aA = smem_u32(sA);

    auto issue_s = [&](int t) -> bool {
        const int e = t / g.ntiles, jt = t % g.ntiles, tile = g.t_first + jt, buf = t & 1, stage = e & 1;
        if (jt == 0 && !mbar_wait(&bars[BAR_A_FULL + stage], (e >> 1) & 1, abort_flag)) return false;
        if (e == 0 && !mbar_wait(&bars[BAR_KV_FULL + tile], 0, abort_flag)) return false;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 4; ++k)
            mma_ss(tmem + buf * 128, smem_desc_sw128(aA + stage * TILE_BYTES + 32 * k),
                   smem_desc_sw128(aK + tile * TILE_BYTES + 32 * k), IDESC_S, k > 0);
        tc_commit(&bars[BAR_S_FULL + buf]);
        if (jt == g.ntiles - 1) tc_commit(&bars[BAR_A_EMPTY + stage]);
        return true;
    };

    if (!issue_s(0)) return ERR_FWD_MMA;
    for (int t = 0; t < g.total; ++t) {
        const int e = t / g.ntiles, jt = t % g.ntiles, tile = g.t_first + jt, buf = t & 1, wb = e & 1;
        if (t + 1 < g.total && !issue_s(t + 1)) return ERR_FWD_MMA;
        if (!mbar_wait(&bars[BAR_P_FULL + buf], (t >> 1) & 1, abort_flag)) return ERR_FWD_MMA;
        if (jt == 0 && e >= 2 && !mbar_wait(&bars[BAR_W_EMPTY + wb], ((e >> 1) - 1) & 1, abort_flag)) return ERR_FWD_MMA;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)
            mma_ts(tmem + 256 + wb * 64, tmem + buf * 128 + 8 * k, smem_desc_sw128(aV + tile * TILE_BYTES + 2048 * k),
                   IDESC_PV, (jt > 0 || k > 0) ? 1u : 0u);
        tc_commit(&bars[BAR_PV_DONE + buf]);
        if (jt == g.ntiles - 1) tc_commit(&bars[BAR_W_FULL + wb]);
    }
    return 0;
}

// ------------------------------------------------------------------ warps 2-5
__device__ __forceinline__ int fwd_softmax(const FwdParams &P, const FwdGeom &g, uint32_t tmem, uint64_t *bars, volatile int *abort_flag) {
    const KernelParams &kp = P.kp;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = (warp & 3) * 32 + lane;            // query row within the tile = TMEM lane
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const int h = blockIdx.y, b = blockIdx.z, hk = h / kp.g;
    const int i = g.i0 + r;
    const bool row_ok = i < kp.n;
    const float c = P.c;
    const __nv_bfloat16 *v2 = reinterpret_cast<const __nv_bfloat16 *>(kp.v2.p);

    float ref = -CUDART_INF_F, m_run = -CUDART_INF_F, l = 0.f;
    float ref_w[2] = {-CUDART_INF_F, -CUDART_INF_F};
    float o[64];
#pragma unroll
    for (int x = 0; x < 64; ++x) o[x] = 0.f;

    // add v2_{i-e} * W_e (TMEM) into the output registers
    auto drain = [&](int e) -> bool {
        const int wb = e & 1;
        if (!warp_wait(&bars[BAR_W_FULL + wb], (e >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const int kk = i + kp.off2 - e;
        const bool ok = row_ok && kk >= 0 && ref_w[wb] > -CUDART_INF_F;
        const float f = ok ? ex2(ref_w[wb] - ref) : 0.f;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            uint32_t w[32];
            tmem_ld32(lane_addr + 256 + wb * 64 + half * 32, w);
            tmem_wait_ld();
            if (ok) {
                const __nv_bfloat16 *vp = v2 + elem_off(kp.v2, b, kk, hk) + half * 32;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint4 raw = *reinterpret_cast<const uint4 *>(vp + u * 8);
                    const uint32_t rr[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                    for (int z = 0; z < 4; ++z) {
                        const __nv_bfloat162 vv = *reinterpret_cast<const __nv_bfloat162 *>(&rr[z]);
                        const int x = half * 32 + u * 8 + z * 2;
                        o[x] = fmaf(f * __uint_as_float(w[u * 8 + z * 2]), __low2float(vv), o[x]);
                        o[x + 1] = fmaf(f * __uint_as_float(w[u * 8 + z * 2 + 1]), __high2float(vv), o[x + 1]);
                    }
                }
            }
        }
        tc_fence_before();
        mbar_arrive(&bars[BAR_W_EMPTY + wb]);
        return true;
    };

    for (int e = 0; e < g.nsweeps; ++e) {
        const bool sweep_ok = row_ok && (i + kp.off2 - e >= 0);
        // move the reference up to the running maximum between sweeps (registers only)
        if (m_run - ref > 8.f) {
            const float f = ex2(ref - m_run);
            l *= f;
#pragma unroll
            for (int x = 0; x < 64; ++x) o[x] *= f;
            ref = m_run;
        }
        ref_w[e & 1] = ref;
        uint32_t pmax2 = 0u;

        for (int jt = 0; jt < g.ntiles; ++jt) {
            const int t = e * g.ntiles + jt, buf = t & 1;
            const int j0 = g.jbase + TJ * (g.t_first + jt);
            // valid columns of this row: lo < col <= hi
            const int d1 = i + kp.off1 - j0;
            const int hi = sweep_ok ? min(d1, TJ - 1) : -1;
            const int lo = max(d1 - kp.w1, -j0 - 1);
            if (!warp_wait(&bars[BAR_S_FULL + buf], (t >> 1) & 1, abort_flag)) return ERR_FWD_SOFTMAX;
            tc_fence_after();
            const bool full = __all_sync(0xffffffffu, lo < 0 && hi >= TJ - 1);

            uint32_t pp[64];
            float tile_sum = 0.f;
            for (int pass = 0; pass < 2; ++pass) {
                tile_sum = 0.f;
                uint32_t tmax2 = 0u;
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint32_t s[32];
                    tmem_ld32(lane_addr + buf * 128 + ch * 32, s);
                    tmem_wait_ld();
                    if (full) {
#pragma unroll
                        for (int x = 0; x < 32; x += 2) {
                            const float p0 = ex2(fmaf(__uint_as_float(s[x]), c, -ref));
                            const float p1 = ex2(fmaf(__uint_as_float(s[x + 1]), c, -ref));
                            tile_sum += p0 + p1;
                            const uint32_t pk = pack_bf16(p0, p1);
                            tmax2 = max_bf16x2(tmax2, pk);
                            pp[ch * 16 + (x >> 1)] = pk;
                        }
                    } else {
#pragma unroll
                        for (int x = 0; x < 32; x += 2) {
                            const int col = ch * 32 + x;
                            float p0 = ex2(fmaf(__uint_as_float(s[x]), c, -ref));
                            float p1 = ex2(fmaf(__uint_as_float(s[x + 1]), c, -ref));
                            p0 = (col > lo && col <= hi) ? p0 : 0.f;
                            p1 = (col + 1 > lo && col + 1 <= hi) ? p1 : 0.f;
                            tile_sum += p0 + p1;
                            const uint32_t pk = pack_bf16(p0, p1);
                            tmax2 = max_bf16x2(tmax2, pk);
                            pp[ch * 16 + (x >> 1)] = pk;
                        }
                    }
                }
                const float tmax = bf16x2_max_as_float(tmax2);
                const bool exceed = !(tmax <= 1.8446744e19f);      // above 2^64, inf or NaN
                if (pass == 1 || !__any_sync(0xffffffffu, exceed)) {
                    pmax2 = max_bf16x2(pmax2, tmax2);
                    break;
                }
                // ---- slow path (whole warp): exact tile maximum, rescale, recompute
                float mx = -CUDART_INF_F;
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint32_t s[32];
                    tmem_ld32(lane_addr + buf * 128 + ch * 32, s);
                    tmem_wait_ld();
#pragma unroll
                    for (int x = 0; x < 32; ++x) {
                        const int col = ch * 32 + x;
                        if (col > lo && col <= hi) mx = fmaxf(mx, __uint_as_float(s[x]));
                    }
                }
                float f = 1.f;
                if (exceed) {
                    // fold what this sweep has seen so far into the running maximum, then re-reference
                    const float seen = bf16x2_max_as_float(pmax2);
                    if (seen > 0.f) m_run = fmaxf(m_run, ref + lg2(seen));
                    const float nref = mx * c;
                    f = ex2(ref - nref);                       // 0 when ref was -inf
                    l *= f;
#pragma unroll
                    for (int x = 0; x < 64; ++x) o[x] *= f;
                    ref = nref;
                    m_run = fmaxf(m_run, nref);
                    ref_w[e & 1] = nref;
                    pmax2 = 0u;
                }
                if (jt > 0) {
                    // W of this sweep already holds partial sums against the old reference
                    const int tp = t - 1;
                    if (!warp_wait(&bars[BAR_PV_DONE + (tp & 1)], (tp >> 1) & 1, abort_flag)) return ERR_FWD_SOFTMAX;
                    tc_fence_after();
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint32_t w[32];
                        tmem_ld32(lane_addr + 256 + (e & 1) * 64 + half * 32, w);
                        tmem_wait_ld();
#pragma unroll
                        for (int x = 0; x < 32; ++x) w[x] = __float_as_uint(__uint_as_float(w[x]) * f);
                        tmem_st32(lane_addr + 256 + (e & 1) * 64 + half * 32, w);
                    }
                    tmem_wait_st();
                }
            }
            l += tile_sum;

            // P (bf16) over the first 64 columns of the S buffer it came from
            {
                uint32_t half0[32], half1[32];
#pragma unroll
                for (int x = 0; x < 32; ++x) { half0[x] = pp[x]; half1[x] = pp[32 + x]; }
                tmem_st32(lane_addr + buf * 128, half0);
                tmem_st32(lane_addr + buf * 128 + 32, half1);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&bars[BAR_P_FULL + buf]);

            if (jt == 0 && e >= 1 && !drain(e - 1)) return ERR_FWD_SOFTMAX;
        }
        const float seen = bf16x2_max_as_float(pmax2);
        if (seen > 0.f) m_run = fmaxf(m_run, ref + lg2(seen));
    }
    if (!drain(g.nsweeps - 1)) return ERR_FWD_SOFTMAX;

    if (row_ok) {
        const float inv = 1.f / l;
        __nv_bfloat16 *op = reinterpret_cast<__nv_bfloat16 *>(kp.out.p) + elem_off(kp.out, b, i, h);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            uint4 v;
            v.x = pack_bf16(o[u * 8 + 0] * inv, o[u * 8 + 1] * inv);
            v.y = pack_bf16(o[u * 8 + 2] * inv, o[u * 8 + 3] * inv);
            v.z = pack_bf16(o[u * 8 + 4] * inv, o[u * 8 + 5] * inv);
            v.w = pack_bf16(o[u * 8 + 6] * inv, o[u * 8 + 7] * inv);
            *reinterpret_cast<uint4 *>(op + u * 8) = v;
        }
        kp.lse[((int64_t)b * kp.hq + h) * kp.n + i] = (ref + lg2(l)) * 0.6931471805599453f;
    }
    return 0;
}

__global__ void __launch_bounds__(FWD_THREADS, 1)
fwd_kernel(const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV, const FwdParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sK = smem;
    uint8_t *sV = sK + (size_t)P.nt * TILE_BYTES;
    uint8_t *sA = sV + (size_t)P.nt * TILE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sA + 2 * TILE_BYTES);
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + BAR_COUNT);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        for (int x = 0; x < BAR_COUNT; ++x) {
            const bool many = (x >= BAR_P_FULL && x < BAR_P_FULL + 2) || (x >= BAR_W_EMPTY && x < BAR_W_EMPTY + 2);
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
    if (warp == 0) {
        err = fwd_producer(P, g, &mapK, &mapV, sK, sV, sA, bars, abort_flag);
    } else if (warp == 1) {
        if ((threadIdx.x & 31) == 0) err = fwd_mma(P, g, tmem, sK, sV, sA, bars, abort_flag);
        __syncwarp();
    } else {
        err = fwd_softmax(P, g, tmem, bars, abort_flag);
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
