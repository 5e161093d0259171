// Backward kernel for dQ, dK2, dV2 on tcgen05 tensor cores (bf16 operands,
// fp32 accumulation in TMEM, head dim 64 or 128), plus the reduction of its
// partials.
//
// A CTA owns 128 query rows i of one (batch, query head) and a subset ("split")
// of the 128-row K1/V1 tiles of their window.  Because the backward recomputes
// probabilities from the saved logsumexp, the splits of one query tile are
// independent; each writes fp32 partials to scratch and a small second kernel
// adds them in a fixed order (splits, then the query heads of a kv group), so
// results are reproducible.
// Head dim 64: a split keeps its (at most three) tiles resident in shared memory; a 5-tile window is
// two splits.
// Head dim 128: a CTA produces 64 of the 128 output channels (blockIdx.x also carries the channel
// half): S and dP contract over all 128 channels, U and W use the 64-channel block of K1 / V1 as their
// B operand, so the fold, its registers and the shared accumulators are those of head dim 64.  Shared
// memory cannot hold a window at this head dim, so one CTA walks the whole window (one split) and its
// 64-row units stream through a three-slot TMA ring (32 KB per slot), once per sweep, from L2: a slot is
// refilled when the U / W products of its unit are done, one unit ahead of the S / dP products that need it.
//
// Per offset e ("sweep") one warp group forms A_e = q_i * k2_{i-e} and B_e = dO_i * v2_{i-e}; per 64-key
// unit the tensor cores compute
//     S = A_e K1^T      dP = B_e V1^T                 (rows i, columns j)
// the compute warps (one thread per query row and half of the unit's columns) form
//     P = exp2(c S - lse2_i)     G = P * (dP - D_i)    (bf16, back into TMEM)
// and the tensor cores accumulate over the sweep
//     U_e += G K1       W_e += P V1                    (K1/V1 as MN-major B)
// At the end of a sweep the row owner folds U_e, W_e into
//     dQ_i += U_e * k2_{i-e}                           (registers)
//     dK2_{i-e} += U_e * q_i,  dV2_{i-e} += W_e * dO_i (fp32 rows in shared memory)
// Row i-e of the shared accumulators is touched by exactly one thread per
// sweep, so the read-modify-write needs no atomics (see BqAcc for how the rows are kept).
//
// Warps (512 threads, four aligned warpgroups): 0 issuer of U (head dim 64: after loading the tiles; head dim 128:
// of U and W); 1 TMEM owner and issuer of S; 2 issuer of dP; 3 issuer of W (head dim 128: TMA producer of the
// ring); 4-7 and 8-11 two compute groups, each forming 32 of the 64 columns of every unit (P, G); 12-15 form A_e
// and B_e of the next sweep, then fold U, W of the last one into dQ / dK2 / dV2 (head dim 64: the q and dO rows
// stay in their registers for both).
// Every thread starts with 128 registers; the issuer warpgroup keeps 40 (setmaxnreg), the compute groups 120
// each and the fold group takes 232.
// TMEM columns: S / dP buffer x -> S/P [128x, 128x+64), dP/G [128x+64, 128x+128); P and G (bf16, 16 columns per
// 32 keys) overwrite the first half of the S and dP columns of the same keys - columns that the writing compute
// group has itself read - so a buffer is busy from the issue of S / dP until the U / W products of its unit are
// done.  Head dim 64 has three such buffers in flight (issue, compute and U / W of different units overlap) and
// one U / W accumulator pair [384, 512), which the fold group reads into registers before the next sweep's
// first product; head dim 128 has two buffers and U / W per sweep parity at [256 + 128p, +128).
#pragma once
#include "sa2_tc_bwd_k1.cuh"

namespace sa2 {
namespace tc {

constexpr int BQ_THREADS = 512;
// Register hand-over between warpgroups.  Four warps per scheduler partition start with 128 registers a
// thread; a group can only grow by what another has released, or its setmaxnreg never returns, so the
// four budgets must add up to 4 * 128.
constexpr int BQ_REGS_LAUNCH = 128, BQ_REGS_ISSUE = 40, BQ_REGS_COMPUTE = 120;
// The fold group (232) holds dQ and, at head dim 64, the q and dO rows, plus either the operand rows of the next
// sweep or a k2 row and chunks of U and W.  (With one compute group at head dim 128 - NCG = 1 - warps 8-11 form
// A_e with 144 registers and the fold group keeps 208.)
template <int D> struct BqCfg {
    static constexpr int CH = D / 64;                            // channel halves = CTAs per (query tile, split)
    static constexpr int KSTEPS = D / 16;                        // K = 16 steps of S and dP
    static constexpr uint32_t BLK = TJ * 128;                    // A_e / B_e: one [128 rows][64 channels] swizzled block
    static constexpr uint32_t TILE = (D / 64) * BLK;             // A_e or B_e
    // K1 / V1 in shared memory: head dim 64 keeps three 128-row tiles of 16 KB resident; head dim 128 has a
    // ring of three 64-row units, each two [64 rows][64 channels] blocks of 8 KB
    static constexpr int NSLOT = 3;
    static constexpr uint32_t KV_BYTES = D == 64 ? 3 * BLK : NSLOT * 16384;
    static constexpr uint32_t UBLK = 8192;                       // one channel block of a 64-row unit (head dim 128)
    static constexpr int NBUF = D == 64 ? 3 : 2;                 // S / dP (P / G) buffers in TMEM
    static constexpr int UWBUF = D == 64 ? 1 : 2;                // U / W accumulator pairs in TMEM
    static constexpr int NCG = 2;                                // compute groups (1 is still supported at head dim 128)
    static constexpr uint32_t UW0 = NBUF * 128;                  // first TMEM column of U / W
};
template <int D> struct BqRegs {
    static constexpr bool BUILDERS = D == 128 && BqCfg<D>::NCG == 1;          // warps 8-11 form A_e instead of computing
    static constexpr int FOLD = BUILDERS ? 208 : 232, BUILD = BUILDERS ? 144 : BQ_REGS_COMPUTE;
};
static_assert(BQ_REGS_ISSUE + BQ_REGS_COMPUTE + BqRegs<64>::FOLD + BqRegs<64>::BUILD == 4 * BQ_REGS_LAUNCH, "register pool must balance");
static_assert(BQ_REGS_ISSUE + BQ_REGS_COMPUTE + BqRegs<128>::FOLD + BqRegs<128>::BUILD == 4 * BQ_REGS_LAUNCH, "register pool must balance");
constexpr int BQ_MAX_TILES = 3;          // K1/V1 tiles of one split (head dim 64)
// Shared accumulators of dK2 / dV2: in sweep e thread r adds to slab row r + w2 - 1 - e, so 128 consecutive rows
// are live at a time.
// Head dim 64 keeps all 127 + w2 rows, 68 floats apart (64 + 4: the row-per-thread accesses of a warp spread over
// all banks, and the offsets inside a row are compile-time constants).
// Head dim 128 needs the space for its K1 / V1 ring and keeps a ring of 128 rows (slab row modulo 128): the top
// row of a sweep is complete when thread 127 has added to it; one warp copies it to the slab in global memory at
// the start of the next sweep, and thread 0 then writes (not adds to) the row that takes its place.  A row is 64
// floats; its sixteen 16-byte chunks are XOR-ed with the row number instead of padding.
constexpr int BQ_ACC_RING = 128;
constexpr int BQ_ACC_STRIDE = 68;
constexpr int BQ_MAX_W2 = 56;            // head dim 64: 127 + w2 accumulator rows must fit; also the tested range
template <int D> struct BqAcc {
    static constexpr bool RING = D == 128;
    __host__ __device__ static int rows(int w2) { return RING ? BQ_ACC_RING : 127 + w2; }
    __host__ __device__ static int row_floats() { return RING ? 64 : BQ_ACC_STRIDE; }
    // float index of (slab row, channel col) inside one accumulator array, col % 4 == 0
    __device__ static int off(int slab_row, int col) {
        if constexpr (RING) {
            const int pr = slab_row & (BQ_ACC_RING - 1);
            return pr * 64 + ((((col >> 2) ^ pr) & 15) << 2);
        } else {
            return slab_row * BQ_ACC_STRIDE + col;
        }
    }
};

enum BqBar {
    BQ_KV_FULL = 0,
    BQ_AB_FULL = 1,
    BQ_AB_EMPTY = 2,
    BQ_S_FULL = 3,       // [3] per buffer
    BQ_P_FULL = 6,       // [3]
    BQ_G_DONE = 9,       // [3] the U / W products of the buffer's unit have completed
    BQ_W_FULL = 12,      // [2] per U / W accumulator pair
    BQ_W_EMPTY = 14,     // [2] the fold group holds U / W of the sweep in registers
    BQ_KV_SLOT = 16,     // [3] head dim 128: the K1/V1 unit of the ring slot has landed
    BQ_KV_FREE = 19,     // [3] head dim 128: the U / W products that read the slot have completed
    BQ_FOLD_SYNC = 22,   // every fold thread has added its sweep into the shared accumulators
    BQ_BAR_COUNT = 23
};

enum { ERR_BQ_PRODUCER = 256, ERR_BQ_MMA = 512, ERR_BQ_COMPUTE = 1024, ERR_BQ_BUILDER = 2048 };

struct BqParams {
    KernelParams kp;
    float c;            // scale * log2(e)
    int nt;             // K1/V1 tiles per query tile
    int nsplit;         // CTAs sharing one query tile
    int tiles_per_split;
    int nqt;            // query tiles
    float *part_dq;     // [nsplit][b][n][hq][d]
    float *part_k2;     // [b][hq][nqt][nsplit][2][acc_rows][d]   (dK2 slab, then dV2 slab)
    int *status;
};

inline int bq_acc_rows(int w2) { return 127 + w2; }
template <int D> inline size_t bq_smem_bytes(int w2) {
    return 1024 + (size_t)2 * BqCfg<D>::KV_BYTES + 2 * BqCfg<D>::TILE +
           (size_t)2 * BqAcc<D>::rows(w2) * BqAcc<D>::row_floats() * sizeof(float) + 256;
}
// (a query tile with one split writes dQ itself and needs no partials)
inline size_t bq_part_dq_bytes(const sa2_shape &s, int nsplit) { return nsplit == 1 ? 0 : (size_t)nsplit * s.b * s.n * s.hq * s.d * sizeof(float); }
inline size_t bq_part_k2_bytes(const sa2_shape &s, int nsplit) {
    const size_t nqt = (s.n + TQ - 1) / TQ;
    return (size_t)s.b * s.hq * nqt * nsplit * 2 * bq_acc_rows(s.w2) * s.d * sizeof(float);
}

struct BqGeom {
    int qt, split, chh;          // query tile, split, channel half of this CTA
    int i0, i_last, nsweeps;
    int ubase;                   // first-key row of the CTA's unit 0; unit x covers rows ubase + 64 x ... + 63
    int nunits;                  // 64-key units the CTA visits in every sweep
    int total;                   // nunits * nsweeps
};

template <int D>
__device__ __forceinline__ BqGeom bq_geom(const BqParams &P) {
    BqGeom g;
    const KernelParams &kp = P.kp;
    g.chh = blockIdx.x % BqCfg<D>::CH;
    const int qs = blockIdx.x / BqCfg<D>::CH;
    g.qt = qs / P.nsplit;
    g.split = qs % P.nsplit;
    g.i0 = g.qt * TQ;
    g.i_last = min(g.i0 + TQ - 1, kp.n - 1);
    g.nsweeps = min(kp.w2, g.i_last + kp.off2 + 1);
    if constexpr (D == 64) {
        const int jbase = g.i0 + kp.off1 + TJ - TJ * P.nt;        // tile t covers rows jbase + 128 t ...
        const int t_first = jbase >= 0 ? 0 : min(P.nt - 1, (-jbase) / TJ);
        const int t_begin = max(t_first, g.split * P.tiles_per_split);
        const int t_end = min(P.nt, (g.split + 1) * P.tiles_per_split);
        g.ubase = jbase + TJ * t_begin;
        g.nunits = 2 * max(0, t_end - t_begin);
    } else {
        const int nh = (kp.w1 + TQ - 1 + 63) / 64;                // 64-row units of the window: ceil((w1 + 127) / 64)
        const int hbase = g.i0 + kp.off1 + TQ - 64 * nh;
        const int h_first = hbase >= 0 ? 0 : min(nh - 1, (-hbase) / 64);
        g.ubase = hbase + 64 * h_first;
        g.nunits = nh - h_first;
    }
    g.total = g.nunits * g.nsweeps;
    return g;
}

// ---------------------------------------------------------------- head dim 128: builders of A_e (warps 8-11)
// One thread per query row forms row r of A_e = q_i * k2_{i-e} for every sweep (the fold group forms B_e, see
// bq_build_b); the whole row is fetched before the wait, so that the stage is rebuilt as soon as the tensor
// cores release it.
template <int D>
__device__ __forceinline__ int bq_builder(const BqParams &P, const BqGeom &g, uint8_t *sA, uint64_t *bars, volatile int *abort_flag) {
    const KernelParams &kp = P.kp;
    const int r = threadIdx.x - 256;
    const int h = blockIdx.y, b = blockIdx.z, hk = h / kp.g;
    const int i = g.i0 + r;
    const bool iv = i < kp.n;
    const __nv_bfloat16 *k2 = reinterpret_cast<const __nv_bfloat16 *>(kp.k2.p);
    const __nv_bfloat16 *qp = reinterpret_cast<const __nv_bfloat16 *>(kp.q.p) + elem_off(kp.q, b, iv ? i : 0, h);
    for (int e = 0; e < g.nsweeps; ++e) {
        const int kk = i + kp.off2 - e;
        const bool ok = iv && kk >= 0;
        const __nv_bfloat16 *kp2 = k2 + elem_off(kp.k2, b, ok ? kk : 0, hk);
        uint4 qv[D / 8], kv[D / 8];
#pragma unroll
        for (int cc = 0; cc < D / 8; ++cc) {
            qv[cc] = ok ? __ldg(reinterpret_cast<const uint4 *>(qp + cc * 8)) : make_uint4(0u, 0u, 0u, 0u);
            kv[cc] = ok ? __ldg(reinterpret_cast<const uint4 *>(kp2 + cc * 8)) : make_uint4(0u, 0u, 0u, 0u);
        }
        if (e >= 1 && !warp_wait(&bars[BQ_AB_EMPTY], (e - 1) & 1, abort_flag, 1)) return ERR_BQ_BUILDER;
#pragma unroll
        for (int cc = 0; cc < D / 8; ++cc) {
            uint4 a;
            a.x = mul_bf16x2(qv[cc].x, kv[cc].x); a.y = mul_bf16x2(qv[cc].y, kv[cc].y);
            a.z = mul_bf16x2(qv[cc].z, kv[cc].z); a.w = mul_bf16x2(qv[cc].w, kv[cc].w);
            *reinterpret_cast<uint4 *>(sA + (cc >> 3) * BqCfg<D>::BLK + sw128_offset(r, cc & 7)) = a;
        }
        fence_proxy_async_smem();
        mbar_arrive(&bars[BQ_AB_FULL]);
    }
    return 0;
}

// ---------------------------------------------------------------- issuers of S (warp 1) and dP (warp 2), one lane each
// Unit u (numbered over the whole kernel) is unit u % nunits of sweep u / nunits and uses TMEM buffer u % NBUF.
// One thread issues about one tcgen05.mma per 60-90 cycles, so the two product stages have an issuing
// thread each; U / W are accumulated by one thread only, which keeps the summation order fixed.
// which = 0: S = A_e K1^T into columns [128 buf, +64); which = 1: dP = B_e V1^T into [128 buf + 64, +64).
template <int D>
__device__ __forceinline__ int bq_mma_first(const BqGeom &g, int which, uint32_t tmem, uint8_t *sKV, uint8_t *sAB,
                                            uint64_t *bars, volatile int *abort_flag) {
    using C = BqCfg<D>;
    constexpr uint32_t IDESC_F = idesc_bf16(128, 64, false, false);
    const uint64_t dT = smem_desc_sw128(smem_u32(sKV)), dA = smem_desc_sw128(smem_u32(sAB));
    if constexpr (D == 64) {
        if (!mbar_wait(&bars[BQ_KV_FULL], 0, abort_flag)) return ERR_BQ_MMA;
    }
    int u = 0, buf = 0, use = 0;                         // use = u / NBUF: how often the buffer has been used before
    int slot = 0, suse = 0;                              // head dim 128: ring slot u % NSLOT and u / NSLOT
    for (int e = 0; e < g.nsweeps; ++e) {
        if (!mbar_wait(&bars[BQ_AB_FULL], e & 1, abort_flag, 0, 1)) return ERR_BQ_MMA;
        for (int w = 0; w < g.nunits; ++w, ++u) {
            // the buffer holds P / G of its previous unit until the U / W products of that unit are done
            if (use >= 1 && !mbar_wait(&bars[BQ_G_DONE + buf], (use - 1) & 1, abort_flag, 0, 2)) return ERR_BQ_MMA;
            if constexpr (D == 128) {
                if (!mbar_wait(&bars[BQ_KV_SLOT + slot], suse & 1, abort_flag, 0, 3)) return ERR_BQ_MMA;
            }
            tc_fence_after();
            SA2_PROF_MARK(seg);
            const uint32_t d = tmem + buf * 128 + which * 64;
            if constexpr (D == 64) {
                const uint64_t t = dT + (uint64_t)((w * 8192) >> 4);       // unit w: rows [64 w, +64) of the resident tiles
#pragma unroll
                for (int k = 0; k < 4; ++k) mma_ss(d, dA + 2 * k, t + 2 * k, IDESC_F, k > 0 ? 1u : 0u);
            } else {
                const uint64_t t = dT + (uint64_t)((slot * 2 * C::UBLK) >> 4);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    mma_ss(d, dA + (uint64_t)(((k >> 2) * C::BLK) >> 4) + (uint64_t)((k & 3) * 2),
                           t + (uint64_t)(((k >> 2) * C::UBLK) >> 4) + (uint64_t)((k & 3) * 2), IDESC_F, k > 0 ? 1u : 0u);
            }
            SA2_PROF_LAP(4, seg);                         // issue of the products
            tc_commit(&bars[BQ_S_FULL + buf]);
            SA2_PROF_LAP(5, seg);                         // the commit
            if (++buf == C::NBUF) { buf = 0; ++use; }
            if (++slot == C::NSLOT) { slot = 0; ++suse; }
        }
        tc_commit(&bars[BQ_AB_EMPTY]);
    }
    return 0;
}

// ---------------------------------------------------------------- head dim 128: TMA producer of the K1/V1 ring (warp 3, one lane)
template <int D>
__device__ __forceinline__ int bq_ring_producer(const BqParams &P, const BqGeom &g, const CUtensorMap *mapK, const CUtensorMap *mapV,
                                                uint8_t *sK, uint8_t *sV, uint64_t *bars, volatile int *abort_flag) {
    using C = BqCfg<D>;
    const int hk = blockIdx.y / P.kp.g;
    prefetch_tmap(mapK);
    prefetch_tmap(mapV);
    int w = 0, slot = 0, suse = 0;
    for (int u = 0; u < g.total; ++u) {
        // the slot is free when the U / W products of the unit it held are done
        if (suse >= 1 && !mbar_wait(&bars[BQ_KV_FREE + slot], (suse - 1) & 1, abort_flag, 32, 1)) return ERR_BQ_PRODUCER;
        const int row = g.ubase + 64 * w;
        mbar_arrive_expect_tx(&bars[BQ_KV_SLOT + slot], 4 * C::UBLK);
#pragma unroll
        for (int cb = 0; cb < 2; ++cb) {
            tma_load_4d(sK + slot * 2 * C::UBLK + cb * C::UBLK, mapK, &bars[BQ_KV_SLOT + slot], cb * 64, hk, row, blockIdx.z);
            tma_load_4d(sV + slot * 2 * C::UBLK + cb * C::UBLK, mapV, &bars[BQ_KV_SLOT + slot], cb * 64, hk, row, blockIdx.z);
        }
        if (++w == g.nunits) w = 0;
        if (++slot == C::NSLOT) { slot = 0; ++suse; }
    }
    // every load must have landed before the CTA may exit, even if the consumers gave up
    for (int u = max(0, g.total - C::NSLOT); u < g.total; ++u)
        if (!mbar_wait(&bars[BQ_KV_SLOT + u % C::NSLOT], (u / C::NSLOT) & 1, abort_flag, 32)) return ERR_BQ_PRODUCER;
    return 0;
}

// ---------------------------------------------------------------- issuers of U, W (one lane each)
// part 0 (warp 0; head dim 64: after loading the tiles): U += G K1; part 1 (warp 3): W += P V1; part 2 (head dim
// 128, warp 0): both.  Each accumulator has one issuing thread, which keeps its summation order fixed.
template <int D>
__device__ __forceinline__ int bq_mma_second(const BqParams &P, const BqGeom &g, int part, const CUtensorMap *mapK, const CUtensorMap *mapV,
                                             uint32_t tmem, uint8_t *sK, uint8_t *sV, uint64_t *bars, volatile int *abort_flag) {
    using C = BqCfg<D>;
    constexpr uint32_t IDESC_G = idesc_bf16(128, 64, false, true);
    if constexpr (D == 64) {
        if (part == 0) {
            const int hk = blockIdx.y / P.kp.g;
            prefetch_tmap(mapK);
            prefetch_tmap(mapV);
            const int nt = g.nunits / 2;
            mbar_arrive_expect_tx(&bars[BQ_KV_FULL], 2 * C::BLK * nt);
            for (int t = 0; t < nt; ++t) {
                const int row = g.ubase + TJ * t;
                tma_load_4d(sK + (size_t)t * C::BLK, mapK, &bars[BQ_KV_FULL], 0, hk, row, blockIdx.z);
                tma_load_4d(sV + (size_t)t * C::BLK, mapV, &bars[BQ_KV_FULL], 0, hk, row, blockIdx.z);
            }
        }
        if (!mbar_wait(&bars[BQ_KV_FULL], 0, abort_flag)) return ERR_BQ_PRODUCER;
    }
    // head dim 128: U / W take the CTA's 64-channel block of the unit as an MN-major B operand
    const uint64_t dK = smem_desc_sw128(smem_u32(sK) + (D == 64 ? 0 : g.chh * C::UBLK));
    const uint64_t dV = smem_desc_sw128(smem_u32(sV) + (D == 64 ? 0 : g.chh * C::UBLK));
    int u = 0, buf = 0, use = 0, slot = 0;
    for (int e = 0; e < g.nsweeps; ++e) {
        const int wb = e % C::UWBUF, wuse = e / C::UWBUF;
        const uint32_t tu = tmem + C::UW0 + wb * 128, tw = tu + 64;
        for (int w = 0; w < g.nunits; ++w, ++u) {
            if (!mbar_wait(&bars[BQ_P_FULL + buf], use & 1, abort_flag, 0, 1)) return ERR_BQ_MMA;
            // the fold group must have read the accumulators of the sweep that used them last
            if (w == 0 && wuse >= 1 && !mbar_wait(&bars[BQ_W_EMPTY + wb], (wuse - 1) & 1, abort_flag, 0, 2)) return ERR_BQ_MMA;
            tc_fence_after();
            const uint64_t off = (uint64_t)((D == 64 ? w * 8192 : slot * 2 * C::UBLK) >> 4);
            const uint64_t kt = dK + off, vt = dV + off;
            const uint32_t a = tmem + buf * 128;
            const uint32_t acc = w > 0 ? 1u : 0u;
            if (part != 1) {
                // keys [32 x, +32) of G are 16 columns at 64 + 32 x, those of P at 32 x
                mma_ts(tu, a + 64, kt, IDESC_G, acc);               // U += G K1
                mma_ts(tu, a + 72, kt + 128, IDESC_G, 1u);
                mma_ts(tu, a + 96, kt + 256, IDESC_G, 1u);
                mma_ts(tu, a + 104, kt + 384, IDESC_G, 1u);
            }
            if (part != 0) {
                mma_ts(tw, a, vt, IDESC_G, acc);                    // W += P V1
                mma_ts(tw, a + 8, vt + 128, IDESC_G, 1u);
                mma_ts(tw, a + 32, vt + 256, IDESC_G, 1u);
                mma_ts(tw, a + 40, vt + 384, IDESC_G, 1u);
            }
            tc_commit(&bars[BQ_G_DONE + buf]);
            if constexpr (D == 128) tc_commit(&bars[BQ_KV_FREE + slot]);
            if (++buf == C::NBUF) { buf = 0; ++use; }
            if (++slot == C::NSLOT) slot = 0;
        }
        tc_commit(&bars[BQ_W_FULL + wb]);
    }
    return 0;
}

// ---------------------------------------------------------------- compute (warps 4-7; head dim 64: and 8-11): P and G
// Head dim 64: group cg forms columns [32 cg, +32) of every unit, which halves the time between S / dP and P / G.
template <int D>
__device__ __forceinline__ int bq_compute(const BqParams &P, const BqGeom &g, int cg, uint32_t tmem, uint64_t *bars, volatile int *abort_flag) {
    using C = BqCfg<D>;
    if (cg >= C::NCG) return 0;
    const KernelParams &kp = P.kp;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = (warp & 3) * 32 + lane;             // query row within the tile = TMEM lane
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const int h = blockIdx.y, b = blockIdx.z;
    const int i = g.i0 + r;
    const bool row_ok = i < kp.n;
    const float c = P.c;
    float lse2 = 0.f, dl = 0.f;
    if (row_ok) {
        const int64_t o = ((int64_t)b * kp.hq + h) * kp.n + i;
        lse2 = kp.lse[o] * 1.4426950408889634f;
        dl = kp.delta[o];
    }
#ifdef SA2_PROF
    long long seg_ld = 0, seg_math = 0, seg_st = 0;       // cycles in TMEM loads, arithmetic, TMEM stores and hand-over
#endif
    {
        int e = 0, w = 0;
        for (int u = 0; u < g.total; ++u, ++w) {
            if (w == g.nunits) { w = 0; ++e; }
            const bool sweep_ok = row_ok && (i + kp.off2 - e >= 0);
            {
                const int buf = u % C::NBUF, use = u / C::NBUF;
                const int j0 = g.ubase + 64 * w;
                const int d1 = i + kp.off1 - j0;
                const int hi = sweep_ok ? min(d1, 63) : -1;         // valid columns: lo < col <= hi
                const int lo = max(d1 - kp.w1, -j0 - 1);
                if (!warp_wait(&bars[BQ_S_FULL + buf], use & 1, abort_flag, 1)) return ERR_BQ_COMPUTE;
                tc_fence_after();
                const bool full = __all_sync(0xffffffffu, lo < 0 && hi >= 63);
                const int ch_end = C::NCG == 2 ? cg + 1 : 2;
#pragma unroll 1
                for (int ch = C::NCG == 2 ? cg : 0; ch < ch_end; ++ch) {
                    uint32_t sv[32], dv[32], pp[16], gg[16];
                    // no row of this warp has a valid column among these 32: P = G = 0 without reading S / dP
                    if (__all_sync(0xffffffffu, hi < ch * 32 || lo >= ch * 32 + 31)) {
#pragma unroll
                        for (int x = 0; x < 16; ++x) { pp[x] = 0u; gg[x] = 0u; }
                        tmem_st16(lane_addr + buf * 128 + ch * 32, pp);
                        tmem_st16(lane_addr + buf * 128 + 64 + ch * 32, gg);
                        continue;
                    }
#ifdef SA2_PROF
                    const long long seg_t0 = clock64();
#endif
                    tmem_ld32(lane_addr + buf * 128 + ch * 32, sv);
                    tmem_ld32(lane_addr + buf * 128 + 64 + ch * 32, dv);
                    tmem_wait_ld();
#ifdef SA2_PROF
                    const long long seg_t1 = clock64();
                    seg_ld += seg_t1 - seg_t0;
#endif
                    if (full) {
#pragma unroll
                        for (int x = 0; x < 32; x += 2) {
                            const float p0 = ex2(fmaf(__uint_as_float(sv[x]), c, -lse2));
                            const float p1 = ex2(fmaf(__uint_as_float(sv[x + 1]), c, -lse2));
                            pp[x >> 1] = pack_bf16(p0, p1);
                            gg[x >> 1] = pack_bf16(p0 * (__uint_as_float(dv[x]) - dl), p1 * (__uint_as_float(dv[x + 1]) - dl));
                        }
                    } else {
                        // valid columns are the integers in (lo, hi]: saturate(half + 1 - |col - mid|) is exactly 1
                        // inside and 0 outside (FMA pipe instead of compares and selects on the ALU pipe); the
                        // exponent is clamped so that a masked-out cell cannot give inf * 0
                        const float mid = 0.5f * (float)(lo + 1 + hi) - (float)(ch * 32), hwp = 0.5f * (float)(hi - lo - 1) + 1.f;
#pragma unroll
                        for (int x = 0; x < 32; x += 2) {
                            const float v0 = __saturatef(hwp - fabsf((float)x - mid));
                            const float v1 = __saturatef(hwp - fabsf((float)(x + 1) - mid));
                            const float p0 = ex2(fminf(fmaf(__uint_as_float(sv[x]), c, -lse2), 100.f)) * v0;
                            const float p1 = ex2(fminf(fmaf(__uint_as_float(sv[x + 1]), c, -lse2), 100.f)) * v1;
                            pp[x >> 1] = pack_bf16(p0, p1);
                            gg[x >> 1] = pack_bf16(p0 * (__uint_as_float(dv[x]) - dl), p1 * (__uint_as_float(dv[x + 1]) - dl));
                        }
                    }
#ifdef SA2_PROF
                    seg_math += clock64() - seg_t1;
#endif
                    // P / G chunk over the first half of the columns of S / dP that this thread has just read (the
                    // other columns of the buffer may still be unread by the other compute group)
                    tmem_st16(lane_addr + buf * 128 + ch * 32, pp);
                    tmem_st16(lane_addr + buf * 128 + 64 + ch * 32, gg);
                }
#ifdef SA2_PROF
                const long long seg_t2 = clock64();
#endif
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(&bars[BQ_P_FULL + buf]);
#ifdef SA2_PROF
                seg_st += clock64() - seg_t2;
#endif
            }
        }
    }
    SA2_PROF_ADD(4, seg_ld);
    SA2_PROF_ADD(5, seg_math);
    SA2_PROF_ADD(6, seg_st);
    return 0;
}

// ---------------------------------------------------------------- fold (warps 8-11): U, W -> dQ, dK2, dV2
__device__ __forceinline__ void bq_fold_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Head dim 128: the fold thread of query row r forms row r of B_e = dO_i * v2_{i-e} for sweep e (the builder
// group forms A_e); the whole row is fetched before the wait for the stage.
template <int D>
__device__ __forceinline__ bool bq_build_b(const BqParams &P, const BqGeom &g, int e, int r, uint8_t *sB, uint64_t *bars,
                                           volatile int *abort_flag) {
    const KernelParams &kp = P.kp;
    const int h = blockIdx.y, b = blockIdx.z, hk = h / kp.g;
    const int i = g.i0 + r;
    const int kk = i + kp.off2 - e;
    const bool ok = i < kp.n && kk >= 0;
    const __nv_bfloat16 *dp = reinterpret_cast<const __nv_bfloat16 *>(kp.dout.p) + elem_off(kp.dout, b, ok ? i : 0, h);
    const __nv_bfloat16 *vp = reinterpret_cast<const __nv_bfloat16 *>(kp.v2.p) + elem_off(kp.v2, b, ok ? kk : 0, hk);
    uint4 dv[16], vv[16];
#pragma unroll
    for (int cc = 0; cc < 16; ++cc) {
        dv[cc] = ok ? __ldg(reinterpret_cast<const uint4 *>(dp + cc * 8)) : make_uint4(0u, 0u, 0u, 0u);
        vv[cc] = ok ? __ldg(reinterpret_cast<const uint4 *>(vp + cc * 8)) : make_uint4(0u, 0u, 0u, 0u);
    }
    if (e >= 1 && !warp_wait(&bars[BQ_AB_EMPTY], (e - 1) & 1, abort_flag, 3)) return false;
#pragma unroll
    for (int cc = 0; cc < 16; ++cc) {
        uint4 bb;
        bb.x = mul_bf16x2(dv[cc].x, vv[cc].x); bb.y = mul_bf16x2(dv[cc].y, vv[cc].y);
        bb.z = mul_bf16x2(dv[cc].z, vv[cc].z); bb.w = mul_bf16x2(dv[cc].w, vv[cc].w);
        *reinterpret_cast<uint4 *>(sB + (cc >> 3) * BqCfg<D>::BLK + sw128_offset(r, cc & 7)) = bb;
    }
    fence_proxy_async_smem();
    mbar_arrive(&bars[BQ_AB_FULL]);
    return true;
}

template <int D>
__device__ __forceinline__ int bq_fold_body(const BqParams &P, const BqGeom &g, uint32_t tmem, float *acc_k, float *acc_v, float *slab,
                                            uint8_t *sA, uint8_t *sB, uint64_t *bars, volatile int *abort_flag) {
    using C = BqCfg<D>;
    const KernelParams &kp = P.kp;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = (warp & 3) * 32 + lane;             // query row within the tile = TMEM lane
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const int h = blockIdx.y, b = blockIdx.z, hk = h / kp.g;
    const int c0 = g.chh * 64;                        // first channel this CTA produces
    const int i = g.i0 + r;
    const bool row_ok = i < kp.n;
    float dq[64];
#pragma unroll
    for (int x = 0; x < 64; ++x) dq[x] = 0.f;
    const __nv_bfloat16 *qrow = reinterpret_cast<const __nv_bfloat16 *>(kp.q.p) + elem_off(kp.q, b, row_ok ? i : 0, h) + c0;
    const __nv_bfloat16 *dorow = reinterpret_cast<const __nv_bfloat16 *>(kp.dout.p) + elem_off(kp.dout, b, row_ok ? i : 0, h) + c0;
    const __nv_bfloat16 *k2 = reinterpret_cast<const __nv_bfloat16 *>(kp.k2.p) + c0;
    const __nv_bfloat16 *v2 = reinterpret_cast<const __nv_bfloat16 *>(kp.v2.p) + c0;

#ifdef SA2_PROF
    long long seg_build = 0, seg_drain = 0;           // cycles after the waits of a build and of a fold
#endif
    // head dim 64: the q and dO rows serve every A_e / B_e and every fold of this thread
    uint4 qv[8], dv[8];
    if constexpr (D == 64) {
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
            qv[cc] = row_ok ? __ldg(reinterpret_cast<const uint4 *>(qrow + cc * 8)) : make_uint4(0u, 0u, 0u, 0u);
            dv[cc] = row_ok ? __ldg(reinterpret_cast<const uint4 *>(dorow + cc * 8)) : make_uint4(0u, 0u, 0u, 0u);
        }
    }

    // row r of A_e and B_e for sweep e (head dim 64): the second-key rows are fetched before the wait for the stage
    auto build = [&](int e) -> bool {
        if constexpr (D == 64) {
            const int kk = i + kp.off2 - e;
            const bool ok = row_ok && kk >= 0;
            const __nv_bfloat16 *kp2 = k2 + elem_off(kp.k2, b, ok ? kk : 0, hk);
            const __nv_bfloat16 *vp2 = v2 + elem_off(kp.v2, b, ok ? kk : 0, hk);
            uint4 kv[8], vv[8];
#pragma unroll
            for (int cc = 0; cc < 8; ++cc) {
                kv[cc] = ok ? __ldg(reinterpret_cast<const uint4 *>(kp2 + cc * 8)) : make_uint4(0u, 0u, 0u, 0u);
                vv[cc] = ok ? __ldg(reinterpret_cast<const uint4 *>(vp2 + cc * 8)) : make_uint4(0u, 0u, 0u, 0u);
            }
            // the products too are formed before the wait: only the stores follow it
#pragma unroll
            for (int cc = 0; cc < 8; ++cc) {
                uint4 a = make_uint4(0u, 0u, 0u, 0u), bb = make_uint4(0u, 0u, 0u, 0u);
                if (ok) {
                    a.x = mul_bf16x2(qv[cc].x, kv[cc].x); a.y = mul_bf16x2(qv[cc].y, kv[cc].y);
                    a.z = mul_bf16x2(qv[cc].z, kv[cc].z); a.w = mul_bf16x2(qv[cc].w, kv[cc].w);
                    bb.x = mul_bf16x2(dv[cc].x, vv[cc].x); bb.y = mul_bf16x2(dv[cc].y, vv[cc].y);
                    bb.z = mul_bf16x2(dv[cc].z, vv[cc].z); bb.w = mul_bf16x2(dv[cc].w, vv[cc].w);
                }
                kv[cc] = a;
                vv[cc] = bb;
            }
            if (e >= 1 && !warp_wait(&bars[BQ_AB_EMPTY], (e - 1) & 1, abort_flag, 3)) return false;
#ifdef SA2_PROF
            const long long seg_t0 = clock64();
#endif
#pragma unroll
            for (int cc = 0; cc < 8; ++cc) {
                *reinterpret_cast<uint4 *>(sA + sw128_offset(r, cc)) = kv[cc];
                *reinterpret_cast<uint4 *>(sB + sw128_offset(r, cc)) = vv[cc];
            }
            fence_proxy_async_smem();
            mbar_arrive(&bars[BQ_AB_FULL]);
#ifdef SA2_PROF
            seg_build += clock64() - seg_t0;
#endif
            return true;
        } else if constexpr (C::NCG == 2) {
            // head dim 128 with two compute groups: this group forms A_e and B_e.  All four rows are fetched and
            // multiplied before the wait (A_e, then B_e in two halves, to stay within the register budget).
            const int kk = i + kp.off2 - e;
            const bool ok = row_ok && kk >= 0;
            const __nv_bfloat16 *qf = qrow - c0, *df = dorow - c0;
            const __nv_bfloat16 *kp2 = k2 - c0 + elem_off(kp.k2, b, ok ? kk : 0, hk);
            const __nv_bfloat16 *vp2 = v2 - c0 + elem_off(kp.v2, b, ok ? kk : 0, hk);
            uint4 a[16], bb[16];
            {
                uint4 x[16];
#pragma unroll
                for (int cc = 0; cc < 16; ++cc) {
                    a[cc] = ok ? __ldg(reinterpret_cast<const uint4 *>(qf + cc * 8)) : make_uint4(0u, 0u, 0u, 0u);
                    x[cc] = ok ? __ldg(reinterpret_cast<const uint4 *>(kp2 + cc * 8)) : make_uint4(0u, 0u, 0u, 0u);
                }
#pragma unroll
                for (int cc = 0; cc < 16; ++cc) {
                    a[cc].x = mul_bf16x2(a[cc].x, x[cc].x); a[cc].y = mul_bf16x2(a[cc].y, x[cc].y);
                    a[cc].z = mul_bf16x2(a[cc].z, x[cc].z); a[cc].w = mul_bf16x2(a[cc].w, x[cc].w);
                }
            }
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                uint4 x[8];
#pragma unroll
                for (int cc = 0; cc < 8; ++cc) {
                    bb[hf * 8 + cc] = ok ? __ldg(reinterpret_cast<const uint4 *>(df + (hf * 8 + cc) * 8)) : make_uint4(0u, 0u, 0u, 0u);
                    x[cc] = ok ? __ldg(reinterpret_cast<const uint4 *>(vp2 + (hf * 8 + cc) * 8)) : make_uint4(0u, 0u, 0u, 0u);
                }
#pragma unroll
                for (int cc = 0; cc < 8; ++cc) {
                    uint4 &t = bb[hf * 8 + cc];
                    t.x = mul_bf16x2(t.x, x[cc].x); t.y = mul_bf16x2(t.y, x[cc].y);
                    t.z = mul_bf16x2(t.z, x[cc].z); t.w = mul_bf16x2(t.w, x[cc].w);
                }
            }
            if (e >= 1 && !warp_wait(&bars[BQ_AB_EMPTY], (e - 1) & 1, abort_flag, 3)) return false;
#pragma unroll
            for (int cc = 0; cc < 16; ++cc) {
                *reinterpret_cast<uint4 *>(sA + (cc >> 3) * C::BLK + sw128_offset(r, cc & 7)) = a[cc];
                *reinterpret_cast<uint4 *>(sB + (cc >> 3) * C::BLK + sw128_offset(r, cc & 7)) = bb[cc];
            }
            fence_proxy_async_smem();
            mbar_arrive(&bars[BQ_AB_FULL]);
            return true;
        } else {
            return bq_build_b<D>(P, g, e, r, sB, bars, abort_flag);
        }
    };

    auto drain = [&](int v) -> bool {
        const int wb = v % C::UWBUF, e = v;
        const int kk = i + kp.off2 - e;
        const bool ok = row_ok && kk >= 0;
        // the first half of the k2 row is fetched before the wait, so that its latency overlaps the end of the
        // sweep; the second half with U
        const __nv_bfloat16 *kr = k2 + elem_off(kp.k2, b, ok ? kk : 0, hk);
        uint4 k2r[4];
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) k2r[cc] = ok ? __ldg(reinterpret_cast<const uint4 *>(kr + cc * 8)) : make_uint4(0u, 0u, 0u, 0u);
        if (!warp_wait(&bars[BQ_W_FULL + wb], (v / C::UWBUF) & 1, abort_flag, 1)) return false;
        // A row of the shared accumulators is written by thread r in this sweep and by another thread in the
        // last one: every fold thread must have finished that one first.
        if (v >= 1 && !warp_wait(&bars[BQ_FOLD_SYNC], (v - 1) & 1, abort_flag, 2)) return false;
        tc_fence_after();
#ifdef SA2_PROF
        const long long seg_t0 = clock64();
#endif
        const int arow = r + kp.w2 - 1 - e;           // slab row of this thread in this sweep
        const bool fresh = BqAcc<D>::RING && (e == 0 || r == 0);      // ring: nothing has been added to the row yet
        if (BqAcc<D>::RING && v >= 1 && warp == 12) {
            // the top row of the last sweep is complete: it goes to the slab before thread 0 reuses its place
            const int trow = TQ - 1 + kp.w2 - e, arr = lane >> 4, c4 = (lane & 15) * 4;
            const float4 t = *reinterpret_cast<const float4 *>((arr ? acc_v : acc_k) + BqAcc<D>::off(trow, c4));
            *reinterpret_cast<float4 *>(slab + ((size_t)arr * (127 + kp.w2) + trow) * D + c4) = t;
            __syncwarp();
        }
        const bool add = ok || BqAcc<D>::RING;       // (a ring row is written even when this thread has nothing to add)
        // eight channels of one accumulator row += x
        auto rmw8 = [&](float *acc, int col, const float (&x)[8]) {
            if constexpr (BqAcc<D>::RING) {
                // both 16-byte pieces are read before either is written: the swizzled addresses hide from the
                // compiler that they are distinct, and it would order the second read after the first write
                float4 *p0 = reinterpret_cast<float4 *>(acc + BqAcc<D>::off(arow, col));
                float4 *p1 = reinterpret_cast<float4 *>(acc + BqAcc<D>::off(arow, col + 4));
                float4 t0 = make_float4(0.f, 0.f, 0.f, 0.f), t1 = t0;
                if (!fresh) { t0 = *p0; t1 = *p1; }
                t0.x += x[0]; t0.y += x[1]; t0.z += x[2]; t0.w += x[3];
                t1.x += x[4]; t1.y += x[5]; t1.z += x[6]; t1.w += x[7];
                *p0 = t0;
                *p1 = t1;
            } else {
                float4 *p = reinterpret_cast<float4 *>(acc + (size_t)arow * BQ_ACC_STRIDE + col);
                float4 t0 = p[0], t1 = p[1];
                t0.x += x[0]; t0.y += x[1]; t0.z += x[2]; t0.w += x[3];
                t1.x += x[4]; t1.y += x[5]; t1.z += x[6]; t1.w += x[7];
                p[0] = t0;
                p[1] = t1;
            }
        };
        // W first, then U, 32 channels at a time: only 32 registers of U / W are live at once, which keeps this
        // group within its budget without spills (the accumulator pair is released after the last read).
        {
            uint4 dr[8];
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
                if constexpr (D == 64) dr[c8] = dv[c8];
                else dr[c8] = __ldg(reinterpret_cast<const uint4 *>(dorow + c8 * 8));
            }
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                uint32_t w[32];
                tmem_ld32(lane_addr + C::UW0 + wb * 128 + 64 + hf * 32, w);
                tmem_wait_ld();
                if (add) {
#pragma unroll
                    for (int c4 = 0; c4 < 4; ++c4) {
                        const int c8 = hf * 4 + c4;
                        const uint32_t dw[4] = {dr[c8].x, dr[c8].y, dr[c8].z, dr[c8].w};
                        float xv[8];
#pragma unroll
                        for (int z = 0; z < 4; ++z) {
                            const __nv_bfloat162 d2 = *reinterpret_cast<const __nv_bfloat162 *>(&dw[z]);
                            const int x = c4 * 8 + z * 2;
                            xv[z * 2] = ok ? __uint_as_float(w[x]) * __low2float(d2) : 0.f;
                            xv[z * 2 + 1] = ok ? __uint_as_float(w[x + 1]) * __high2float(d2) : 0.f;
                        }
                        rmw8(acc_v, c8 * 8, xv);
                    }
                }
            }
        }
        {
            uint4 qr[8];
#pragma unroll
            for (int c8 = 0; c8 < 8; ++c8) {
                if constexpr (D == 64) qr[c8] = qv[c8];
                else qr[c8] = __ldg(reinterpret_cast<const uint4 *>(qrow + c8 * 8));
            }
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                uint32_t u[32];
                tmem_ld32(lane_addr + C::UW0 + wb * 128 + hf * 32, u);
                if (hf == 1) {
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc)
                        k2r[cc] = ok ? __ldg(reinterpret_cast<const uint4 *>(kr + 32 + cc * 8)) : make_uint4(0u, 0u, 0u, 0u);
                }
                tmem_wait_ld();
                if (hf == 1) {
                    // U and W of the sweep are in registers (or already used): the tensor cores may overwrite them
                    tc_fence_before();
                    mbar_arrive(&bars[BQ_W_EMPTY + wb]);
                }
                if (add) {
#pragma unroll
                    for (int c4 = 0; c4 < 4; ++c4) {
                        const int c8 = hf * 4 + c4;
                        const uint4 kraw = k2r[c4];
                        const uint32_t kw[4] = {kraw.x, kraw.y, kraw.z, kraw.w};
                        const uint32_t qw[4] = {qr[c8].x, qr[c8].y, qr[c8].z, qr[c8].w};
                        float xk[8];
#pragma unroll
                        for (int z = 0; z < 4; ++z) {
                            const __nv_bfloat162 k2v = *reinterpret_cast<const __nv_bfloat162 *>(&kw[z]);
                            const __nv_bfloat162 q2 = *reinterpret_cast<const __nv_bfloat162 *>(&qw[z]);
                            const int x = c4 * 8 + z * 2;
                            const float a0 = __uint_as_float(u[x]), a1 = __uint_as_float(u[x + 1]);
                            dq[c8 * 8 + z * 2] = fmaf(a0, __low2float(k2v), dq[c8 * 8 + z * 2]);
                            dq[c8 * 8 + z * 2 + 1] = fmaf(a1, __high2float(k2v), dq[c8 * 8 + z * 2 + 1]);
                            xk[z * 2] = ok ? a0 * __low2float(q2) : 0.f;
                            xk[z * 2 + 1] = ok ? a1 * __high2float(q2) : 0.f;
                        }
                        rmw8(acc_k, c8 * 8, xk);
                    }
                }
            }
        }
        mbar_arrive(&bars[BQ_FOLD_SYNC]);
#ifdef SA2_PROF
        seg_drain += clock64() - seg_t0;
#endif
        return true;
    };

    const int nv = g.total > 0 ? g.nsweeps : 0;       // a split whose tiles all lie before the sequence start has no work
    int err = 0;
    if (nv > 0 && !build(0)) err = ERR_BQ_COMPUTE;
    for (int v = 0; v < nv && err == 0; ++v) {
        // the operands of the next sweep first: the tensor cores wait for them, U / W of this sweep arrive later
        if (v + 1 < nv && !build(v + 1)) { err = ERR_BQ_COMPUTE; break; }
        if (!drain(v)) err = ERR_BQ_COMPUTE;
    }

    SA2_PROF_ADD(4, seg_build);
    SA2_PROF_ADD(5, seg_drain);
    // dQ of this row (NaN when a wait ran out, so that the failure is visible in the result): with one split per
    // query tile it is final and goes straight to the gradient, otherwise a partial for the reduction kernel
    if (row_ok) {
        const bool bad = err != 0 || *abort_flag != 0;
        if (P.nsplit == 1) {
            const bool gbf16 = kp.grad_bf16 != 0;
            const int64_t o = elem_off(kp.dq, b, i, h) + c0;
#pragma unroll
            for (int x = 0; x < 64; x += 4) {
                float v[4];
#pragma unroll
                for (int z = 0; z < 4; ++z) v[z] = bad ? CUDART_NAN_F : dq[x + z] * kp.scale;
                store_vec<4>(kp.dq.p, o + x, gbf16, v);
            }
        } else {
            float *dst = P.part_dq + ((((size_t)g.split * kp.b + b) * kp.n + i) * kp.hq + h) * D + c0;
#pragma unroll
            for (int x = 0; x < 64; x += 4)
                *reinterpret_cast<float4 *>(dst + x) = bad ? make_float4(CUDART_NAN_F, CUDART_NAN_F, CUDART_NAN_F, CUDART_NAN_F)
                                                           : make_float4(dq[x], dq[x + 1], dq[x + 2], dq[x + 3]);
        }
    }
    return err;
}

template <int D>
__device__ __forceinline__ int bq_fold(const BqParams &P, const BqGeom &g, uint32_t tmem, float *acc_k, float *acc_v, uint8_t *sA, uint8_t *sB,
                                       uint64_t *bars, volatile int *abort_flag) {
    const KernelParams &kp = P.kp;
    const int ft = threadIdx.x - 384;                 // 0..127 among the fold threads
    const int h = blockIdx.y, b = blockIdx.z;
    const int slab_rows = 127 + kp.w2;
    // this CTA's 64 channels of its slab (dK2 rows, then dV2 rows)
    float *slab = P.part_k2 + ((((size_t)b * kp.hq + h) * P.nqt + g.qt) * P.nsplit + g.split) * (size_t)(2 * slab_rows * D) + g.chh * 64;
    if constexpr (!BqAcc<D>::RING) {
        // zero the accumulators (acc_v follows acc_k); only this group touches them
        for (int x = ft; x < 2 * slab_rows * BQ_ACC_STRIDE; x += 128) acc_k[x] = 0.f;
        bq_fold_sync();
    }
    const int err = bq_fold_body<D>(P, g, tmem, acc_k, acc_v, slab, sA, sB, bars, abort_flag);
    // The barrier sits outside the body so that a warp that gave up on a wait still reaches it.
    bq_fold_sync();
    // Ring: rows above the live ones went to the slab when they were completed; the live rows follow now, and
    // the rows below them (second keys before the sequence start, when fewer than w2 sweeps ran) are zero.
    const int nv = g.total > 0 ? g.nsweeps : 0;
    const int live0 = BqAcc<D>::RING ? kp.w2 - nv : 0;                 // first slab row held in shared memory
    const int rows = BqAcc<D>::RING && nv > 0 ? live0 + BQ_ACC_RING : slab_rows;
    const bool held = !BqAcc<D>::RING || nv > 0;
    const bool bad = err != 0 || *abort_flag != 0;     // a CTA in which a wait ran out reports NaN
    for (int x = ft; x < 2 * rows * 16; x += 128) {
        const int arr = x / (rows * 16), y = x - arr * rows * 16;
        const int row = y >> 4, c4 = (y & 15) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (held && row >= live0) v = *reinterpret_cast<const float4 *>((arr ? acc_v : acc_k) + BqAcc<D>::off(row, c4));
        if (bad) v = make_float4(CUDART_NAN_F, CUDART_NAN_F, CUDART_NAN_F, CUDART_NAN_F);
        *reinterpret_cast<float4 *>(slab + ((size_t)arr * slab_rows + row) * D + c4) = v;
    }
    return err;
}

template <int D>
__global__ void __launch_bounds__(BQ_THREADS, 1)
bwd_q_kernel(const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV, const BqParams P) {
    using C = BqCfg<D>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sK = smem;
    uint8_t *sV = sK + C::KV_BYTES;
    uint8_t *sA = sV + C::KV_BYTES;
    uint8_t *sB = sA + C::TILE;
    float *acc_k = reinterpret_cast<float *>(sB + C::TILE);
    const int acc_floats = BqAcc<D>::rows(P.kp.w2) * BqAcc<D>::row_floats();
    float *acc_v = acc_k + acc_floats;
    uint64_t *bars = reinterpret_cast<uint64_t *>(acc_v + acc_floats);
    uint32_t *tmem_holder = reinterpret_cast<uint32_t *>(bars + BQ_BAR_COUNT);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int x = 0; x < BQ_BAR_COUNT; ++x) {
            const bool pfull = x >= BQ_P_FULL && x < BQ_P_FULL + 3;          // every compute thread
            const bool many = (x >= BQ_W_EMPTY && x < BQ_W_EMPTY + 2) || x == BQ_FOLD_SYNC;
            // S_FULL and AB_EMPTY collect one commit from each of the two first-product issuers; head dim 64:
            // G_DONE and W_FULL one from each of the two second-product issuers
            const bool two = (x >= BQ_S_FULL && x < BQ_S_FULL + 3) || x == BQ_AB_EMPTY ||
                             (D == 64 && ((x >= BQ_G_DONE && x < BQ_G_DONE + 3) || (x >= BQ_W_FULL && x < BQ_W_FULL + 2)));
            // head dim 64: the fold group forms A_e and B_e; head dim 128: the builders A_e, the fold group B_e
            mbar_init(&bars[x], x == BQ_AB_FULL ? (BqRegs<D>::BUILDERS ? 256u : 128u) : pfull ? 128u * C::NCG : many ? 128u : two ? 2u : 1u);
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
    const BqGeom g = bq_geom<D>(P);

    int err = 0;
#ifdef SA2_PROF
    const long long prof_t0 = clock64();
    sa2::sm100::prof_begin();
#endif
    if (warp < 4) {
        reg_dealloc<BQ_REGS_ISSUE>();                 // one instruction for the whole warpgroup
        if (warp == 0 || (D == 64 && warp == 3)) {
            if (lane == 0 && g.total > 0)
                err = bq_mma_second<D>(P, g, D == 64 ? (warp == 0 ? 0 : 1) : 2, &mapK, &mapV, tmem, sK, sV, bars, abort_flag);
            __syncwarp();
        } else if (warp == 1 || warp == 2) {
            if (lane == 0 && g.total > 0)
                err = bq_mma_first<D>(g, warp - 1, tmem, warp == 1 ? sK : sV, warp == 1 ? sA : sB, bars, abort_flag);
            __syncwarp();
        } else if constexpr (D == 128) {
            if (lane == 0 && g.total > 0) err = bq_ring_producer<D>(P, g, &mapK, &mapV, sK, sV, bars, abort_flag);
            __syncwarp();
        }
    } else if (warp < 4 + 4 * C::NCG) {
        // one call site for both compute groups: they run the same instructions, which the instruction caches
        // of a scheduler then hold once
        reg_dealloc<BQ_REGS_COMPUTE>();
        err = bq_compute<D>(P, g, (warp >> 2) - 1, tmem, bars, abort_flag);
    } else if (warp < 12) {
        if constexpr (BqRegs<D>::BUILDERS) {
            reg_alloc<BqRegs<D>::BUILD>();
            if (g.total > 0) err = bq_builder<D>(P, g, sA, bars, abort_flag);
        } else {
            reg_dealloc<BQ_REGS_COMPUTE>();
        }
    } else {
        reg_alloc<BqRegs<D>::FOLD>();
        err = bq_fold<D>(P, g, tmem, acc_k, acc_v, sA, sB, bars, abort_flag);
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

// ---------------------------------------------------------------------------
// Reduction of the partials: one thread per 4 channels of an output row.
//   dq[b,i,h]   = scale * sum_split part_dq[split][b][i][h]        (two or more splits only)
//   dk2[b,k,hk] = scale * sum_{h in group} sum_{tiles touching k} sum_split slab_k[...]
//   dv2[b,k,hk] =         same over slab_v
// Row k (position k - off2 in query coordinates) lies in the slab of query tile
// T at slab row k - off2 - 128 T + (w2 - 1), for the one or two tiles where
// that index falls inside [0, 127 + w2).
// ---------------------------------------------------------------------------
template <int D>
__global__ void bwd_q_reduce_kernel(const BqParams P) {
    constexpr int TPR = D / 4;                          // threads per row
    const KernelParams &kp = P.kp;
    const int acc_rows = 127 + kp.w2;
    const int64_t nq = P.nsplit == 1 ? 0 : (int64_t)kp.b * kp.n * kp.hq * TPR;      // one split: dQ is already in place
    const int64_t nk = (int64_t)kp.b * kp.nk2 * kp.hk * TPR;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool gbf16 = kp.grad_bf16 != 0;
    if (idx < nq) {
        const int c4 = (int)(idx % TPR) * 4;
        int64_t rest = idx / TPR;
        const int h = (int)(rest % kp.hq); rest /= kp.hq;
        const int i = (int)(rest % kp.n);
        const int b = (int)(rest / kp.n);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < P.nsplit; ++s) {
            const float4 v = *reinterpret_cast<const float4 *>(P.part_dq + ((((size_t)s * kp.b + b) * kp.n + i) * kp.hq + h) * D + c4);
            acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
        }
#pragma unroll
        for (int z = 0; z < 4; ++z) acc[z] *= kp.scale;
        store_vec<4>(kp.dq.p, elem_off(kp.dq, b, i, h) + c4, gbf16, acc);
    } else if (idx < nq + nk) {
        const int64_t id2 = idx - nq;
        const int c4 = (int)(id2 % TPR) * 4;
        int64_t rest = id2 / TPR;
        const int hk = (int)(rest % kp.hk); rest /= kp.hk;
        const int k = (int)(rest % kp.nk2);
        const int b = (int)(rest / kp.nk2);
        float ak[4] = {0.f, 0.f, 0.f, 0.f}, av[4] = {0.f, 0.f, 0.f, 0.f};
        const int pos = k - kp.off2;                    // in query coordinates (may be negative for halo rows)
        for (int hh = 0; hh < kp.g; ++hh) {
            const int h = hk * kp.g + hh;
            // tiles T with 0 <= pos - 128 T + w2 - 1 < acc_rows
            const int t_hi = min(P.nqt - 1, (pos + kp.w2 - 1) >= 0 ? (pos + kp.w2 - 1) / TQ : -1);
            for (int T = max(0, t_hi - 1); T <= t_hi; ++T) {
                const int row = pos - TQ * T + kp.w2 - 1;
                if (row < 0 || row >= acc_rows) continue;
                for (int s = 0; s < P.nsplit; ++s) {
                    const float *slab = P.part_k2 + ((((size_t)b * kp.hq + h) * P.nqt + T) * P.nsplit + s) * (size_t)(2 * acc_rows * D);
                    const float4 vk = *reinterpret_cast<const float4 *>(slab + (size_t)row * D + c4);
                    const float4 vv = *reinterpret_cast<const float4 *>(slab + (size_t)(acc_rows + row) * D + c4);
                    ak[0] += vk.x; ak[1] += vk.y; ak[2] += vk.z; ak[3] += vk.w;
                    av[0] += vv.x; av[1] += vv.y; av[2] += vv.z; av[3] += vv.w;
                }
            }
        }
#pragma unroll
        for (int z = 0; z < 4; ++z) ak[z] *= kp.scale;
        store_vec<4>(kp.dk2.p, elem_off(kp.dk2, b, k, hk) + c4, gbf16, ak);
        store_vec<4>(kp.dv2.p, elem_off(kp.dv2, b, k, hk) + c4, gbf16, av);
    }
}

}  // namespace tc
}  // namespace sa2
