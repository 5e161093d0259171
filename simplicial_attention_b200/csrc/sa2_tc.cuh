// Host side of the tcgen05 / TMEM / TMA kernels (bf16 operands, fp32
// accumulation): applicability checks, tensor maps, launches.
#pragma once
#include "sa2.h"
#include "sa2_common.cuh"
#include "sa2_simt.cuh"
#include "sa2_tc_fwd.cuh"
#include "sa2_tc_bwd_k1.cuh"
#include "sa2_tc_bwd_q.cuh"
#include "sa2_tc_fwd128.cuh"
#include "sa2_tc_bwd_k1_128.cuh"
#include "sa2_tmap.cuh"
#include <cstdlib>

namespace sa2 {
namespace tc {

inline int tiles_per_query_tile(int w1) { return (w1 + TJ - 1 + TJ - 1) / TJ; }   // ceil((w1 + 127) / 128)

// The tensor-core forward handles bf16 with head dim 64 and first-key windows whose
// tiles fit in shared memory (w1 <= 513), or head dim 128 with any window (the
// window is walked in passes).
inline bool fwd_supported(const sa2_shape &s) {
    if (s.dtype != SA2_BF16) return false;
    return s.d == 128 || (s.d == 64 && tiles_per_query_tile(s.w1) <= MAX_NT);
}
// The tensor-core backward handles bf16 and head dim 64 or 128, any window.
inline bool bwd_supported(const sa2_shape &s) { return s.dtype == SA2_BF16 && (s.d == 64 || s.d == 128); }
inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }
// CTAs sharing one query tile in the dQ/dK2/dV2 kernel (head dim 128 walks the whole window in one CTA)
inline int bq_splits(int w1, int d) { return d == 128 ? 1 : (tiles_per_query_tile(w1) + BQ_MAX_TILES - 1) / BQ_MAX_TILES; }
// Diagnostic switch: SA2_MMA_N64=1 issues every head-dim-128 product over the channels as two N = 64
// instructions instead of one N = 128 instruction.
inline int n64_products() {
    static const int v = [] { const char *e = std::getenv("SA2_MMA_N64"); return (e && e[0] == '1') ? 1 : 0; }();
    return v;
}
// dQ/dK2/dV2 run on the tensor cores when their shared accumulators (127 + w2 rows) fit
inline bool bq_supported(const sa2_shape &s) { return bwd_supported(s) && s.w2 <= BQ_MAX_W2; }
// scratch after the D vector: per-split partial dQ, then the per-CTA dK2/dV2 slabs
inline size_t bwd_extra_workspace_bytes(const sa2_shape &s) {
    if (!bq_supported(s)) return 0;
    const int ns = bq_splits(s.w1, s.d);
    return align256(bq_part_dq_bytes(s, ns)) + align256(bq_part_k2_bytes(s, ns));
}
// forward: 1 kernel; backward: D = rowsum(O*dO), dK1/dV1, dQ/dK2/dV2 partials, their reduction
// (or, when w2 is too large for the shared accumulators, two fp32 kernels for dQ and dK2/dV2)
inline int launches(const sa2_shape &, bool backward) { return backward ? 4 : 1; }

inline bool tma_addressable(const TensorRef &t) {
    return (reinterpret_cast<uintptr_t>(t.p) & 15u) == 0 && t.sb % 8 == 0 && t.sn % 8 == 0 && t.sh % 8 == 0;
}

// Device status word (one per device): kernels OR error bits into it when a
// bounded wait expires.
__device__ int g_status_word;

inline int *status_word() {
    static int *ptrs[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!ptrs[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
        ptrs[dev] = reinterpret_cast<int *>(p);
    }
    return ptrs[dev];
}

// 16-byte vector access and TMA need 16-byte aligned bases and strides that are multiples of 8 elements
inline bool fwd_addressable(const KernelParams &kp) {
    return tma_addressable(kp.k1) && tma_addressable(kp.v1) && tma_addressable(kp.q) && tma_addressable(kp.k2) &&
           tma_addressable(kp.v2) && tma_addressable(kp.out);
}

inline int fwd128(const KernelParams &kp, const sa2_shape &s, cudaStream_t st) {
    f128::Params P;
    P.kp = kp;
    P.nh = (s.w1 + TQ - 1 + f128::UNIT - 1) / f128::UNIT;       // ceil((w1 + 127) / 64)
    P.c = s.scale * 1.4426950408889634f;
    P.pv_split = n64_products();
    P.status = status_word();
    if (!P.status) return SA2_ERR_CUDA;
    CUtensorMap mapK, mapV;     // 64-row, 64-channel boxes
    if (!tmap::make_rows_map(&mapK, kp.k1.p, kp.b, kp.nk1, kp.hk, 128, kp.k1.sb, kp.k1.sn, kp.k1.sh, f128::UNIT) ||
        !tmap::make_rows_map(&mapV, kp.v1.p, kp.b, kp.nk1, kp.hk, 128, kp.v1.sb, kp.v1.sn, kp.v1.sh, f128::UNIT))
        return SA2_ERR_CUDA;
    const size_t smem = f128::smem_bytes();
    if (cudaFuncSetAttribute(f128::fwd128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return SA2_ERR_CUDA;
    dim3 grid((kp.n + TQ - 1) / TQ, kp.hq, kp.b);
    f128::fwd128_kernel<<<grid, f128::THREADS, smem, st>>>(mapK, mapV, P);
    return cudaGetLastError() == cudaSuccess ? SA2_OK : SA2_ERR_CUDA;
}

inline int fwd(const KernelParams &kp, const sa2_shape &s, cudaStream_t st) {
    if (!fwd_addressable(kp)) return SA2_ERR_INVALID;
    if (s.d == 128) return fwd128(kp, s, st);
    FwdParams P;
    P.kp = kp;
    P.nt = tiles_per_query_tile(s.w1);
    P.c = s.scale * 1.4426950408889634f;
    P.status = status_word();
    if (!P.status) return SA2_ERR_CUDA;
    CUtensorMap mapK, mapV;
    if (!tmap::make_rows_map(&mapK, kp.k1.p, kp.b, kp.nk1, kp.hk, 64, kp.k1.sb, kp.k1.sn, kp.k1.sh, TJ) ||
        !tmap::make_rows_map(&mapV, kp.v1.p, kp.b, kp.nk1, kp.hk, 64, kp.v1.sb, kp.v1.sn, kp.v1.sh, TJ))
        return SA2_ERR_CUDA;
    CUtensorMap mapK2;      // second keys, 32-row boxes
    if (!tmap::make_rows_map(&mapK2, kp.k2.p, kp.b, kp.nk2, kp.hk, 64, kp.k2.sb, kp.k2.sn, kp.k2.sh, 32)) return SA2_ERR_CUDA;
    const size_t smem = fwd_smem_bytes(P.nt);
    if (cudaFuncSetAttribute(fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return SA2_ERR_CUDA;
    dim3 grid((kp.n + TQ - 1) / TQ, kp.hq, kp.b);
    fwd_kernel<<<grid, FWD_THREADS, smem, st>>>(mapK, mapV, mapK2, P);
    return cudaGetLastError() == cudaSuccess ? SA2_OK : SA2_ERR_CUDA;
}

inline bool bwd_addressable(const KernelParams &kp) {
    return fwd_addressable(kp) && tma_addressable(kp.dout);
}

template <int D>
inline int bwd_q_launch(const KernelParams &kp, const sa2_shape &s, const CUtensorMap &mapK, const CUtensorMap &mapV,
                        float c, int *status, void *extra, cudaStream_t st) {
    // dQ, dK2, dV2: query-tile-owned tcgen05 kernel + deterministic reduction of its partials
    BqParams Q;
    Q.kp = kp;
    Q.c = c;
    Q.nt = tiles_per_query_tile(s.w1);
    Q.nsplit = bq_splits(s.w1, D);
    Q.tiles_per_split = (Q.nt + Q.nsplit - 1) / Q.nsplit;
    Q.nqt = (kp.n + TQ - 1) / TQ;
    Q.part_dq = reinterpret_cast<float *>(extra);
    Q.part_k2 = reinterpret_cast<float *>(reinterpret_cast<char *>(extra) + align256(bq_part_dq_bytes(s, Q.nsplit)));
    Q.status = status;
    const size_t smem = bq_smem_bytes<D>(s.w2);
    if (cudaFuncSetAttribute(bwd_q_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return SA2_ERR_CUDA;
    CUtensorMap ringK = mapK, ringV = mapV;
    if (D == 128) {     // the streamed units are 64-row boxes
        if (!tmap::make_rows_map(&ringK, kp.k1.p, kp.b, kp.nk1, kp.hk, D, kp.k1.sb, kp.k1.sn, kp.k1.sh, 64) ||
            !tmap::make_rows_map(&ringV, kp.v1.p, kp.b, kp.nk1, kp.hk, D, kp.v1.sb, kp.v1.sn, kp.v1.sh, 64))
            return SA2_ERR_CUDA;
    }
    bwd_q_kernel<D><<<dim3(Q.nqt * Q.nsplit * BqCfg<D>::CH, kp.hq, kp.b), BQ_THREADS, smem, st>>>(ringK, ringV, Q);
    if (cudaGetLastError() != cudaSuccess) return SA2_ERR_CUDA;
    const int64_t work = ((Q.nsplit == 1 ? 0 : (int64_t)kp.b * kp.n * kp.hq) + (int64_t)kp.b * kp.nk2 * kp.hk) * (D / 4);
    bwd_q_reduce_kernel<D><<<(unsigned)((work + 255) / 256), 256, 0, st>>>(Q);
    return cudaGetLastError() == cudaSuccess ? SA2_OK : SA2_ERR_CUDA;
}

template <int D>
inline int bwd_q_simt(const KernelParams &kp, cudaStream_t st) {
    // dQ and dK2/dV2: fp32 SIMT kernels (second-key windows too long for the shared accumulators)
    using namespace sa2::simt;
    auto kq = row_kernel<D, MODE_BWD_Q>;
    auto kk2 = row_kernel<D, MODE_BWD_K2>;
    if (cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<D>::smem_bwd) != cudaSuccess ||
        cudaFuncSetAttribute(kk2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<D>::smem_bwd) != cudaSuccess)
        return SA2_ERR_CUDA;
    kq<<<dim3((kp.n + TILE - 1) / TILE, kp.hq, kp.b), NTHREADS, Cfg<D>::smem_bwd, st>>>(kp);
    if (cudaGetLastError() != cudaSuccess) return SA2_ERR_CUDA;
    kk2<<<dim3((kp.nk2 + TILE - 1) / TILE, kp.hk, kp.b), NTHREADS, Cfg<D>::smem_bwd, st>>>(kp);
    return cudaGetLastError() == cudaSuccess ? SA2_OK : SA2_ERR_CUDA;
}

inline int bwd(const KernelParams &kp, const sa2_shape &s, void *extra, cudaStream_t st, int phases = 0) {
    if (!bwd_addressable(kp)) return SA2_ERR_INVALID;
    const float c = s.scale * 1.4426950408889634f;
    int *status = status_word();
    if (!status) return SA2_ERR_CUDA;
    if (phases == 0) phases = SA2_BWD_ROWSUM | SA2_BWD_K1 | SA2_BWD_Q;

    // D_i = sum_c O_ic dO_ic
    if (phases & SA2_BWD_ROWSUM) {
        const int64_t rows = (int64_t)kp.b * kp.n * kp.hq;
        simt::delta_kernel<<<(unsigned)((rows * 32 + 255) / 256), 256, 0, st>>>(kp, s.d);
        if (cudaGetLastError() != cudaSuccess) return SA2_ERR_CUDA;
    }

    // 128-row, 64-channel boxes of K1 / V1 (a head-dim-128 tile is two boxes)
    CUtensorMap mapK, mapV;
    if (!tmap::make_rows_map(&mapK, kp.k1.p, kp.b, kp.nk1, kp.hk, s.d, kp.k1.sb, kp.k1.sn, kp.k1.sh, TJ) ||
        !tmap::make_rows_map(&mapV, kp.v1.p, kp.b, kp.nk1, kp.hk, s.d, kp.v1.sb, kp.v1.sn, kp.v1.sh, TJ))
        return SA2_ERR_CUDA;

    // dK1, dV1: key-tile-owned tcgen05 kernel
    if (phases & SA2_BWD_K1) {
        CUtensorMap mapK2, mapV2;      // second keys / values, 32-row boxes of 64 channels
        if (!tmap::make_rows_map(&mapK2, kp.k2.p, kp.b, kp.nk2, kp.hk, s.d, kp.k2.sb, kp.k2.sn, kp.k2.sh, 32) ||
            !tmap::make_rows_map(&mapV2, kp.v2.p, kp.b, kp.nk2, kp.hk, s.d, kp.v2.sb, kp.v2.sn, kp.v2.sh, 32))
            return SA2_ERR_CUDA;
        const dim3 grid((kp.nk1 + TJ - 1) / TJ, kp.hk, kp.b);
        if (s.d == 128) {
            k128::Params P;
            P.kp = kp;
            P.c = c;
            P.n_split = n64_products();
            P.status = status;
            if (cudaFuncSetAttribute(k128::bwd_k1_128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)k128::smem_bytes()) != cudaSuccess)
                return SA2_ERR_CUDA;
            k128::bwd_k1_128_kernel<<<grid, k128::THREADS, k128::smem_bytes(), st>>>(mapK, mapV, mapK2, mapV2, P);
        } else {
            BwdParams P;
            P.kp = kp;
            P.c = c;
            P.status = status;
            if (cudaFuncSetAttribute(bwd_k1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bk1_smem_bytes()) != cudaSuccess)
                return SA2_ERR_CUDA;
            bwd_k1_kernel<<<grid, BK1_THREADS, bk1_smem_bytes(), st>>>(mapK, mapV, mapK2, mapV2, P);
        }
        if (cudaGetLastError() != cudaSuccess) return SA2_ERR_CUDA;
    }

    if (!(phases & SA2_BWD_Q)) return SA2_OK;
    if (bq_supported(s))
        return s.d == 128 ? bwd_q_launch<128>(kp, s, mapK, mapV, c, status, extra, st)
                          : bwd_q_launch<64>(kp, s, mapK, mapV, c, status, extra, st);
    return s.d == 128 ? bwd_q_simt<128>(kp, st) : bwd_q_simt<64>(kp, st);
}

}  // namespace tc
}  // namespace sa2
