// Host side of the tcgen05 / TMEM / TMA kernels (bf16 operands, fp32
// accumulation): applicability checks, tensor maps, launches.
#pragma once
#include "sa2.h"
#include "sa2_common.cuh"
#include "sa2_tc_fwd.cuh"
#include "sa2_tmap.cuh"

namespace sa2 {
namespace tc {

inline int tiles_per_query_tile(int w1) { return (w1 + TJ - 1 + TJ - 1) / TJ; }   // ceil((w1 + 127) / 128)

// The tensor-core forward handles bf16, head dim 64 and first-key windows whose
// tiles fit in shared memory (w1 <= 513).
inline bool fwd_supported(const sa2_shape &s) {
    return s.dtype == SA2_BF16 && s.d == 64 && tiles_per_query_tile(s.w1) <= MAX_NT;
}
inline bool bwd_supported(const sa2_shape &) { return false; }
inline size_t bwd_extra_workspace_bytes(const sa2_shape &) { return 0; }
inline int launches(const sa2_shape &, bool backward) { return backward ? 0 : 1; }

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

inline int fwd(const KernelParams &kp, const sa2_shape &s, cudaStream_t st) {
    if (!fwd_addressable(kp)) return SA2_ERR_INVALID;
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
    const size_t smem = fwd_smem_bytes(P.nt);
    if (cudaFuncSetAttribute(fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return SA2_ERR_CUDA;
    dim3 grid((kp.n + TQ - 1) / TQ, kp.hq, kp.b);
    fwd_kernel<<<grid, FWD_THREADS, smem, st>>>(mapK, mapV, P);
    return cudaGetLastError() == cudaSuccess ? SA2_OK : SA2_ERR_CUDA;
}

inline int bwd(const KernelParams &, const sa2_shape &, void *, cudaStream_t) { return SA2_ERR_UNSUPPORTED; }

}  // namespace tc
}  // namespace sa2
