// tcgen05 / TMEM / TMA kernels (bf16 operands, fp32 accumulation) for sm_100a.
#pragma once
#include "sa2.h"
#include "sa2_common.cuh"

namespace sa2 {
namespace tc {

inline bool fwd_supported(const sa2_shape &) { return false; }
inline bool bwd_supported(const sa2_shape &) { return false; }
inline size_t bwd_extra_workspace_bytes(const sa2_shape &) { return 0; }
inline int launches(const sa2_shape &, bool) { return 0; }
inline int fwd(const KernelParams &, const sa2_shape &, cudaStream_t) { return SA2_ERR_UNSUPPORTED; }
inline int bwd(const KernelParams &, const sa2_shape &, void *, cudaStream_t) { return SA2_ERR_UNSUPPORTED; }

}  // namespace tc
}  // namespace sa2
