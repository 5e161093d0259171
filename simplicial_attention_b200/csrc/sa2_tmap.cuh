// Host-side construction of TMA tensor maps for [batch][seq][head][channel]
// bf16 tensors.  The driver entry point is looked up at run time so that the
// library does not link against libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sa2 {
namespace tmap {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Map over a bf16 tensor [b][rows][h][d] with element strides (sb, sn, sh, 1).
// A box is `box_rows` consecutive rows of one (batch, head), 64 channels wide
// (128 bytes), stored with the 128-byte swizzle; rows outside [0, rows) read
// as zero.  Coordinates are (channel, head, row, batch).
inline bool make_rows_map(CUtensorMap *out, const void *base, int b, int rows, int h, int d,
                          int64_t sb, int64_t sn, int64_t sh, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)h, (cuuint64_t)rows, (cuuint64_t)b};
    cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)sn * 2, (cuuint64_t)sb * 2};
    cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    // a dimension of extent 1 may carry any stride; keep it a non-zero multiple of 16 bytes
    for (int i = 0; i < 3; ++i)
        if (strides[i] == 0) strides[i] = 16;
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace tmap
}  // namespace sa2
