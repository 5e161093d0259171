// Shared device-side types and load/store helpers for the sliding-window
// 2-simplicial attention kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace sa2 {

// One [batch][seq][head][channel] tensor: base pointer and element strides
// (channel stride is 1).
struct TensorRef {
    void *p;
    int64_t sb, sn, sh;
};

struct KernelParams {
    TensorRef q, k1, k2, v1, v2, out, dout;
    TensorRef dq, dk1, dk2, dv1, dv2;
    float *lse;     // [b][hq][n]
    float *delta;   // [b][hq][n], D_i = sum_c O_ic dO_ic (backward scratch)
    int b, n, hq, hk, g;
    int w1, w2, off1, off2;
    int nk1, nk2;   // rows of k1/v1 and k2/v2: n + off1, n + off2
    int in_bf16, grad_bf16;
    float scale;
};

__device__ __forceinline__ int64_t elem_off(const TensorRef &t, int b, int n, int h) {
    return (int64_t)b * t.sb + (int64_t)n * t.sn + (int64_t)h * t.sh;
}

// Vector loads of VEC (2 or 4) consecutive channels, converted to fp32.
template <int VEC>
__device__ __forceinline__ void load_vec(const void *base, int64_t off, bool bf16, float (&v)[VEC]) {
    if (bf16) {
        const __nv_bfloat16 *p = reinterpret_cast<const __nv_bfloat16 *>(base) + off;
        if constexpr (VEC == 4) {
            const uint2 u = *reinterpret_cast<const uint2 *>(p);
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162 *>(&u.x);
            const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162 *>(&u.y);
            v[0] = __low2float(a); v[1] = __high2float(a);
            v[2] = __low2float(c); v[3] = __high2float(c);
        } else {
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162 *>(p);
            v[0] = __low2float(a); v[1] = __high2float(a);
        }
    } else {
        const float *p = reinterpret_cast<const float *>(base) + off;
        if constexpr (VEC == 4) {
            const float4 f = *reinterpret_cast<const float4 *>(p);
            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        } else {
            const float2 f = *reinterpret_cast<const float2 *>(p);
            v[0] = f.x; v[1] = f.y;
        }
    }
}

template <int VEC>
__device__ __forceinline__ void store_vec(void *base, int64_t off, bool bf16, const float (&v)[VEC]) {
    if (bf16) {
        __nv_bfloat16 *p = reinterpret_cast<__nv_bfloat16 *>(base) + off;
        if constexpr (VEC == 4) {
            __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
            __nv_bfloat162 c = __floats2bfloat162_rn(v[2], v[3]);
            uint2 u;
            u.x = *reinterpret_cast<uint32_t *>(&a);
            u.y = *reinterpret_cast<uint32_t *>(&c);
            *reinterpret_cast<uint2 *>(p) = u;
        } else {
            *reinterpret_cast<__nv_bfloat162 *>(p) = __floats2bfloat162_rn(v[0], v[1]);
        }
    } else {
        float *p = reinterpret_cast<float *>(base) + off;
        if constexpr (VEC == 4) {
            *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
            *reinterpret_cast<float2 *>(p) = make_float2(v[0], v[1]);
        }
    }
}

}  // namespace sa2
