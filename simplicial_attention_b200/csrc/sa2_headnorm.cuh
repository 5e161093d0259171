// Per-head RMSNorm of a packed projection, forward and backward.
//
// The reference's module normalises q, k, k', v, v' per head with five separate
// RMSNorm modules after splitting the fused projection (simplicial_mha.py:124-127).
// Here the whole projection [rows][channels] is normalised in one pass: every
// group of d consecutive channels is one head, and `weight` holds the learned
// gain per channel (the caller tiles each norm's d gains over its heads).
//
//   y[r, c]  = x[r, c] * rstd[r, g] * weight[c],  rstd[r, g] = rsqrt(mean_{c in g} x^2 + eps)
//   dx       = rstd * (gy - xh * mean_g(gy * xh)),  gy = dy * weight,  xh = x * rstd
//   dweight[c] = sum_r dy[r, c] * xh[r, c]
//
// One warp per (row, head): HBM-bound, every element is read once and written
// once.  dweight is reduced without atomics: each CTA sums its rows in shared
// memory in warp order and writes one partial row; a second kernel adds the
// partial rows in a fixed order (eight interleaved slices, then the slices).
#pragma once
#include "sa2_common.cuh"
#include <cuda_bf16.h>

namespace sa2 {
namespace headnorm {

constexpr int WARPS = 8;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// channel of a lane's k-th element within its head: a few contiguous elements per lane for narrow heads (one
// 4- or 8-byte access), interleaved by warp for wide ones (every access of the warp is one contiguous run)
template <int PER> __device__ __forceinline__ int chan(int lane, int k) { return PER <= 4 ? lane * PER + k : k * 32 + lane; }

struct Params {
    const void *x;        // [rows][x_stride], channels contiguous
    const void *dy;       // backward only: [rows][dy_stride]
    const float *weight;  // [channels]
    void *y;              // forward: [rows][y_stride]; backward: dx
    float *rstd;          // [rows][groups]
    float *partial;       // backward: [gridDim.x][channels]
    int64_t rows, x_stride, y_stride, dy_stride;
    int channels, d;      // d in {32, 64, 128, 256, 512}: d / 32 elements per lane
    float eps;
};

// grid-stride over (row, head) pairs: pair p -> row p / groups, head p % groups
template <typename TX, typename TY, int PER>
__global__ void __launch_bounds__(WARPS * 32) fwd_kernel(const Params P) {
    const int groups = P.channels / P.d;
    const int lane = threadIdx.x & 31;
    const int64_t pairs = P.rows * groups;
    const TX *x = reinterpret_cast<const TX *>(P.x);
    TY *y = reinterpret_cast<TY *>(P.y);
    for (int64_t p = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5); p < pairs; p += (int64_t)gridDim.x * WARPS) {
        const int64_t r = p / groups;
        const int c0 = (int)(p % groups) * P.d;
        float v[PER], ss = 0.f;
#pragma unroll
        for (int k = 0; k < PER; ++k) { v[k] = to_f<TX>(x[r * P.x_stride + c0 + chan<PER>(lane, k)]); ss += v[k] * v[k]; }
        const float rs = rsqrtf(warp_sum(ss) / (float)P.d + P.eps);
#pragma unroll
        for (int k = 0; k < PER; ++k) {
            const int c = c0 + chan<PER>(lane, k);
            y[r * P.y_stride + c] = from_f<TY>(v[k] * rs * P.weight[c]);
        }
        if (lane == 0) P.rstd[p] = rs;
    }
}

// Each CTA owns a contiguous range of rows, so that its warps' dweight terms can be summed in row order.
template <typename TX, typename TY, int PER>
__global__ void __launch_bounds__(WARPS * 32) bwd_kernel(const Params P) {
    extern __shared__ float acc[];                     // [WARPS][channels]
    const int groups = P.channels / P.d;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const TX *x = reinterpret_cast<const TX *>(P.x);
    const TY *dy = reinterpret_cast<const TY *>(P.dy);
    TX *dx = reinterpret_cast<TX *>(P.y);
    for (int c = threadIdx.x; c < WARPS * P.channels; c += WARPS * 32) acc[c] = 0.f;
    __syncthreads();
    const int64_t rows_per_cta = (P.rows + gridDim.x - 1) / gridDim.x;
    const int64_t r_begin = (int64_t)blockIdx.x * rows_per_cta;
    const int64_t r_end = r_begin + rows_per_cta < P.rows ? r_begin + rows_per_cta : P.rows;
    float *mine = acc + (size_t)warp * P.channels;
    for (int64_t r = r_begin + warp; r < r_end; r += WARPS) {
        for (int g = 0; g < groups; ++g) {
            const int c0 = g * P.d;
            const float rs = P.rstd[r * groups + g];
            float xh[PER], gy[PER], dot = 0.f;
#pragma unroll
            for (int k = 0; k < PER; ++k) {
                const int c = c0 + chan<PER>(lane, k);
                xh[k] = to_f<TX>(x[r * P.x_stride + c]) * rs;
                const float d_ = to_f<TY>(dy[r * P.dy_stride + c]);
                gy[k] = d_ * P.weight[c];
                dot += gy[k] * xh[k];
                mine[c] += d_ * xh[k];
            }
            const float m = warp_sum(dot) / (float)P.d;
#pragma unroll
            for (int k = 0; k < PER; ++k) dx[r * P.y_stride + c0 + chan<PER>(lane, k)] = from_f<TX>(rs * (gy[k] - xh[k] * m));
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < P.channels; c += WARPS * 32) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) s += acc[(size_t)w * P.channels + c];
        P.partial[(size_t)blockIdx.x * P.channels + c] = s;
    }
}

// 32 channels x 8 slices per CTA: slice j adds partial rows j, j + 8, ... in order, then the eight slice sums
// are added in order - a fixed summation tree, so the result does not depend on scheduling.
__global__ void __launch_bounds__(256) dweight_reduce_kernel(const float *partial, float *dweight, int nparts, int channels) {
    __shared__ float part[8][32];
    const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    float s = 0.f;
    if (c < channels)
        for (int p = slice; p < nparts; p += 8) s += partial[(size_t)p * channels + c];
    part[slice][lane] = s;
    __syncthreads();
    if (slice == 0 && c < channels) {
        float t = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) t += part[j][lane];
        dweight[c] = t;
    }
}

}  // namespace headnorm
}  // namespace sa2
