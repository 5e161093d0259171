// fp32 SIMT kernels for sliding-window causal 2-simplicial attention.
//
// These are the exact-arithmetic tier: inputs (fp32 or bf16) are widened to
// fp32, every product and sum is fp32, and nothing is rounded to bf16 on the
// way.  They handle every head dim in {32, 64, 128}, any sequence length, any
// window and grouped-query heads, and they are the kernels the tensor-core
// path is checked against on the device.
//
// Formulation ("k'-offset"): for an offset e = i - k in [0, w2) every query
// row i is paired with ONE second key k2[i-e].  A_e[i,:] = scale*q_i*k2_{i-e}
// turns the trilinear logits into an ordinary GEMM S_e = A_e K1^T, and
// W_e = P_e V1 followed by O += v2_{i-e} * W_e gives the output.  The softmax
// runs jointly over all (j, e).  The same tiles serve the three gradient
// kernels:
//   rows = query rows i          -> dQ            (MODE_BWD_Q)
//   rows = second-key rows k=i-e -> dK2, dV2      (MODE_BWD_K2)
//   rows = first-key rows j      -> dK1, dV1      (k1_kernel, S^T tiles)
// Each output row is owned by exactly one CTA, so there are no atomics and
// results are bitwise reproducible.
//
// Tile: 64 rows x 64 first-key columns, 256 threads as a 16x16 grid; thread
// (ty, tx) owns rows ty+16*ii and columns tx+16*jj of the logit tile and rows
// ty+16*ii, channels tx*VEC.. of the accumulators.
#pragma once
#include "sa2_common.cuh"
#include <math_constants.h>

namespace sa2 {
namespace simt {

enum { MODE_FWD = 0, MODE_BWD_Q = 1, MODE_BWD_K2 = 2 };

constexpr int TILE = 64;
constexpr int LP = TILE + 4;   // row stride of the probability tiles
constexpr int NTHREADS = 256;

template <int D> struct Cfg {
    static constexpr int LD = D + 4;                 // row stride of [64][D] tiles
    static constexpr int CPT = D / 16;               // channels per thread
    static constexpr int VEC = (D >= 64) ? 4 : 2;    // vector width of a channel group
    static constexpr int NV = CPT / VEC;             // channel groups per thread
    static constexpr size_t smem_fwd = sizeof(float) * (3 * TILE * LD + TILE * LP);
    static constexpr size_t smem_bwd = sizeof(float) * (4 * TILE * LD + 2 * TILE * LP);
};

// first channel of channel group u for thread column tx
template <int D> __device__ __forceinline__ int chan(int tx, int u) {
    return u * (16 * Cfg<D>::VEC) + tx * Cfg<D>::VEC;
}

// acc[ii][jj] = sum_c A[ty+16ii][c] * B[tx+16jj][c]
template <int D>
__device__ __forceinline__ void gemm_nt(const float *__restrict__ A, const float *__restrict__ B,
                                        int ty, int tx, float (&acc)[4][4]) {
    constexpr int LD = Cfg<D>::LD;
#pragma unroll
    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) acc[ii][jj] = 0.f;
#pragma unroll 4
    for (int c = 0; c < D; c += 4) {
        float4 a[4], b[4];
#pragma unroll
        for (int ii = 0; ii < 4; ++ii) a[ii] = *reinterpret_cast<const float4 *>(A + (ty + 16 * ii) * LD + c);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) b[jj] = *reinterpret_cast<const float4 *>(B + (tx + 16 * jj) * LD + c);
#pragma unroll
        for (int ii = 0; ii < 4; ++ii)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                acc[ii][jj] = fmaf(a[ii].x, b[jj].x, acc[ii][jj]);
                acc[ii][jj] = fmaf(a[ii].y, b[jj].y, acc[ii][jj]);
                acc[ii][jj] = fmaf(a[ii].z, b[jj].z, acc[ii][jj]);
                acc[ii][jj] = fmaf(a[ii].w, b[jj].w, acc[ii][jj]);
            }
    }
}

// acc[ii][u*VEC+e] += sum_j P[ty+16ii][j] * X[j][chan(tx,u)+e]
template <int D>
__device__ __forceinline__ void gemm_pv(const float *__restrict__ P, const float *__restrict__ X,
                                        int ty, int tx, float (&acc)[4][Cfg<D>::CPT]) {
    constexpr int LD = Cfg<D>::LD, VEC = Cfg<D>::VEC, NV = Cfg<D>::NV;
#pragma unroll 2
    for (int j = 0; j < TILE; j += 4) {
        float4 pr[4];
#pragma unroll
        for (int ii = 0; ii < 4; ++ii) pr[ii] = *reinterpret_cast<const float4 *>(P + (ty + 16 * ii) * LP + j);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
#pragma unroll
            for (int u = 0; u < NV; ++u) {
                float x[VEC];
                const float *xp = X + (j + jj) * LD + chan<D>(tx, u);
                if constexpr (VEC == 4) {
                    const float4 f = *reinterpret_cast<const float4 *>(xp);
                    x[0] = f.x; x[1] = f.y; x[2] = f.z; x[3] = f.w;
                } else {
                    const float2 f = *reinterpret_cast<const float2 *>(xp);
                    x[0] = f.x; x[1] = f.y;
                }
#pragma unroll
                for (int ii = 0; ii < 4; ++ii) {
                    const float pv = jj == 0 ? pr[ii].x : jj == 1 ? pr[ii].y : jj == 2 ? pr[ii].z : pr[ii].w;
#pragma unroll
                    for (int e = 0; e < VEC; ++e) acc[ii][u * VEC + e] = fmaf(pv, x[e], acc[ii][u * VEC + e]);
                }
            }
        }
    }
}

// Fill a [64][D] fp32 tile from rows row0.. of a tensor (zero past nrows).
template <int D>
__device__ __forceinline__ void fill_tile(float *S, const TensorRef &t, int b, int h, int row0, int nrows, bool bf16) {
    constexpr int LD = Cfg<D>::LD;
    constexpr int C4 = D / 4;
    for (int idx = threadIdx.x; idx < TILE * C4; idx += NTHREADS) {
        const int r = idx / C4, c = (idx % C4) * 4;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        const int row = row0 + r;
        if (row >= 0 && row < nrows) load_vec<4>(t.p, elem_off(t, b, row, h) + c, bf16, v);
        *reinterpret_cast<float4 *>(S + r * LD + c) = make_float4(v[0], v[1], v[2], v[3]);
    }
}

// Build A[r][c] = mul * x[i(r)][c] * y[k(r)][c] for the 64 rows of a tile;
// rows whose (i, k) pair is invalid become zero.  i(r) = i_base + r,
// k(r) = k_base + r.
template <int D>
__device__ __forceinline__ void build_prod_tile(float *S, const TensorRef &x, int hx, const TensorRef &y, int hy,
                                                int b, int i_base, int n_i, int k_base, int n_k, float mul, bool bf16) {
    constexpr int LD = Cfg<D>::LD;
    constexpr int C4 = D / 4;
    for (int idx = threadIdx.x; idx < TILE * C4; idx += NTHREADS) {
        const int r = idx / C4, c = (idx % C4) * 4;
        const int i = i_base + r, k = k_base + r;
        float o[4] = {0.f, 0.f, 0.f, 0.f};
        if (i >= 0 && i < n_i && k >= 0 && k < n_k) {
            float a[4], e[4];
            load_vec<4>(x.p, elem_off(x, b, i, hx) + c, bf16, a);
            load_vec<4>(y.p, elem_off(y, b, k, hy) + c, bf16, e);
#pragma unroll
            for (int u = 0; u < 4; ++u) o[u] = mul * a[u] * e[u];
        }
        *reinterpret_cast<float4 *>(S + r * LD + c) = make_float4(o[0], o[1], o[2], o[3]);
    }
}

__device__ __forceinline__ float half_warp_max(float v) {
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------------------
// Row-owned kernel: forward, dQ, or dK2/dV2.
// grid = (ceil(rows/64), heads, b); heads = hq (FWD, BWD_Q) or hk (BWD_K2).
// ---------------------------------------------------------------------------
template <int D, int MODE>
__global__ void __launch_bounds__(NTHREADS) row_kernel(const KernelParams p) {
    using C = Cfg<D>;
    constexpr int LD = C::LD, CPT = C::CPT, VEC = C::VEC, NV = C::NV;
    extern __shared__ __align__(16) float smem[];
    float *As = smem;
    float *Ks = As + TILE * LD;
    float *Vs = Ks + TILE * LD;
    float *Ps = Vs + TILE * LD;
    float *dOvs = Ps + TILE * LP;     // backward only
    float *Gs = dOvs + TILE * LD;     // backward only

    const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
    const int r0 = blockIdx.x * TILE;
    const int bi = blockIdx.z;
    const bool bf16 = p.in_bf16 != 0;
    const int hk_i = (MODE == MODE_BWD_K2) ? (int)blockIdx.y : (int)blockIdx.y / p.g;
    const int h_begin = (MODE == MODE_BWD_K2) ? hk_i * p.g : (int)blockIdx.y;
    const int h_end = (MODE == MODE_BWD_K2) ? h_begin + p.g : h_begin + 1;

    // query rows this tile can touch, over all offsets e
    int i_min, i_max;
    if (MODE == MODE_BWD_K2) {
        const int k_hi = min(r0 + TILE - 1, p.nk2 - 1);
        i_min = max(0, r0 - p.off2);
        i_max = min(p.n - 1, k_hi - p.off2 + p.w2 - 1);
    } else {
        i_min = r0;
        i_max = min(p.n - 1, r0 + TILE - 1);
    }
    const int j_lo = max(0, i_min + p.off1 - p.w1 + 1);
    const int j_hi = i_max + p.off1;

    float acc0[4][CPT];   // FWD: O   BWD_Q: dQ   BWD_K2: dK2
    float acc1[4][CPT];   // BWD_K2: dV2
    float m_run[4], l_run[4];
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
        m_run[ii] = -CUDART_INF_F;
        l_run[ii] = 0.f;
#pragma unroll
        for (int c = 0; c < CPT; ++c) { acc0[ii][c] = 0.f; acc1[ii][c] = 0.f; }
    }

    for (int h = h_begin; h < h_end; ++h) {
        for (int j0 = (j_lo / TILE) * TILE; j0 <= j_hi; j0 += TILE) {
            __syncthreads();
            fill_tile<D>(Ks, p.k1, bi, hk_i, j0, p.nk1, bf16);
            fill_tile<D>(Vs, p.v1, bi, hk_i, j0, p.nk1, bf16);

            for (int e = 0; e < p.w2; ++e) {
                // rows of this tile that are valid for offset e (uniform over the CTA)
                int i_base, k_base, ilo, ihi;
                if (MODE == MODE_BWD_K2) {
                    k_base = r0; i_base = r0 - p.off2 + e;
                } else {
                    i_base = r0; k_base = r0 + p.off2 - e;
                }
                ilo = max(i_base, max(0, i_base - k_base));            // i >= 0 and k >= 0
                ihi = min(min(i_base + TILE - 1, p.n - 1), i_base + (p.nk2 - 1 - k_base));
                if (ilo > ihi) continue;
                if (ihi + p.off1 < j0 || ilo + p.off1 - p.w1 + 1 > j0 + TILE - 1) continue;

                __syncthreads();
                build_prod_tile<D>(As, p.q, h, p.k2, hk_i, bi, i_base, p.n, k_base, p.nk2, p.scale, bf16);
                if (MODE != MODE_FWD)
                    build_prod_tile<D>(dOvs, p.dout, h, p.v2, hk_i, bi, i_base, p.n, k_base, p.nk2, 1.f, bf16);
                __syncthreads();

                float s[4][4];
                gemm_nt<D>(As, Ks, ty, tx, s);

                bool ok[4][4];
                bool rvalid[4];
#pragma unroll
                for (int ii = 0; ii < 4; ++ii) {
                    const int r = ty + 16 * ii;
                    const int i = i_base + r, k = k_base + r;
                    rvalid[ii] = (i >= 0 && i < p.n && k >= 0 && k < p.nk2);
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        const int j = j0 + tx + 16 * jj;
                        const int dist = i + p.off1 - j;
                        ok[ii][jj] = rvalid[ii] && dist >= 0 && dist < p.w1;
                    }
                }

                if (MODE == MODE_FWD) {
#pragma unroll
                    for (int ii = 0; ii < 4; ++ii) {
                        float mx = -CUDART_INF_F;
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) if (ok[ii][jj]) mx = fmaxf(mx, s[ii][jj]);
                        mx = half_warp_max(mx);
                        const float m_new = fmaxf(m_run[ii], mx);
                        float alpha = 1.f, rs = 0.f;
                        if (m_new > -CUDART_INF_F) {
                            alpha = __expf(m_run[ii] - m_new);   // exp(-inf) = 0 on the first hit
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj) {
                                const float pv = ok[ii][jj] ? __expf(s[ii][jj] - m_new) : 0.f;
                                s[ii][jj] = pv;
                                rs += pv;
                            }
                        } else {
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj) s[ii][jj] = 0.f;
                        }
                        rs = half_warp_sum(rs);
                        l_run[ii] = l_run[ii] * alpha + rs;
                        m_run[ii] = m_new;
#pragma unroll
                        for (int c = 0; c < CPT; ++c) acc0[ii][c] *= alpha;
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) Ps[(ty + 16 * ii) * LP + tx + 16 * jj] = s[ii][jj];
                    }
                    __syncthreads();
                    float w[4][CPT];
#pragma unroll
                    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
                        for (int c = 0; c < CPT; ++c) w[ii][c] = 0.f;
                    gemm_pv<D>(Ps, Vs, ty, tx, w);
#pragma unroll
                    for (int ii = 0; ii < 4; ++ii) {
                        if (!rvalid[ii]) continue;
                        const int k = k_base + ty + 16 * ii;
#pragma unroll
                        for (int u = 0; u < NV; ++u) {
                            float x[VEC];
                            load_vec<VEC>(p.v2.p, elem_off(p.v2, bi, k, hk_i) + chan<D>(tx, u), bf16, x);
#pragma unroll
                            for (int q = 0; q < VEC; ++q)
                                acc0[ii][u * VEC + q] = fmaf(w[ii][u * VEC + q], x[q], acc0[ii][u * VEC + q]);
                        }
                    }
                } else {
                    float dp[4][4];
                    gemm_nt<D>(dOvs, Vs, ty, tx, dp);
#pragma unroll
                    for (int ii = 0; ii < 4; ++ii) {
                        const int i = i_base + ty + 16 * ii;
                        float lse_i = 0.f, dl_i = 0.f;
                        if (rvalid[ii]) {
                            const int64_t o = ((int64_t)bi * p.hq + h) * p.n + i;
                            lse_i = p.lse[o];
                            dl_i = p.delta[o];
                        }
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) {
                            const float pv = ok[ii][jj] ? __expf(s[ii][jj] - lse_i) : 0.f;
                            Gs[(ty + 16 * ii) * LP + tx + 16 * jj] = pv * (dp[ii][jj] - dl_i);
                            if (MODE == MODE_BWD_K2) Ps[(ty + 16 * ii) * LP + tx + 16 * jj] = pv;
                        }
                    }
                    __syncthreads();
                    float u_[4][CPT];
#pragma unroll
                    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
                        for (int c = 0; c < CPT; ++c) u_[ii][c] = 0.f;
                    gemm_pv<D>(Gs, Ks, ty, tx, u_);
                    if (MODE == MODE_BWD_Q) {
#pragma unroll
                        for (int ii = 0; ii < 4; ++ii) {
                            if (!rvalid[ii]) continue;
                            const int k = k_base + ty + 16 * ii;
#pragma unroll
                            for (int u = 0; u < NV; ++u) {
                                float x[VEC];
                                load_vec<VEC>(p.k2.p, elem_off(p.k2, bi, k, hk_i) + chan<D>(tx, u), bf16, x);
#pragma unroll
                                for (int q = 0; q < VEC; ++q)
                                    acc0[ii][u * VEC + q] = fmaf(u_[ii][u * VEC + q], x[q], acc0[ii][u * VEC + q]);
                            }
                        }
                    } else {
                        float w[4][CPT];
#pragma unroll
                        for (int ii = 0; ii < 4; ++ii)
#pragma unroll
                            for (int c = 0; c < CPT; ++c) w[ii][c] = 0.f;
                        gemm_pv<D>(Ps, Vs, ty, tx, w);
#pragma unroll
                        for (int ii = 0; ii < 4; ++ii) {
                            if (!rvalid[ii]) continue;
                            const int i = i_base + ty + 16 * ii;
#pragma unroll
                            for (int u = 0; u < NV; ++u) {
                                float xq[VEC], xd[VEC];
                                load_vec<VEC>(p.q.p, elem_off(p.q, bi, i, h) + chan<D>(tx, u), bf16, xq);
                                load_vec<VEC>(p.dout.p, elem_off(p.dout, bi, i, h) + chan<D>(tx, u), bf16, xd);
#pragma unroll
                                for (int q = 0; q < VEC; ++q) {
                                    acc0[ii][u * VEC + q] = fmaf(u_[ii][u * VEC + q], xq[q], acc0[ii][u * VEC + q]);
                                    acc1[ii][u * VEC + q] = fmaf(w[ii][u * VEC + q], xd[q], acc1[ii][u * VEC + q]);
                                }
                            }
                        }
                    }
                }
            }
        }
    }

    // epilogue: each thread stores its rows
    const bool gbf16 = p.grad_bf16 != 0;
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
        const int r = r0 + ty + 16 * ii;
        if (MODE == MODE_FWD) {
            if (r >= p.n) continue;
            const float inv = 1.f / l_run[ii];
#pragma unroll
            for (int u = 0; u < NV; ++u) {
                float x[VEC];
#pragma unroll
                for (int q = 0; q < VEC; ++q) x[q] = acc0[ii][u * VEC + q] * inv;
                store_vec<VEC>(p.out.p, elem_off(p.out, bi, r, h_begin) + chan<D>(tx, u), bf16, x);
            }
            if (tx == 0) p.lse[((int64_t)bi * p.hq + h_begin) * p.n + r] = m_run[ii] + __logf(l_run[ii]);
        } else if (MODE == MODE_BWD_Q) {
            if (r >= p.n) continue;
#pragma unroll
            for (int u = 0; u < NV; ++u) {
                float x[VEC];
#pragma unroll
                for (int q = 0; q < VEC; ++q) x[q] = acc0[ii][u * VEC + q] * p.scale;
                store_vec<VEC>(p.dq.p, elem_off(p.dq, bi, r, h_begin) + chan<D>(tx, u), gbf16, x);
            }
        } else {
            if (r >= p.nk2) continue;
#pragma unroll
            for (int u = 0; u < NV; ++u) {
                float x[VEC], y[VEC];
#pragma unroll
                for (int q = 0; q < VEC; ++q) { x[q] = acc0[ii][u * VEC + q] * p.scale; y[q] = acc1[ii][u * VEC + q]; }
                store_vec<VEC>(p.dk2.p, elem_off(p.dk2, bi, r, hk_i) + chan<D>(tx, u), gbf16, x);
                store_vec<VEC>(p.dv2.p, elem_off(p.dv2, bi, r, hk_i) + chan<D>(tx, u), gbf16, y);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// First-key-owned kernel: dK1, dV1.  grid = (ceil(nk1/64), hk, b).
// Works on transposed tiles S^T[j][i] so that the accumulators are row-owned.
// ---------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(NTHREADS) k1_kernel(const KernelParams p) {
    using C = Cfg<D>;
    constexpr int LD = C::LD, CPT = C::CPT, VEC = C::VEC, NV = C::NV;
    extern __shared__ __align__(16) float smem[];
    float *As = smem;
    float *Ks = As + TILE * LD;
    float *Vs = Ks + TILE * LD;
    float *Ps = Vs + TILE * LD;
    float *dOvs = Ps + TILE * LP;
    float *Gs = dOvs + TILE * LD;

    const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
    const int j0 = blockIdx.x * TILE;
    const int hk_i = blockIdx.y, bi = blockIdx.z;
    const bool bf16 = p.in_bf16 != 0;

    fill_tile<D>(Ks, p.k1, bi, hk_i, j0, p.nk1, bf16);
    fill_tile<D>(Vs, p.v1, bi, hk_i, j0, p.nk1, bf16);

    float dk[4][CPT], dv[4][CPT];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj)
#pragma unroll
        for (int c = 0; c < CPT; ++c) { dk[jj][c] = 0.f; dv[jj][c] = 0.f; }

    const int i_lo = max(0, j0 - p.off1);
    const int i_hi = min(p.n - 1, min(j0 + TILE - 1, p.nk1 - 1) + p.w1 - 1 - p.off1);

    for (int h = hk_i * p.g; h < (hk_i + 1) * p.g; ++h) {
        for (int i0 = i_lo; i0 <= i_hi; i0 += TILE) {
            const int it_hi = min(i0 + TILE - 1, i_hi);
            // column statistics of this query tile
            float lse_c[4], dl_c[4];
#pragma unroll
            for (int ii = 0; ii < 4; ++ii) {
                const int i = i0 + tx + 16 * ii;
                lse_c[ii] = 0.f; dl_c[ii] = 0.f;
                if (i <= it_hi) {
                    const int64_t o = ((int64_t)bi * p.hq + h) * p.n + i;
                    lse_c[ii] = p.lse[o];
                    dl_c[ii] = p.delta[o];
                }
            }
            for (int e = 0; e < p.w2; ++e) {
                const int k_base = i0 + p.off2 - e;
                if (it_hi + p.off2 - e < 0) break;   // no valid second key for any row, nor for larger e
                __syncthreads();
                build_prod_tile<D>(As, p.q, h, p.k2, hk_i, bi, i0, it_hi + 1, k_base, p.nk2, p.scale, bf16);
                build_prod_tile<D>(dOvs, p.dout, h, p.v2, hk_i, bi, i0, it_hi + 1, k_base, p.nk2, 1.f, bf16);
                __syncthreads();
                float st[4][4], dpt[4][4];
                gemm_nt<D>(Ks, As, ty, tx, st);      // st[jj][ii]: row j, column i
                gemm_nt<D>(Vs, dOvs, ty, tx, dpt);
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int j = j0 + ty + 16 * jj;
#pragma unroll
                    for (int ii = 0; ii < 4; ++ii) {
                        const int i = i0 + tx + 16 * ii;
                        const int dist = i + p.off1 - j;
                        const bool ok = (i <= it_hi) && (i + p.off2 - e >= 0) && dist >= 0 && dist < p.w1 && j < p.nk1;
                        const float pv = ok ? __expf(st[jj][ii] - lse_c[ii]) : 0.f;
                        Ps[(ty + 16 * jj) * LP + tx + 16 * ii] = pv;
                        Gs[(ty + 16 * jj) * LP + tx + 16 * ii] = pv * (dpt[jj][ii] - dl_c[ii]);
                    }
                }
                __syncthreads();
                gemm_pv<D>(Ps, dOvs, ty, tx, dv);
                gemm_pv<D>(Gs, As, ty, tx, dk);
            }
        }
    }

    const bool gbf16 = p.grad_bf16 != 0;
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
        const int j = j0 + ty + 16 * jj;
        if (j >= p.nk1) continue;
#pragma unroll
        for (int u = 0; u < NV; ++u) {
            float x[VEC], y[VEC];
#pragma unroll
            for (int q = 0; q < VEC; ++q) { x[q] = dk[jj][u * VEC + q]; y[q] = dv[jj][u * VEC + q]; }
            store_vec<VEC>(p.dk1.p, elem_off(p.dk1, bi, j, hk_i) + chan<D>(tx, u), gbf16, x);
            store_vec<VEC>(p.dv1.p, elem_off(p.dv1, bi, j, hk_i) + chan<D>(tx, u), gbf16, y);
        }
    }
}

// D_i = sum_c O_ic dO_ic, one warp per (b, i, h) row.
__global__ void delta_kernel(const KernelParams p, int d) {
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int64_t rows = (int64_t)p.b * p.n * p.hq;
    if (warp >= rows) return;
    const int h = (int)(warp % p.hq);
    const int i = (int)((warp / p.hq) % p.n);
    const int b = (int)(warp / ((int64_t)p.hq * p.n));
    const bool bf16 = p.in_bf16 != 0;
    float s = 0.f;
    for (int c = lane * 2; c < d; c += 64) {
        float a[2], e[2];
        load_vec<2>(p.out.p, elem_off(p.out, b, i, h) + c, bf16, a);
        load_vec<2>(p.dout.p, elem_off(p.dout, b, i, h) + c, bf16, e);
        s = fmaf(a[0], e[0], s);
        s = fmaf(a[1], e[1], s);
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) p.delta[((int64_t)b * p.hq + h) * p.n + i] = s;
}

}  // namespace simt
}  // namespace sa2
