// C ABI of the library (declared in include/sa2.h): argument checks, kernel
// selection and launches.  No torch types, no allocation, no host sync.
#include "sa2.h"
#include "sa2_common.cuh"
#include "sa2_simt.cuh"
#include "sa2_tc.cuh"
#include "sa2_headnorm.cuh"
#include <nvtx3/nvToolsExt.h>

namespace sa2 {
namespace nvtx {
// NVTX range around an entry point (header-only NVTX v3: a no-op unless a profiler is attached)
struct Range {
    explicit Range(const char *name) { nvtxRangePushA(name); }
    ~Range() { nvtxRangePop(); }
};
}  // namespace nvtx
}  // namespace sa2

namespace {

using sa2::KernelParams;
using sa2::TensorRef;

inline TensorRef ref(const void *p, const sa2_strides &s) {
    return TensorRef{const_cast<void *>(p), s.batch, s.seq, s.head};
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool strides_ok(const sa2_strides &s) { return s.batch % 4 == 0 && s.seq % 4 == 0 && s.head % 4 == 0; }

int check_shape(const sa2_shape &s) {
    if (s.b <= 0 || s.n <= 0 || s.hq <= 0 || s.hk <= 0 || s.w1 <= 0 || s.w2 <= 0) return SA2_ERR_INVALID;
    if (s.off1 < 0 || s.off2 < 0) return SA2_ERR_INVALID;
    if (s.hq % s.hk != 0) return SA2_ERR_INVALID;
    if (s.d != 32 && s.d != 64 && s.d != 128) return SA2_ERR_UNSUPPORTED;
    if (s.dtype != SA2_F32 && s.dtype != SA2_BF16) return SA2_ERR_UNSUPPORTED;
    if (s.kernel != SA2_KERNEL_AUTO && s.kernel != SA2_KERNEL_SIMT && s.kernel != SA2_KERNEL_TCGEN05)
        return SA2_ERR_UNSUPPORTED;
    return SA2_OK;
}

void fill_common(KernelParams &p, const sa2_shape &s) {
    p.b = s.b; p.n = s.n; p.hq = s.hq; p.hk = s.hk; p.g = s.hq / s.hk;
    p.w1 = s.w1; p.w2 = s.w2; p.off1 = s.off1; p.off2 = s.off2;
    p.nk1 = s.n + s.off1; p.nk2 = s.n + s.off2;
    p.in_bf16 = (s.dtype == SA2_BF16);
    p.grad_bf16 = 0;
    p.scale = s.scale;
}

template <typename K>
int set_smem(K kernel, size_t bytes) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) == cudaSuccess
               ? SA2_OK : SA2_ERR_CUDA;
}

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? SA2_OK : SA2_ERR_CUDA; }

template <int D>
int simt_fwd(const KernelParams &p, cudaStream_t st) {
    using namespace sa2::simt;
    auto k = row_kernel<D, MODE_FWD>;
    if (int e = set_smem(k, Cfg<D>::smem_fwd)) return e;
    dim3 grid((p.n + TILE - 1) / TILE, p.hq, p.b);
    k<<<grid, NTHREADS, Cfg<D>::smem_fwd, st>>>(p);
    return launch_status();
}

template <int D>
int simt_bwd(const KernelParams &p, cudaStream_t st, int phases = 0) {
    using namespace sa2::simt;
    if (phases == 0) phases = SA2_BWD_ROWSUM | SA2_BWD_K1 | SA2_BWD_Q;
    if (phases & SA2_BWD_ROWSUM) {
        const int64_t rows = (int64_t)p.b * p.n * p.hq;
        delta_kernel<<<(unsigned)((rows * 32 + 255) / 256), 256, 0, st>>>(p, D);
        if (int e = launch_status()) return e;
    }

    auto kq = row_kernel<D, MODE_BWD_Q>;
    auto kk2 = row_kernel<D, MODE_BWD_K2>;
    auto kk1 = k1_kernel<D>;
    if (int e = set_smem(kq, Cfg<D>::smem_bwd)) return e;
    if (int e = set_smem(kk2, Cfg<D>::smem_bwd)) return e;
    if (int e = set_smem(kk1, Cfg<D>::smem_bwd)) return e;

    if (phases & SA2_BWD_Q) {
        kq<<<dim3((p.n + TILE - 1) / TILE, p.hq, p.b), NTHREADS, Cfg<D>::smem_bwd, st>>>(p);
        if (int e = launch_status()) return e;
        kk2<<<dim3((p.nk2 + TILE - 1) / TILE, p.hk, p.b), NTHREADS, Cfg<D>::smem_bwd, st>>>(p);
        if (int e = launch_status()) return e;
    }
    if (phases & SA2_BWD_K1) {
        kk1<<<dim3((p.nk1 + TILE - 1) / TILE, p.hk, p.b), NTHREADS, Cfg<D>::smem_bwd, st>>>(p);
        return launch_status();
    }
    return SA2_OK;
}

// argument checks shared by sa2_bwd and sa2_bwd_static_scratch
int check_bwd_args(const sa2_bwd_args *a) {
    if (!a) return SA2_ERR_INVALID;
    if (int e = check_shape(a->shape)) return e;
    if (!a->q || !a->k1 || !a->k2 || !a->v1 || !a->v2 || !a->out || !a->dout || !a->lse) return SA2_ERR_INVALID;
    if (!a->dq || !a->dk1 || !a->dk2 || !a->dv1 || !a->dv2) return SA2_ERR_INVALID;
    if (a->grad_dtype != SA2_F32 && a->grad_dtype != SA2_BF16) return SA2_ERR_UNSUPPORTED;
    const void *ptrs[] = {a->q, a->k1, a->k2, a->v1, a->v2, a->out, a->dout, a->dq, a->dk1, a->dk2, a->dv1, a->dv2};
    for (const void *p : ptrs) if (!aligned16(p)) return SA2_ERR_INVALID;
    const sa2_strides *ss[] = {&a->sq, &a->sk1, &a->sk2, &a->sv1, &a->sv2, &a->sout, &a->sdout,
                               &a->sdq, &a->sdk1, &a->sdk2, &a->sdv1, &a->sdv2};
    for (const sa2_strides *s : ss) if (!strides_ok(*s)) return SA2_ERR_INVALID;
    return SA2_OK;
}

void fill_bwd_params(KernelParams &p, const sa2_bwd_args *a, float *rowsum) {
    fill_common(p, a->shape);
    p.grad_bf16 = (a->grad_dtype == SA2_BF16);
    p.q = ref(a->q, a->sq); p.k1 = ref(a->k1, a->sk1); p.k2 = ref(a->k2, a->sk2);
    p.v1 = ref(a->v1, a->sv1); p.v2 = ref(a->v2, a->sv2);
    p.out = ref(a->out, a->sout); p.dout = ref(a->dout, a->sdout);
    p.dq = ref(a->dq, a->sdq); p.dk1 = ref(a->dk1, a->sdk1); p.dk2 = ref(a->dk2, a->sdk2);
    p.dv1 = ref(a->dv1, a->sdv1); p.dv2 = ref(a->dv2, a->sdv2);
    p.lse = const_cast<float *>(a->lse);
    p.delta = rowsum;
}

// One block of one warp waits on a barrier that nobody arrives on, with the given limit: the self-test of
// the bounded waits.  The wait runs out, the block records ERR_SELFTEST and leaves through the normal path.
__global__ void selftest_wait_kernel(long long limit_cycles, int *status) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        sa2::sm100::mbar_init(&bar, 1);
        abort_flag = 0;
        sa2::sm100::fence_barrier_init();
    }
    __syncthreads();
    const bool ok = sa2::sm100::mbar_wait(&bar, 0, &abort_flag, 32, -1, limit_cycles);
    if (!ok && threadIdx.x == 0) atomicOr(status, SA2_SELFTEST_WAIT_BIT);
}

}  // namespace

extern "C" {

int sa2_version(void) { return 100; }

int sa2_selftest_wait(long long limit_cycles, void *stream) {
    if (limit_cycles <= 0 || limit_cycles > 2000000000LL) return SA2_ERR_INVALID;
    int *word = sa2::tc::status_word();
    if (!word) return SA2_ERR_CUDA;
    selftest_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(limit_cycles, word);
    return launch_status();
}

#ifdef SA2_PROF
// diagnostic builds only (-DSA2_PROF=<CTA index>): read and clear the wait-accounting table
int sa2_prof_read(unsigned long long *host, int n) {
    if (cudaMemcpyFromSymbol(host, sa2::sm100::g_prof, sizeof(unsigned long long) * n) != cudaSuccess) return -1;
    static unsigned long long zeros[512] = {0};
    return cudaMemcpyToSymbol(sa2::sm100::g_prof, zeros, sizeof(unsigned long long) * n) == cudaSuccess ? 0 : -1;
}
#endif

int sa2_device_status(int reset) {
    int *word = sa2::tc::status_word();
    if (!word) return -1;
    int v = 0;
    if (cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (reset && v != 0) {
        const int zero = 0;
        if (cudaMemcpy(word, &zero, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) return -1;
    }
    return v;
}

int sa2_check_device(int reset) {
    const int v = sa2_device_status(reset);
    if (v < 0) return SA2_ERR_CUDA;
    return v == 0 ? SA2_OK : SA2_ERR_DEVICE;
}

const char *sa2_strerror(int status) {
    switch (status) {
        case SA2_OK: return "ok";
        case SA2_ERR_INVALID: return "invalid argument (null pointer, bad size, hq % hk != 0, misaligned pointer or stride)";
        case SA2_ERR_UNSUPPORTED: return "unsupported configuration (head dim must be 32, 64 or 128; dtype fp32 or bf16; "
                                         "the tcgen05 kernels need bf16)";
        case SA2_ERR_WORKSPACE: return "workspace missing, misaligned or smaller than sa2_bwd_workspace_bytes()";
        case SA2_ERR_CUDA: return "a CUDA call failed";
        case SA2_ERR_DEVICE: return "a kernel gave up on a bounded wait; the rows it owned hold NaN";
        case SA2_ERR_TOO_LARGE: return "problem too large for the library's built-in scratch: b * hq * n exceeds "
                                       "SA2_STATIC_SCRATCH_ROWS (use sa2_bwd with a caller-provided workspace)";
        default: return "unknown status";
    }
}

int sa2_kernel_launches(const sa2_shape *s, int backward) {
    if (!s || check_shape(*s) != SA2_OK) return -1;
    const bool tc_ok = backward ? sa2::tc::bwd_supported(*s) : sa2::tc::fwd_supported(*s);
    if (s->kernel == SA2_KERNEL_TCGEN05 && !tc_ok) return -1;
    if (tc_ok && s->kernel != SA2_KERNEL_SIMT) return sa2::tc::launches(*s, backward != 0);
    return backward ? 4 : 1;   // SIMT: delta + dQ + dK2/dV2 + dK1/dV1
}

size_t sa2_bwd_workspace_bytes(const sa2_shape *s) {
    if (!s || check_shape(*s) != SA2_OK) return 0;
    size_t delta = (size_t)s->b * s->hq * s->n * sizeof(float);
    delta = (delta + 255) & ~(size_t)255;
    return delta + sa2::tc::bwd_extra_workspace_bytes(*s);
}

int sa2_fwd(const sa2_fwd_args *a) {
    sa2::nvtx::Range range("sa2_fwd");
    if (!a) return SA2_ERR_INVALID;
    if (int e = check_shape(a->shape)) return e;
    if (!a->q || !a->k1 || !a->k2 || !a->v1 || !a->v2 || !a->out || !a->lse) return SA2_ERR_INVALID;
    const void *ptrs[] = {a->q, a->k1, a->k2, a->v1, a->v2, a->out};
    for (const void *p : ptrs) if (!aligned16(p)) return SA2_ERR_INVALID;
    const sa2_strides *ss[] = {&a->sq, &a->sk1, &a->sk2, &a->sv1, &a->sv2, &a->sout};
    for (const sa2_strides *s : ss) if (!strides_ok(*s)) return SA2_ERR_INVALID;

    KernelParams p{};
    fill_common(p, a->shape);
    p.q = ref(a->q, a->sq); p.k1 = ref(a->k1, a->sk1); p.k2 = ref(a->k2, a->sk2);
    p.v1 = ref(a->v1, a->sv1); p.v2 = ref(a->v2, a->sv2); p.out = ref(a->out, a->sout);
    p.lse = a->lse;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);

    const bool tc_ok = sa2::tc::fwd_supported(a->shape) && sa2::tc::fwd_addressable(p);
    if (a->shape.kernel == SA2_KERNEL_TCGEN05 && !tc_ok) return SA2_ERR_UNSUPPORTED;
    if (tc_ok && a->shape.kernel != SA2_KERNEL_SIMT) return sa2::tc::fwd(p, a->shape, st);

    switch (a->shape.d) {
        case 32: return simt_fwd<32>(p, st);
        case 64: return simt_fwd<64>(p, st);
        default: return simt_fwd<128>(p, st);
    }
}

int sa2_bwd(const sa2_bwd_args *a) {
    sa2::nvtx::Range range("sa2_bwd");
    if (int e = check_bwd_args(a)) return e;
    if (a->phases < 0 || a->phases > (SA2_BWD_ROWSUM | SA2_BWD_K1 | SA2_BWD_Q)) return SA2_ERR_INVALID;
    const size_t need = sa2_bwd_workspace_bytes(&a->shape);
    if (!a->workspace || a->workspace_bytes < need || (reinterpret_cast<uintptr_t>(a->workspace) & 255u))
        return SA2_ERR_WORKSPACE;

    KernelParams p{};
    fill_bwd_params(p, a, reinterpret_cast<float *>(a->workspace));
    cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);

    const bool tc_ok = sa2::tc::bwd_supported(a->shape) && sa2::tc::bwd_addressable(p);
    if (a->shape.kernel == SA2_KERNEL_TCGEN05 && !tc_ok) return SA2_ERR_UNSUPPORTED;
    if (tc_ok && a->shape.kernel != SA2_KERNEL_SIMT) {
        size_t delta = (size_t)a->shape.b * a->shape.hq * a->shape.n * sizeof(float);
        delta = (delta + 255) & ~(size_t)255;
        return sa2::tc::bwd(p, a->shape, reinterpret_cast<char *>(a->workspace) + delta, st, a->phases);
    }

    switch (a->shape.d) {
        case 32: return simt_bwd<32>(p, st, a->phases);
        case 64: return simt_bwd<64>(p, st, a->phases);
        default: return simt_bwd<128>(p, st, a->phases);
    }
}

// ---------------------------------------------------------------------------
// Backward without caller-provided scratch.
//
// Some hosts of this library cannot hand it a workspace: an inference or
// training engine that claimed all device memory for its own pools at start-up,
// a plug-in that is only allowed to launch kernels, a latency-critical loop in
// which every allocator call is forbidden.  For them the row sums
// D_i = sum_c O_ic dO_ic live in the fixed device array below instead.  The
// array is part of the library image: every GPU that loads the library keeps
// SA2_STATIC_SCRATCH_ROWS * 4 bytes (1 MiB) for it until the process exits.
// ---------------------------------------------------------------------------
static __device__ __align__(256) float g_static_rowsum[SA2_STATIC_SCRATCH_ROWS];

namespace {

// Device address of g_static_rowsum on the current device.  In host code the
// array's name is only a handle, never a device pointer, so the address is
// asked for once per device (with that device current) and remembered.
float *static_rowsum_ptr() {
    static float *ptrs[64] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    float *p = ptrs[dev];
    if (!p) {
        void *addr = nullptr;
        if (cudaGetSymbolAddress(&addr, g_static_rowsum) != cudaSuccess || !addr) return nullptr;
        p = reinterpret_cast<float *>(addr);
        ptrs[dev] = p;      // racing first calls store the same value
    }
    return p;
}

}  // namespace

int sa2_bwd_static_scratch(const sa2_bwd_args *a) {
    sa2::nvtx::Range range("sa2_bwd_static_scratch");
    if (int e = check_bwd_args(a)) return e;
    // only the fp32 kernels get by with the row sums alone
    if (a->shape.kernel == SA2_KERNEL_TCGEN05) return SA2_ERR_UNSUPPORTED;
    const long long rows = (long long)a->shape.b * a->shape.hq * a->shape.n;
    if (rows > (long long)SA2_STATIC_SCRATCH_ROWS) return SA2_ERR_TOO_LARGE;

    float *rowsum = static_rowsum_ptr();
    if (!rowsum) return SA2_ERR_CUDA;

    KernelParams p{};
    fill_bwd_params(p, a, rowsum);    // every entry the kernels read is rewritten first: nothing has to start at zero
    cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);
    switch (a->shape.d) {
        case 32: return simt_bwd<32>(p, st);
        case 64: return simt_bwd<64>(p, st);
        default: return simt_bwd<128>(p, st);
    }
}

}  // extern "C"

// ---------------------------------------------------------------- per-head RMSNorm
namespace {

int headnorm_grid(int64_t rows) {
    const int64_t want = (rows + sa2::headnorm::WARPS - 1) / sa2::headnorm::WARPS;
    return (int)(want < 592 ? (want > 0 ? want : 1) : 592);          // 4 CTAs per SM
}

int headnorm_check(const sa2_headnorm_args *a, bool backward) {
    if (!a || !a->x || !a->weight || !a->y || !a->rstd || a->rows <= 0 || a->channels <= 0) return SA2_ERR_INVALID;
    if (a->d != 32 && a->d != 64 && a->d != 128 && a->d != 256 && a->d != 512) return SA2_ERR_UNSUPPORTED;
    if (a->channels % a->d != 0) return SA2_ERR_INVALID;
    if ((a->x_dtype != SA2_F32 && a->x_dtype != SA2_BF16) || (a->y_dtype != SA2_F32 && a->y_dtype != SA2_BF16)) return SA2_ERR_UNSUPPORTED;
    if (a->x_stride < a->channels || a->y_stride < a->channels) return SA2_ERR_INVALID;
    if (backward) {
        if (!a->dy || !a->dweight || a->dy_stride < a->channels) return SA2_ERR_INVALID;
        if (!a->partial || a->partial_bytes < sa2_headnorm_partial_bytes(a->rows, a->channels)) return SA2_ERR_WORKSPACE;
    }
    return SA2_OK;
}

template <typename TX, typename TY>
int headnorm_launch(const sa2_headnorm_args *a, const sa2::headnorm::Params &P, bool backward) {
    using namespace sa2::headnorm;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);
    if (!backward) {
        const int64_t pairs = a->rows * (a->channels / a->d);
        const int grid = (int)((pairs + WARPS - 1) / WARPS < 148 * 16 ? (pairs + WARPS - 1) / WARPS : 148 * 16);
        if (a->d == 32) fwd_kernel<TX, TY, 1><<<grid, WARPS * 32, 0, st>>>(P);
        else if (a->d == 64) fwd_kernel<TX, TY, 2><<<grid, WARPS * 32, 0, st>>>(P);
        else if (a->d == 128) fwd_kernel<TX, TY, 4><<<grid, WARPS * 32, 0, st>>>(P);
        else if (a->d == 256) fwd_kernel<TX, TY, 8><<<grid, WARPS * 32, 0, st>>>(P);
        else fwd_kernel<TX, TY, 16><<<grid, WARPS * 32, 0, st>>>(P);
    } else {
        const int grid = headnorm_grid(a->rows);
        const size_t smem = (size_t)WARPS * a->channels * sizeof(float);
        auto run = [&](auto kern) -> int {
            if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return SA2_ERR_CUDA;
            kern<<<grid, WARPS * 32, smem, st>>>(P);
            return SA2_OK;
        };
        int rc;
        if (a->d == 32) rc = run(bwd_kernel<TX, TY, 1>);
        else if (a->d == 64) rc = run(bwd_kernel<TX, TY, 2>);
        else if (a->d == 128) rc = run(bwd_kernel<TX, TY, 4>);
        else if (a->d == 256) rc = run(bwd_kernel<TX, TY, 8>);
        else rc = run(bwd_kernel<TX, TY, 16>);
        if (rc != SA2_OK) return rc;
        dweight_reduce_kernel<<<(a->channels + 31) / 32, 256, 0, st>>>(P.partial, a->dweight, grid, a->channels);
    }
    return cudaGetLastError() == cudaSuccess ? SA2_OK : SA2_ERR_CUDA;
}

int headnorm_dispatch(const sa2_headnorm_args *a, bool backward) {
    const int rc = headnorm_check(a, backward);
    if (rc != SA2_OK) return rc;
    // only the backward keeps per-warp partial rows of the gain gradient in shared memory
    if (backward && (size_t)sa2::headnorm::WARPS * a->channels * sizeof(float) > 200 * 1024) return SA2_ERR_UNSUPPORTED;
    sa2::headnorm::Params P;
    P.x = a->x; P.dy = a->dy; P.weight = a->weight; P.y = a->y; P.rstd = a->rstd;
    P.partial = reinterpret_cast<float *>(a->partial);
    P.rows = a->rows; P.x_stride = a->x_stride; P.y_stride = a->y_stride; P.dy_stride = a->dy_stride;
    P.channels = a->channels; P.d = a->d; P.eps = a->eps;
    const bool xb = a->x_dtype == SA2_BF16, yb = a->y_dtype == SA2_BF16;
    if (xb && yb) return headnorm_launch<__nv_bfloat16, __nv_bfloat16>(a, P, backward);
    if (xb) return headnorm_launch<__nv_bfloat16, float>(a, P, backward);
    if (yb) return headnorm_launch<float, __nv_bfloat16>(a, P, backward);
    return headnorm_launch<float, float>(a, P, backward);
}

}  // namespace

extern "C" {

size_t sa2_headnorm_partial_bytes(int64_t rows, int32_t channels) {
    if (rows <= 0 || channels <= 0) return 0;
    return (size_t)headnorm_grid(rows) * (size_t)channels * sizeof(float);
}
int sa2_headnorm_fwd(const sa2_headnorm_args *a) {
    sa2::nvtx::Range range("sa2_headnorm_fwd");
    return headnorm_dispatch(a, false);
}
int sa2_headnorm_bwd(const sa2_headnorm_args *a) {
    sa2::nvtx::Range range("sa2_headnorm_bwd");
    return headnorm_dispatch(a, true);
}

}  // extern "C"
