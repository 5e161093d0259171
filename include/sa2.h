/*
 * sa2.h - C ABI of the sliding-window causal 2-simplicial attention kernels
 * for NVIDIA B200 (sm_100a).
 *
 * The library replaces the Triton kernels and the autograd launcher of
 * lucidrains/simplicial-attention; each entry point names the reference code
 * it stands in for (paths relative to the reference project).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer owned by the caller; the library
 *     allocates nothing and keeps no reference after the call returns;
 *   - tensors are addressed as [batch][seq][head][channel] with explicit
 *     element strides for batch, seq and head; the channel stride is 1
 *     (the reference requires the same: triton_two_simplicial_attention.py:39-40,731);
 *   - launches are asynchronous on `stream` (a cudaStream_t passed as void*);
 *   - every function returns an sa2_status; nothing throws, aborts or traps.
 *
 * Semantics (one batch b, query head h, kv head h / (hq/hk)):
 *   S_ijk = scale * sum_c q_ic k1_jc k2_kc   for 0 <= i-j < w1, 0 <= i-k < w2
 *   LSE_i = log sum_jk exp S_ijk             (natural log)
 *   O_ic  = sum_jk exp(S_ijk - LSE_i) v1_jc v2_kc
 * Query row i sits at key position i + off1 of k1/v1 and i + off2 of k2/v2:
 * off1/off2 are the numbers of extra ("halo") key rows that precede the first
 * query row, used when a long sequence is split into blocks across GPUs.  With
 * off1 = off2 = 0 this is the reference's operator.
 */
#ifndef SA2_H
#define SA2_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum sa2_status {
    SA2_OK = 0,
    SA2_ERR_INVALID = 1,       /* null pointer, non-positive size, hq % hk != 0 ... */
    SA2_ERR_UNSUPPORTED = 2,   /* head dim not in {32, 64, 128}, unknown dtype, kernel not applicable */
    SA2_ERR_WORKSPACE = 3,     /* workspace missing or smaller than sa2_bwd_workspace_bytes() */
    SA2_ERR_CUDA = 4,          /* a CUDA runtime / driver call failed */
    SA2_ERR_DEVICE = 5,        /* a kernel gave up on a bounded wait */
    SA2_ERR_TOO_LARGE = 6      /* beyond the capacity of sa2_bwd_static_scratch */
} sa2_status;

typedef enum sa2_dtype { SA2_F32 = 0, SA2_BF16 = 1 } sa2_dtype;

/* Which implementation runs.  AUTO picks the tcgen05 tensor-core path when the
 * problem fits it (bf16, supported head dim) and the fp32 SIMT path otherwise. */
typedef enum sa2_kernel { SA2_KERNEL_AUTO = 0, SA2_KERNEL_SIMT = 1, SA2_KERNEL_TCGEN05 = 2 } sa2_kernel;

/* element strides of one [batch][seq][head][channel] tensor */
typedef struct sa2_strides {
    int64_t batch, seq, head;
} sa2_strides;

typedef struct sa2_shape {
    int32_t b;        /* batch */
    int32_t n;        /* query rows (= rows of out, dout, dq) */
    int32_t hq;       /* query heads */
    int32_t hk;       /* key/value heads, hq % hk == 0 */
    int32_t d;        /* head dim: 32, 64 or 128 */
    int32_t w1;       /* window over k1/v1: 0 <= i-j < w1 */
    int32_t w2;       /* window over k2/v2: 0 <= i-k < w2 */
    int32_t off1;     /* halo rows in k1/v1 (they hold n + off1 rows) */
    int32_t off2;     /* halo rows in k2/v2 (they hold n + off2 rows) */
    int32_t dtype;    /* sa2_dtype of q, k1, k2, v1, v2, out, dout */
    int32_t kernel;   /* sa2_kernel */
    float   scale;    /* logit scale; the reference uses d^-0.5 */
} sa2_shape;

/*
 * Parts of the backward that sa2_bwd_args.phases can select (0 runs all of them).  ROWSUM writes
 * D_i = sum_c O_ic dO_ic into the workspace; K1 (dK1, dV1) and Q (dQ, dK2, dV2) read it and are
 * independent of each other, so a caller may time them apart or run them on different streams
 * after ROWSUM has been ordered before both.
 */
typedef enum sa2_bwd_phase { SA2_BWD_ROWSUM = 1, SA2_BWD_K1 = 2, SA2_BWD_Q = 4 } sa2_bwd_phase;

typedef struct sa2_fwd_args {
    sa2_shape shape;
    const void *q, *k1, *k2, *v1, *v2;
    void  *out;               /* [b][n][hq][d], dtype */
    float *lse;               /* [b][hq][n] fp32 contiguous, natural log */
    sa2_strides sq, sk1, sk2, sv1, sv2, sout;
    void *stream;
} sa2_fwd_args;

typedef struct sa2_bwd_args {
    sa2_shape shape;
    const void *q, *k1, *k2, *v1, *v2;
    const void *out, *dout;   /* saved forward output and its gradient */
    const float *lse;         /* saved logsumexp from sa2_fwd */
    void *dq;                 /* [b][n][hq][d] */
    void *dk1, *dv1;          /* [b][n+off1][hk][d], summed over each kv head's query group */
    void *dk2, *dv2;          /* [b][n+off2][hk][d] */
    sa2_strides sq, sk1, sk2, sv1, sv2, sout, sdout, sdq, sdk1, sdk2, sdv1, sdv2;
    int32_t grad_dtype;       /* sa2_dtype of dq, dk1, dk2, dv1, dv2 */
    int32_t phases;           /* 0: the whole backward; otherwise an OR of sa2_bwd_phase */
    void  *workspace;         /* >= sa2_bwd_workspace_bytes(&shape) bytes, 256-byte aligned */
    size_t workspace_bytes;
    void *stream;
} sa2_bwd_args;

/*
 * Forward: writes out and lse.
 * Replaces two_simplicial_attn_fwd_kernel
 * (simplicial_attention/triton_two_simplicial_attention.py:48-228) and its
 * launch in SlidingTwoSimplicialAttention.forward (:721-807).  Unlike the
 * reference it needs no padding of the sequence, reads grouped-query heads in
 * place (no repeat, :1029-1034) and returns the logsumexp to the caller.
 */
int sa2_fwd(const sa2_fwd_args *args);

/*
 * Backward: writes dq, dk1, dk2, dv1, dv2 (every element; no zero-fill needed).
 * Replaces backward_preprocess_do_o_dot (:230-286),
 * two_simplicial_attn_bwd_kv1_kernel (:288-503), the two passes of
 * two_simplicial_attn_bwd_kv2q_kernel (:505-712) and their launches in
 * SlidingTwoSimplicialAttention.backward (:809-1006).  No floating-point
 * atomics: results are bitwise reproducible run to run.
 */
int sa2_bwd(const sa2_bwd_args *args);

/*
 * Scratch bytes sa2_bwd needs for this shape (the per-row dot products
 * D_i = sum_c O_ic dO_ic, which the reference keeps in a tensor it allocates
 * itself at :825).  The forward needs none.
 */
size_t sa2_bwd_workspace_bytes(const sa2_shape *shape);

/*
 * Backward for callers that cannot supply scratch memory.  It has no
 * counterpart in the reference, which allocates whatever it needs from torch.
 *
 * Who needs it: a host that gave all device memory to its own pools before this
 * library was loaded, a plug-in that may launch kernels but not call an
 * allocator, a loop in which allocation is ruled out for latency reasons.
 * `args->workspace` and `args->workspace_bytes` are ignored; the row sums
 * D_i = sum_c O_ic dO_ic go into an array compiled into the library
 * (SA2_STATIC_SCRATCH_ROWS floats = 1 MiB, held by every GPU that loads the
 * library until the process ends).  The call allocates and frees nothing.
 *
 *   - Limit: b * hq * n <= SA2_STATIC_SCRATCH_ROWS, otherwise SA2_ERR_TOO_LARGE.
 *   - Runs the fp32 kernels (any head dim in {32, 64, 128}, fp32 or bf16
 *     tensors); shape.kernel == SA2_KERNEL_TCGEN05 is SA2_ERR_UNSUPPORTED
 *     because the tensor-core backward needs far more scratch than this.
 *     Results equal sa2_bwd with shape.kernel == SA2_KERNEL_SIMT.
 *   - The first call on each device looks up the array's device address (the
 *     device must be current, as for every call); make that first call before
 *     starting any stream capture.
 *   - All calls share the one array, which keeps whatever the previous call
 *     left in it.  Nothing in it has to start at zero - each call rewrites the
 *     entries it reads - but two calls that overlap in time on the same GPU
 *     (different streams, or different threads) race on it: keep them ordered.
 */
#define SA2_STATIC_SCRATCH_ROWS 262144
int sa2_bwd_static_scratch(const sa2_bwd_args *args);

/*
 * Number of kernel launches sa2_fwd (backward == 0) or sa2_bwd (backward != 0)
 * issues for this shape, or -1 for a shape they would reject.  The reference
 * launches 1 forward and 4 backward kernels plus 5 memsets (:749,834,868,938,972,853-857).
 */
int sa2_kernel_launches(const sa2_shape *shape, int backward);

/*
 * Device status word of the current device: 0 when every kernel ran to
 * completion, otherwise the OR of the error bits of kernels that gave up on a
 * bounded wait (the rows they owned are then written as NaN).  Synchronises the device;
 * meant for tests and diagnostics, not for the hot path.  `reset` != 0 clears
 * the word.  Returns -1 if the word cannot be read.  No counterpart in the
 * reference, whose Triton kernels contain no waits.
 */
int sa2_device_status(int reset);

/*
 * The same check as a status: SA2_OK when the status word is 0, SA2_ERR_DEVICE
 * when a kernel gave up on a bounded wait since the last reset (the rows that
 * kernel owned were written as NaN), SA2_ERR_CUDA if the word cannot be read.
 * Synchronises the device.  No counterpart in the reference.
 */
int sa2_check_device(int reset);

/*
 * Self-test of the bounded waits: launches one warp that waits, for at most `limit_cycles` SM clock
 * cycles (1 ... 2e9), on a barrier nobody arrives on.  The wait runs out, the kernel sets
 * SA2_SELFTEST_WAIT_BIT in the device status word and ends normally - nothing faults or hangs.
 * sa2_check_device() then reports SA2_ERR_DEVICE once.  No counterpart in the reference.
 */
#define SA2_SELFTEST_WAIT_BIT 0x10000
int sa2_selftest_wait(long long limit_cycles, void *stream);

/* Static, human-readable text for a status code. */
const char *sa2_strerror(int status);

/* Library version as major*10000 + minor*100 + patch. */
int sa2_version(void);

/*
 * Per-head RMSNorm of a packed projection - stands in for the five RMSNorm
 * modules the reference applies to q, k, k', v, v' after splitting its fused
 * projection (simplicial_attention/simplicial_mha.py:69-73,124-127).
 *
 * x is [rows][channels] with row stride x_stride (elements), channels
 * contiguous; every group of d consecutive channels is one head; weight holds
 * one gain per channel (each norm's d gains tiled over its heads):
 *   rstd[r][g] = rsqrt(mean_{c in head g} x[r][c]^2 + eps)
 *   y[r][c]    = x[r][c] * rstd[r][c / d] * weight[c]
 * sa2_headnorm_bwd returns dx (layout and dtype of x) and dweight[channels];
 * `partial` is caller-owned scratch of sa2_headnorm_partial_bytes().  d must be
 * 32, 64, 128, 256 or 512 (with channels = d it is an ordinary RMSNorm over the
 * whole row) and channels a multiple of d.  x_dtype / y_dtype are the
 * element types of x (and dx) and of y (and dy).
 */
typedef struct sa2_headnorm_args {
    const void *x;
    const void *dy;        /* backward only */
    const float *weight;
    void *y;               /* forward: y; backward: dx */
    float *rstd;           /* [rows][channels / d]: written by the forward, read by the backward */
    float *dweight;        /* backward only: [channels] */
    void *partial;         /* backward only */
    size_t partial_bytes;
    int64_t rows, x_stride, y_stride, dy_stride;
    int32_t channels, d;
    int32_t x_dtype, y_dtype;
    float eps;
    void *stream;
} sa2_headnorm_args;

int sa2_headnorm_fwd(const sa2_headnorm_args *args);
int sa2_headnorm_bwd(const sa2_headnorm_args *args);
size_t sa2_headnorm_partial_bytes(int64_t rows, int32_t channels);

#ifdef __cplusplus
}
#endif
#endif /* SA2_H */
