/*
 * kda_b200.h — C ABI of the B200 (sm_100a) Kimi Delta Attention kernels.
 *
 * The reference has no C/FFI interface for this path: its fast path is one Python call,
 * fla.ops.kda.chunk_kda(...) at k3mini/model.py:197-216, selected by
 * k3mini/backends.py:155-243.  The entry points below are what a binding for that call
 * needs: plain pointers and sizes in, an int status out.  They never allocate device
 * memory, never synchronise the device and never abort; every buffer (inputs, outputs and
 * the workspace) is owned by the caller and must live on the current CUDA device.
 *
 * Tensor layouts (row-major, innermost last):
 *   q, k, g : [B, T, H, dk]      v, o, do : [B, T, H, dv]      beta : [B, T, H]
 *   A_log   : [H] float          dt_bias  : [H * dk] float (may be NULL)
 *   h0/ht/dh0/dht : [N, H, dk, dv] float, or [N, H, dv, dk] with KDA_FLAG_STATE_V_FIRST
 *   cu_seqlens : [N + 1] int64 on the device (requires B == 1), or NULL for N == B
 * q, k, v, g, beta, o, do and the gradients of the first five share one element type
 * (KDA_DTYPE_F32 or KDA_DTYPE_BF16); parameters, states and their gradients are float.
 */
#ifndef KDA_B200_H
#define KDA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KDA_CHUNK 64

enum { KDA_DTYPE_F32 = 0, KDA_DTYPE_BF16 = 1 };

enum {
    KDA_FLAG_QK_L2NORM = 1,     /* use_qk_l2norm_in_kernel   (k3mini/model.py:209) */
    KDA_FLAG_GATE = 2,          /* use_gate_in_kernel        (k3mini/model.py:210) */
    KDA_FLAG_BETA_SIGMOID = 4,  /* use_beta_sigmoid_in_kernel(k3mini/model.py:211) */
    KDA_FLAG_STATE_V_FIRST = 8, /* state_v_first             (k3mini/model.py:214) */
    KDA_FLAG_FORCE_SIMT = 16,   /* FP32 CUDA-core arithmetic in every stage (validation mode) */
    /* per-stage variants of the same switch (debugging / A-B measurements) */
    KDA_FLAG_SIMT_FWD_INTRA = 32, KDA_FLAG_SIMT_FWD_STATE = 64,
    KDA_FLAG_SIMT_BWD_STATE = 128, KDA_FLAG_SIMT_BWD_CHUNK = 256, KDA_FLAG_SIMT_BWD_WY = 512,
    /* Forward-only call: nothing is kept for a backward (no T, chunk-entry states, V' or prologue
     * records are written) and kda_workspace_bytes reports the smaller workspace.  This is the
     * forward the reference replays under activation checkpointing (k3mini/model.py:825-831) and
     * the first forward of the recompute policy (disable_recompute = False, k3mini/model.py:215);
     * o and the final state are bit-identical to the saving forward.  kda_bwd rejects the flag. */
    KDA_FLAG_NO_SAVE = 1024,
    /* Move the [64 x 128] tiles of the token-major tensors (q, k, v, g in, o and dv out) row by row instead of
     * with one bulk-tensor copy per tile.  Same bytes either way; the library falls back to this by itself
     * where the driver's tensor-map encoder is not available, and uses it for partial chunks. */
    KDA_FLAG_ROW_COPIES = 2048
};

enum {
    KDA_OK = 0,
    KDA_ERR_NULL = 1,        /* a required pointer is NULL */
    KDA_ERR_SHAPE = 2,       /* unsupported or inconsistent sizes */
    KDA_ERR_DTYPE = 3,
    KDA_ERR_WORKSPACE = 4,   /* workspace too small or misaligned */
    KDA_ERR_ALIGN = 5,       /* a tensor pointer is not 16-byte aligned */
    KDA_ERR_LAUNCH = 6,      /* the CUDA runtime refused a launch (see kda_last_cuda_error) */
    KDA_ERR_DEVICE_WAIT = 7, /* a bounded device-side wait gave up (read from the status word) */
    KDA_ERR_GUARD = 8,       /* guard span is not a finite value <= 232 (or negative = exact) */
    KDA_ERR_STATIC_LIMIT = 9, /* size beyond the built-in scratch of an allocation-free entry point */
    KDA_ERR_UNSUPPORTED = 10 /* the fused short convolution needs the BF16, d = 128 tensor-core path */
};

/* One call's description.  Replaces the keyword arguments of chunk_kda
 * (k3mini/model.py:200-216) plus the tensors autograd hands to its backward. */
typedef struct KdaParams {
    int32_t B, T, H, dk, dv;
    int32_t N;             /* number of sequences: B, or len(cu_seqlens) - 1 */
    int32_t NT;            /* total number of 64-token chunks over all sequences */
    int32_t dtype;         /* KDA_DTYPE_* */
    int32_t flags;         /* KDA_FLAG_* */
    float scale;           /* k3mini/model.py:208 */
    float guard_span;      /* log2 span limit of the guarded diagonal (k3mini/backends.py:18);
                              negative forces the exact pairwise path everywhere */
    /* forward inputs */
    const void *q, *k, *v, *g, *beta;
    const float *A_log, *dt_bias;
    const float *h0;            /* may be NULL (zero state) */
    const int64_t *cu_seqlens;  /* device, may be NULL */
    const int32_t *chunk_seq;   /* device [NT]: sequence of each chunk (needed with cu_seqlens) */
    const int32_t *seq_chunk_off; /* device [N+1]: first chunk of each sequence (with cu_seqlens) */
    /* forward outputs */
    void *o;
    float *ht;                  /* may be NULL */
    /* workspace: kda_workspace_bytes(); written by kda_fwd, read by kda_bwd */
    void *workspace;
    size_t workspace_bytes;
    /* backward inputs / outputs (ignored by kda_fwd) */
    const void *grad_o;
    const float *grad_ht;       /* may be NULL */
    void *grad_q, *grad_k, *grad_v, *grad_g, *grad_beta;
    float *grad_A_log, *grad_dt_bias; /* may be NULL unless KDA_FLAG_GATE */
    float *grad_h0;             /* may be NULL */
    void *bwd_scratch;          /* kda_workspace_bytes() second result */
    size_t bwd_scratch_bytes;
    int32_t *status;            /* device word, zero-initialised by the caller; a kernel whose
                                   bounded wait gives up ORs a non-zero code into it */
    /* Optional: the three causal depthwise short convolutions + SiLU in front of the op
     * (k3mini/model.py:181-185, conv1d of k3mini/model.py:76-88) fused into the load stage.
     * When conv_q is non-NULL, q, k, v above are the PRE-convolution projections; the taps are
     * FP32 [H*dk][conv_ksize] (channel = head * dk + d; tap j multiplies x[t - (ksize-1) + j]),
     * the window restarts at every sequence start, and the convolved rows are rounded to the
     * element type exactly as the stand-alone kda_short_conv_fwd does.  grad_q, grad_k, grad_v
     * are then gradients of the CONVOLVED rows (feed them to kda_short_conv_bwd) unless
     * grad_conv_q/k/v below are given.  All three or none; BF16 with dk = 128 only (else
     * KDA_ERR_UNSUPPORTED). */
    const float *conv_q, *conv_k, *conv_v;
    int32_t conv_ksize;         /* 1..4 */
    /* Optional with cu_seqlens: device [NT][4] int32 = {sequence, chunk inside the sequence, first
     * flattened token, valid rows} of every chunk, so that a CTA finds its chunk with one 16-byte load
     * instead of three dependent ones through chunk_seq / seq_chunk_off / cu_seqlens (16-byte aligned). */
    const int32_t *chunk_tab;
    /* Optional: a word of PINNED (device-mapped) host memory.  When set, the thread whose wait gave up
     * stores the status word into it as well, so that the host can notice by reading its own memory,
     * without a copy engine, a synchronisation or one more launch. */
    int32_t *status_host;
    /* Optional, with conv_q/k/v (kda_bwd only): FP32 [H*dk][conv_ksize] gradients of the three filters.
     * When all three are given, the backward of the short convolutions runs inside the KDA backward
     * kernels: grad_q, grad_k, grad_v then receive the gradients of the PRE-convolution projections
     * (the gradient of the convolved rows never goes to memory) and kda_workspace_bytes reports a
     * slightly larger backward scratch.  When NULL, grad_q/k/v are gradients of the convolved rows as
     * before (feed them to kda_short_conv_bwd). */
    float *grad_conv_q, *grad_conv_k, *grad_conv_v;
} KdaParams;

/* Bytes of forward workspace (saved for the backward) and of backward scratch for these
 * sizes.  Replaces the torch.empty calls inside the reference's third-party op. */
int kda_workspace_bytes(const KdaParams *p, size_t *fwd_bytes, size_t *bwd_bytes);

/* Forward of chunk_kda (k3mini/model.py:200-216): o, optional final state, and the
 * per-chunk intermediates in the workspace. */
int kda_fwd(const KdaParams *p, void *cuda_stream);

/* Backward of chunk_kda (what autograd runs for k3mini/model.py:200-216):
 * dq, dk, dv, dg, dbeta, dA_log, ddt_bias, dh0 from do, dht and the forward workspace. */
int kda_bwd(const KdaParams *p, void *cuda_stream);

/* One decoding step: the recurrence of k3mini/model.py:121-128 for ONE token per (sequence, head),
 * with the same optional prologue as chunk_kda (KDA_FLAG_QK_L2NORM / GATE / BETA_SIGMOID,
 * k3mini/model.py:217-223) and the same state layouts (KDA_FLAG_STATE_V_FIRST, model.py:214).  The
 * reference has no generation path; this is the step its final-state interface implies (the
 * third-party package it builds on ships it as fused_recurrent_kda).
 *   q, k, g : [N, H, dk]     v, o : [N, H, dv]     beta : [N, H]     states : [N, H, dk, dv] float
 * state_out may equal state_in (updated in place).  status may be NULL, else a device word that
 * receives a non-zero code if the bounded wait for the state copy gives up. */
int kda_recurrent_step(const void *q, const void *k, const void *v, const void *g, const void *beta,
                       const float *A_log, const float *dt_bias, const float *state_in, float *state_out,
                       void *o, int32_t N, int32_t H, int32_t dk, int32_t dv, int32_t dtype, int32_t flags,
                       float scale, int32_t *status, void *cuda_stream);

/* Causal depthwise short convolution + SiLU over [B, T, C] (k3mini/model.py:76-88; the
 * fast path's fla.modules.ShortConvolution at k3mini/model.py:147-155).  weight is
 * [C, 1, ksize] float, ksize <= 4; cu_seqlens as above (no tap crosses a document). */
int kda_short_conv_fwd(const void *x, const float *weight, void *y, int32_t B, int32_t T, int32_t C,
                       int32_t ksize, int32_t dtype, const int64_t *cu_seqlens, int32_t N,
                       void *cuda_stream);
/* dweight [C, ksize] is reduced in a fixed order from partial [n_partial, C, ksize]
 * (caller scratch; n_partial token-tile groups run in parallel, 64..512 is a good range). */
int kda_short_conv_bwd(const void *x, const float *weight, const void *dy, void *dx, float *dweight,
                       float *partial, int32_t n_partial, int32_t B, int32_t T, int32_t C, int32_t ksize,
                       int32_t dtype, const int64_t *cu_seqlens, int32_t N, void *cuda_stream);

/* Allocation-free variant of kda_short_conv_bwd.  It has no counterpart in the reference; it
 * exists for hosts that may not create device memory at call time: a plugin running under a
 * memory plan that was frozen at start-up, a real-time loop that forbids allocator calls, a
 * process whose memory pool is owned by another runtime.  Such a caller still passes its input
 * and output tensors, but no scratch: the per-token-group partial sums of dweight live in a
 * 2 MiB array that is part of the library image on every GPU that loads it.
 *   - Limit: C * ksize <= 8192 (e.g. 2048 channels with 4 taps); larger sizes return
 *     KDA_ERR_STATIC_LIMIT and launch nothing.
 *   - The first call on each device looks up that device's address of the array (the device
 *     must be current); make that first call outside any stream capture.  Later calls do no
 *     set-up.  No call allocates or frees device memory.
 *   - All calls on a device share the one array.  Every element that is read is rewritten by
 *     the same call first, so nothing needs clearing, but two calls that overlap on the GPU
 *     (different streams) race on it: serialise them.
 *   - Results equal kda_short_conv_bwd with n_partial = 64 bit for bit.
 *   - The per-device address table holds device ordinals 0..63 (a higher ordinal returns
 *     KDA_ERR_STATIC_LIMIT), and an address looked up before cudaDeviceReset() is stale afterwards:
 *     do not reset a device between calls. */
int kda_short_conv_bwd_static(const void *x, const float *weight, const void *dy, void *dx, float *dweight,
                              int32_t B, int32_t T, int32_t C, int32_t ksize, int32_t dtype,
                              const int64_t *cu_seqlens, int32_t N, void *cuda_stream);

/* Headwise RMSNorm(x) * sigmoid(gate) over [rows, dim] (k3mini/model.py:91-98; the fast
 * path's fla.modules.FusedRMSNormGated at k3mini/model.py:171-175). */
int kda_norm_gate_fwd(const void *x, const void *gate, const float *weight, void *y, float *rstd,
                      int64_t rows, int32_t dim, float eps, int32_t dtype, void *cuda_stream);
/* dweight [dim] is reduced in a fixed order from partial [n_partial, dim] (caller scratch). */
int kda_norm_gate_bwd(const void *x, const void *gate, const float *weight, const void *dy, void *dx,
                      void *dgate, float *dweight, float *partial, int32_t n_partial, int64_t rows,
                      int32_t dim, float eps, int32_t dtype, void *cuda_stream);

/* The guarded diagonal tile with the interface of the reference's device-independent contract
 * (experiments/kda_sm90/guarded_diagonal_oracle.py:110-180, reference_policy="midpoint"):
 * float tensors gate, q, k [n_tiles,16,32], beta [n_tiles,16], dAqk, dAkk [n_tiles,16,16] ->
 * dq, dk, dkt [n_tiles,16,32] and hits [n_tiles] (1 = midpoint factorisation used).  Same
 * guard and evaluation rules as the intra-chunk backward; a negative span rejects every tile.
 * The oracle accepts spans in (0, 252); this entry also accepts negative values. */
int kda_guarded_diagonal_tiles(const float *gate, const float *q, const float *k, const float *beta,
                               const float *dAqk, const float *dAkk, float *dq, float *dk, float *dkt,
                               int *hits, int n_tiles, float max_log2_span, void *cuda_stream);

/* Gate-span statistic of the reference's span profiler (scripts/profile_kda_gate_spans.py:21-56):
 * raw [B, T, H, d] (T a multiple of 64, d a multiple of 32, d <= 256), a_log [H], dt_bias [H * d] ->
 * out [B * T/64 * 4 * H * d/32] float: per [16 rows x 32 channels] tile of the within-chunk cumulative
 * log2 decay -exp(A_log) softplus(raw + dt_bias) / ln 2, the largest drop below the tile's first row. */
int kda_gate_tile_spans(const void *raw, const float *a_log, const float *dt_bias, float *out, int32_t B,
                        int32_t T, int32_t H, int32_t d, int32_t dtype, void *cuda_stream);

/* Guarded-diagonal contract of the reference's backend check (k3mini/backends.py:17-19,
 * 68-109): version 1, "tf32x3"-class precision, span <= 232. */
int kda_guard_version(void);
float kda_guard_max_span(void);
const char *kda_guard_dot_precision(void);

/* Benchmark instrumentation (no reference counterpart; the reference times its op from
 * Python with CUDA events, scripts/benchmark_kda_backends.py:119-165).  After
 * kda_profile_begin(n) the next n kda_fwd / kda_bwd calls bracket each of their kernels with
 * CUDA events on the caller's stream.  After the stream is synchronised,
 * kda_profile_read(call, &kind, ms, max) returns the number of stages of that call
 * (kind 0 = forward, 1 = backward) and their durations in milliseconds, or -1. */
int kda_profile_begin(int max_calls);
int kda_profile_read(int call, int *kind, float *stage_ms, int max_stages);

/* Device self-test of the tcgen05 building block (no reference counterpart): one CTA
 * computes D[128,N] = A[128,K] * B[K,N] (FP32 in, BF16 operands, FP32 accumulate) with the
 * operand view (shared K-major / MN-major, or A in tensor memory) and the descriptor strides
 * given by the caller.  Used by the tests to pin the operand layouts the kernels rely on. */
int kda_selftest_mma(const float *A, const float *B, float *D, int N, int K, int a_mode, int b_mode,
                     int lbo_a, int sbo_a, int step_a, int lbo_b, int sbo_b, int step_b, int neg_a,
                     int m_rows, int *status, void *cuda_stream);

/* Device self-test of the bounded wait (no reference counterpart): one CTA arms an mbarrier for
 * twice the 256 bytes its single bulk copy delivers and polls at most poll_limit (1..4096) times.
 * The wait runs out by construction; the kernel ORs `code` (1..255) into *status, waits for the
 * copy that is in flight, copies the 64 floats src -> dst, frees its tensor memory and returns.
 * The device stays usable; the tests use it to check that a given-up wait is reported. */
int kda_selftest_wait(const float *src, float *dst, int poll_limit, int code, int *status, void *cuda_stream);

/* Launches a one-thread kernel on the given stream that copies a non-zero *status into *status_host
 * (pinned, device-mapped): for entry points that take a bare status pointer, such as kda_recurrent_step. */
int kda_status_publish(const int32_t *status, int32_t *status_host, void *cuda_stream);

const char *kda_status_string(int status);
const char *kda_last_cuda_error(void);
int kda_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* KDA_B200_H */
