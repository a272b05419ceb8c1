/*
 * sb_b200.h -- C ABI of the B200 (sm_100a) stick-breaking attention kernels.
 *
 * Plain C: device pointers, sizes and element strides only; no framework types.  The caller owns
 * every buffer (inputs, outputs, saved state, workspace, status word); the library keeps nothing
 * between calls except per-process caches of driver entry points and kernel attributes.  Every
 * entry point only enqueues work on the given stream and never synchronises.  Calls on different
 * streams or devices may run concurrently as long as they do not share output or workspace memory.
 *
 * Tensor convention (same as the reference operators): q, k, v, o and their gradients are
 * (batch, heads, tokens, head_dim) with arbitrary element strides for the first three axes and a
 * unit stride on head_dim.  A packed variable-length batch is batch == 1 with `cu_seqlens` holding
 * the END offset of every sequence (no leading zero), exactly what
 * stickbreaking_attention/sb_varlen/__init__.py:71-78 hands to its kernels after stripping the zero.
 * A fixed-length batch passes cu_seqlens == NULL.
 */
#ifndef SB_B200_H_
#define SB_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SB_ABI_VERSION 2

#if defined(__GNUC__)
#define SB_EXPORT __attribute__((visibility("default")))
#else
#define SB_EXPORT
#endif

enum SbDtype { SB_DTYPE_F32 = 0, SB_DTYPE_BF16 = 1, SB_DTYPE_F16 = 2 };

enum SbStatus {
  SB_OK = 0,
  SB_ERR_ARGUMENT = 1,     /* bad shape, stride, pointer or struct size; see sb_last_error()  */
  SB_ERR_WORKSPACE = 2,    /* workspace missing or smaller than sb_workspace_bytes()          */
  SB_ERR_CUDA = 3,         /* a CUDA runtime/driver call failed; see sb_last_error()          */
  SB_ERR_NO_DEVICE_CODE = 4 /* device is not sm_100: there is no other code path              */
};

/* Codes the kernels write to status[0] (device memory, 4 x int32, caller-zeroed). */
enum SbDeviceStatus {
  SB_DEV_OK = 0,
  SB_DEV_BAD_CU_SEQLENS = 1, /* not non-decreasing, beyond `tokens`, or longer than max_seqlen;
                                status[1] = index of the offending sequence.  No kernel of the
                                call then computes anything, and every row of the call's outputs
                                is filled with NaN (where the reference raises on the host,
                                sb_varlen/__init__.py:72-74)                                   */
  SB_DEV_WAIT_TIMEOUT = 2    /* a bounded on-chip wait gave up; status[1] = which barrier      */
};

enum SbKernelPath {
  SB_PATH_SIMT = 0,     /* fp32 arithmetic on CUDA cores: fp32 tensors and irregular head_dim  */
  SB_PATH_TCGEN05 = 1   /* tcgen05 MMAs with TMEM accumulators, TMA-staged tiles: bf16 / fp16  */
};

enum SbFlags {
  SB_FLAG_FORCE_SIMT = 1, /* run the CUDA-core kernels even where the tensor-core ones apply   */
  SB_FLAG_CHECK_LEADING_ZERO = 2, /* cu_seqlens points one past the caller's leading 0 (the
                            `zero_start` form of sb_varlen/__init__.py:72-74): the element before
                            cu_seqlens[0] is read and must be 0, else SB_DEV_BAD_CU_SEQLENS with
                            status[1] = -1.  Replaces the reference's host-side assert, which
                            forces a device synchronisation.                                    */
  SB_FLAG_BWD_SKIP_DKV = 4, /* timing aid: sb_bwd enqueues only the dQ kernel                   */
  SB_FLAG_BWD_SKIP_DQ = 8,  /* timing aid: sb_bwd enqueues only the dK/dV kernel, which then reads
                            what a previous full sb_bwd left in the same workspace              */
  SB_FLAG_BWD_RECOMPUTE = 16, /* small-workspace backward.  By default (16-bit tensors, head_dim up to 128)
                            the dQ kernel stores its A and dz tiles -- 64 KiB per (query tile, key tile)
                            pair and head, heads processed in chunks that fit the scratch budget (8 GiB
                            unless sb_set_backward_scratch_budget changed it) -- and the dK/dV kernel is
                            two plain GEMMs over them.  With this flag, or when one head alone exceeds the
                            budget, the dK/dV kernel recomputes the tiles from boundary values (a few KiB
                            per pair).  Same 16-bit tiles either way.                             */
  SB_FLAG_FUSE_REM_V = 32,  /* the caller wants out = o + rem[..., None] * v, what every caller of the
                            reference computes right after the operator (tests/test_varlen.py:101,
                            tests/test_attn.py:64).  sb_fwd writes `out` to `o` (rem and log_rem as usual).
                            sb_bwd takes d_out in `d_o`, adds <d_out, v> per row to d_rem (which may then be
                            NULL = zero) and rem * d_out to dv, and needs 4 more workspace bytes per
                            (batch, head, token).                                                  */
  SB_FLAG_DENSE_ROW_PASS = 64 /* measuring aid.  The attention weight of a key is its beta times the product of
                            (1 - beta) over the keys between it and the query; in fp32 that product underflows to
                            exactly 0 once the keys in between carry about 126 bits of -log2(1 - beta).  From
                            there on everything a row computes per score (p in the forward; A, G and dz in the
                            backward) is exactly 0, and the tensor-core kernels skip that arithmetic wherever it
                            is 0 for all 32 rows of a warp: they keep only the running log-space sum.  Every MMA
                            is still issued and the results are bit-identical.  With this flag the arithmetic is
                            done for every score regardless.                                      */
};

typedef struct SbTensor {
  void *ptr;        /* device pointer to element (0,0,0,0)                   */
  int64_t stride_b; /* element strides; the head_dim stride is 1 by contract */
  int64_t stride_h;
  int64_t stride_t;
} SbTensor;

typedef struct SbParams {
  int32_t struct_bytes; /* = sizeof(SbParams); checked                                          */
  int32_t dtype;        /* SbDtype of q,k,v,o,rem and all gradients                             */
  int32_t batch;        /* 1 for a packed variable-length batch                                 */
  int32_t heads;
  int32_t head_dim;     /* 1..256                                                               */
  int32_t num_seq;      /* entries in cu_seqlens (0 when cu_seqlens == NULL)                    */
  int64_t tokens;       /* size of the tokens axis                                              */
  int32_t max_seqlen;   /* upper bound on any sequence length; 0 means `tokens`                 */
  int32_t attend_current; /* 0: key j < query i (default of the reference); 1: j <= i           */
  int32_t cu_seqlens_int64; /* element type of cu_seqlens: 0 = int32, 1 = int64                 */
  float logit_scale;    /* multiplies <q,k>; the reference default is 1/sqrt(head_dim)          */
  int32_t flags;        /* SbFlags                                                              */
  int32_t reserved;     /* must be 0                                                            */
  const void *cu_seqlens; /* device, num_seq sequence END offsets, or NULL                      */

  SbTensor q, k, v;     /* in                                                                    */
  SbTensor o;           /* out (forward)                                                         */
  void *rem;            /* out (forward): (batch, heads, tokens) contiguous, `dtype`             */
  double *log_rem;      /* forward out / backward in: (batch, heads, tokens) contiguous fp64,    *
                         * sum over allowed keys of log2(1 - beta).  Plays the part of the       *
                         * reference's fp32 `neg_log_acc` (sb_varlen_fwd.py:420,205).            */

  SbTensor d_o;         /* in  (backward)                                                        */
  const void *d_rem;    /* in  (backward): (batch, heads, tokens) contiguous, `dtype`            */
  SbTensor dq, dk, dv;  /* out (backward); every covered row is written, none is accumulated     */

  void *workspace;      /* device scratch of at least sb_workspace_bytes() bytes, 256-B aligned  */
  size_t workspace_bytes;
  int32_t *status;      /* device int32[4], zeroed by the caller, or NULL                        */

  float *attn_weights;  /* optional out (forward), NULL otherwise: fp32 (batch, heads, tokens, attn_cols)  *
                         * contiguous and ZEROED by the caller.  Row t receives the attention weights of   *
                         * token t, entry j being the weight on the j-th key of t's own sequence (j <      *
                         * attn_cols).  This is the `return_attention` / W output the reference marks TODO *
                         * (sb_varlen_fwd.py:195-202, 421-425): same fp32, caller-zeroed, sequence-local   *
                         * key index.  A debugging aid: the call then runs the CUDA-core kernels, whatever *
                         * the dtype.                                                                       */
  int64_t attn_cols;    /* columns of attn_weights (>= the longest sequence to get every weight)          */
} SbParams;

/* Scratch bytes sb_fwd (backward == 0) or sb_bwd (backward != 0) needs for these shapes.  Looks at
 * shapes, dtype, max_seqlen and flags only, never at device memory.  Stands in for the per-call
 * allocations the reference makes inside its launchers (lock and count arrays,
 * sb_varlen_bwd.py:568-573).  Returns (size_t)-1 for invalid parameters. */
SB_EXPORT size_t sb_workspace_bytes(const SbParams *p, int backward);

/* Forward: writes o, rem, log_rem for every token covered by a sequence (tokens past the last
 * sequence end are zero-filled).  Replaces `_compileable_forward`, i.e. the custom ops
 * stickbreaking_attention::varlen_fwd (sb_varlen_fwd.py:454-522) and ::attn_fwd
 * (sb_attn/sb_fwd.py:177-253).  `stream` is a cudaStream_t.  Returns an SbStatus. */
SB_EXPORT int sb_fwd(const SbParams *p, void *stream);

/* Backward: reads q, k, v, log_rem, d_o, d_rem and writes dq, dk, dv.  Deterministic: no atomics,
 * no locks, bitwise identical from run to run.  Replaces `_compileable_backward`, i.e. the custom
 * ops ::varlen_bwd (sb_varlen_bwd.py:542-641) and ::attn_bwd (sb_attn/sb_bwd.py:208-297). */
SB_EXPORT int sb_bwd(const SbParams *p, void *stream);

/* Forward pass for callers that cannot allocate device memory.  No counterpart in the reference, which
 * allocates freely inside its launchers.
 *
 * Who needs it: a host that hands an operator a fixed memory arena at start-up and forbids later allocation
 * (inference servers, embedded runtimes); a latency-critical loop in which cudaMalloc's implicit device-wide
 * synchronisation is unacceptable; a plain C caller that only holds the tensors it was given and has no
 * allocator to ask.  Such a caller still passes q, k, v, o, rem and log_rem, but leaves `workspace` and
 * `workspace_bytes` unset: the forward's scratch (the sequence table built from cu_seqlens) lives in an array
 * of SB_STATIC_SCRATCH_BYTES bytes inside the library's device image.  Every GPU that loads the library holds
 * that array until the process exits.
 *
 * Same results as sb_fwd.  A call fits when sb_workspace_bytes(p, 0) <= SB_STATIC_SCRATCH_BYTES; that is the whole
 * rule.  (The scratch holds the sequence table: a few hundred bytes plus about 12 bytes per packed sequence and 8
 * bytes per work item, an item being 256 tokens on the tensor-core path (128 tokens for head sizes up to 64 with
 * max_seqlen <= 1024) and 32 tokens on the CUDA-core path that fp32 tensors and irregular head sizes take; a
 * fixed-length batch always fits.)  A call that does not fit returns
 * SB_ERR_WORKSPACE with a message and launches nothing.  The function calls no cudaMalloc, cudaFree or any other
 * allocating routine.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 * current); make that first call before any stream capture begins.  All calls on a device share the one
 * array, which keeps whatever the previous call left in it; each call rewrites the parts it reads.  Two calls
 * whose kernels may overlap on the GPU (different streams, or different threads) race on it: serialise them. */
#define SB_STATIC_SCRATCH_BYTES 65536
SB_EXPORT int sb_fwd_static_scratch(const SbParams *p, void *stream);

/* Upper bound, in bytes, on the scratch one chunk of heads of sb_bwd may take (default 8 GiB); returns the previous
 * value, and with bytes == 0 only reports it.  Process-wide; affects sb_workspace_bytes(p, 1) and sb_bwd alike, so
 * set it before sizing a workspace.  The backward works through the heads in chunks whose stored attention tiles
 * (64 KiB per 128 x 128 tile pair and head) fit the bound, and takes the recomputing dK/dV kernel when one head alone
 * does not fit.  The reference has no counterpart: its backward keeps nothing but lock arrays
 * (sb_varlen_bwd.py:568-573). */
SB_EXPORT size_t sb_set_backward_scratch_budget(size_t bytes);

/* Which kernels sb_fwd / sb_bwd run for these parameters (an SbKernelPath), or -1 if invalid. */
SB_EXPORT int sb_kernel_path(const SbParams *p);

/* Number of kernel launches the last sb_fwd / sb_bwd call of this thread enqueued. */
SB_EXPORT int sb_last_launch_count(void);

/* Text of the last error returned to this thread ("" if none). */
SB_EXPORT const char *sb_last_error(void);

SB_EXPORT int sb_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SB_B200_H_ */
