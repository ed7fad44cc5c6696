/*
 * nb_attn.h -- C ABI of the B200 (sm_100a) bidirectional attention library.
 *
 * The library computes O = softmax(Q K^T * scale) V and its gradients for bf16 tensors with
 * head_dim 64, non-causal, no mask, no dropout: the arithmetic behind the single call
 *     x = F.scaled_dot_product_attention(q, k, v, is_causal=self.causal)
 * in nanobrain's Attention block (src/nanobrain/modules.py:62), whose backward is reached by
 * autograd from loss.backward() (src/nanobrain/misc.py:371).
 *
 * Conventions
 *  - All pointers except the argument structs themselves are DEVICE pointers. Buffers are
 *    borrowed for the duration of the launch; the library allocates no device memory and keeps
 *    no pointer after the call returns.
 *  - Calls enqueue work on `stream` (a cudaStream_t passed as void*) and return without
 *    synchronising. A non-zero return value is a validation or launch error (nothing was
 *    enqueued); decode it with nb_attn_strerror.
 *  - Tensors are addressed as element [batch b][token t][head h][dim d] =
 *    ptr + b*stride_batch + t*stride_token + h*stride_head + d, strides in ELEMENTS, the
 *    head_dim stride is 1. Pointers must be 16-byte aligned and strides multiples of 8.
 *    This covers the [B, L, H, 64] memory that modules.py:59-61 produces (transposed views of
 *    Linear outputs) as well as a contiguous [B, H, L, 64] tensor.
 *  - Dense mode (cu_seqlens_q == NULL): batch sequences of max_seqlen_q / max_seqlen_k tokens.
 *    Varlen mode: tokens of all sequences are packed along the token axis; sequence i owns
 *    tokens [cu_seqlens[i], cu_seqlens[i+1]); stride_batch is ignored.
 *  - lse holds the natural-log row log-sum-exp of the scaled scores, fp32, laid out
 *    [batch][heads][max_seqlen_q] in dense mode and [heads][total_q] in varlen mode.
 *  - status (optional, may be NULL) points at one int32 in device memory that the caller has
 *    zeroed. Kernels never trap: if a bounded wait inside a kernel gives up, the kernel writes
 *    a non-zero code there and still runs to completion.
 */
#ifndef NB_ATTN_H_
#define NB_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NB_ATTN_ABI_VERSION 1

enum nb_attn_error {
  NB_ATTN_OK = 0,
  NB_ATTN_ERR_NULL = 1,        /* a required pointer is NULL */
  NB_ATTN_ERR_HEAD_DIM = 2,    /* head_dim != 64 */
  NB_ATTN_ERR_SHAPE = 3,       /* non-positive or inconsistent sizes */
  NB_ATTN_ERR_ALIGN = 4,       /* pointer not 16-byte aligned or stride not a multiple of 8 */
  NB_ATTN_ERR_WORKSPACE = 5,   /* workspace missing or too small */
  NB_ATTN_ERR_TENSOR_MAP = 6,  /* the driver rejected a TMA tensor map */
  NB_ATTN_ERR_LAUNCH = 7,      /* a CUDA runtime call failed */
  NB_ATTN_ERR_DEVICE = 8,      /* the current device is not sm_100 */
  NB_ATTN_ERR_TOO_LARGE = 9    /* problem exceeds the built-in scratch of nb_attn_bwd_builtin_scratch */
};

typedef struct nb_attn_tensor {
  void* ptr;            /* bf16 */
  int64_t stride_batch; /* elements; ignored in varlen mode */
  int64_t stride_token;
  int64_t stride_head;
} nb_attn_tensor;

typedef struct nb_attn_shape {
  int32_t batch;        /* number of sequences */
  int32_t heads;
  int32_t head_dim;     /* must be 64 */
  int32_t max_seqlen_q; /* dense: the query length; varlen: an upper bound on any length */
  int32_t max_seqlen_k;
  int64_t total_q;      /* varlen: packed query tokens; dense: batch * max_seqlen_q */
  int64_t total_k;
  const int32_t* cu_seqlens_q; /* device int32 [batch + 1], or NULL for dense mode */
  const int32_t* cu_seqlens_k; /* device int32 [batch + 1], or NULL for dense mode */
  float scale;          /* softmax scale; F.scaled_dot_product_attention's default is 1/sqrt(64) */
} nb_attn_shape;

/* Forward: replaces the forward of F.scaled_dot_product_attention at
 * src/nanobrain/modules.py:62. Writes o (bf16) and lse (fp32, saved for backward). */
typedef struct nb_attn_fwd_args {
  nb_attn_shape shape;
  nb_attn_tensor q, k, v; /* inputs */
  nb_attn_tensor o;       /* output */
  float* lse;
  int32_t* status;
} nb_attn_fwd_args;

int nb_attn_fwd(const nb_attn_fwd_args* args, void* stream);

/* Backward: replaces the autograd backward of the same call (reached from
 * src/nanobrain/misc.py:368-371). Reads q, k, v, o, d_o, lse; writes dq, dk, dv (bf16).
 * `workspace` is caller-owned scratch of at least nb_attn_bwd_workspace_bytes(...) bytes,
 * 256-byte aligned; its contents on entry do not matter and are garbage on return. */
typedef struct nb_attn_bwd_args {
  nb_attn_shape shape;
  nb_attn_tensor q, k, v, o, d_o; /* inputs */
  nb_attn_tensor dq, dk, dv;      /* outputs */
  const float* lse;
  void* workspace;
  size_t workspace_bytes;
  int32_t* status;
  /* Optional profiling hooks: cudaEvent_t handles (or NULL) recorded on `stream` immediately
   * before and after the main backward kernel, i.e. between the row-dot prologue and the dQ
   * conversion epilogue, so a caller can time the dominant kernel alone. */
  void* event_main_begin;
  void* event_main_end;
} nb_attn_bwd_args;

int nb_attn_bwd(const nb_attn_bwd_args* args, void* stream);

/* Scratch bytes nb_attn_bwd needs: an fp32 dQ accumulator [total_q][heads][64] plus the
 * per-row dO.O dot products [heads * total_q]. */
size_t nb_attn_bwd_workspace_bytes(int64_t total_q, int32_t heads, int32_t head_dim);

/* Backward for callers that cannot allocate device memory (no counterpart in the reference).
 *
 * Who needs it: code that runs where a device allocation is forbidden or unavailable -- inside a
 * region that must not touch the allocator (for example between two phases of a memory-planned
 * training step whose pool is fully committed), in a host process that only borrows device
 * pointers from another runtime and owns no allocator of its own, or in a latency-critical loop
 * where a cudaMalloc would serialise the device. Such a caller still passes every input and output
 * buffer, but not the scratch: this entry point ignores args->workspace / workspace_bytes and uses
 * a fixed array that lives inside the library image on each GPU (NB_ATTN_BUILTIN_SCRATCH_ROWS rows
 * of 260 bytes, about 16.3 MiB per GPU that loads the library, held until the process exits).
 *
 * Limits and rules
 *  - total_q * heads must not exceed NB_ATTN_BUILTIN_SCRATCH_ROWS; larger problems are refused
 *    with NB_ATTN_ERR_TOO_LARGE and nothing is launched. Use nb_attn_bwd with your own workspace.
 *  - The call performs no cudaMalloc / cudaFree and calls no allocating library routine.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress with
 *    that device current). Make that first call outside any CUDA stream capture.
 *  - All calls on a GPU share the one array. It keeps whatever the previous call left in it; the
 *    kernels clear what has to start at zero themselves. Two calls whose kernels overlap on the
 *    same GPU (different streams) race on it: serialise them.
 * Results are the same as nb_attn_bwd's up to the order of the fp32 dQ additions. */
#define NB_ATTN_BUILTIN_SCRATCH_ROWS 65536
int nb_attn_bwd_builtin_scratch(const nb_attn_bwd_args* args, void* stream);

/* Human-readable text for a return code. */
const char* nb_attn_strerror(int code);

/* NB_ATTN_ABI_VERSION the library was built with. */
int nb_attn_abi_version(void);

/* Single-tile self-test of the tensor-core operand forms the kernels use (no counterpart in the
 * reference). a and b are row-major bf16 [128][128]; d receives fp32:
 *   mode 0: d[128][128] = a[:, 0:64] * b[:, 0:64]^T     mode 1, 2: d[128][64] = a * b[:, 0:64]
 *   mode 3: d[128][64]  = a^T * b[:, 0:64]
 * Modes 1 and 2 differ in where the kernel stages a (tensor memory / shared memory). */
int nb_attn_selftest_mma(int mode, const void* a, const void* b, float* d, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* NB_ATTN_H_ */
