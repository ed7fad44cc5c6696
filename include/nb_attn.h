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
 *  - status (optional, may be NULL) points at one int32 that the caller has zeroed, in device
 *    memory or in pinned host memory that the device can address. Kernels never trap: they write a
 *    non-zero code there and still run to completion. NB_ATTN_STATUS_WAIT_TIMEOUT: a bounded wait
 *    inside a kernel gave up (results are garbage). NB_ATTN_STATUS_BAD_SEQLENS: the device-side
 *    check of cu_seqlens failed -- offsets negative or decreasing, a sequence longer than
 *    max_seqlen_q / max_seqlen_k, or the last offset beyond total_q / total_k; the attention
 *    kernels then do nothing and the outputs are left unwritten.
 *  - Varlen contract: max_seqlen_q / max_seqlen_k must be true upper bounds of the sequence
 *    lengths in cu_seqlens (they size tensor maps and the work list); the kernels verify this on
 *    the device and report NB_ATTN_STATUS_BAD_SEQLENS instead of dropping tiles.
 *  - Varlen scheduling: every call turns cu_seqlens into a work list of (sequence, 128-row tile)
 *    items on the device, most expensive items first and ragged last tiles at the end; the forward
 *    launches one CTA per item and head, the backward one persistent CTA per SM that takes the
 *    (item, head) pairs in list order. The list lives in the call's workspace.
 *  - Varlen padding: cu_seqlens[batch] may be smaller than total_q / total_k (tokens packed into
 *    a buffer of fixed capacity). The rows past the last sequence belong to no sequence; the
 *    kernels write zeros to them in o, dq, dk and dv (and -inf in lse), so every output row is
 *    defined.
 */
#ifndef NB_ATTN_H_
#define NB_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NB_ATTN_ABI_VERSION 2

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

/* Codes a kernel may write to the status word. */
enum nb_attn_status {
  NB_ATTN_STATUS_OK = 0,
  NB_ATTN_STATUS_WAIT_TIMEOUT = 1,
  NB_ATTN_STATUS_BAD_SEQLENS = 2
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
 * src/nanobrain/modules.py:62. Writes o (bf16) and lse (fp32, saved for backward).
 * Varlen mode needs `workspace`: caller-owned scratch of at least
 * nb_attn_fwd_workspace_bytes(&shape) bytes, 256-byte aligned, for the work list (contents on
 * entry do not matter). Dense mode ignores it. */
typedef struct nb_attn_fwd_args {
  nb_attn_shape shape;
  nb_attn_tensor q, k, v; /* inputs */
  nb_attn_tensor o;       /* output */
  float* lse;
  int32_t* status;
  void* workspace;
  size_t workspace_bytes;
} nb_attn_fwd_args;

int nb_attn_fwd(const nb_attn_fwd_args* args, void* stream);

/* Scratch bytes nb_attn_fwd needs: the work list of query tiles in varlen mode, 0 in dense mode. */
size_t nb_attn_fwd_workspace_bytes(const nb_attn_shape* shape);

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

/* Scratch bytes nb_attn_bwd needs: an fp32 dQ accumulator [total_q][heads][64], the per-row
 * dO.O dot products [heads * total_q] and, in varlen mode, the work list of key tiles. */
size_t nb_attn_bwd_workspace_bytes(const nb_attn_shape* shape);

/* Backward for callers that cannot allocate device memory (no counterpart in the reference).
 *
 * Who needs it: code that runs where a device allocation is forbidden or unavailable -- inside a
 * region that must not touch the allocator (for example between two phases of a memory-planned
 * training step whose pool is fully committed), in a host process that only borrows device
 * pointers from another runtime and owns no allocator of its own, or in a latency-critical loop
 * where a cudaMalloc would serialise the device. Such a caller still passes every input and output
 * buffer, but not the scratch: this entry point ignores args->workspace / workspace_bytes and uses
 * a fixed array that lives inside the library image on each GPU (NB_ATTN_BUILTIN_SCRATCH_ROWS rows
 * of 260 bytes plus NB_ATTN_BUILTIN_SCRATCH_ITEMS work-list entries of 32 bytes, about 16.8 MiB per
 * GPU that loads the library, held until the process exits).
 *
 * Limits and rules
 *  - total_q * heads must not exceed NB_ATTN_BUILTIN_SCRATCH_ROWS and, in varlen mode,
 *    total_k / 128 + batch + 1 must not exceed NB_ATTN_BUILTIN_SCRATCH_ITEMS; larger problems are
 *    refused with NB_ATTN_ERR_TOO_LARGE and nothing is launched. Use nb_attn_bwd with your own
 *    workspace.
 *  - The call performs no cudaMalloc / cudaFree and calls no allocating library routine.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress with
 *    that device current). Make that first call outside any CUDA stream capture.
 *  - All calls on a GPU share the one array. It keeps whatever the previous call left in it; the
 *    kernels clear what has to start at zero themselves. Two calls whose kernels overlap on the
 *    same GPU (different streams) race on it: serialise them.
 * Results are the same as nb_attn_bwd's up to the order of the fp32 dQ additions. */
#define NB_ATTN_BUILTIN_SCRATCH_ROWS 65536
#define NB_ATTN_BUILTIN_SCRATCH_ITEMS 16384
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

/* Bounded-wait self-test (no counterpart in the reference): one CTA waits, with `limit_ns` instead
 * of the kernels' two-second limit, on a barrier that nothing arrives on. The wait gives up, the
 * kernel writes NB_ATTN_STATUS_WAIT_TIMEOUT to *status, frees its tensor memory and returns; this
 * is the path every attention kernel takes if one of its waits runs out. out (device int32[2],
 * optional) receives {first wait gave up, a later wait returned at once}. */
int nb_attn_selftest_wait(uint64_t limit_ns, int32_t* status, int32_t* out, void* stream);

/* The varlen scheduler's work list, exposed for inspection and tests (no counterpart in the
 * reference; its ragged consumer there is src/nanobrain/model.py:254-270).
 *
 * side 0: items are query tiles, cost = key tiles of the sequence (what nb_attn_fwd builds);
 * side 1: items are key tiles, cost = query tiles (what nb_attn_bwd builds).
 * An item is a 32-byte record (below): sequence, tile, and the sequence's offsets and lengths on
 * both sides, so that a CTA learns its work from one read. Unused entries have seq = -1; sequence
 * index `batch` stands for the rows past the last sequence (cost 0). Items are ordered by
 * decreasing cost, all full tiles before all ragged last tiles; the order inside one cost class
 * is unspecified on the device and ascending by sequence in the host version.
 * nb_attn_schedule_capacity: entries a list needs (total / 128 + batch + 1).
 * nb_attn_schedule_build:    build on the device into items (device array of n_items records) on `stream`.
 * nb_attn_schedule_host:     the same rule on host arrays (cu_seqlens on the host); returns
 *                            NB_ATTN_ERR_SHAPE where the device would report BAD_SEQLENS. */
typedef struct nb_attn_sched_item {
  int32_t seq;          /* sequence index; `batch` = the rows past the last sequence; -1 = unused */
  int32_t tile;         /* 128-row tile of the sequence on the item's own side */
  int32_t own_begin;    /* first packed row of the sequence on the own side */
  int32_t own_len;      /* its length there */
  int32_t other_begin;  /* the same on the side the item's inner loop walks */
  int32_t other_len;
  int32_t reserved[2];
} nb_attn_sched_item;

int64_t nb_attn_schedule_capacity(int64_t total_tokens, int32_t batch);
int nb_attn_schedule_build(const nb_attn_shape* shape, int side, nb_attn_sched_item* items, int64_t n_items,
                           int32_t* status, void* stream);
int nb_attn_schedule_host(const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int32_t batch,
                          int32_t max_seqlen_q, int32_t max_seqlen_k, int64_t total_q, int64_t total_k, int side,
                          nb_attn_sched_item* items, int64_t n_items);

#ifdef __cplusplus
}
#endif

#endif /* NB_ATTN_H_ */
