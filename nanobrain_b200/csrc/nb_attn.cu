// Host side of the C ABI declared in include/nb_attn.h: argument validation, TMA tensor-map
// construction and kernel launches. No device memory is allocated here and nothing is kept
// between calls except per-process one-time state (the driver entry point used to encode
// tensor maps and the per-device "large dynamic shared memory" opt-in).
#include "../../include/nb_attn.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <utility>
#include <vector>

#include "bwd_kernel.cuh"
#include "fwd_kernel.cuh"
#include "sched_kernel.cuh"
#include "selftest_kernel.cuh"

// Build-time switch: 0 launches every kernel with plain stream order instead of programmatic
// dependent launch (the kernels' griddepcontrol instructions are then no-ops).
#ifndef NB_ATTN_PDL
#define NB_ATTN_PDL 1
#endif

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;

EncodeTiledFn get_encode() {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
  });
  return g_encode;
}

constexpr int kMaxDevices = 64;
std::mutex g_dev_mutex;
int g_dev_state[kMaxDevices];  // 0 = not set up, 1 = ready, <0 = error code (negated)
int g_dev_sms[kMaxDevices];    // SM count, valid once the device is ready

// Once per device: check the architecture and opt the kernels into their dynamic shared memory.
int ensure_device_ready() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return NB_ATTN_ERR_LAUNCH;
  if (dev < 0 || dev >= kMaxDevices) return NB_ATTN_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (g_dev_state[dev] == 1) return NB_ATTN_OK;
  if (g_dev_state[dev] < 0) return -g_dev_state[dev];
  int major = 0;
  int rc = NB_ATTN_OK;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&g_dev_sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      g_dev_sms[dev] <= 0) {
    rc = NB_ATTN_ERR_LAUNCH;
  } else if (major != 10) {
    rc = NB_ATTN_ERR_DEVICE;
  } else if (cudaFuncSetAttribute(nb::attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  nb::kFwdSmemBytes) != cudaSuccess ||
             cudaFuncSetAttribute(nb::attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  nb::kBwdSmemBytes) != cudaSuccess ||
             cudaFuncSetAttribute(nb::mma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  nb::kSelftestSmemBytes) != cudaSuccess) {
    rc = NB_ATTN_ERR_LAUNCH;
  }
  g_dev_state[dev] = rc == NB_ATTN_OK ? 1 : -rc;
  return rc;
}

// SM count of the current device (after ensure_device_ready succeeded on it).
int device_sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 1;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  return g_dev_sms[dev] > 0 ? g_dev_sms[dev] : 1;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_tensor(const nb_attn_tensor& t, bool dense) {
  if (t.ptr == nullptr) return NB_ATTN_ERR_NULL;
  if (!aligned16(t.ptr)) return NB_ATTN_ERR_ALIGN;
  if (t.stride_token <= 0 || t.stride_head <= 0 || (t.stride_token % 8) != 0 || (t.stride_head % 8) != 0)
    return NB_ATTN_ERR_ALIGN;
  if (dense && (t.stride_batch <= 0 || (t.stride_batch % 8) != 0)) return NB_ATTN_ERR_ALIGN;
  return NB_ATTN_OK;
}

int check_shape(const nb_attn_shape& s) {
  if (s.head_dim != nb::kHeadDim) return NB_ATTN_ERR_HEAD_DIM;
  if (s.batch <= 0 || s.heads <= 0 || s.max_seqlen_q <= 0 || s.max_seqlen_k <= 0) return NB_ATTN_ERR_SHAPE;
  if (s.batch > 65534 || s.heads > 65535) return NB_ATTN_ERR_SHAPE;
  if ((s.cu_seqlens_q == nullptr) != (s.cu_seqlens_k == nullptr)) return NB_ATTN_ERR_SHAPE;
  if (s.total_q <= 0 || s.total_k <= 0) return NB_ATTN_ERR_SHAPE;
  if (s.cu_seqlens_q == nullptr) {
    if (s.total_q != int64_t(s.batch) * s.max_seqlen_q || s.total_k != int64_t(s.batch) * s.max_seqlen_k)
      return NB_ATTN_ERR_SHAPE;
    // The backward kernel counts its work units (key tiles x heads x sequences) in 32 bits.
    if ((int64_t(s.max_seqlen_k) + nb::kTile - 1) / nb::kTile * s.heads * s.batch > INT32_MAX) return NB_ATTN_ERR_SHAPE;
  } else {
    if (s.total_q > INT32_MAX || s.total_k > INT32_MAX) return NB_ATTN_ERR_SHAPE;
    // The grid is items x heads.
    if (nb::sched_capacity(s.total_q, s.batch) * s.heads > INT32_MAX ||
        nb::sched_capacity(s.total_k, s.batch) * s.heads > INT32_MAX)
      return NB_ATTN_ERR_SHAPE;
  }
  if (!(s.scale > 0.f)) return NB_ATTN_ERR_SHAPE;
  return NB_ATTN_OK;
}

// 4-D map over (head_dim, token, head, batch) with a 64 x 128 x 1 x 1 box and 128-byte swizzle.
// Rows outside the token extent read as zeros.
int make_tmap(CUtensorMap* map, const nb_attn_tensor& t, const nb_attn_shape& s, bool is_q) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return NB_ATTN_ERR_TENSOR_MAP;
  const bool dense = s.cu_seqlens_q == nullptr;
  const uint64_t tokens = dense ? uint64_t(is_q ? s.max_seqlen_q : s.max_seqlen_k) : uint64_t(is_q ? s.total_q : s.total_k);
  const uint64_t nbatch = dense ? uint64_t(s.batch) : 1u;
  cuuint64_t dims[4] = {uint64_t(nb::kHeadDim), tokens, uint64_t(s.heads), nbatch};
  const uint64_t batch_stride = dense ? uint64_t(t.stride_batch) : tokens * uint64_t(t.stride_token);
  cuuint64_t strides[3] = {uint64_t(t.stride_token) * 2u, uint64_t(t.stride_head) * 2u, batch_stride * 2u};
  cuuint32_t box[4] = {uint32_t(nb::kHeadDim), uint32_t(nb::kTile), 1u, 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, t.ptr, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? NB_ATTN_OK : NB_ATTN_ERR_TENSOR_MAP;
}

// 3-D fp32 map over the dQ accumulator [token][head][64]: (64, tokens, heads), box 32 x 32 x 1 with
// 128-byte swizzle, used by the backward kernel's TMA add-reductions.
int make_dq_accum_tmap(CUtensorMap* map, float* accum, int64_t total_q, int heads) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return NB_ATTN_ERR_TENSOR_MAP;
  cuuint64_t dims[3] = {uint64_t(nb::kHeadDim), uint64_t(total_q), uint64_t(heads)};
  cuuint64_t strides[2] = {uint64_t(heads) * nb::kHeadDim * sizeof(float), uint64_t(nb::kHeadDim) * sizeof(float)};
  cuuint32_t box[3] = {32u, 32u, 1u};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, accum, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? NB_ATTN_OK : NB_ATTN_ERR_TENSOR_MAP;
}

constexpr float kLog2e = 1.4426950408889634f;

// Launch with programmatic stream serialization: the kernel may become resident while its
// predecessor in the stream drains; it orders itself with griddepcontrol.wait (ptx.cuh).
template <typename... KArgs, typename... Args>
cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = NB_ATTN_PDL ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// side 0: query tiles are the items; side 1: key tiles are.
nb::SchedParams make_sched(const nb_attn_shape& s, int side, nb::SchedItem* items, int64_t n_items, int32_t* status) {
  nb::SchedParams sp;
  const bool fwd = side == 0;
  sp.cu_own = fwd ? s.cu_seqlens_q : s.cu_seqlens_k;
  sp.cu_other = fwd ? s.cu_seqlens_k : s.cu_seqlens_q;
  sp.batch = s.batch;
  sp.max_own = fwd ? s.max_seqlen_q : s.max_seqlen_k;
  sp.max_other = fwd ? s.max_seqlen_k : s.max_seqlen_q;
  sp.total_own = fwd ? s.total_q : s.total_k;
  sp.total_other = fwd ? s.total_k : s.total_q;
  sp.items = items;
  sp.n_items = int32_t(n_items);
  sp.status = status;
  return sp;
}

// Layout of the backward workspace: fp32 dQ accumulator | fp32 delta | work list (varlen only).
size_t bwd_accum_bytes(const nb_attn_shape& s) { return size_t(s.total_q) * size_t(s.heads) * nb::kHeadDim * sizeof(float); }
size_t bwd_delta_bytes(const nb_attn_shape& s) { return size_t(s.total_q) * size_t(s.heads) * sizeof(float); }
size_t bwd_items_offset(const nb_attn_shape& s) { return align_up(bwd_accum_bytes(s) + bwd_delta_bytes(s), 256); }

int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Scratch for nb_attn_bwd_builtin_scratch: one fixed array in the library image per GPU. The name
// below is only a host-side handle; kernels get the device address looked up per device.
constexpr size_t kBuiltinScratchBytes =
    size_t(NB_ATTN_BUILTIN_SCRATCH_ROWS) * (nb::kHeadDim * sizeof(float) + sizeof(float)) + 256 +
    size_t(NB_ATTN_BUILTIN_SCRATCH_ITEMS) * sizeof(nb::SchedItem);
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];
void* g_builtin_scratch_addr[kMaxDevices];  // device address of the array, per device, once looked up

// Once per device, with that device current: resolve the array's device address.
int builtin_scratch_address(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return NB_ATTN_ERR_LAUNCH;
  if (dev < 0 || dev >= kMaxDevices) return NB_ATTN_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (g_builtin_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_builtin_scratch) != cudaSuccess || ptr == nullptr) return NB_ATTN_ERR_LAUNCH;
    g_builtin_scratch_addr[dev] = ptr;
  }
  *out = g_builtin_scratch_addr[dev];
  return NB_ATTN_OK;
}

// Everything about a backward call that can be checked without touching CUDA.
int validate_bwd(const nb_attn_bwd_args* a) {
  if (a == nullptr) return NB_ATTN_ERR_NULL;
  int rc = check_shape(a->shape);
  if (rc) return rc;
  const bool dense = a->shape.cu_seqlens_q == nullptr;
  const nb_attn_tensor* ts[] = {&a->q, &a->k, &a->v, &a->o, &a->d_o, &a->dq, &a->dk, &a->dv};
  for (const nb_attn_tensor* t : ts)
    if ((rc = check_tensor(*t, dense))) return rc;
  if (a->lse == nullptr) return NB_ATTN_ERR_NULL;
  return NB_ATTN_OK;
}

// `a` has passed validate_bwd and the device is ready.
int launch_bwd(const nb_attn_bwd_args* a, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = NB_ATTN_OK;
  const nb_attn_shape& s = a->shape;
  const bool dense = s.cu_seqlens_q == nullptr;
  if (workspace_bytes < nb_attn_bwd_workspace_bytes(&s)) return NB_ATTN_ERR_WORKSPACE;

  CUtensorMap tq, tk, tv, tg, tdq;
  if ((rc = make_tmap(&tq, a->q, s, true)) || (rc = make_tmap(&tk, a->k, s, false)) ||
      (rc = make_tmap(&tv, a->v, s, false)) || (rc = make_tmap(&tg, a->d_o, s, true)) ||
      (rc = make_dq_accum_tmap(&tdq, static_cast<float*>(workspace), s.total_q, s.heads)))
    return rc;

  nb::BwdParams p;
  p.o = static_cast<const __nv_bfloat16*>(a->o.ptr);
  p.d_o = static_cast<const __nv_bfloat16*>(a->d_o.ptr);
  p.o_sb = dense ? a->o.stride_batch : 0;
  p.o_st = a->o.stride_token;
  p.o_sh = a->o.stride_head;
  p.do_sb = dense ? a->d_o.stride_batch : 0;
  p.do_st = a->d_o.stride_token;
  p.do_sh = a->d_o.stride_head;
  p.dq = static_cast<__nv_bfloat16*>(a->dq.ptr);
  p.dk = static_cast<__nv_bfloat16*>(a->dk.ptr);
  p.dv = static_cast<__nv_bfloat16*>(a->dv.ptr);
  p.dq_sb = dense ? a->dq.stride_batch : 0;
  p.dq_st = a->dq.stride_token;
  p.dq_sh = a->dq.stride_head;
  p.dk_sb = dense ? a->dk.stride_batch : 0;
  p.dk_st = a->dk.stride_token;
  p.dk_sh = a->dk.stride_head;
  p.dv_sb = dense ? a->dv.stride_batch : 0;
  p.dv_st = a->dv.stride_token;
  p.dv_sh = a->dv.stride_head;
  p.lse = a->lse;
  p.dq_accum = static_cast<float*>(workspace);
  p.delta = p.dq_accum + size_t(s.total_q) * s.heads * nb::kHeadDim;
  p.cu_q = s.cu_seqlens_q;
  p.cu_k = s.cu_seqlens_k;
  p.batch = s.batch;
  p.heads = s.heads;
  p.lq = s.max_seqlen_q;
  p.lk = s.max_seqlen_k;
  p.total_q = s.total_q;
  p.total_k = s.total_k;
  p.scale = s.scale;
  p.scale_log2 = s.scale * kLog2e;
  p.status = a->status;
  // The main kernel's CTAs are persistent: one per SM, each walking its share of the work units
  // (key tiles x heads x sequences, or work-list entries x heads).
  int64_t n_work = 0;
  p.n_kt = ceil_div(s.max_seqlen_k, nb::kTile);
  if (dense) {
    p.items = nullptr;
    p.sched = nb::SchedParams{};
    n_work = int64_t(p.n_kt) * s.heads * s.batch;
  } else {
    // Block 0 of the prologue builds the list of key tiles; the main kernel runs items x heads CTAs.
    const int64_t n_items = nb::sched_capacity(s.total_k, s.batch);
    nb::SchedItem* items =
        reinterpret_cast<nb::SchedItem*>(static_cast<unsigned char*>(workspace) + bwd_items_offset(s));
    p.items = items;
    p.sched = make_sched(s, 1, items, n_items, a->status);
    n_work = n_items * s.heads;
  }
  p.n_work = int32_t(n_work);
  p.div_heads = nb::make_fast_div(uint32_t(s.heads));
  p.div_n_kt = nb::make_fast_div(uint32_t(p.n_kt));
  const int sms = device_sm_count();
  const dim3 grid(unsigned(n_work < sms ? n_work : sms), 1, 1);

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t rows = s.total_q * s.heads;
  const int64_t want_blocks = (rows * 8 + 255) / 256;
  const int aux_blocks = int(want_blocks < 148 * 16 ? want_blocks : 148 * 16);
  bool ok = launch(nb::attn_bwd_prologue_kernel, dim3(aux_blocks), dim3(256), 0, st, p) == cudaSuccess;
  if (a->event_main_begin) cudaEventRecord(static_cast<cudaEvent_t>(a->event_main_begin), st);
  ok = ok && launch(nb::attn_bwd_kernel, grid, dim3(nb::kBwdThreads), nb::kBwdSmemBytes, st, tq, tk, tv, tg, tdq, p) ==
                 cudaSuccess;
  if (a->event_main_end) cudaEventRecord(static_cast<cudaEvent_t>(a->event_main_end), st);
  ok = ok && launch(nb::attn_bwd_epilogue_kernel, dim3(aux_blocks), dim3(256), 0, st, p) == cudaSuccess;
  if (!ok) {
    cudaGetLastError();  // leave no sticky "last error" behind for the caller's own checks
    return NB_ATTN_ERR_LAUNCH;
  }
  return cudaGetLastError() == cudaSuccess ? NB_ATTN_OK : NB_ATTN_ERR_LAUNCH;
}

}  // namespace

extern "C" {

int nb_attn_abi_version(void) { return NB_ATTN_ABI_VERSION; }

const char* nb_attn_strerror(int code) {
  switch (code) {
    case NB_ATTN_OK: return "ok";
    case NB_ATTN_ERR_NULL: return "a required pointer is NULL";
    case NB_ATTN_ERR_HEAD_DIM: return "head_dim must be 64";
    case NB_ATTN_ERR_SHAPE: return "invalid or inconsistent sizes";
    case NB_ATTN_ERR_ALIGN: return "pointers must be 16-byte aligned and strides positive multiples of 8 elements";
    case NB_ATTN_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case NB_ATTN_ERR_TENSOR_MAP: return "could not encode a TMA tensor map";
    case NB_ATTN_ERR_LAUNCH: return "a CUDA runtime call failed";
    case NB_ATTN_ERR_DEVICE: return "the current device is not an sm_100 GPU";
    case NB_ATTN_ERR_TOO_LARGE:
      return "total_q * heads exceeds NB_ATTN_BUILTIN_SCRATCH_ROWS; use nb_attn_bwd with a caller workspace";
    default: return "unknown error code";
  }
}

size_t nb_attn_bwd_workspace_bytes(const nb_attn_shape* shape) {
  if (shape == nullptr || check_shape(*shape) != NB_ATTN_OK) return 0;
  const nb_attn_shape& s = *shape;
  if (s.cu_seqlens_q == nullptr) return bwd_accum_bytes(s) + bwd_delta_bytes(s);
  return bwd_items_offset(s) + size_t(nb::sched_capacity(s.total_k, s.batch)) * sizeof(nb::SchedItem);
}

size_t nb_attn_fwd_workspace_bytes(const nb_attn_shape* shape) {
  if (shape == nullptr || check_shape(*shape) != NB_ATTN_OK || shape->cu_seqlens_q == nullptr) return 0;
  return size_t(nb::sched_capacity(shape->total_q, shape->batch)) * sizeof(nb::SchedItem);
}

int nb_attn_fwd(const nb_attn_fwd_args* a, void* stream) {
  if (a == nullptr) return NB_ATTN_ERR_NULL;
  int rc = check_shape(a->shape);
  if (rc) return rc;
  const nb_attn_shape& s = a->shape;
  const bool dense = s.cu_seqlens_q == nullptr;
  if ((rc = check_tensor(a->q, dense)) || (rc = check_tensor(a->k, dense)) || (rc = check_tensor(a->v, dense)) ||
      (rc = check_tensor(a->o, dense)))
    return rc;
  if (a->lse == nullptr) return NB_ATTN_ERR_NULL;
  const size_t ws_need = nb_attn_fwd_workspace_bytes(&s);
  if (ws_need > 0 && (a->workspace == nullptr || a->workspace_bytes < ws_need ||
                      (reinterpret_cast<uintptr_t>(a->workspace) & 255u) != 0))
    return NB_ATTN_ERR_WORKSPACE;
  if ((rc = ensure_device_ready())) return rc;

  CUtensorMap tq, tk, tv;
  if ((rc = make_tmap(&tq, a->q, s, true)) || (rc = make_tmap(&tk, a->k, s, false)) ||
      (rc = make_tmap(&tv, a->v, s, false)))
    return rc;

  nb::FwdParams p;
  p.o = static_cast<__nv_bfloat16*>(a->o.ptr);
  p.o_sb = dense ? a->o.stride_batch : 0;
  p.o_st = a->o.stride_token;
  p.o_sh = a->o.stride_head;
  p.lse = a->lse;
  p.cu_q = s.cu_seqlens_q;
  p.cu_k = s.cu_seqlens_k;
  p.batch = s.batch;
  p.heads = s.heads;
  p.lq = s.max_seqlen_q;
  p.lk = s.max_seqlen_k;
  p.total_q = s.total_q;
  p.total_k = s.total_k;
  p.scale_log2 = s.scale * kLog2e;
  p.status = a->status;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(ceil_div(s.max_seqlen_q, nb::kFwdQRows), s.heads, s.batch);
  bool ok = true;
  p.items = nullptr;
  if (!dense) {
    // The scheduler's list of query tiles, then one CTA per item and head.
    const int64_t n_items = nb::sched_capacity(s.total_q, s.batch);
    nb::SchedItem* items = static_cast<nb::SchedItem*>(a->workspace);
    const nb::SchedParams sp = make_sched(s, 0, items, n_items, a->status);
    ok = launch(nb::attn_sched_kernel, dim3(1), dim3(nb::kSchedThreads), 0, st, sp) == cudaSuccess;
    p.items = items;
    grid = dim3(unsigned(n_items * s.heads), 1, 1);
  }
  ok = ok && launch(nb::attn_fwd_kernel, grid, dim3(nb::kFwdThreads), nb::kFwdSmemBytes, st, tq, tk, tv, p) == cudaSuccess;
  if (!ok) {
    cudaGetLastError();
    return NB_ATTN_ERR_LAUNCH;
  }
  return cudaGetLastError() == cudaSuccess ? NB_ATTN_OK : NB_ATTN_ERR_LAUNCH;
}

int nb_attn_bwd(const nb_attn_bwd_args* a, void* stream) {
  int rc = validate_bwd(a);
  if (rc) return rc;
  if (a->workspace == nullptr || a->workspace_bytes < nb_attn_bwd_workspace_bytes(&a->shape) ||
      (reinterpret_cast<uintptr_t>(a->workspace) & 255u) != 0)
    return NB_ATTN_ERR_WORKSPACE;
  if ((rc = ensure_device_ready())) return rc;
  return launch_bwd(a, a->workspace, a->workspace_bytes, stream);
}

int nb_attn_bwd_builtin_scratch(const nb_attn_bwd_args* a, void* stream) {
  // Same argument checks, in the same order, as nb_attn_bwd; CUDA is touched only after them.
  int rc = validate_bwd(a);
  if (rc) return rc;
  const nb_attn_shape& s = a->shape;
  if (s.total_q * int64_t(s.heads) > int64_t(NB_ATTN_BUILTIN_SCRATCH_ROWS)) return NB_ATTN_ERR_TOO_LARGE;
  if (s.cu_seqlens_q != nullptr && nb::sched_capacity(s.total_k, s.batch) > int64_t(NB_ATTN_BUILTIN_SCRATCH_ITEMS))
    return NB_ATTN_ERR_TOO_LARGE;
  if ((rc = ensure_device_ready())) return rc;
  void* scratch = nullptr;
  if ((rc = builtin_scratch_address(&scratch))) {
    cudaGetLastError();
    return rc;
  }
  return launch_bwd(a, scratch, kBuiltinScratchBytes, stream);
}

int nb_attn_selftest_mma(int mode, const void* a, const void* b, float* d, int32_t* status, void* stream) {
  if (a == nullptr || b == nullptr || d == nullptr) return NB_ATTN_ERR_NULL;
  if (mode < 0 || mode > 3) return NB_ATTN_ERR_SHAPE;
  if (!aligned16(a) || !aligned16(b)) return NB_ATTN_ERR_ALIGN;
  int rc = ensure_device_ready();
  if (rc) return rc;
  nb::mma_selftest_kernel<<<1, 128, nb::kSelftestSmemBytes, static_cast<cudaStream_t>(stream)>>>(
      mode, static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), d, status);
  return cudaGetLastError() == cudaSuccess ? NB_ATTN_OK : NB_ATTN_ERR_LAUNCH;
}

int nb_attn_selftest_wait(uint64_t limit_ns, int32_t* status, int32_t* out, void* stream) {
  if (status == nullptr) return NB_ATTN_ERR_NULL;
  if (limit_ns == 0 || limit_ns > 1000000000ull) return NB_ATTN_ERR_SHAPE;  // at most one second
  int rc = ensure_device_ready();
  if (rc) return rc;
  nb::wait_selftest_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns, status, out);
  return cudaGetLastError() == cudaSuccess ? NB_ATTN_OK : NB_ATTN_ERR_LAUNCH;
}

int64_t nb_attn_schedule_capacity(int64_t total_tokens, int32_t batch) {
  if (total_tokens < 0 || batch <= 0) return 0;
  return nb::sched_capacity(total_tokens, batch);
}

int nb_attn_schedule_build(const nb_attn_shape* shape, int side, nb_attn_sched_item* items, int64_t n_items,
                           int32_t* status, void* stream) {
  if (shape == nullptr || items == nullptr) return NB_ATTN_ERR_NULL;
  int rc = check_shape(*shape);
  if (rc) return rc;
  if (shape->cu_seqlens_q == nullptr || (side != 0 && side != 1)) return NB_ATTN_ERR_SHAPE;
  if (n_items < nb::sched_capacity(side == 0 ? shape->total_q : shape->total_k, shape->batch) || n_items > INT32_MAX)
    return NB_ATTN_ERR_WORKSPACE;
  if ((rc = ensure_device_ready())) return rc;
  const nb::SchedParams sp = make_sched(*shape, side, reinterpret_cast<nb::SchedItem*>(items), n_items, status);
  if (launch(nb::attn_sched_kernel, dim3(1), dim3(nb::kSchedThreads), 0, static_cast<cudaStream_t>(stream), sp) !=
      cudaSuccess) {
    cudaGetLastError();
    return NB_ATTN_ERR_LAUNCH;
  }
  return NB_ATTN_OK;
}

int nb_attn_schedule_host(const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int32_t batch,
                          int32_t max_seqlen_q, int32_t max_seqlen_k, int64_t total_q, int64_t total_k, int side,
                          nb_attn_sched_item* items_out, int64_t n_items) {
  if (cu_seqlens_q == nullptr || cu_seqlens_k == nullptr || items_out == nullptr) return NB_ATTN_ERR_NULL;
  nb::SchedItem* items = reinterpret_cast<nb::SchedItem*>(items_out);
  if (batch <= 0 || batch > 65534 || (side != 0 && side != 1) || n_items > INT32_MAX) return NB_ATTN_ERR_SHAPE;
  nb_attn_shape s = {};
  s.batch = batch;
  s.max_seqlen_q = max_seqlen_q;
  s.max_seqlen_k = max_seqlen_k;
  s.total_q = total_q;
  s.total_k = total_k;
  s.cu_seqlens_q = cu_seqlens_q;
  s.cu_seqlens_k = cu_seqlens_k;
  const nb::SchedParams sp = make_sched(s, side, items, n_items, nullptr);
  if (n_items < nb::sched_capacity(sp.total_own, batch)) return NB_ATTN_ERR_WORKSPACE;
  // Same classification as the device kernel; buckets in order, sequences ascending inside one.
  std::vector<std::vector<int>> by_bucket(nb::kSchedBuckets);
  for (int i = 0; i <= batch; ++i) {  // i == batch: the rows past the last sequence
    const nb::SchedSeq q = nb::sched_classify(sp, i);
    if (!q.ok) return NB_ATTN_ERR_SHAPE;
    by_bucket[q.bucket].push_back(i);
  }
  int64_t at = 0;
  for (const auto& seqs : by_bucket)
    for (int i : seqs) {
      const nb::SchedSeq q = nb::sched_classify(sp, i);
      for (int t = 0; t < q.full; ++t) items[at++] = nb::sched_item(q, i, t);
    }
  for (const auto& seqs : by_bucket)
    for (int i : seqs) {
      const nb::SchedSeq q = nb::sched_classify(sp, i);
      if (q.ragged) items[at++] = nb::sched_item(q, i, q.full);
    }
  for (; at < n_items; ++at) items[at] = nb::sched_no_item();
  return NB_ATTN_OK;
}

}  // extern "C"
