// Host side of the C ABI declared in include/nb_attn.h: argument validation, TMA tensor-map
// construction and kernel launches. No device memory is allocated here and nothing is kept
// between calls except per-process one-time state (the driver entry point used to encode
// tensor maps and the per-device "large dynamic shared memory" opt-in).
#include "../../include/nb_attn.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "bwd_kernel.cuh"
#include "fwd_kernel.cuh"
#include "selftest_kernel.cuh"

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
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
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
  if (s.batch > 65535 || s.heads > 65535) return NB_ATTN_ERR_SHAPE;
  if ((s.cu_seqlens_q == nullptr) != (s.cu_seqlens_k == nullptr)) return NB_ATTN_ERR_SHAPE;
  if (s.total_q <= 0 || s.total_k <= 0) return NB_ATTN_ERR_SHAPE;
  if (s.cu_seqlens_q == nullptr) {
    if (s.total_q != int64_t(s.batch) * s.max_seqlen_q || s.total_k != int64_t(s.batch) * s.max_seqlen_k)
      return NB_ATTN_ERR_SHAPE;
  } else {
    if (s.total_q > INT32_MAX || s.total_k > INT32_MAX) return NB_ATTN_ERR_SHAPE;
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

int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Scratch for nb_attn_bwd_builtin_scratch: one fixed array in the library image per GPU. The name
// below is only a host-side handle; kernels get the device address looked up per device.
constexpr size_t kBuiltinScratchBytes = size_t(NB_ATTN_BUILTIN_SCRATCH_ROWS) * (nb::kHeadDim * sizeof(float) + sizeof(float));
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

int launch_bwd(const nb_attn_bwd_args* a, void* workspace, size_t workspace_bytes, void* stream) {
  if (a == nullptr) return NB_ATTN_ERR_NULL;
  int rc = check_shape(a->shape);
  if (rc) return rc;
  const nb_attn_shape& s = a->shape;
  const bool dense = s.cu_seqlens_q == nullptr;
  const nb_attn_tensor* ts[] = {&a->q, &a->k, &a->v, &a->o, &a->d_o, &a->dq, &a->dk, &a->dv};
  for (const nb_attn_tensor* t : ts)
    if ((rc = check_tensor(*t, dense))) return rc;
  if (a->lse == nullptr) return NB_ATTN_ERR_NULL;
  const size_t need = nb_attn_bwd_workspace_bytes(s.total_q, s.heads, s.head_dim);
  if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return NB_ATTN_ERR_WORKSPACE;
  if ((rc = ensure_device_ready())) return rc;

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
  p.scale = s.scale;
  p.scale_log2 = s.scale * kLog2e;
  p.status = a->status;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t rows = s.total_q * s.heads;
  const int64_t want_blocks = (rows * 8 + 255) / 256;
  const int aux_blocks = int(want_blocks < 148 * 16 ? want_blocks : 148 * 16);
  nb::attn_bwd_prologue_kernel<<<aux_blocks, 256, 0, st>>>(p);
  if (a->event_main_begin) cudaEventRecord(static_cast<cudaEvent_t>(a->event_main_begin), st);
  const dim3 grid(ceil_div(s.max_seqlen_k, nb::kTile), s.heads, s.batch);
  nb::attn_bwd_kernel<<<grid, nb::kBwdThreads, nb::kBwdSmemBytes, st>>>(tq, tk, tv, tg, tdq, p);
  if (a->event_main_end) cudaEventRecord(static_cast<cudaEvent_t>(a->event_main_end), st);
  nb::attn_bwd_epilogue_kernel<<<aux_blocks, 256, 0, st>>>(p);
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

size_t nb_attn_bwd_workspace_bytes(int64_t total_q, int32_t heads, int32_t head_dim) {
  if (total_q <= 0 || heads <= 0 || head_dim <= 0) return 0;
  const size_t rows = size_t(total_q) * size_t(heads);
  return rows * size_t(head_dim) * sizeof(float) + rows * sizeof(float);
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
  p.scale_log2 = s.scale * kLog2e;
  p.status = a->status;

  const dim3 grid(ceil_div(s.max_seqlen_q, nb::kFwdQRows), s.heads, s.batch);
  nb::attn_fwd_kernel<<<grid, nb::kFwdThreads, nb::kFwdSmemBytes, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? NB_ATTN_OK : NB_ATTN_ERR_LAUNCH;
}

int nb_attn_bwd(const nb_attn_bwd_args* a, void* stream) {
  if (a == nullptr) return NB_ATTN_ERR_NULL;
  return launch_bwd(a, a->workspace, a->workspace_bytes, stream);
}

int nb_attn_bwd_builtin_scratch(const nb_attn_bwd_args* a, void* stream) {
  if (a == nullptr) return NB_ATTN_ERR_NULL;
  int rc = check_shape(a->shape);
  if (rc) return rc;
  if (a->shape.total_q * int64_t(a->shape.heads) > int64_t(NB_ATTN_BUILTIN_SCRATCH_ROWS)) return NB_ATTN_ERR_TOO_LARGE;
  void* scratch = nullptr;
  if ((rc = builtin_scratch_address(&scratch))) return rc;
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

}  // extern "C"
