// Single-tile self-test of the four tcgen05.mma operand forms the attention kernels rely on.
// It fills shared memory with plain stores in the 128-byte-swizzled layout (so it checks the
// matrix descriptors independently of TMA), runs one MMA chain and dumps the fp32 accumulator.
//
//   mode 0: D[128x128] = A[:, 0:64] * B[:, 0:64]^T   A, B K-major from shared memory      (S, dP)
//   mode 1: D[128x64]  = A * B[:, 0:64]              A (bf16) from tensor memory, B MN-major (PV, dV)
//   mode 2: D[128x64]  = A * B[:, 0:64]              A K-major from shared memory (two 64-column
//                                                    halves), B MN-major                    (dK)
//   mode 3: D[128x64]  = A^T * B[:, 0:64]            A MN-major (same bytes as mode 2), B MN-major (dQ)
// A and B are row-major [128][128] bf16 in global memory; D is row-major fp32 [128][128] or [128][64].
#pragma once

#include "fwd_kernel.cuh"
#include "ptx.cuh"

namespace nb {

constexpr int kSelftestSmemBytes = 4 * kTileBytes + 1024;

__global__ void __launch_bounds__(128)
mma_selftest_kernel(int mode, const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ B,
                    float* __restrict__ D, int32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  uint8_t* smem_al = smem_raw + (((smem_u32(smem_raw) + 1023u) & ~1023u) - smem_u32(smem_raw));
  const uint32_t sA = smem_u32(smem_al);             // two 16 KB halves: columns 0..63 | 64..127
  const uint32_t sB = sA + 2 * kTileBytes;           // two halves likewise
  if (tid == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_base_slot), 256);
    tmem_relinquish();
  }
  // Row `tid` of A and B into the swizzled blocks.
  for (int half = 0; half < 2; ++half) {
    for (int ch = 0; ch < 8; ++ch) {
      const uint4 va = *reinterpret_cast<const uint4*>(A + tid * 128 + half * 64 + ch * 8);
      const uint4 vb = *reinterpret_cast<const uint4*>(B + tid * 128 + half * 64 + ch * 8);
      *reinterpret_cast<uint4*>(smem_al + half * kTileBytes + swz128(tid, ch)) = va;
      *reinterpret_cast<uint4*>(smem_al + (2 + half) * kTileBytes + swz128(tid, ch)) = vb;
    }
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t lane_off = uint32_t(warp * 32) << 16;
  const uint32_t tm_d = tmem_base, tm_a = tmem_base + 128;

  if (mode == 1) {
    // A row `tid` (bf16 pairs) into tensor memory columns [128, 192).
    for (int c = 0; c < 4; ++c) {
      uint32_t pk[16];
      const uint32_t* src = reinterpret_cast<const uint32_t*>(A + tid * 128 + c * 32);
      for (int i = 0; i < 16; ++i) pk[i] = src[i];
      tmem_st16(tm_a + lane_off + c * 16, pk);
    }
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();

  if (tid == 0) {
    tc_fence_after();
    if (mode == 0) {
      const uint64_t ad = make_sdesc(sA, 16, 1024), bd = make_sdesc(sB, 16, 1024);
      for (int k = 0; k < 4; ++k) mma_ss(tm_d, ad + 2 * k, bd + 2 * k, make_idesc(128, 128, 0, 0), k > 0);
    } else if (mode == 1) {
      const uint64_t bd = make_sdesc(sB, 1024, 1024);
      for (int k = 0; k < 8; ++k) mma_ts(tm_d, tm_a + 8 * k, bd + 128 * k, make_idesc(128, 64, 0, 1), k > 0);
    } else if (mode == 2) {
      const uint64_t bd = make_sdesc(sB, 1024, 1024);
      for (int k = 0; k < 8; ++k) {
        const uint64_t ad = make_sdesc(sA + (k >> 2) * kTileBytes, 16, 1024) + 2 * (k & 3);
        mma_ss(tm_d, ad, bd + 128 * k, make_idesc(128, 64, 0, 1), k > 0);
      }
    } else {
      const uint64_t ad = make_sdesc(sA, kTileBytes, 1024), bd = make_sdesc(sB, 1024, 1024);
      for (int k = 0; k < 8; ++k) mma_ss(tm_d, ad + 128 * k, bd + 128 * k, make_idesc(128, 64, 1, 1), k > 0);
    }
    tc_commit(smem_u32(&bar));
  }
  __syncwarp();
  mbar_wait(smem_u32(&bar), 0, &abort_flag, status);
  tc_fence_after();
  const int ncols = mode == 0 ? 128 : 64;
  for (int c = 0; c < ncols / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(tm_d + lane_off + c * 32, r);
    tmem_wait_ld();
    for (int i = 0; i < 32; ++i) D[tid * ncols + c * 32 + i] = __uint_as_float(r[i]);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// Self-test of the bounded wait: one CTA allocates tensor memory, then all its warps wait on an
// mbarrier that nothing will ever arrive on, with the caller's limit instead of the kernels' two
// seconds. The wait gives up, the status word receives kStatusWaitTimeout, the tensor memory is
// freed and the kernel returns -- what every attention kernel does if one of its waits runs out.
// out[0] = 1 if the first wait returned "gave up", out[1] = 1 if a later wait returned at once
// because of the CTA-wide abort flag.
__global__ void __launch_bounds__(128) wait_selftest_kernel(uint64_t limit_ns, int32_t* status, int32_t* out) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_base_slot), 512);  // everything: a leak would block the next kernel
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const bool first = mbar_wait(smem_u32(&bar), 0, &abort_flag, status, limit_ns);
  __syncthreads();
  const uint64_t t0 = globaltimer_ns();
  const bool second = mbar_wait(smem_u32(&bar), 0, &abort_flag, status, limit_ns);
  const uint64_t waited = globaltimer_ns() - t0;
  if (tid == 0 && out != nullptr) {
    out[0] = first ? 0 : 1;
    out[1] = (!second && waited < limit_ns) ? 1 : 0;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base_slot, 512);
  }
}

}  // namespace nb
