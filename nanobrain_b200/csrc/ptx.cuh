// Thin inline-PTX wrappers for the sm_100a features the attention kernels use:
// mbarriers, TMA tiled loads (cp.async.bulk.tensor, one CTA per load), tensor memory
// (tcgen05.alloc / ld / st) and the 5th-generation tensor-core MMA (tcgen05.mma).
//
// Every wait in this file is bounded: after roughly two seconds without progress a
// waiter raises a CTA-wide abort flag in shared memory, records a code in the caller's
// status word in global memory and returns; later waits see the flag and return at once,
// so a kernel always runs to its end and frees its tensor memory.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nb {

// ----------------------------------------------------------------------------------------
// Addresses and fences
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// Programmatic dependent launch: a kernel launched with the programmatic-stream-serialization
// attribute may start while its predecessor in the stream is still running. pdl_wait() blocks until
// the predecessor has completed and its writes are visible; pdl_launch_dependents() lets the
// successor's CTAs be scheduled as soon as every CTA of this grid has called it or exited. Each
// kernel here calls pdl_launch_dependents() only after its own pdl_wait(), so when a CTA of kernel N
// runs, everything before kernel N-1 in the stream is complete: before its wait a kernel may read
// whatever kernel N-1 does not write.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ----------------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Status codes written to the caller's status word: a bounded wait gave up, or the work-list
// builder found cu_seqlens that are not a valid packing (see sched_kernel.cuh).
enum : int { kStatusOk = 0, kStatusWaitTimeout = 1, kStatusBadSeqlens = 2 };

constexpr uint64_t kWaitLimitNs = 2000000000ull;  // about two seconds

// Bounded wait. `abort_flag` lives in shared memory and is shared by the whole CTA. The attention
// kernels use the default limit (a compile-time constant); the wait self-test passes its own
// (at most 4 s: the clock is the low word of the nanosecond timer).
// The loop is kept as small as it can be -- 32-bit timer arithmetic, the flag and the status word
// touched with plain state-space stores: the warp-specialised kernels have dozens of wait sites,
// every one of them inlined, and their hot code has to fit the SM's instruction cache (with a
// larger loop the backward kernel's instruction-cache hit rate was 92 % at best and instruction
// fetch was its top stall).
__device__ __forceinline__ uint32_t globaltimer_lo() {
  uint32_t t;
  asm volatile("mov.u32 %0, %%globaltimer_lo;" : "=r"(t));
  return t;
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status_word, uint64_t limit_ns = kWaitLimitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint32_t flag_addr = smem_u32(const_cast<int*>(abort_flag));
  const uint32_t limit = uint32_t(limit_ns);
  const uint32_t t0 = globaltimer_lo();
#pragma unroll 1
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    uint32_t flag;
    asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(flag) : "r"(flag_addr) : "memory");
    if (flag) return false;
    if (globaltimer_lo() - t0 > limit) break;
  }
  asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(flag_addr), "r"(1) : "memory");
  if (status_word)
    asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(status_word), "r"((int)kStatusWaitTimeout) : "memory");
  return false;
}

// ----------------------------------------------------------------------------------------
// TMA: tiled 4-D load global -> shared, completion on an mbarrier (CTA-local).
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t smem_dst, const CUtensorMap* tmap, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4, %5}], [%6];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
        "r"(bar)
      : "memory");
}

// Tiled 3-D add-reduction shared -> global (fp32 tensor map): global[box] += shared[box]. The
// operation joins the thread's current bulk async-group.
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* tmap, uint32_t smem_src, int c0, int c1,
                                                  int c2) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
      :
      : "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(smem_src)
      : "memory");
}
// L2 eviction-priority policies. They are hints attached to single accesses (no cache state is
// configured): the fp32 dQ accumulator is cleared, added into and read back within one backward
// call and fits the L2, so its lines are marked "evict last" while the call runs and "evict first"
// on their final read.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void st_global_v4_hint(void* ptr, float4 v, uint64_t pol) {
  asm volatile("st.global.L2::cache_hint.v4.f32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(ptr), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w), "l"(pol)
               : "memory");
}
__device__ __forceinline__ float4 ld_global_v4_hint(const void* ptr, uint64_t pol) {
  float4 v;
  asm volatile("ld.global.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(ptr), "l"(pol)
               : "memory");
  return v;
}
// The add-reduction above with an L2 policy.
__device__ __forceinline__ void tma_reduce_add_3d_hint(const CUtensorMap* tmap, uint32_t smem_src, int c0, int c1,
                                                       int c2, uint64_t pol) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group.L2::cache_hint [%0, {%1, %2, %3}], "
      "[%4], %5;"
      :
      : "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(smem_src), "l"(pol)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until the shared-memory sources of all committed bulk groups have been read.
__device__ __forceinline__ void bulk_wait_group_read0() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// Waits until all committed bulk groups have completed.
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ----------------------------------------------------------------------------------------
// Tensor memory
// ----------------------------------------------------------------------------------------
// One full warp allocates `ncols` (power of two, >= 32) columns; the base address lands in
// shared memory at `smem_result`.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has finished.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// 32 lanes x 32 bit, repeated 32 times along columns: thread t of the warp receives columns
// [col, col+32) of lane (lane_base + t). taddr = (lane << 16) | column.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
        "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
      : "memory");
}

// 16 lanes x 256 bit, repeated 4 times along columns (32 columns): thread t of the warp receives,
// for column block i (8 columns each), r[4i+0..1] = row (lane_base + t/4), columns 8i + 2(t%4) + {0,1}
// and r[4i+2..3] = row (lane_base + 8 + t/4), same columns. Four neighbouring threads thus hold
// 32 contiguous bytes of one row, which makes a warp-wide vector store or reduction hit whole
// 32-byte sectors.
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Fire-and-forget fp32 vector reduction into global memory (two adjacent floats).
__device__ __forceinline__ void red_add_v2(float* addr, float a, float b) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(addr), "f"(a), "f"(b) : "memory");
}

// Register re-partitioning between warpgroups (all four warps of an aligned warpgroup execute it).
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}

// Waits for two barriers with the two polls in flight together (their latencies overlap).
__device__ __forceinline__ void mbar_wait2(uint32_t bar_a, uint32_t par_a, uint32_t bar_b, uint32_t par_b,
                                           volatile int* abort_flag, int* status_word) {
  const bool a = mbar_try_wait(bar_a, par_a);
  const bool b = mbar_try_wait(bar_b, par_b);
  if (!a) mbar_wait(bar_a, par_a, abort_flag, status_word);
  if (!b) mbar_wait(bar_b, par_b, abort_flag, status_word);
}

// ----------------------------------------------------------------------------------------
// tcgen05.mma descriptors (bf16 inputs, fp32 accumulate, cta_group::1)
// ----------------------------------------------------------------------------------------
// Instruction descriptor, kind::f16: D=f32 (bits 4-5 = 1), A=B=bf16 (bits 7-9, 10-12 = 1),
// bit 15/16 = A/B major (0 = K-major, 1 = MN-major), bits 17-22 = N/8, bits 24-28 = M/16.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(a_mn_major) << 15) |
         (uint32_t(b_mn_major) << 16) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}
// The same descriptor with another N (a multiple of 16 for M = 128), for MMAs over a ragged tile.
__host__ __device__ constexpr uint32_t idesc_with_n(uint32_t idesc, int n) {
  return (idesc & ~(0x3Fu << 17)) | (uint32_t(n >> 3) << 17);
}

// Shared-memory matrix descriptor for the 128-byte-swizzled layouts used here. Every operand
// tile is stored as rows of 128 bytes (64 bf16) at a 128-byte pitch, 16-byte chunks XOR-ed with
// (row & 7) (what TMA's SWIZZLE_128B writes), in blocks whose base is 1024-byte aligned.
//   bits 0-13  start address >> 4      bits 16-29 leading byte offset >> 4
//   bits 32-45 stride byte offset >> 4 bits 46-47 version (1 on sm_100)
//   bits 61-63 layout (2 = SWIZZLE_128B)
// K-major operand (rows = M or N index, the 64 elements of a row run along K): stride offset =
// 1024 (eight rows); the leading offset is unused. One MMA consumes 16 K elements = 32 bytes of
// each row, so the next K step adds 32 bytes to the start address.
// MN-major operand (rows = K index, the 64 elements of a row run along M or N): stride offset =
// 1024 (eight K rows), leading offset = distance between 64-element blocks along M/N. One MMA
// consumes 16 K rows, so the next K step adds 2048 bytes.
__device__ __forceinline__ uint64_t make_sdesc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3FFFF) >> 4);
  d |= uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ----------------------------------------------------------------------------------------
// Small math helpers
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed pairs of fp32 (one issue slot for two lanes of work on sm_100).
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// Three-input maximum (one instruction on sm_100).
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// exp2 of a packed pair on the FMA and integer pipes instead of the MUFU unit (16 results per clock
// per SM), for arguments <= ~100: clamp at -126, split x = n + f with n = round(x) by adding
// 1.5*2^23, evaluate a degree-3 minimax polynomial for 2^f on [-0.5, 0.5] (relative error 7.5e-5,
// far below the bf16 rounding the result receives), and add n to the exponent field.
__device__ __forceinline__ uint64_t exp2_poly_f32x2(uint64_t x2) {
  float x0, x1;
  unpack_f32x2(x2, x0, x1);
  const uint64_t xc = pack_f32x2(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
  const uint64_t t = add_f32x2(xc, pack_f32x2(12582912.f, 12582912.f));
  const uint64_t n = add_f32x2(t, pack_f32x2(-12582912.f, -12582912.f));
  const uint64_t f = fma_f32x2(n, pack_f32x2(-1.f, -1.f), xc);
  uint64_t p = fma_f32x2(f, pack_f32x2(0.05517164617776871f, 0.05517164617776871f),
                         pack_f32x2(0.2426111251115799f, 0.2426111251115799f));
  p = fma_f32x2(p, f, pack_f32x2(0.6932609677314758f, 0.6932609677314758f));
  p = fma_f32x2(p, f, pack_f32x2(0.9999280571937561f, 0.9999280571937561f));
  const uint32_t r0 = uint32_t(p) + (uint32_t(t) << 23);
  const uint32_t r1 = uint32_t(p >> 32) + (uint32_t(t >> 32) << 23);
  return (uint64_t(r1) << 32) | r0;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Byte offset of the 16-byte chunk `chunk` (0..7) of row `row` inside a 128-byte-swizzled
// block with 128-byte rows.
__device__ __forceinline__ uint32_t swz128(uint32_t row, uint32_t chunk) {
  return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

}  // namespace nb
