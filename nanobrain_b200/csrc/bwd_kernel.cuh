// Backward attention kernels (head_dim 64, bf16 tensors, fp32 accumulation):
//
//   attn_bwd_prologue_kernel : delta[row] = sum_d dO[row,d] * O[row,d] (warp-shuffle row dot) and
//                              clears the fp32 dQ accumulator. HBM-bound.
//   attn_bwd_kernel          : a work unit is one 128-row K/V tile of one (sequence, head), walked
//                              over the sequence's queries in 128-row steps. Everything is computed
//                              transposed so that a thread owns a key row (tensor-memory lane):
//                                S^T  = K Q^T                       (tcgen05, smem x smem)
//                                dP^T = V dO^T                      (tcgen05, smem x smem)
//                                P^T  = exp2(S^T*scale_log2 - lse)  (recomputed from the saved LSE)
//                                dS^T = P^T o (dP^T - delta)
//                                dV  += P^T dO                      (A = P^T from tensor memory)
//                                dK  += dS^T Q                      (A = dS^T from shared memory)
//                                dQ   = dS K                        (same dS bytes read MN-major)
//                              dQ tiles are added into the fp32 accumulator with TMA add-reductions
//                              because every K/V tile of a sequence contributes to every dQ row.
//                              CTAs are persistent (one per SM): each walks its share of the work
//                              units and the step pipeline runs on through the boundary between
//                              two units -- K is double-buffered, V is reloaded as soon as the
//                              unit's last dP^T MMA has read it, dV / dK leave through the drain
//                              warps while the next unit's first steps run -- so a unit's start-up
//                              and tail (a third of a CTA's life on ~800-token sequences) overlap
//                              its neighbours' steps.
//                              Warp roles (640 threads): warps 0-7 are two compute warpgroups that
//                              split the 128 query columns of a step (64 each); warps 8-11 are
//                              four MMA issuers (S^T/dP^T, dV, dK, dQ: one elected thread each --
//                              a single thread can issue a tcgen05.mma only every ~55 cycles, so
//                              the 32 MMAs of a step need several issuers to keep the tensor pipe
//                              fed); warps 12-15 drain the dQ tiles (one tensor-memory lane
//                              quadrant each) into the accumulator and, at the end of a unit, dV
//                              and dK into their tensors; warp 16 drives TMA; warp 17 stages the
//                              steps' LSE/delta rows and control words (warps 18-19 only complete
//                              its warpgroup for the register re-partitioning). The loaders and
//                              the drain warps read the work list; the compute warps and the
//                              issuers learn about a step from its control word alone.
//                              Code size is a first-order concern here: five roles' loops run at
//                              the same time and have to share the SM's instruction cache (at
//                              67 KB of code its hit rate was 68 % and instruction fetch was the
//                              top stall; at 48 KB it is above 93 %). Hence the compact wait loop,
//                              rolled MMA-issue loops, divisions by multiply-high, and the compute
//                              role as a function that is not inlined.
//   attn_bwd_epilogue_kernel : dQ = bf16(scale * accumulator). HBM-bound.
//
// Packed mode: block 0 of the prologue also builds the scheduler's work list of key tiles
// (sched_kernel.cuh); the main kernel's work units are list entries x heads (the heads of one entry
// adjacent), dealt to the CTAs in the list's order of decreasing cost.
// A ragged tile is computed at full width and masked: rows of the NEXT packed sequence that it
// brings into shared memory are
// multiplied by exact zeros of P^T / dS^T. For finite data that is exact; if the next sequence's
// first rows hold Inf or NaN, 0 x Inf makes this sequence's gradients NaN as well (the forward
// kernel clears such rows and keeps sequences isolated; measured here, clearing them in this
// kernel cost 7 % of its time, and cutting the MMAs of ragged tiles to their live rows gained
// nothing, so neither is done).
#pragma once

#include "fwd_kernel.cuh"
#include "ptx.cuh"

namespace nb {

// Division of a number below 2^31 by a fixed divisor as a multiply-high and a shift (the divisor's
// magic numbers come from the host). The work-index split is inlined in four warp roles, and an
// integer division routine in each of them is code the instruction cache has no room for.
struct FastDiv {
  uint32_t mul, shr, div;
  __device__ __forceinline__ uint32_t quot(uint32_t n) const { return div == 1u ? n : __umulhi(n, mul) >> shr; }
};
inline FastDiv make_fast_div(uint32_t d) {
  FastDiv f;
  f.div = d, f.mul = 0, f.shr = 0;
  if (d > 1) {
    uint32_t lg = 0;
    while ((1ull << lg) < d) ++lg;  // ceil(log2 d)
    const uint64_t p = 31 + lg;
    f.mul = uint32_t(((1ull << p) + d - 1) / d);
    f.shr = uint32_t(p - 32);
  }
  return f;
}

#ifndef NB_BWD_L2_HINTS
#define NB_BWD_L2_HINTS 1
#endif

struct BwdParams {
  const __nv_bfloat16 *o, *d_o;
  int64_t o_sb, o_st, o_sh, do_sb, do_st, do_sh;
  __nv_bfloat16 *dq, *dk, *dv;
  int64_t dq_sb, dq_st, dq_sh, dk_sb, dk_st, dk_sh, dv_sb, dv_st, dv_sh;
  const float* lse;
  float* delta;     // same indexing as lse
  float* dq_accum;  // fp32 [total_q][heads][64]
  const int32_t* cu_q;
  const int32_t* cu_k;
  const SchedItem* items;  // packed mode: work list of key tiles; CTA x runs entry x / heads for head x % heads
  SchedParams sched;      // packed mode: what block 0 of the prologue builds (items == NULL: nothing)
  int32_t batch, heads;
  int32_t lq, lk;
  int32_t n_work;  // work units of the main kernel: key tiles x heads x sequences, or list entries x heads
  int32_t n_kt;    // dense mode: key tiles per (sequence, head)
  FastDiv div_heads, div_n_kt;  // the main kernel splits a work index without a division routine
  int64_t total_q, total_k;
  float scale, scale_log2;
  int32_t* status;
};

// ----------------------------------------------------------------------------------------
// Prologue: one quarter-warp (8 lanes x 16 bytes) per (token, head) row.
// ----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) attn_bwd_prologue_kernel(const BwdParams p) {
  __shared__ SchedShared sched_sm;
  pdl_wait();  // O comes from the forward kernel, dO from whatever ran before this call
  pdl_launch_dependents();
  if (blockIdx.x == 0 && p.sched.items != nullptr) sched_build<256>(p.sched, sched_sm);
  const int64_t n_rows = p.total_q * p.heads;
  const int lane8 = threadIdx.x & 7;
  int64_t row = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 3;
  const int64_t row_step = (int64_t(gridDim.x) * blockDim.x) >> 3;
#if NB_BWD_L2_HINTS
  const uint64_t keep = l2_policy_evict_last();
#endif
  for (; row < n_rows; row += row_step) {
    const int64_t t = row / p.heads;
    const int h = int(row - t * p.heads);
    int64_t b = 0, tok = t, didx;
    if (p.cu_q == nullptr) {
      b = t / p.lq;
      tok = t - b * p.lq;
      didx = (b * p.heads + h) * p.lq + tok;
    } else {
      didx = int64_t(h) * p.total_q + t;
    }
    const uint4 ov = *reinterpret_cast<const uint4*>(p.o + b * p.o_sb + tok * p.o_st + h * p.o_sh + lane8 * 8);
    const uint4 gv =
        *reinterpret_cast<const uint4*>(p.d_o + b * p.do_sb + tok * p.do_st + h * p.do_sh + lane8 * 8);
    const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&ov);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = __bfloat1622float2(o2[i]);
      const float2 g = __bfloat1622float2(g2[i]);
      acc = fmaf(a.x, g.x, acc);
      acc = fmaf(a.y, g.y, acc);
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    if (lane8 == 0) p.delta[didx] = acc;
    float4* acc_row = reinterpret_cast<float4*>(p.dq_accum + row * kHeadDim);
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
#if NB_BWD_L2_HINTS
    st_global_v4_hint(acc_row + lane8 * 2, z, keep);
    st_global_v4_hint(acc_row + lane8 * 2 + 1, z, keep);
#else
    acc_row[lane8 * 2] = z;
    acc_row[lane8 * 2 + 1] = z;
#endif
  }
}

// ----------------------------------------------------------------------------------------
// Epilogue: dQ = bf16(scale * accumulator), 8 lanes per (token, head) row.
// ----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) attn_bwd_epilogue_kernel(const BwdParams p) {
  pdl_wait();  // the accumulator is complete when the main kernel is
  pdl_launch_dependents();
#if NB_BWD_L2_HINTS
  const uint64_t drop = l2_policy_evict_first();
#endif
  const int64_t n_rows = p.total_q * p.heads;
  const int lane8 = threadIdx.x & 7;
  int64_t row = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 3;
  const int64_t row_step = (int64_t(gridDim.x) * blockDim.x) >> 3;
  for (; row < n_rows; row += row_step) {
    const int64_t t = row / p.heads;
    const int h = int(row - t * p.heads);
    int64_t b = 0, tok = t;
    if (p.cu_q == nullptr) {
      b = t / p.lq;
      tok = t - b * p.lq;
    }
    const float4* acc_row = reinterpret_cast<const float4*>(p.dq_accum + row * kHeadDim);
#if NB_BWD_L2_HINTS
    const float4 x = ld_global_v4_hint(acc_row + lane8 * 2, drop), y = ld_global_v4_hint(acc_row + lane8 * 2 + 1, drop);
#else
    const float4 x = acc_row[lane8 * 2], y = acc_row[lane8 * 2 + 1];
#endif
    uint4 v;
    v.x = pack_bf16(x.x * p.scale, x.y * p.scale);
    v.y = pack_bf16(x.z * p.scale, x.w * p.scale);
    v.z = pack_bf16(y.x * p.scale, y.y * p.scale);
    v.w = pack_bf16(y.z * p.scale, y.w * p.scale);
    *reinterpret_cast<uint4*>(p.dq + b * p.dq_sb + tok * p.dq_st + h * p.dq_sh + lane8 * 8) = v;
  }
}

// ----------------------------------------------------------------------------------------
// Main backward kernel
// ----------------------------------------------------------------------------------------
constexpr int kBwdThreads = 640;
constexpr int kBwdStages = 3;  // Q/dO ring
constexpr int kBwdOutStageBytes = 8192;  // dK/dV read-out: 2 KB per drain warp
// K (two buffers), V, 3x(Q, dO), dS (two 64-column halves), fp32 dQ staging (two 32-column halves),
// the dK/dV read-out staging, LSE/delta stages, the steps' control words and alignment slack
constexpr int kBwdSmemBytes =
    (3 + 2 * kBwdStages + 4) * kTileBytes + kBwdOutStageBytes + kBwdStages * 2 * kTile * 4 + 32 + 1024;
constexpr int kBwdTmemCols = 512;  // S^T 0, dP^T 128, P^T 256, dV 320, dK 384, dQ 448
// Register re-partitioning. The CTA launches with 640 threads x 96 registers (the most the
// register file allows); setmaxnreg only moves registers inside that allocation, so the budget
// must balance exactly or the growing warps would wait for ever:
//   2 compute warpgroups x 128 x 168 + issuers 128 x 56 + dQ drainers 128 x 56 + loader group 128 x 32
//   = 43008 + 7168 + 7168 + 4096 = 61440 = 640 x 96.
// Every warp of an aligned warpgroup executes the same setmaxnreg instruction.
constexpr int kBwdLaunchRegs = 96;
constexpr int kBwdComputeRegs = 168;
constexpr int kBwdIssuerRegs = 56;
constexpr int kBwdDrainRegs = 56;
constexpr int kBwdLoaderRegs = 32;
static_assert(256 * kBwdComputeRegs + 128 * (kBwdIssuerRegs + kBwdDrainRegs + kBwdLoaderRegs) ==
                  kBwdThreads * kBwdLaunchRegs, "register budget");

enum BwdBar : int {
  kBarKFull = 0,                            // [2] K is double-buffered across a CTA's work items
  kBarKFree = 2,                            // [2] the item's last dQ MMA has read K
  kBarVFull = 4,
  kBarVFree,                                // the item's last dP^T MMA has read V
  kBarQdoFull,                              // [kBwdStages] TMA issue + LSE/delta staged
  kBarQdoEmpty = kBarQdoFull + kBwdStages,  // [kBwdStages], 3 arrivals: S/dP, dV and dK issuers
  kBarSFull = kBarQdoEmpty + kBwdStages,
  kBarSFree,    // 8 arrivals (one per compute warp)
  kBarDpFull,
  kBarDpFree,   // 8
  kBarPFull,    // 8
  kBarPtFree,   // dV MMAs of the step have consumed P^T
  kBarDsFull,   // 8 arrivals
  kBarDsFree,   // 2 arrivals: dK and dQ issuers
  kBarDqFull,
  kBarDqFree,   // 4 (dQ drain warps)
  kBarDvDone,   // the item's last dV MMA is complete
  kBarDkDone,
  kBarDvOut,    // 4: the drain warps have read the item's dV accumulator
  kBarDkOut,    // 4
  kBwdNumBars
};

// One unit of a CTA's work: a 128-row K/V tile of one (sequence, head).
struct BwdWork {
  int n_q;  // query tiles to walk; 0: keys without queries (dK = dV = 0); -1: no more work
  int kt, h, b, bcoord;
  int k_begin, lk, q_begin, lq;
};

// CTAs are persistent: CTA c of G takes the work units c, 2G-1-c, 2G+c, ... ("snake" order over
// rounds of G). The list is ordered by decreasing cost, so this hands every CTA nearly the same
// total, without a shared counter: every warp role of a CTA walks the same sequence on its own.
__device__ __forceinline__ uint32_t bwd_work_index(uint32_t round) {
  const uint32_t c = (round & 1u) ? gridDim.x - 1u - blockIdx.x : blockIdx.x;
  return round * gridDim.x + c;
}

__device__ __forceinline__ BwdWork bwd_work(const BwdParams& p, uint32_t round) {
  BwdWork w;
  w.n_q = -1, w.kt = 0, w.h = 0, w.b = 0, w.bcoord = 0, w.k_begin = 0, w.lk = 0, w.q_begin = 0, w.lq = 0;
  const uint32_t g = bwd_work_index(round);
  if (g >= uint32_t(p.n_work)) return w;
  if (p.cu_q != nullptr) {
    // One 32-byte read tells all about the item (the sequence index `batch` stands for the rows past
    // the last sequence: keys without queries). Unused entries sit at the end of the list.
    const uint32_t idx = p.div_heads.quot(g);
    const SchedItem item = sched_load(p.items, idx);
    if (item.seq < 0) return w;
    w.h = int(g - idx * uint32_t(p.heads));
    w.b = item.seq, w.kt = item.tile;
    w.k_begin = item.own_begin, w.lk = item.own_len;
    w.q_begin = item.other_begin, w.lq = item.other_len;
  } else {
    const uint32_t t = p.div_n_kt.quot(g);
    w.kt = int(g - t * uint32_t(p.n_kt));
    w.b = w.bcoord = int(p.div_heads.quot(t));
    w.h = int(t - uint32_t(w.b) * uint32_t(p.heads));
    w.lk = p.lk, w.lq = p.lq;
  }
  w.n_q = (w.lq + kTile - 1) / kTile;
  return w;
}

// Query tile an item starts at. Concurrent CTAs work on the key tiles of one (sequence, head) and
// all add into the same dQ tiles, so they start at different ones: key tile kt at query tile kt,
// and where there are more key tiles than query tiles at a tile picked by a multiplicative hash
// (a multiply-high maps it into [0, n_q) without a division routine).
__device__ __forceinline__ int bwd_first_tile(int kt, int n_q) {
  return kt < n_q ? kt : int(__umulhi(uint32_t(kt) * 0x9E3779B9u, uint32_t(n_q)));
}

// Running position of a role in the CTA's stream of steps: step count, Q/dO stage and the phase of
// that stage's barriers. Steps run on through the boundaries between work items.
struct BwdStepPos {
  uint32_t s = 0, qs = 0, qph = 0;
  __device__ __forceinline__ void advance() {
    ++s;
    if (++qs == uint32_t(kBwdStages)) qs = 0, qph ^= 1u;
  }
};

// Control word of a step, staged with the step's LSE/delta rows (one per Q/dO stage). The compute
// warps and the MMA issuers learn everything about a step from it, so they never read the work
// list or leave their step loops: between two items of a persistent CTA they would otherwise run
// cold code behind a global-memory read (measured: 1500-3000 cycles per item boundary).
enum BwdCtrl : uint32_t {
  kCtrlFirst = 1u,  // first step of a work item
  kCtrlLast = 2u,   // last step of a work item
  kCtrlKb = 4u,     // which K buffer the item uses
  kCtrlStop = 8u,   // no step: the CTA's work has ended
  // bits 8-15: live query columns of the step's tile (1..128); bits 16-23: live key rows of the item's tile
};

// The compute warps' role: for every step of the CTA, P^T from S^T, then dS^T from dP^T.
// Not inlined on purpose: compiled by itself the step body keeps its instruction schedule (it sits
// at the compute warps' 168-register cap, and inlined into the kernel it came out 10-60 % slower
// whenever the code around it changed).
__device__ __noinline__ void bwd_compute_role(const uint32_t bar0, int* abort_flag, int32_t* status,
                                              const uint32_t tmem_base, const float* sLse, const float* sDelta,
                                              const volatile uint32_t* sCtrl, uint8_t* sDS_ptr,
                                              const float scale_log2) {
  const int warp = threadIdx.x >> 5;
  const int w = warp >> 2;                       // warpgroup: query columns [64w, 64w+64)
  const int krow_in_tile = threadIdx.x & 127;    // key row of this thread = tensor-memory lane
  const uint32_t tm_lane = tmem_base + (uint32_t((warp & 3) * 32) << 16);
  uint8_t* ds_half = sDS_ptr + w * kTileBytes;
  BwdStepPos pos;
  for (;; pos.advance()) {
  const uint32_t s = pos.s, qs = pos.qs, qph = pos.qph;
  auto bar = [&](int i) { return bar0 + 8u * uint32_t(i); };
  const int lane = threadIdx.x & 31;
  const uint32_t tm_s = tm_lane, tm_dp = tm_lane + 128, tm_pt = tm_lane + 256;
  const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2);
  const float4* lse4 = reinterpret_cast<const float4*>(sLse + qs * kTile + 64 * w);   // -lse (log2)
  const float4* dl4 = reinterpret_cast<const float4*>(sDelta + qs * kTile + 64 * w);  // -delta
  uint64_t pf[32];  // P^T values of this thread as packed fp32 pairs

  bool pt_ok, dp_ok;
  // ---- phase A: P^T = exp2(S^T * scale_log2 - lse) ----
  mbar_wait2(bar(kBarQdoFull + qs), qph, bar(kBarSFull), s & 1, abort_flag, status);
  const uint32_t ctrl = sCtrl[qs];
  if ((ctrl & kCtrlStop) || *reinterpret_cast<volatile int*>(abort_flag)) break;
  // Key rows past the end of the sequence must not contribute to dQ; on the ragged last query tile
  // this warpgroup's half has fewer than 64 live columns.
  const bool zero_row = krow_in_tile >= int((ctrl >> 16) & 0xFFu);
  const int valid_cols = int((ctrl >> 8) & 0xFFu) - 64 * w;
  tc_fence_after();
  {
    uint32_t ra[32], rb[32];
    tmem_ld32(tm_s + 64 * w, ra);
    tmem_ld32(tm_s + 64 * w + 32, rb);
    tmem_wait_ld();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(bar(kBarSFree));
    // Poll the barriers needed after the exponentials now; the polls' latency overlaps them.
    pt_ok = s > 0 ? mbar_try_wait(bar(kBarPtFree), (s - 1) & 1) : true;
    dp_ok = mbar_try_wait(bar(kBarDpFull), s & 1);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t* src = i < 8 ? &ra[4 * i] : &rb[4 * (i - 8)];
      const float4 l = lse4[i];
      float x0, x1, x2, x3;
      unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(src[0]), __uint_as_float(src[1])), scale2,
                             pack_f32x2(l.x, l.y)), x0, x1);
      unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(src[2]), __uint_as_float(src[3])), scale2,
                             pack_f32x2(l.z, l.w)), x2, x3);
      pf[2 * i] = pack_f32x2(fast_exp2(x0), fast_exp2(x1));
      // Every other second pair goes to the FMA pipe: the exponentials are this phase's
      // bottleneck (both warps of an SM sub-partition run it together on one MUFU unit).
      if (i & 1) pf[2 * i + 1] = exp2_poly_f32x2(pack_f32x2(x2, x3));
      else pf[2 * i + 1] = pack_f32x2(fast_exp2(x2), fast_exp2(x3));
    }
  }
  if (zero_row) {
    // Key rows past the end of the sequence must not contribute to dQ.
#pragma unroll
    for (int i = 0; i < 32; ++i) pf[i] = 0ull;
  }
  if (valid_cols < 64) {
    // Query columns past the end of the sequence: the hardware exponential already gave exactly 0
    // for their -inf argument, but the polynomial's clamp gave 2^-126. Zero those too (the second
    // pair of every odd group of four columns), so that nothing at all is added to the dQ rows of
    // the next packed sequence.
#pragma unroll
    for (int i = 1; i < 16; i += 2) {
      float a0, a1;
      unpack_f32x2(pf[2 * i + 1], a0, a1);
      pf[2 * i + 1] = pack_f32x2(4 * i + 2 < valid_cols ? a0 : 0.f, 4 * i + 3 < valid_cols ? a1 : 0.f);
    }
  }
  if (s > 0) {
    if (!pt_ok) mbar_wait(bar(kBarPtFree), (s - 1) & 1, abort_flag, status);
    tc_fence_after();
  }
  {
    uint32_t pk[16];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float a0, a1;
        unpack_f32x2(pf[16 * c + i], a0, a1);
        pk[i] = pack_bf16(a0, a1);
      }
      tmem_st16(tm_pt + 32 * w + 16 * c, pk);
    }
  }

  // ---- middle: pull dP^T of this tile out of tensor memory ----
  uint32_t ra[32], rb[32];
  if (!dp_ok) mbar_wait(bar(kBarDpFull), s & 1, abort_flag, status);
  tc_fence_after();
  const bool ds_ok = s > 0 ? mbar_try_wait(bar(kBarDsFree), (s - 1) & 1) : true;
  tmem_ld32(tm_dp + 64 * w, ra);
  tmem_ld32(tm_dp + 64 * w + 32, rb);
  tmem_wait_ld();
  tmem_wait_st();
  tc_fence_before();
  __syncwarp();
  if (lane == 0) {
    mbar_arrive(bar(kBarPFull));
    mbar_arrive(bar(kBarDpFree));
  }

  // ---- phase B: dS^T = P^T o (dP^T - delta) -> shared memory ----
  if (!ds_ok) mbar_wait(bar(kBarDsFree), (s - 1) & 1, abort_flag, status);
#pragma unroll
  for (int c = 0; c < 8; ++c) {  // 16-byte chunk c = query columns [8c, 8c+8) of this half
    const uint32_t* src = c < 4 ? &ra[8 * c] : &rb[8 * (c - 4)];
    const float4 d0 = dl4[2 * c], d1 = dl4[2 * c + 1];
    const uint64_t nd[4] = {pack_f32x2(d0.x, d0.y), pack_f32x2(d0.z, d0.w), pack_f32x2(d1.x, d1.y),
                            pack_f32x2(d1.z, d1.w)};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint64_t dp2 = pack_f32x2(__uint_as_float(src[2 * i]), __uint_as_float(src[2 * i + 1]));
      float a0, a1;
      unpack_f32x2(mul_f32x2(pf[4 * c + i], add_f32x2(dp2, nd[i])), a0, a1);
      o[i] = pack_bf16(a0, a1);
    }
    *reinterpret_cast<uint4*>(ds_half + swz128(krow_in_tile, c)) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) mbar_arrive(bar(kBarDsFull));
  }
}

__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                const __grid_constant__ CUtensorMap tmap_dq, const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[kBwdNumBars];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // delta, the cleared dQ accumulator and the work list come from the prologue kernel.
  pdl_wait();
  pdl_launch_dependents();

  uint8_t* smem_al = smem_raw + (((smem_u32(smem_raw) + 1023u) & ~1023u) - smem_u32(smem_raw));
  const uint32_t smem_base = smem_u32(smem_al);
  auto sK = [&](uint32_t kb) { return smem_base + kb * kTileBytes; };
  const uint32_t sV = smem_base + 2 * kTileBytes;
  auto sQ = [&](uint32_t s) { return smem_base + (3 + 2 * s) * kTileBytes; };
  auto sDO = [&](uint32_t s) { return smem_base + (4 + 2 * s) * kTileBytes; };
  constexpr int kDsTile0 = 3 + 2 * kBwdStages;
  const uint32_t sDS = smem_base + kDsTile0 * kTileBytes;  // 32 KB bf16: q columns 0..63 | 64..127
  uint8_t* sDS_ptr = smem_al + kDsTile0 * kTileBytes;
  uint8_t* sDQ_ptr = smem_al + (kDsTile0 + 2) * kTileBytes;  // 32 KB fp32: d columns 0..31 | 32..63
  uint8_t* sOut_ptr = smem_al + (kDsTile0 + 4) * kTileBytes;  // dK/dV read-out staging
  float* sLse = reinterpret_cast<float*>(sOut_ptr + kBwdOutStageBytes);  // [stages][128], log2 domain
  float* sDelta = sLse + kBwdStages * kTile;                             // [stages][128]
  uint32_t* sCtrl = reinterpret_cast<uint32_t*>(sDelta + kBwdStages * kTile);  // [stages], see BwdCtrl
  uint32_t* sCtrlQ = sCtrl + 4;  // [4], indexed by step & 3: the dQ issuer's copy (it does not hold the stage)

  const uint32_t bar0 = smem_u32(&bars[0]);
  auto bar = [&](int i) { return bar0 + 8u * uint32_t(i); };

  if (tid == 16 * 32) {
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_do);
    abort_flag = 0;
    for (int i = 0; i < kBwdNumBars; ++i) {
      uint32_t count = 1;
      if (i >= kBarQdoFull && i < kBarQdoFull + kBwdStages) count = 2;  // TMA issue + LSE/delta staged
      if (i >= kBarQdoEmpty && i < kBarQdoEmpty + kBwdStages) count = 3;
      if (i == kBarSFree || i == kBarDpFree || i == kBarPFull || i == kBarDsFull) count = 8;
      if (i == kBarDqFree || i == kBarDvOut || i == kBarDkOut) count = 4;
      if (i == kBarDsFree) count = 2;
      mbar_init(bar(i), count);
    }
    fence_mbar_init();
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(&tmem_base_slot), kBwdTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128, tm_pt = tmem_base + 256;
  const uint32_t tm_dv = tmem_base + 320, tm_dk = tmem_base + 384, tm_dq = tmem_base + 448;

  constexpr uint32_t kIdescS = make_idesc(128, 128, 0, 0);   // K-major x K-major, N = 128
  constexpr uint32_t kIdescKN = make_idesc(128, 64, 0, 1);   // A K-major / tensor memory, B MN-major
  constexpr uint32_t kIdescNN = make_idesc(128, 64, 1, 1);   // A MN-major, B MN-major
  const bool packed = p.cu_q != nullptr;

  if (warp >= 16) {
    setmaxnreg_dec<kBwdLoaderRegs>();
    if (warp == 16) {
      // ---------------- TMA producer (one lane) ----------------
      // K of the next item goes into the other K buffer; V is reloaded as soon as the item's last
      // dP^T MMA has read it; Q/dO tiles run through the ring without regard to item boundaries.
      if (lane == 0) {
        BwdStepPos pos;
        uint32_t ni = 0;  // items with queries so far
#pragma unroll 1
        for (uint32_t round = 0;; ++round) {
          const BwdWork wk = bwd_work(p, round);
          if (wk.n_q < 0) break;
          if (wk.n_q == 0) continue;
          const uint32_t kb = ni & 1u;
          const int krow = wk.k_begin + wk.kt * kTile;
          if (ni >= 2) mbar_wait(bar(kBarKFree + kb), ((ni >> 1) - 1) & 1, &abort_flag, p.status);
          mbar_arrive_expect_tx(bar(kBarKFull + kb), kTileBytes);
          tma_load_4d(sK(kb), &tmap_k, bar(kBarKFull + kb), 0, krow, wk.h, wk.bcoord);
          int jt = bwd_first_tile(wk.kt, wk.n_q);
#pragma unroll 1
          for (int j = 0; j < wk.n_q; ++j) {
            if (pos.s >= uint32_t(kBwdStages))
              mbar_wait(bar(kBarQdoEmpty + pos.qs), pos.qph ^ 1u, &abort_flag, p.status);
            mbar_arrive_expect_tx(bar(kBarQdoFull + pos.qs), 2 * kTileBytes);
            tma_load_4d(sQ(pos.qs), &tmap_q, bar(kBarQdoFull + pos.qs), 0, wk.q_begin + jt * kTile, wk.h, wk.bcoord);
            tma_load_4d(sDO(pos.qs), &tmap_do, bar(kBarQdoFull + pos.qs), 0, wk.q_begin + jt * kTile, wk.h,
                        wk.bcoord);
            if (j == 0) {
              if (ni >= 1) mbar_wait(bar(kBarVFree), (ni - 1) & 1, &abort_flag, p.status);
              mbar_arrive_expect_tx(bar(kBarVFull), kTileBytes);
              tma_load_4d(sV, &tmap_v, bar(kBarVFull), 0, krow, wk.h, wk.bcoord);
            }
            pos.advance();
            jt = jt + 1 == wk.n_q ? 0 : jt + 1;
          }
          ++ni;
        }
        // One more stage carries the stop mark (no data).
        if (pos.s >= uint32_t(kBwdStages)) mbar_wait(bar(kBarQdoEmpty + pos.qs), pos.qph ^ 1u, &abort_flag, p.status);
        mbar_arrive(bar(kBarQdoFull + pos.qs));
      }
    } else if (warp == 17) {
      // ---------------- LSE/delta staging and the steps' control words ----------------
      // A step's rows are requested before the wait for a free stage, so that this latency does not
      // sit between a stage becoming free and becoming full again. They are staged negated: -lse in
      // the log2 domain and -delta. Rows past the end of the sequence get -lse = -inf, which makes
      // their P^T column 0.
      BwdStepPos pos;
      uint32_t ni = 0;
#pragma unroll 1
      for (uint32_t round = 0;; ++round) {
        const BwdWork wk = bwd_work(p, round);
        if (wk.n_q < 0) break;
        if (wk.n_q == 0) continue;
        const int rows_live = min(wk.lk - wk.kt * kTile, kTile);
        const int64_t stat_base =
            packed ? int64_t(wk.h) * p.total_q + wk.q_begin : (int64_t(wk.b) * p.heads + wk.h) * p.lq;
        int jt = bwd_first_tile(wk.kt, wk.n_q);
#pragma unroll 1
        for (int j = 0; j < wk.n_q; ++j) {
          float l2[4], dl[4];
#pragma unroll
          for (int r4 = 0; r4 < 4; ++r4) {
            const int r = jt * kTile + r4 * 32 + lane;
            l2[r4] = -INFINITY, dl[r4] = 0.f;
            if (r < wk.lq) {
              l2[r4] = p.lse[stat_base + r] * -1.4426950408889634f;
              dl[r4] = -p.delta[stat_base + r];
            }
          }
          if (pos.s >= uint32_t(kBwdStages) && lane == 0)
            mbar_wait(bar(kBarQdoEmpty + pos.qs), pos.qph ^ 1u, &abort_flag, p.status);
          __syncwarp();
#pragma unroll
          for (int r4 = 0; r4 < 4; ++r4) {
            sLse[pos.qs * kTile + r4 * 32 + lane] = l2[r4];
            sDelta[pos.qs * kTile + r4 * 32 + lane] = dl[r4];
          }
          if (lane == 0) {
            const int cols_live = min(wk.lq - jt * kTile, kTile);
            const uint32_t ctrl = (j == 0 ? kCtrlFirst : 0u) | (j == wk.n_q - 1 ? kCtrlLast : 0u) |
                                  ((ni & 1u) ? kCtrlKb : 0u) | (uint32_t(cols_live) << 8) |
                                  (uint32_t(rows_live) << 16);
            sCtrl[pos.qs] = ctrl;
            sCtrlQ[pos.s & 3u] = ctrl;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(kBarQdoFull + pos.qs));
          pos.advance();
          jt = jt + 1 == wk.n_q ? 0 : jt + 1;
        }
        ++ni;
      }
      if (lane == 0) {
        if (pos.s >= uint32_t(kBwdStages)) mbar_wait(bar(kBarQdoEmpty + pos.qs), pos.qph ^ 1u, &abort_flag, p.status);
        sCtrl[pos.qs] = kCtrlStop;
        sCtrlQ[pos.s & 3u] = kCtrlStop;
        mbar_arrive(bar(kBarQdoFull + pos.qs));
      }
    }
  } else if (warp >= 12) {
    // ---------------- drain warps: dQ tiles every step, dV and dK once per item ----------------
    // Warp 12+q owns tensor-memory lane quadrant q. dQ: it stages its 32 rows (two 32-column
    // halves, 128-byte swizzled rows) in shared memory and one lane issues the TMA add-reductions,
    // so only warp-level synchronisation is needed and L2 receives whole 128-byte lines. Rows past
    // the end of the sequence are staged as exact zeros, so adding them is harmless. dV / dK: when
    // the item's last MMA into the accumulator is complete every lane pulls its row into registers
    // as bf16 and the warp stores the rows through a 2 KB scratch area; the issuers start the next
    // item's first dV / dK MMA as soon as the accumulator has been read. dV is complete half a step
    // before the item's last dQ tile, so it is taken out before that tile is drained; dK follows the
    // tile. (With both after it, every item's second step waited ~2900 cycles for the next dV / dK
    // MMA.)
    setmaxnreg_dec<kBwdDrainRegs>();
    const int quad = warp & 3;
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    uint8_t* stage = sDQ_ptr + quad * 4096;
    uint8_t* ostage = sOut_ptr + quad * (kBwdOutStageBytes / 4);
    uint32_t s = 0, ni = 0;
#if NB_BWD_L2_HINTS
    const uint64_t keep = l2_policy_evict_last();
#endif
#pragma unroll 1
    for (uint32_t round = 0;; ++round) {
      const BwdWork wk = bwd_work(p, round);
      const int n_q = wk.n_q;
      if (n_q < 0) break;
      const int h = wk.h;
      const int rows_live = wk.lk - wk.kt * kTile - quad * 32;  // this warp's rows below that exist
      const int64_t out_row = int64_t(wk.k_begin + wk.kt * kTile + quad * 32);
      const int64_t dv_off = int64_t(wk.bcoord) * p.dv_sb + int64_t(h) * p.dv_sh + out_row * p.dv_st;
      const int64_t dk_off = int64_t(wk.bcoord) * p.dk_sb + int64_t(h) * p.dk_sh + out_row * p.dk_st;
      if (n_q == 0) {
        // No queries at all: dK = dV = 0.
        if (lane < rows_live) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            reinterpret_cast<uint4*>(p.dv + dv_off + int64_t(lane) * p.dv_st)[c] = make_uint4(0, 0, 0, 0);
            reinterpret_cast<uint4*>(p.dk + dk_off + int64_t(lane) * p.dk_st)[c] = make_uint4(0, 0, 0, 0);
          }
        }
        continue;
      }
      int row = (packed ? 0 : wk.b * p.lq) + wk.q_begin + quad * 32 + bwd_first_tile(wk.kt, n_q) * kTile;
      const int row_end = (packed ? 0 : wk.b * p.lq) + wk.q_begin + quad * 32 + n_q * kTile;
      // Events of an item, in order: the dQ tiles of steps 0 .. n_q-2, dV, the last dQ tile, dK.
#pragma unroll 1
      for (int e = 0; e < n_q + 2; ++e) {
        if (e == n_q - 1 || e == n_q + 1) {
          const bool is_dk = e > n_q;
          mbar_wait(bar(is_dk ? kBarDkDone : kBarDvDone), ni & 1, &abort_flag, p.status);
          tc_fence_after();
          const uint32_t tm_acc = (is_dk ? tm_dk : tm_dv) + lane_off;
          const float out_scale = is_dk ? p.scale : 1.f;
          __nv_bfloat16* out = is_dk ? p.dk + dk_off : p.dv + dv_off;
          const int64_t out_st = is_dk ? p.dk_st : p.dv_st;
          // The whole 64-column row of this lane becomes 32 packed registers (four 16-column loads)
          // and the accumulator is handed back at once. The rows then go out 32 columns at a time
          // through a 2 KB scratch area, four lanes per 64-byte half row (a row per lane straight
          // from the registers was measured slower: 32 separate lines per store instruction).
          uint32_t pk[32];
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t r[16];
            tmem_ld16(tm_acc + 16 * q4, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 8; ++i)
              pk[8 * q4 + i] =
                  pack_bf16(__uint_as_float(r[2 * i]) * out_scale, __uint_as_float(r[2 * i + 1]) * out_scale);
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(is_dk ? kBarDkOut : kBarDvOut));  // the accumulator is free
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            // Row `lane` of the scratch holds 32 bf16 = four 16-byte chunks, XOR-ed with the row
            // pair's index so that neither the writes (a row per lane) nor the reads (four lanes per
            // row) collide on banks.
#pragma unroll
            for (int c = 0; c < 4; ++c)
              *reinterpret_cast<uint4*>(ostage + lane * 64 + ((c ^ ((lane >> 1) & 3)) << 4)) = make_uint4(
                  pk[16 * half + 4 * c], pk[16 * half + 4 * c + 1], pk[16 * half + 4 * c + 2], pk[16 * half + 4 * c + 3]);
            __syncwarp();
#pragma unroll
            for (int it = 0; it < 4; ++it) {
              const int rloc = it * 8 + (lane >> 2), c = lane & 3;
              const uint4 v = *reinterpret_cast<const uint4*>(ostage + rloc * 64 + ((c ^ ((rloc >> 1) & 3)) << 4));
              if (rloc < rows_live) *reinterpret_cast<uint4*>(out + int64_t(rloc) * out_st + half * 32 + c * 8) = v;
            }
            __syncwarp();
          }
          continue;
        }
        mbar_wait(bar(kBarDqFull), s & 1, &abort_flag, p.status);
        tc_fence_after();
        if (lane == 0) bulk_wait_group_read0();  // the previous reductions have read the staging rows
        __syncwarp();
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tmem_ld32(tm_dq + lane_off + 32 * half, r);
          tmem_wait_ld();
          if (half == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kBarDqFree));  // the dQ tile is out of tensor memory
          }
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<uint4*>(stage + half * kTileBytes + swz128(lane, c)) =
                make_uint4(r[4 * c], r[4 * c + 1], r[4 * c + 2], r[4 * c + 3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
#if NB_BWD_L2_HINTS
          tma_reduce_add_3d_hint(&tmap_dq, smem_u32(stage), 0, row, h, keep);
          tma_reduce_add_3d_hint(&tmap_dq, smem_u32(stage + kTileBytes), 32, row, h, keep);
#else
          tma_reduce_add_3d(&tmap_dq, smem_u32(stage), 0, row, h);
          tma_reduce_add_3d(&tmap_dq, smem_u32(stage + kTileBytes), 32, row, h);
#endif
          bulk_commit_group();
        }
        ++s;
        row += kTile;
        if (row == row_end) row -= n_q * kTile;
      }
      ++ni;
    }
    if (lane == 0) bulk_wait_group_read0();  // the staging rows must outlive the TMA engine's reads
  } else if (warp >= 8) {
    setmaxnreg_dec<kBwdIssuerRegs>();
    // Each issuer is one elected thread that walks the CTA's steps by their control words.
    if (elect_one()) {
      BwdStepPos pos;
      uint32_t ni = 0;  // items started
      volatile uint32_t* ctrl_ring = sCtrl;
      if (warp == 8) {
        // ---------------- MMA issuer: S^T = K Q^T and dP^T = V dO^T ----------------
        const uint64_t vd = make_sdesc(sV, 16, 1024);
        uint64_t kd = 0;
#pragma unroll 1
        for (;; pos.advance()) {
          if (!mbar_wait(bar(kBarQdoFull + pos.qs), pos.qph, &abort_flag, p.status)) break;
          const uint32_t ctrl = ctrl_ring[pos.qs];
          if (ctrl & kCtrlStop) {
            // The compute warps wait for the stage and for S^T together, so the stop mark needs an
            // arrival on the S^T barrier -- once they have consumed the previous step's phase (a
            // barrier must never run two phases ahead of a waiter that tests by parity).
            if (pos.s > 0) mbar_wait(bar(kBarSFree), (pos.s - 1) & 1, &abort_flag, p.status);
            mbar_arrive(bar(kBarSFull));
            break;
          }
          if (ctrl & kCtrlFirst) {
            const uint32_t kb = (ctrl & kCtrlKb) ? 1u : 0u;
            kd = make_sdesc(sK(kb), 16, 1024);
            mbar_wait(bar(kBarKFull + kb), (ni >> 1) & 1, &abort_flag, p.status);
          }
          if (pos.s > 0) mbar_wait(bar(kBarSFree), (pos.s - 1) & 1, &abort_flag, p.status);
          tc_fence_after();
          const uint64_t qd = make_sdesc(sQ(pos.qs), 16, 1024), gd = make_sdesc(sDO(pos.qs), 16, 1024);
#pragma unroll 1
          for (int k = 0; k < 4; ++k) mma_ss(tm_s, kd + 2 * k, qd + 2 * k, kIdescS, k > 0);
          tc_commit(bar(kBarSFull));
          if (ctrl & kCtrlFirst) mbar_wait(bar(kBarVFull), ni & 1, &abort_flag, p.status);
          if (pos.s > 0) mbar_wait(bar(kBarDpFree), (pos.s - 1) & 1, &abort_flag, p.status);
          tc_fence_after();
#pragma unroll 1
          for (int k = 0; k < 4; ++k) mma_ss(tm_dp, vd + 2 * k, gd + 2 * k, kIdescS, k > 0);
          tc_commit(bar(kBarDpFull));
          tc_commit(bar(kBarQdoEmpty + pos.qs));
          if (ctrl & kCtrlLast) {
            tc_commit(bar(kBarVFree));
            ++ni;
          }
        }
      } else if (warp == 9) {
        // ---------------- MMA issuer: dV += P^T dO ----------------
#pragma unroll 1
        for (;; pos.advance()) {
          if (!mbar_wait(bar(kBarQdoFull + pos.qs), pos.qph, &abort_flag, p.status)) break;
          const uint32_t ctrl = ctrl_ring[pos.qs];
          if (ctrl & kCtrlStop) break;
          const bool first = (ctrl & kCtrlFirst) != 0;
          // The previous item's dV has to be out of tensor memory before this one's first MMA.
          if (first && ni > 0) mbar_wait(bar(kBarDvOut), (ni - 1) & 1, &abort_flag, p.status);
          mbar_wait(bar(kBarPFull), pos.s & 1, &abort_flag, p.status);
          tc_fence_after();
          const uint64_t gd_mn = make_sdesc(sDO(pos.qs), 1024, 1024);
#pragma unroll 1
          for (int k = 0; k < 8; ++k) mma_ts(tm_dv, tm_pt + 8 * k, gd_mn + 128 * k, kIdescKN, !first || (k > 0));
          tc_commit(bar(kBarPtFree));
          tc_commit(bar(kBarQdoEmpty + pos.qs));
          if (ctrl & kCtrlLast) {
            tc_commit(bar(kBarDvDone));
            ++ni;
          }
        }
      } else if (warp == 10) {
        // ---------------- MMA issuer: dK += dS^T Q ----------------
#pragma unroll 1
        for (;; pos.advance()) {
          if (!mbar_wait(bar(kBarQdoFull + pos.qs), pos.qph, &abort_flag, p.status)) break;
          const uint32_t ctrl = ctrl_ring[pos.qs];
          if (ctrl & kCtrlStop) break;
          const bool first = (ctrl & kCtrlFirst) != 0;
          if (first && ni > 0) mbar_wait(bar(kBarDkOut), (ni - 1) & 1, &abort_flag, p.status);
          mbar_wait(bar(kBarDsFull), pos.s & 1, &abort_flag, p.status);
          tc_fence_after();
          const uint64_t qd_mn = make_sdesc(sQ(pos.qs), 1024, 1024);
#pragma unroll 1
          for (int k = 0; k < 8; ++k) {
            // A: K-major view of the dS buffer; one K step = 16 query columns.
            const uint64_t ad = make_sdesc(sDS + (k >> 2) * kTileBytes, 16, 1024) + 2 * (k & 3);
            mma_ss(tm_dk, ad, qd_mn + 128 * k, kIdescKN, !first || (k > 0));
          }
          tc_commit(bar(kBarDsFree));
          tc_commit(bar(kBarQdoEmpty + pos.qs));
          if (ctrl & kCtrlLast) {
            tc_commit(bar(kBarDkDone));
            ++ni;
          }
        }
      } else {
        // ---------------- MMA issuer: dQ = dS K ----------------
        // A: MN-major view of the same dS bytes; one K step = 16 key rows.
        const uint64_t ds_mn = make_sdesc(sDS, kTileBytes, 1024);
        uint64_t kd_mn = 0;
        uint32_t kb = 0;
#pragma unroll 1
        for (;; pos.advance()) {
          if (!mbar_wait(bar(kBarQdoFull + pos.qs), pos.qph, &abort_flag, p.status)) break;
          // This issuer does not hold the stage (the path from a stage becoming free to becoming full
          // again is the tightest in the pipeline), so it reads a copy that is overwritten four steps
          // later: that write comes after the dK MMA of step s+1, which follows this step's dQ MMA.
          const uint32_t ctrl = (reinterpret_cast<volatile uint32_t*>(sCtrlQ))[pos.s & 3u];
          if (ctrl & kCtrlStop) break;
          if (ctrl & kCtrlFirst) {
            kb = (ctrl & kCtrlKb) ? 1u : 0u;
            kd_mn = make_sdesc(sK(kb), 1024, 1024);
            mbar_wait(bar(kBarKFull + kb), (ni >> 1) & 1, &abort_flag, p.status);
          }
          mbar_wait(bar(kBarDsFull), pos.s & 1, &abort_flag, p.status);
          if (pos.s > 0) mbar_wait(bar(kBarDqFree), (pos.s - 1) & 1, &abort_flag, p.status);
          tc_fence_after();
#pragma unroll 1
          for (int k = 0; k < 8; ++k) mma_ss(tm_dq, ds_mn + 128 * k, kd_mn + 128 * k, kIdescNN, k > 0);
          tc_commit(bar(kBarDqFull));
          tc_commit(bar(kBarDsFree));
          if (ctrl & kCtrlLast) {
            tc_commit(bar(kBarKFree + kb));
            ++ni;
          }
        }
      }
    }
  } else {
    // ---------------- compute warpgroups: w = 0 / 1 owns query columns [64w, 64w+64) ----------------
    setmaxnreg_inc<kBwdComputeRegs>();
    bwd_compute_role(bar0, &abort_flag, p.status, tmem_base, sLse, sDelta, sCtrl, sDS_ptr, p.scale_log2);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kBwdTmemCols);
  }
}

}  // namespace nb
