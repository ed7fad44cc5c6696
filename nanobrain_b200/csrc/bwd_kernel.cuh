// Backward attention kernels (head_dim 64, bf16 tensors, fp32 accumulation):
//
//   attn_bwd_prologue_kernel : delta[row] = sum_d dO[row,d] * O[row,d] (warp-shuffle row dot) and
//                              clears the fp32 dQ accumulator. HBM-bound.
//   attn_bwd_kernel          : one CTA owns one 128-row K/V tile of one (sequence, head) and walks
//                              the sequence's queries in 128-row tiles. Everything is computed
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
//                              Warp roles (640 threads): warps 0-7 are two compute warpgroups that
//                              split the 128 query columns of a tile (64 each); warps 8-11 are
//                              four MMA issuers (S^T/dP^T, dV, dK, dQ: one elected thread each --
//                              a single thread can issue a tcgen05.mma only every ~55 cycles, so
//                              the 32 MMAs of a tile need several issuers to keep the tensor pipe
//                              fed); warps 12-15 drain the dQ tiles (one tensor-memory lane
//                              quadrant each) into the accumulator; warp 16 drives TMA and stages
//                              LSE/delta rows (warps 17-19 only complete its warpgroup for the
//                              register re-partitioning).
//   attn_bwd_epilogue_kernel : dQ = bf16(scale * accumulator). HBM-bound.
//
// Packed mode: block 0 of the prologue also builds the scheduler's work list of key tiles
// (sched_kernel.cuh) and the main kernel's grid is items x heads (the heads of one item adjacent).
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
    acc_row[lane8 * 2] = z;
    acc_row[lane8 * 2 + 1] = z;
  }
}

// ----------------------------------------------------------------------------------------
// Epilogue: dQ = bf16(scale * accumulator), 8 lanes per (token, head) row.
// ----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) attn_bwd_epilogue_kernel(const BwdParams p) {
  pdl_wait();  // the accumulator is complete when the main kernel is
  pdl_launch_dependents();
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
    const float4 x = acc_row[lane8 * 2], y = acc_row[lane8 * 2 + 1];
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
// K, V, 3x(Q, dO), dS (two 64-column halves), fp32 dQ staging (two 32-column halves) + LSE/delta
// stages + alignment slack
constexpr int kBwdSmemBytes = (2 + 2 * kBwdStages + 4) * kTileBytes + kBwdStages * 2 * kTile * 4 + 1024;
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
  kBarKvFull = 0,
  kBarQdoFull = 1,                       // [kBwdStages]
  kBarQdoEmpty = kBarQdoFull + kBwdStages,  // [kBwdStages], 3 arrivals: S/dP, dV and dK issuers
  kBarSFull = kBarQdoEmpty + kBwdStages,
  kBarSFree,    // 8 arrivals (one per compute warp)
  kBarDpFull,
  kBarDpFree,   // 8
  kBarPFull,    // 8
  kBarPtFree,   // dV MMAs of the tile have consumed P^T
  kBarDsFull,   // 8 arrivals
  kBarDsFree,   // 2 arrivals: dK and dQ issuers
  kBarDqFull,
  kBarDqFree,   // 4 (dQ drain warps)
  kBarDkDone,
  kBwdNumBars
};

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
  int kt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;

  // delta, the cleared dQ accumulator and the work list come from the prologue kernel.
  pdl_wait();
  pdl_launch_dependents();

  int q_begin = 0, k_begin = 0, lq = p.lq, lk = p.lk, bcoord = b;
  if (p.cu_q != nullptr) {
    // One read tells the CTA everything about its item (the sequence index `batch` stands for the
    // rows past the last sequence: keys without queries, which get dK = dV = 0).
    const SchedItem item = sched_load(p.items, blockIdx.x / uint32_t(p.heads));
    if (item.seq < 0) return;
    h = blockIdx.x % uint32_t(p.heads);
    b = item.seq;
    kt = item.tile;
    k_begin = item.own_begin;
    lk = item.own_len;
    q_begin = item.other_begin;
    lq = item.other_len;
    bcoord = 0;
  }
  const int k_row0 = kt * kTile;
  if (k_row0 >= lk) return;
  const int n_q = (lq + kTile - 1) / kTile;

  uint8_t* smem_al = smem_raw + (((smem_u32(smem_raw) + 1023u) & ~1023u) - smem_u32(smem_raw));
  const uint32_t smem_base = smem_u32(smem_al);
  const uint32_t sK = smem_base;
  const uint32_t sV = smem_base + 1 * kTileBytes;
  auto sQ = [&](int s) { return smem_base + (2 + 2 * s) * kTileBytes; };
  auto sDO = [&](int s) { return smem_base + (3 + 2 * s) * kTileBytes; };
  constexpr int kDsTile0 = 2 + 2 * kBwdStages;
  const uint32_t sDS = smem_base + kDsTile0 * kTileBytes;  // 32 KB bf16: q columns 0..63 | 64..127
  uint8_t* sDS_ptr = smem_al + kDsTile0 * kTileBytes;
  uint8_t* sDQ_ptr = smem_al + (kDsTile0 + 2) * kTileBytes;  // 32 KB fp32: d columns 0..31 | 32..63
  float* sLse = reinterpret_cast<float*>(smem_al + (kDsTile0 + 4) * kTileBytes);  // [stages][128], log2 domain
  float* sDelta = sLse + kBwdStages * kTile;                                      // [stages][128]

  const uint32_t bar0 = smem_u32(&bars[0]);
  auto bar = [&](int i) { return bar0 + 8u * uint32_t(i); };

  // The producer's own thread initialises the barriers, so it can request K, V and the first Q/dO
  // tiles at once; the other threads meet the barriers only after the __syncthreads below.
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
      if (i == kBarSFree || i == kBarDpFree || i == kBarPFull) count = 8;
      if (i == kBarDqFree) count = 4;
      if (i == kBarDsFull) count = 8;
      if (i == kBarDsFree) count = 2;
      mbar_init(bar(i), count);
    }
    fence_mbar_init();
    if (n_q > 0) {
      const int jt0 = kt % n_q;
      mbar_arrive_expect_tx(bar(kBarKvFull), 2 * kTileBytes);
      tma_load_4d(sK, &tmap_k, bar(kBarKvFull), 0, k_begin + k_row0, h, bcoord);
      tma_load_4d(sV, &tmap_v, bar(kBarKvFull), 0, k_begin + k_row0, h, bcoord);
      mbar_arrive_expect_tx(bar(kBarQdoFull), 2 * kTileBytes);
      tma_load_4d(sQ(0), &tmap_q, bar(kBarQdoFull), 0, q_begin + jt0 * kTile, h, bcoord);
      tma_load_4d(sDO(0), &tmap_do, bar(kBarQdoFull), 0, q_begin + jt0 * kTile, h, bcoord);
    }
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
  const int64_t stat_base = p.cu_q != nullptr ? int64_t(h) * p.total_q + q_begin : (int64_t(b) * p.heads + h) * p.lq;

  if (n_q > 0) {
    if (warp >= 16) {
      // ---------------- TMA producer + LSE/delta staging (warp 16; 17-19 idle) ----------------
      setmaxnreg_dec<kBwdLoaderRegs>();
      if (warp == 16) {
      for (int j = 0; j < n_q; ++j) {
        const int qs = j % kBwdStages;
        const int jt = (j + kt) % n_q;  // staggered start: concurrent CTAs touch different dQ tiles
        // The tile's LSE/delta rows are requested before the wait for a free stage, so that this
        // latency does not sit between a stage becoming free and becoming full again. They are
        // staged negated: -lse in the log2 domain and -delta. Rows past the end of the sequence get
        // -lse = -inf, which makes their P^T column 0.
        float l2[4], dl[4];
#pragma unroll
        for (int r4 = 0; r4 < 4; ++r4) {
          const int r = jt * kTile + r4 * 32 + lane;
          l2[r4] = -INFINITY, dl[r4] = 0.f;
          if (r < lq) {
            l2[r4] = p.lse[stat_base + r] * -1.4426950408889634f;
            dl[r4] = -p.delta[stat_base + r];
          }
        }
        if (j >= kBwdStages && lane == 0)
          mbar_wait(bar(kBarQdoEmpty + qs), ((j / kBwdStages) - 1) & 1, &abort_flag, p.status);
        __syncwarp();
        if (lane == 0 && j > 0) {  // tile 0 is already on its way
          mbar_arrive_expect_tx(bar(kBarQdoFull + qs), 2 * kTileBytes);
          tma_load_4d(sQ(qs), &tmap_q, bar(kBarQdoFull + qs), 0, q_begin + jt * kTile, h, bcoord);
          tma_load_4d(sDO(qs), &tmap_do, bar(kBarQdoFull + qs), 0, q_begin + jt * kTile, h, bcoord);
        }
#pragma unroll
        for (int r4 = 0; r4 < 4; ++r4) {
          sLse[qs * kTile + r4 * 32 + lane] = l2[r4];
          sDelta[qs * kTile + r4 * 32 + lane] = dl[r4];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(kBarQdoFull + qs));
      }
      }
    } else if (warp >= 12) {
      // ---------------- dQ drain warps: tensor memory -> staged fp32 rows -> TMA add-reduction ----------------
      // Warp 12+q owns tensor-memory lane quadrant q. It stages its 32 rows (two 32-column halves,
      // 128-byte swizzled rows) in shared memory and one lane issues the TMA add-reductions, so
      // only warp-level synchronisation is needed and L2 receives whole 128-byte lines. Rows past
      // the end of the sequence are staged as exact zeros, so adding them is harmless.
      setmaxnreg_dec<kBwdDrainRegs>();
      const int quad = warp & 3;
      const uint32_t lane_off = uint32_t(quad * 32) << 16;
      const int64_t acc_batch_row = int64_t(p.cu_q != nullptr ? 0 : b) * p.lq + q_begin;
      uint8_t* stage = sDQ_ptr + quad * 4096;
      for (int j = 0; j < n_q; ++j) {
        const int tile = (j + kt) % n_q;
        mbar_wait(bar(kBarDqFull), j & 1, &abort_flag, p.status);
        tc_fence_after();
        if (lane == 0) bulk_wait_group_read0();  // the previous reductions have read the staging rows
        __syncwarp();
#pragma unroll
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
          const int row = int(acc_batch_row) + tile * kTile + quad * 32;
          tma_reduce_add_3d(&tmap_dq, smem_u32(stage), 0, row, h);
          tma_reduce_add_3d(&tmap_dq, smem_u32(stage + kTileBytes), 32, row, h);
          bulk_commit_group();
        }
      }
      if (lane == 0) bulk_wait_group_read0();  // the staging rows must outlive the TMA engine's reads
    } else if (warp >= 8) {
      setmaxnreg_dec<kBwdIssuerRegs>();
      if (warp == 8) {
      // ---------------- MMA issuer: S^T = K Q^T and dP^T = V dO^T ----------------
      if (elect_one()) {
        const uint64_t kd = make_sdesc(sK, 16, 1024), vd = make_sdesc(sV, 16, 1024);
        mbar_wait(bar(kBarKvFull), 0, &abort_flag, p.status);
        for (int j = 0; j < n_q; ++j) {
          const int qs = j % kBwdStages;
          mbar_wait(bar(kBarQdoFull + qs), (j / kBwdStages) & 1, &abort_flag, p.status);
          if (j > 0) mbar_wait(bar(kBarSFree), (j - 1) & 1, &abort_flag, p.status);
          tc_fence_after();
          const uint64_t qd = make_sdesc(sQ(qs), 16, 1024), gd = make_sdesc(sDO(qs), 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_ss(tm_s, kd + 2 * k, qd + 2 * k, kIdescS, k > 0);
          tc_commit(bar(kBarSFull));
          if (j > 0) mbar_wait(bar(kBarDpFree), (j - 1) & 1, &abort_flag, p.status);
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_ss(tm_dp, vd + 2 * k, gd + 2 * k, kIdescS, k > 0);
          tc_commit(bar(kBarDpFull));
          tc_commit(bar(kBarQdoEmpty + qs));
        }
      }
      } else if (warp == 9) {
      // ---------------- MMA issuer: dV += P^T dO ----------------
      if (elect_one()) {
        for (int j = 0; j < n_q; ++j) {
          const int qs = j % kBwdStages;
          mbar_wait(bar(kBarPFull), j & 1, &abort_flag, p.status);
          mbar_wait(bar(kBarQdoFull + qs), (j / kBwdStages) & 1, &abort_flag, p.status);
          tc_fence_after();
          const uint64_t gd_mn = make_sdesc(sDO(qs), 1024, 1024);
#pragma unroll
          for (int k = 0; k < 8; ++k) mma_ts(tm_dv, tm_pt + 8 * k, gd_mn + 128 * k, kIdescKN, (j > 0) || (k > 0));
          tc_commit(bar(kBarPtFree));
          tc_commit(bar(kBarQdoEmpty + qs));
        }
      }
      } else if (warp == 10) {
      // ---------------- MMA issuer: dK += dS^T Q ----------------
      if (elect_one()) {
        for (int j = 0; j < n_q; ++j) {
          const int qs = j % kBwdStages;
          mbar_wait(bar(kBarDsFull), j & 1, &abort_flag, p.status);
          mbar_wait(bar(kBarQdoFull + qs), (j / kBwdStages) & 1, &abort_flag, p.status);
          tc_fence_after();
          const uint64_t qd_mn = make_sdesc(sQ(qs), 1024, 1024);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            // A: K-major view of the dS buffer; one K step = 16 query columns.
            const uint64_t ad = make_sdesc(sDS + (k >> 2) * kTileBytes, 16, 1024) + 2 * (k & 3);
            mma_ss(tm_dk, ad, qd_mn + 128 * k, kIdescKN, (j > 0) || (k > 0));
          }
          tc_commit(bar(kBarDsFree));
          tc_commit(bar(kBarQdoEmpty + qs));
        }
        tc_commit(bar(kBarDkDone));
      }
      } else {
      // ---------------- MMA issuer: dQ = dS K ----------------
      if (elect_one()) {
        const uint64_t kd_mn = make_sdesc(sK, 1024, 1024);
        mbar_wait(bar(kBarKvFull), 0, &abort_flag, p.status);
        for (int j = 0; j < n_q; ++j) {
          mbar_wait(bar(kBarDsFull), j & 1, &abort_flag, p.status);
          if (j > 0) mbar_wait(bar(kBarDqFree), (j - 1) & 1, &abort_flag, p.status);
          tc_fence_after();
          // A: MN-major view of the same dS bytes; one K step = 16 key rows.
          const uint64_t ds_mn = make_sdesc(sDS, kTileBytes, 1024);
#pragma unroll
          for (int k = 0; k < 8; ++k) mma_ss(tm_dq, ds_mn + 128 * k, kd_mn + 128 * k, kIdescNN, k > 0);
          tc_commit(bar(kBarDqFull));
          tc_commit(bar(kBarDsFree));
        }
      }
      }
    } else {
      // ---------------- compute warpgroups: w = 0 / 1 owns query columns [64w, 64w+64) ----------------
      setmaxnreg_inc<kBwdComputeRegs>();
      const int w = warp >> 2;
      const int krow_in_tile = tid & 127;  // key row of this thread = tensor-memory lane
      const uint32_t lane_off = uint32_t((warp & 3) * 32) << 16;
      const bool row_valid = (k_row0 + krow_in_tile) < lk;
      const bool partial = (k_row0 + kTile) > lk;
      const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
      // Iteration that visits the last, ragged query tile (-1 if the length is a multiple of the tile).
      const int j_ragged = (lq % kTile) != 0 ? (n_q - 1 - kt % n_q + n_q) % n_q : -1;
      for (int j = 0; j < n_q; ++j) {
        const int qs = j % kBwdStages;
        const float4* lse4 = reinterpret_cast<const float4*>(sLse + qs * kTile + 64 * w);   // -lse (log2)
        const float4* dl4 = reinterpret_cast<const float4*>(sDelta + qs * kTile + 64 * w);  // -delta
        uint64_t pf[32];  // P^T values of this thread as packed fp32 pairs

        bool pt_ok, dp_ok;
        // ---- phase A: P^T = exp2(S^T * scale_log2 - lse) ----
        mbar_wait2(bar(kBarQdoFull + qs), (j / kBwdStages) & 1, bar(kBarSFull), j & 1, &abort_flag, p.status);
        tc_fence_after();
        {
          uint32_t ra[32], rb[32];
          tmem_ld32(tm_s + lane_off + 64 * w, ra);
          tmem_ld32(tm_s + lane_off + 64 * w + 32, rb);
          tmem_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(kBarSFree));
          // Poll the barriers needed after the exponentials now; the polls' latency overlaps them.
          pt_ok = j > 0 ? mbar_try_wait(bar(kBarPtFree), (j - 1) & 1) : true;
          dp_ok = mbar_try_wait(bar(kBarDpFull), j & 1);
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
        if (partial && !row_valid) {
          // Key rows past the end of the sequence must not contribute to dQ.
#pragma unroll
          for (int i = 0; i < 32; ++i) pf[i] = 0ull;
        }
        if (j == j_ragged) {
          // Query columns past the end of the sequence: the hardware exponential already gave 0 for
          // their -inf argument, the polynomial's clamp gave 2^-126. Make all of them exactly 0, so
          // that nothing at all is added to the dQ rows of the next packed sequence.
          const int valid = lq - (n_q - 1) * kTile - 64 * w;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float a0, a1;
            unpack_f32x2(pf[i], a0, a1);
            pf[i] = pack_f32x2(2 * i < valid ? a0 : 0.f, 2 * i + 1 < valid ? a1 : 0.f);
          }
        }
        if (j > 0) {
          if (!pt_ok) mbar_wait(bar(kBarPtFree), (j - 1) & 1, &abort_flag, p.status);
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
            tmem_st16(tm_pt + lane_off + 32 * w + 16 * c, pk);
          }
        }

        // ---- middle: pull dP^T of this tile out of tensor memory ----
        uint32_t ra[32], rb[32];
        if (!dp_ok) mbar_wait(bar(kBarDpFull), j & 1, &abort_flag, p.status);
        tc_fence_after();
        const bool ds_ok = j > 0 ? mbar_try_wait(bar(kBarDsFree), (j - 1) & 1) : true;
        tmem_ld32(tm_dp + lane_off + 64 * w, ra);
        tmem_ld32(tm_dp + lane_off + 64 * w + 32, rb);
        tmem_wait_ld();
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bar(kBarPFull));
          mbar_arrive(bar(kBarDpFree));
        }

        // ---- phase B: dS^T = P^T o (dP^T - delta) -> shared memory ----
        if (!ds_ok) mbar_wait(bar(kBarDsFree), (j - 1) & 1, &abort_flag, p.status);
        uint8_t* half = sDS_ptr + w * kTileBytes;
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
          *reinterpret_cast<uint4*>(half + swz128(krow_in_tile, c)) = make_uint4(o[0], o[1], o[2], o[3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(kBarDsFull));
      }
      // ---- epilogue: warpgroup 0 stores dV, warpgroup 1 stores dK (scaled) ----
      // Warpgroup 0 needs dV complete (the last P^T consumed), warpgroup 1 needs dK complete.
      if (w == 0) mbar_wait(bar(kBarPtFree), (n_q - 1) & 1, &abort_flag, p.status);
      else mbar_wait(bar(kBarDkDone), 0, &abort_flag, p.status);
      tc_fence_after();
      // Each warp turns its 32 accumulator rows into bf16 in a 4 KB scratch area and writes them out
      // with eight lanes per 128-byte row, so the stores are whole lines. Only warp-level
      // synchronisation is needed: a warp reads back what it wrote. The scratch is dead operand
      // space: warpgroup 0 uses the V tile (last read by the final dP^T MMA, long complete when the
      // final dV MMA is), warpgroup 1 the first Q stage (read only by S^T and dK MMAs, all complete).
      uint8_t* scratch = smem_al + (1 + w) * kTileBytes + (warp & 3) * 4096;
      const float out_scale = w == 0 ? 1.f : p.scale;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32((w == 0 ? tm_dv : tm_dk) + lane_off + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(r[8 * i + 0]) * out_scale, __uint_as_float(r[8 * i + 1]) * out_scale);
          v.y = pack_bf16(__uint_as_float(r[8 * i + 2]) * out_scale, __uint_as_float(r[8 * i + 3]) * out_scale);
          v.z = pack_bf16(__uint_as_float(r[8 * i + 4]) * out_scale, __uint_as_float(r[8 * i + 5]) * out_scale);
          v.w = pack_bf16(__uint_as_float(r[8 * i + 6]) * out_scale, __uint_as_float(r[8 * i + 7]) * out_scale);
          *reinterpret_cast<uint4*>(scratch + swz128(lane, c * 4 + i)) = v;
        }
      }
      __syncwarp();
      __nv_bfloat16* out_base = w == 0 ? p.dv + int64_t(bcoord) * p.dv_sb + int64_t(h) * p.dv_sh
                                       : p.dk + int64_t(bcoord) * p.dk_sb + int64_t(h) * p.dk_sh;
      const int64_t out_st = w == 0 ? p.dv_st : p.dk_st;
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int rloc = it * 4 + (lane >> 3);
        const int krow = k_row0 + (warp & 3) * 32 + rloc;
        const uint4 v = *reinterpret_cast<const uint4*>(scratch + swz128(rloc, lane & 7));
        if (krow < lk) *reinterpret_cast<uint4*>(out_base + int64_t(k_begin + krow) * out_st + (lane & 7) * 8) = v;
      }
    }
  } else if (warp < 8) {
    // No queries at all: dK = dV = 0.
    const int w = warp >> 2;
    const int krow = k_row0 + (tid & 127);
    if (krow < lk) {
      __nv_bfloat16* out_ptr =
          w == 0 ? p.dv + int64_t(bcoord) * p.dv_sb + int64_t(k_begin + krow) * p.dv_st + int64_t(h) * p.dv_sh
                 : p.dk + int64_t(bcoord) * p.dk_sb + int64_t(k_begin + krow) * p.dk_st + int64_t(h) * p.dk_sh;
      for (int c = 0; c < 8; ++c) reinterpret_cast<uint4*>(out_ptr)[c] = make_uint4(0, 0, 0, 0);
    }
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
