// Forward attention kernel: O = softmax(Q K^T * scale) V, bf16 in / bf16 out, fp32 softmax
// statistics and accumulation, head_dim 64, non-causal.
//
// One CTA owns one 128-row query tile of one (sequence, head) and walks the sequence's keys in
// 128-row tiles. In packed mode the CTA takes its (sequence, tile) from the scheduler's work list
// (sched_kernel.cuh: grid = items x heads with the heads of one item adjacent, so that launch order
// is most expensive first over the whole grid; running the list once per head instead was measured
// slower on mixes of short and long sequences); in dense mode the grid is
// (tiles, heads, batch). Two CTAs are resident per SM (256 tensor-memory columns and 80 KB of shared
// memory each), so one CTA's softmax, prologue and epilogue overlap the other's MMAs. A ragged last
// key tile is trimmed: its score MMA runs with N rounded up to 16, the P V MMA with as many K steps,
// and the softmax warps touch only the live 32-column chunks. Warp roles (192 threads):
//
//   warps 0-3 : softmax warpgroup. Thread r owns row r of the tile (tensor-memory lane r). Per key
//               tile it pulls the whole fp32 score row into registers (which frees the score
//               buffer for the next S MMA at once), takes the row max, and writes
//               P = exp2(S*scale_log2 - m) as bf16 into a separate tensor-memory buffer. The
//               offset m is the row max of the first tile; later tiles do not compute a max at
//               all: they exponentiate against m and look at the tile's row sum, and only if a sum
//               shows that some exponent ran far above m (sum > 2^14, or Inf / NaN) is the tile
//               redone with its true max, m refreshed and the O accumulator in tensor memory
//               rescaled. At the end it normalises and stores O and the log-sum-exp.
//   warp 4    : one elected thread issues every tcgen05.mma: S = Q K^T (both operands from shared
//               memory) and O += P V (P from tensor memory, V from shared memory, MN-major).
//   warp 5    : one elected thread drives TMA: the Q tile once, then K and V tiles through a
//               two-stage ring (SWIZZLE_128B; every CTA loads its own tiles).
//
// Tensor memory (256 columns): S [0,128) O [128,192) P [192,256).
#pragma once

#include <type_traits>

#include "ptx.cuh"
#include "sched_kernel.cuh"

namespace nb {

struct FwdParams {
  __nv_bfloat16* o;
  int64_t o_sb, o_st, o_sh;  // element strides of O: batch, token, head
  float* lse;
  const int32_t* cu_q;  // NULL => dense
  const int32_t* cu_k;
  const SchedItem* items;  // packed mode: the scheduler's work list; CTA x runs entry x / heads for head x % heads
  int32_t batch, heads;
  int32_t lq, lk;  // dense lengths (max_seqlen in varlen mode)
  int64_t total_q, total_k;
  float scale_log2;  // scale * log2(e)
  int32_t* status;
};

constexpr int kTile = 128;  // rows per Q tile and per K/V tile
constexpr int kHeadDim = 64;
constexpr int kTileBytes = kTile * kHeadDim * 2;  // 16 KB

constexpr int kFwdThreads = 192;
constexpr int kFwdQRows = kTile;  // query rows per CTA
constexpr int kFwdStages = 2;
constexpr int kFwdSmemBytes = (1 + 2 * kFwdStages) * kTileBytes + 1024;
constexpr int kFwdTmemCols = 256;
constexpr float kRescaleThreshold = 8.f;  // log2 units
// Build-time switch: 1 = skip the row max after the first key tile (see the softmax warps); 0 takes
// the row max of every tile.
#ifndef NB_FWD_LAZY_MAX
#define NB_FWD_LAZY_MAX 1
#endif
constexpr float kLazySumLimit = 16384.f;

// Row maximum of 32 raw scores with two independent chains of 3-input max.
__device__ __forceinline__ void chunk_max(const uint32_t (&r)[32], float& mx0, float& mx1) {
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    mx0 = max3(mx0, __uint_as_float(r[j]), __uint_as_float(r[j + 1]));
    mx1 = max3(mx1, __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
  }
}

// Columns >= valid (only on a ragged last key tile) count as -inf.
__device__ __forceinline__ void chunk_mask(uint32_t (&r)[32], int col0, int valid) {
#pragma unroll
  for (int j = 0; j < 32; ++j)
    if (col0 + j >= valid) r[j] = 0xff800000u;
}

// P = exp2(s*scale_log2 - m_scaled) for 32 scores, packed to bf16; four partial row sums kept as
// two packed fp32 pairs. Packed f32x2 arithmetic halves the issue slots of the FMA and the add.
__device__ __forceinline__ void chunk_exp(const uint32_t (&r)[32], uint64_t scale2, uint64_t neg_m2,
                                          uint64_t& l01, uint64_t& l23, uint32_t (&pk)[16]) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    float x0, x1;
    unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])), scale2, neg_m2),
                 x0, x1);
    float p0, p1;
    // One pair in eight takes the polynomial on the FMA pipe; the other exponentials keep the MUFU
    // unit (16 results per clock per SM) as busy as the rest of the loop allows.
    if ((j & 7) == 7) unpack_f32x2(exp2_poly_f32x2(pack_f32x2(x0, x1)), p0, p1);
    else p0 = fast_exp2(x0), p1 = fast_exp2(x1);
    if (j & 1) l23 = add_f32x2(l23, pack_f32x2(p0, p1)); else l01 = add_f32x2(l01, pack_f32x2(p0, p1));
    pk[j] = pack_bf16(p0, p1);
  }
}

__global__ void __launch_bounds__(kFwdThreads, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  // q_full, k_full[2], v_full[2], kv_empty[2], s_full, s_free, p_full, pv_done
  __shared__ __align__(8) uint64_t bars[11];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  // What only the epilogue needs of the work item (re-read there, so that the softmax warps do not
  // hold it in registers through their loop): q_begin, lq, head, sequence, first row of the tile.
  __shared__ int epi_meta[5];

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;

  // Everything this kernel reads may come from the kernel right before it in the stream.
  pdl_wait();
  pdl_launch_dependents();

  int q_begin = 0, k_begin = 0, lq = p.lq, lk = p.lk, bcoord = b;
  if (p.cu_q != nullptr) {
    // One read tells the CTA everything about its item (the sequence index `batch` stands for the
    // rows past the last sequence: queries without keys, which get O = 0 and LSE = -inf).
    const SchedItem item = sched_load(p.items, blockIdx.x / uint32_t(p.heads));
    if (item.seq < 0) return;
    h = blockIdx.x % uint32_t(p.heads);
    b = item.seq;
    qt = item.tile;
    q_begin = item.own_begin;
    lq = item.own_len;
    k_begin = item.other_begin;
    lk = item.other_len;
    bcoord = 0;
  }
  const int q_row0 = qt * kTile;
  if (q_row0 >= lq) return;  // this tile lies past the end of the sequence
  const int n_kv = (lk + kTile - 1) / kTile;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = smem_base;
  auto sK = [&](int s) { return smem_base + (1 + 2 * s) * kTileBytes; };
  auto sV = [&](int s) { return smem_base + (2 + 2 * s) * kTileBytes; };
  const uint32_t bar0 = smem_u32(&bars[0]);
  const uint32_t bar_q_full = bar0;
  auto bar_k_full = [&](int s) { return bar0 + 8 * (1 + s); };
  auto bar_v_full = [&](int s) { return bar0 + 8 * (3 + s); };
  auto bar_kv_empty = [&](int s) { return bar0 + 8 * (5 + s); };
  const uint32_t bar_s_full = bar0 + 8 * 7, bar_s_free = bar0 + 8 * 8;
  const uint32_t bar_p_full = bar0 + 8 * 9, bar_pv_done = bar0 + 8 * 10;

  // The producer's own thread initialises the barriers, so it can start the first loads (Q and both
  // K/V stages) at once; the other threads meet the barriers only after the __syncthreads below.
  if (tid == 5 * 32) {
    epi_meta[0] = q_begin, epi_meta[1] = lq, epi_meta[2] = h, epi_meta[3] = b, epi_meta[4] = q_row0;
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    abort_flag = 0;
    for (int i = 0; i < 11; ++i) mbar_init(bar0 + 8 * i, (i == 8 || i == 9) ? 4 : 1);  // s_free, p_full: per warp
    fence_mbar_init();
    if (n_kv > 0) {
      mbar_arrive_expect_tx(bar_q_full, kTileBytes);
      tma_load_4d(sQ, &tmap_q, bar_q_full, 0, q_begin + q_row0, h, bcoord);
      for (int i = 0; i < kFwdStages && i < n_kv; ++i) {
        mbar_arrive_expect_tx(bar_k_full(i), kTileBytes);
        tma_load_4d(sK(i), &tmap_k, bar_k_full(i), 0, k_begin + i * kTile, h, bcoord);
        mbar_arrive_expect_tx(bar_v_full(i), kTileBytes);
        tma_load_4d(sV(i), &tmap_v, bar_v_full(i), 0, k_begin + i * kTile, h, bcoord);
      }
    }
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(&tmem_base_slot), kFwdTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t tm_s = tmem_base, tm_o = tmem_base + 128, tm_p = tmem_base + 192;

  if (n_kv > 0) {
    if (warp == 5) {
      // ---------------- TMA producer ----------------
      if (elect_one()) {
        for (int i = kFwdStages; i < n_kv; ++i) {  // the first tiles were requested at start-up
          const int s = i % kFwdStages;
          mbar_wait(bar_kv_empty(s), ((i / kFwdStages) - 1) & 1, &abort_flag, p.status);
          mbar_arrive_expect_tx(bar_k_full(s), kTileBytes);
          tma_load_4d(sK(s), &tmap_k, bar_k_full(s), 0, k_begin + i * kTile, h, bcoord);
          mbar_arrive_expect_tx(bar_v_full(s), kTileBytes);
          tma_load_4d(sV(s), &tmap_v, bar_v_full(s), 0, k_begin + i * kTile, h, bcoord);
        }
      }
    } else if (warp == 4) {
      // ---------------- MMA issuer ----------------
      if (elect_one()) {
        constexpr uint32_t kIdescS = make_idesc(128, 128, 0, 0);
        constexpr uint32_t kIdescPV = make_idesc(128, 64, 0, 1);
        const uint64_t qd = make_sdesc(sQ, 16, 1024);
        // Live key columns of the last tile, rounded up to the MMA's granularity of 16.
        const int last_n16 = (lk - (n_kv - 1) * kTile + 15) & ~15;
        auto issue_s = [&](int i) {
          const uint64_t kd = make_sdesc(sK(i % kFwdStages), 16, 1024);
          const uint32_t idesc = i == n_kv - 1 ? idesc_with_n(kIdescS, last_n16) : kIdescS;
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_ss(tm_s, qd + 2 * k, kd + 2 * k, idesc, k > 0);
          tc_commit(bar_s_full);
        };
        mbar_wait(bar_q_full, 0, &abort_flag, p.status);
        mbar_wait(bar_k_full(0), 0, &abort_flag, p.status);
        tc_fence_after();
        issue_s(0);
        for (int i = 0; i < n_kv; ++i) {
          const int s = i % kFwdStages;
          if (i + 1 < n_kv) {
            // Next scores as soon as the softmax warps hold S(i) in registers.
            mbar_wait(bar_s_free, i & 1, &abort_flag, p.status);
            mbar_wait(bar_k_full((i + 1) % kFwdStages), ((i + 1) / kFwdStages) & 1, &abort_flag, p.status);
            tc_fence_after();
            issue_s(i + 1);
          }
          mbar_wait(bar_p_full, i & 1, &abort_flag, p.status);
          mbar_wait(bar_v_full(s), (i / kFwdStages) & 1, &abort_flag, p.status);
          tc_fence_after();
          const uint64_t vd = make_sdesc(sV(s), 1024, 1024);
          if (i + 1 < n_kv || last_n16 == kTile) {
#pragma unroll
            for (int k = 0; k < 8; ++k) mma_ts(tm_o, tm_p + 8 * k, vd + 128 * k, kIdescPV, (i > 0) || (k > 0));
          } else {
            // Ragged last tile: only the K steps that cover live keys (the softmax warps have cleared
            // the rows between the last live key and the next multiple of 16).
#pragma unroll 1
            for (int k = 0; k < (last_n16 >> 4); ++k)
              mma_ts(tm_o, tm_p + 8 * k, vd + 128 * k, kIdescPV, (i > 0) || (k > 0));
          }
          tc_commit(bar_pv_done);
          tc_commit(bar_kv_empty(s));
        }
      }
    } else {
      // ---------------- softmax warpgroup ----------------
      const uint32_t lane_off = uint32_t(warp * 32) << 16;
      const uint32_t s_addr = tm_s + lane_off, p_addr = tm_p + lane_off, o_addr = tm_o + lane_off;
      const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
      float m_run = -INFINITY;  // raw (unscaled) running max used as the exp offset
      float l_run = 0.f;
      // One key tile. kRagged is true only for a last tile with fewer than 128 live keys: then only
      // the live 32-column chunks are loaded, exponentiated and stored (the trimmed MMAs neither
      // write the other score columns nor read the other P columns).
      auto softmax_tile = [&](const int i, auto ragged_tag) __attribute__((always_inline)) {
        constexpr bool kRagged = decltype(ragged_tag)::value;
        const int valid = kRagged ? lk - i * kTile : kTile;
        const int nchunk = kRagged ? (valid + 31) >> 5 : 4;  // live 32-column chunks
        mbar_wait(bar_s_full, i & 1, &abort_flag, p.status);
        tc_fence_after();
        uint32_t ra[32], rb[32], rc[32], rd[32], pk[16];
        tmem_ld32(s_addr, ra);
        if (nchunk > 1) tmem_ld32(s_addr + 32, rb);
        if (nchunk > 2) tmem_ld32(s_addr + 64, rc);
        if (nchunk > 3) tmem_ld32(s_addr + 96, rd);
        tmem_wait_ld();
        // The whole row is in registers: the score buffer may be overwritten.
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_s_free);
        if (kRagged) {
          chunk_mask(ra, 0, valid);
          chunk_mask(rb, 32, valid);
          chunk_mask(rc, 64, valid);
          chunk_mask(rd, 96, valid);
        }
#if NB_FWD_LAZY_MAX
        // After the first tile the row max is not computed at all: P is evaluated against the
        // running offset m_run, and only if some row's tile sum shows that an exponent ran far
        // above the offset (or overflowed) is the tile redone with the true max.
        bool with_max = i == 0;
#else
        constexpr bool with_max = true;
#endif
        bool waited = i == 0;
        float tile_sum;
        for (;;) {
          if (with_max) {
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
            chunk_max(ra, mx0, mx1);
            if (nchunk > 1) chunk_max(rb, mx2, mx3);
            if (nchunk > 2) chunk_max(rc, mx0, mx1);
            if (nchunk > 3) chunk_max(rd, mx2, mx3);
            const float m_new = fmaxf(m_run, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)));
            const bool need = (m_new - m_run) * p.scale_log2 > kRescaleThreshold;
            // P and O of the previous tile must have been consumed / completed first.
            if (!waited) {
              mbar_wait(bar_pv_done, (i - 1) & 1, &abort_flag, p.status);
              tc_fence_after();
              waited = true;
            }
            if (__any_sync(0xffffffffu, need)) {
              // Rare after the first tile: refresh the max of the rows that need it, rescale their
              // running sum and their row of the O accumulator.
              const float alpha = need ? fast_exp2((m_run - m_new) * p.scale_log2) : 1.f;
              if (need) m_run = m_new;
              l_run *= alpha;
              if (i > 0) {
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {
                  uint32_t o[32];
                  tmem_ld32(o_addr + c * 32, o);
                  tmem_wait_ld();
#pragma unroll
                  for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
                  tmem_st32(o_addr + c * 32, o);
                }
              }
            }
          } else if (!waited) {
            mbar_wait(bar_pv_done, (i - 1) & 1, &abort_flag, p.status);
            tc_fence_after();
            waited = true;
          }
          const float nm = -m_run * p.scale_log2;
          const uint64_t neg_m2 = pack_f32x2(nm, nm);
          uint64_t l01 = 0ull, l23 = 0ull;
          chunk_exp(ra, scale2, neg_m2, l01, l23, pk);
          tmem_st16(p_addr, pk);
          if (nchunk > 1) {
            chunk_exp(rb, scale2, neg_m2, l01, l23, pk);
            tmem_st16(p_addr + 16, pk);
          }
          if (nchunk > 2) {
            chunk_exp(rc, scale2, neg_m2, l01, l23, pk);
            tmem_st16(p_addr + 32, pk);
          }
          if (nchunk > 3) {
            chunk_exp(rd, scale2, neg_m2, l01, l23, pk);
            tmem_st16(p_addr + 48, pk);
          }
          float a0, a1, a2, a3;
          unpack_f32x2(l01, a0, a1);
          unpack_f32x2(l23, a2, a3);
          tile_sum = (a0 + a1) + (a2 + a3);
#if NB_FWD_LAZY_MAX
          // A tile sum above 2^14 (or Inf / NaN) means some exponent was far above the offset.
          if (!with_max && __any_sync(0xffffffffu, !(tile_sum <= kLazySumLimit))) {
            with_max = true;
            tmem_wait_st();  // the P columns are rewritten
            continue;
          }
#endif
          break;
        }
        l_run += tile_sum;
        if (kRagged && warp == 0 && p.cu_q != nullptr) {
          // Packed mode: V rows [valid, valid rounded up to 16) of this tile belong to the next
          // sequence. Their P columns are 0, but 0 x Inf would still poison this sequence, so the rows
          // are cleared before P is handed to the MMA warp. (The swizzle only permutes 16-byte chunks
          // inside a 128-byte row: whole rows are contiguous.)
          const int st = i % kFwdStages;
          mbar_wait(bar_v_full(st), (i / kFwdStages) & 1, &abort_flag, p.status);
          uint8_t* v_rows = smem_raw + (sV(st) - smem_u32(smem_raw));
          for (int c = valid * 8 + lane; c < ((valid + 15) & ~15) * 8; c += 32)
            reinterpret_cast<uint4*>(v_rows)[c] = make_uint4(0, 0, 0, 0);
          fence_proxy_async_smem();
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p_full);
      };
      const bool last_ragged = lk - (n_kv - 1) * kTile < kTile;
      const int n_full = last_ragged ? n_kv - 1 : n_kv;
      for (int i = 0; i < n_full; ++i) softmax_tile(i, std::false_type{});
      if (last_ragged) softmax_tile(n_kv - 1, std::true_type{});

      // Epilogue: O / l -> bf16, natural-log LSE.
      mbar_wait(bar_pv_done, (n_kv - 1) & 1, &abort_flag, p.status);
      tc_fence_after();
      const volatile int* meta = epi_meta;
      const int e_q_begin = meta[0], e_lq = meta[1], e_h = meta[2], e_b = meta[3], e_row0 = meta[4];
      const int e_bcoord = p.cu_q != nullptr ? 0 : e_b;
      const int row = e_row0 + tid;
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      // Each warp turns its 32 rows into bf16 in a 4 KB scratch area (the Q tile, dead once the
      // last S MMA has run -- which the completed P V MMA implies) and writes them out with eight
      // lanes per 128-byte row, so the stores are whole lines; a warp only reads what it wrote.
      uint8_t* scratch = smem_raw + (smem_base - smem_u32(smem_raw)) + warp * 4096;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t o[32];
        tmem_ld32(o_addr + c * 32, o);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(o[8 * j + 0]) * inv_l, __uint_as_float(o[8 * j + 1]) * inv_l);
          v.y = pack_bf16(__uint_as_float(o[8 * j + 2]) * inv_l, __uint_as_float(o[8 * j + 3]) * inv_l);
          v.z = pack_bf16(__uint_as_float(o[8 * j + 4]) * inv_l, __uint_as_float(o[8 * j + 5]) * inv_l);
          v.w = pack_bf16(__uint_as_float(o[8 * j + 6]) * inv_l, __uint_as_float(o[8 * j + 7]) * inv_l);
          *reinterpret_cast<uint4*>(scratch + swz128(lane, c * 4 + j)) = v;
        }
      }
      __syncwarp();
      __nv_bfloat16* out_base = p.o + int64_t(e_bcoord) * p.o_sb + int64_t(e_h) * p.o_sh;
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int rloc = it * 4 + (lane >> 3);
        const int orow = e_row0 + warp * 32 + rloc;
        const uint4 v = *reinterpret_cast<const uint4*>(scratch + swz128(rloc, lane & 7));
        if (orow < e_lq) *reinterpret_cast<uint4*>(out_base + int64_t(e_q_begin + orow) * p.o_st + (lane & 7) * 8) = v;
      }
      if (row < e_lq) {
        const float lse = (m_run * p.scale_log2 + log2f(l_run)) * 0.6931471805599453f;
        const int64_t lse_idx = p.cu_q != nullptr ? int64_t(e_h) * p.total_q + e_q_begin + row
                                                  : (int64_t(e_b) * p.heads + e_h) * p.lq + row;
        p.lse[lse_idx] = lse;
      }
    }
  } else if (warp < 4) {
    // No keys at all: the output is defined as zero and the LSE as -inf.
    const int row = q_row0 + tid;
    if (row < lq) {
      __nv_bfloat16* optr = p.o + int64_t(bcoord) * p.o_sb + int64_t(q_begin + row) * p.o_st + int64_t(h) * p.o_sh;
      for (int c = 0; c < 8; ++c) reinterpret_cast<uint4*>(optr)[c] = make_uint4(0, 0, 0, 0);
      const int64_t lse_idx = p.cu_q != nullptr ? int64_t(h) * p.total_q + q_begin + row
                                                : (int64_t(b) * p.heads + h) * p.lq + row;
      p.lse[lse_idx] = -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kFwdTmemCols);
  }
}

}  // namespace nb
