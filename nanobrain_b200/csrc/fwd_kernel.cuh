// Forward attention kernel: O = softmax(Q K^T * scale) V, bf16 in / bf16 out, fp32 softmax
// statistics and accumulation, head_dim 64, non-causal.
//
// One CTA owns up to two 128-row query tiles (256 consecutive rows) of one (sequence, head) and
// walks the sequence's keys in 128-row tiles. Warp roles (320 threads):
//
//   warps 0-3, 4-7 : softmax warpgroup for query tile 0 / tile 1. Thread r owns row r of its tile
//                    (tensor-memory lane r). Per key tile it streams the fp32 score row out of
//                    tensor memory in 32-column chunks, computes P = exp2(S*scale_log2 - m) against
//                    the CURRENT running max while tracking the tile's own max, and writes P as
//                    bf16 into a separate tensor-memory buffer. Only if some row's max grew by
//                    more than 2^8 (rare after the first tile) does the warp refresh the max,
//                    rescale its rows of the O accumulator and redo the tile's exponentials.
//   warp 8         : one elected thread issues every tcgen05.mma: S_t = Q_t K^T (both operands from
//                    shared memory) and O_t += P_t V (P from tensor memory, V from shared memory,
//                    MN-major). When tile t's P is ready it first issues S_t of the next key tile,
//                    then P_t V, so the softmax warps get their next scores a single MMA later.
//   warp 9         : one elected thread drives TMA: both Q tiles once, then K and V tiles through
//                    a three-stage ring (SWIZZLE_128B, no multicast).
//
// Tensor memory (all 512 columns): S0 [0,128) S1 [128,256) O0 [256,320) O1 [320,384)
// P0 [384,448) P1 [448,512).
#pragma once

#include "ptx.cuh"

namespace nb {

struct FwdParams {
  __nv_bfloat16* o;
  int64_t o_sb, o_st, o_sh;  // element strides of O: batch, token, head
  float* lse;
  const int32_t* cu_q;  // NULL => dense
  const int32_t* cu_k;
  int32_t batch, heads;
  int32_t lq, lk;  // dense lengths (max_seqlen in varlen mode)
  int64_t total_q;
  float scale_log2;  // scale * log2(e)
  int32_t* status;
};

constexpr int kTile = 128;  // rows per Q tile and per K/V tile
constexpr int kHeadDim = 64;
constexpr int kTileBytes = kTile * kHeadDim * 2;  // 16 KB

constexpr int kFwdThreads = 320;
constexpr int kFwdQRows = 2 * kTile;  // query rows per CTA
constexpr int kFwdStages = 3;
constexpr int kFwdSmemBytes = (2 + 2 * kFwdStages) * kTileBytes + 1024;
constexpr int kFwdTmemCols = 512;
constexpr float kRescaleThreshold = 8.f;  // log2 units

// Running statistics of one score row while a key tile streams through.
struct RowStats {
  uint64_t l01, l23;  // four partial row sums as two packed fp32 pairs
  float mx0, mx1;     // two partial row maxima of the raw scores
  __device__ __forceinline__ void reset() {
    l01 = l23 = 0ull;
    mx0 = mx1 = -INFINITY;
  }
  __device__ __forceinline__ float sum() const {
    float a, b, c, d;
    unpack_f32x2(l01, a, b);
    unpack_f32x2(l23, c, d);
    return (a + b) + (c + d);
  }
  __device__ __forceinline__ float max() const { return fmaxf(mx0, mx1); }
};

// One 32-column chunk of a score row: P = exp2(s*scale_log2 - m_scaled) packed to bf16, row sums
// and row maxima accumulated on the side. Columns >= valid (only on a ragged last key tile)
// count as -inf. Packed f32x2 arithmetic and the 3-input max halve the issue slots.
__device__ __forceinline__ void softmax_chunk(uint32_t (&r)[32], int col0, int valid, uint64_t scale2,
                                              uint64_t neg_m2, RowStats& st, uint32_t (&pk)[16]) {
  if (valid < kTile) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j >= valid) r[j] = 0xff800000u;  // -inf
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float s0 = __uint_as_float(r[2 * j]), s1 = __uint_as_float(r[2 * j + 1]);
    if (j & 1) st.mx1 = max3(st.mx1, s0, s1); else st.mx0 = max3(st.mx0, s0, s1);
    float x0, x1;
    unpack_f32x2(fma_f32x2(pack_f32x2(s0, s1), scale2, neg_m2), x0, x1);
    const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
    if (j & 1) st.l23 = add_f32x2(st.l23, pack_f32x2(p0, p1)); else st.l01 = add_f32x2(st.l01, pack_f32x2(p0, p1));
    pk[j] = pack_bf16(p0, p1);
  }
}

__device__ __forceinline__ float chunk_max(const uint32_t (&r)[32], int col0, int valid) {
  float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
  for (int j = 0; j < 32; j += 2) {
    if (col0 + j < valid) mx0 = fmaxf(mx0, __uint_as_float(r[j]));
    if (col0 + j + 1 < valid) mx1 = fmaxf(mx1, __uint_as_float(r[j + 1]));
  }
  return fmaxf(mx0, mx1);
}

__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  // q_full, k_full[3], v_full[3], kv_empty[3], s_full[2], p_full[2], pv_done[2]
  __shared__ __align__(8) uint64_t bars[16];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int qp = blockIdx.x, h = blockIdx.y, b = blockIdx.z;

  int q_begin = 0, k_begin = 0, lq = p.lq, lk = p.lk, bcoord = b;
  if (p.cu_q != nullptr) {
    q_begin = p.cu_q[b];
    lq = p.cu_q[b + 1] - q_begin;
    k_begin = p.cu_k[b];
    lk = p.cu_k[b + 1] - k_begin;
    bcoord = 0;
  }
  const int q_row0 = qp * kFwdQRows;
  if (q_row0 >= lq) return;  // whole CTA lies past the end of the sequence
  const int n_tiles = (q_row0 + kTile < lq) ? 2 : 1;
  const int n_kv = (lk + kTile - 1) / kTile;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  auto sQ = [&](int t) { return smem_base + t * kTileBytes; };
  auto sK = [&](int s) { return smem_base + (2 + 2 * s) * kTileBytes; };
  auto sV = [&](int s) { return smem_base + (3 + 2 * s) * kTileBytes; };
  const uint32_t bar0 = smem_u32(&bars[0]);
  auto bar_q_full = [&]() { return bar0; };
  auto bar_k_full = [&](int s) { return bar0 + 8 * (1 + s); };
  auto bar_v_full = [&](int s) { return bar0 + 8 * (4 + s); };
  auto bar_kv_empty = [&](int s) { return bar0 + 8 * (7 + s); };
  auto bar_s_full = [&](int t) { return bar0 + 8 * (10 + t); };
  auto bar_p_full = [&](int t) { return bar0 + 8 * (12 + t); };
  auto bar_pv_done = [&](int t) { return bar0 + 8 * (14 + t); };

  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < 16; ++i) mbar_init(bar0 + 8 * i, (i == 12 || i == 13) ? kTile : 1);
    fence_mbar_init();
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(&tmem_base_slot), kFwdTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  auto tm_s = [&](int t) { return tmem_base + t * 128; };
  auto tm_o = [&](int t) { return tmem_base + 256 + t * 64; };
  auto tm_p = [&](int t) { return tmem_base + 384 + t * 64; };

  if (n_kv > 0) {
    if (warp == 9) {
      // ---------------- TMA producer ----------------
      if (elect_one()) {
        tma_prefetch_desc(&tmap_q);
        tma_prefetch_desc(&tmap_k);
        tma_prefetch_desc(&tmap_v);
        mbar_arrive_expect_tx(bar_q_full(), n_tiles * kTileBytes);
        for (int t = 0; t < n_tiles; ++t)
          tma_load_4d(sQ(t), &tmap_q, bar_q_full(), 0, q_begin + q_row0 + t * kTile, h, bcoord);
        for (int i = 0; i < n_kv; ++i) {
          const int s = i % kFwdStages;
          if (i >= kFwdStages) mbar_wait(bar_kv_empty(s), ((i / kFwdStages) - 1) & 1, &abort_flag, p.status);
          mbar_arrive_expect_tx(bar_k_full(s), kTileBytes);
          tma_load_4d(sK(s), &tmap_k, bar_k_full(s), 0, k_begin + i * kTile, h, bcoord);
          mbar_arrive_expect_tx(bar_v_full(s), kTileBytes);
          tma_load_4d(sV(s), &tmap_v, bar_v_full(s), 0, k_begin + i * kTile, h, bcoord);
        }
      }
    } else if (warp == 8) {
      // ---------------- MMA issuer ----------------
      if (elect_one()) {
        constexpr uint32_t kIdescS = make_idesc(128, 128, 0, 0);
        constexpr uint32_t kIdescPV = make_idesc(128, 64, 0, 1);
        auto issue_s = [&](int t, int s) {
          const uint64_t a = make_sdesc(sQ(t), 16, 1024), bd = make_sdesc(sK(s), 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_ss(tm_s(t), a + 2 * k, bd + 2 * k, kIdescS, k > 0);
          tc_commit(bar_s_full(t));
        };
        mbar_wait(bar_q_full(), 0, &abort_flag, p.status);
        mbar_wait(bar_k_full(0), 0, &abort_flag, p.status);
        tc_fence_after();
        for (int t = 0; t < n_tiles; ++t) issue_s(t, 0);
        for (int i = 0; i < n_kv; ++i) {
          const int s = i % kFwdStages;
          const int s1 = (i + 1) % kFwdStages;
          for (int t = 0; t < n_tiles; ++t) {
            mbar_wait(bar_p_full(t), i & 1, &abort_flag, p.status);
            tc_fence_after();
            if (i + 1 < n_kv) {
              // The softmax warps have consumed S_t(i): compute the next scores first.
              if (t == 0) {
                mbar_wait(bar_k_full(s1), ((i + 1) / kFwdStages) & 1, &abort_flag, p.status);
                tc_fence_after();
              }
              issue_s(t, s1);
            }
            if (t == 0) {
              mbar_wait(bar_v_full(s), (i / kFwdStages) & 1, &abort_flag, p.status);
              tc_fence_after();
            }
            const uint64_t vd = make_sdesc(sV(s), 1024, 1024);
#pragma unroll
            for (int k = 0; k < 8; ++k) mma_ts(tm_o(t), tm_p(t) + 8 * k, vd + 128 * k, kIdescPV, (i > 0) || (k > 0));
            tc_commit(bar_pv_done(t));
          }
          tc_commit(bar_kv_empty(s));
        }
      }
    } else {
      // ---------------- softmax warpgroups ----------------
      const int t = warp >> 2;
      if (t < n_tiles) {
        const int row_in_tile = tid & 127;
        const uint32_t lane_off = uint32_t((warp & 3) * 32) << 16;
        const uint32_t s_addr = tm_s(t) + lane_off, p_addr = tm_p(t) + lane_off, o_addr = tm_o(t) + lane_off;
        float m_run = -INFINITY;  // raw (unscaled) running max used as the exp offset
        float l_run = 0.f;
        for (int i = 0; i < n_kv; ++i) {
          const int valid = lk - i * kTile;  // >= kTile except on a ragged last tile
          mbar_wait(bar_s_full(t), i & 1, &abort_flag, p.status);
          tc_fence_after();
          uint32_t ra[32], rb[32], pk[16];
          RowStats st;
          st.reset();
          const uint64_t scale2 = pack_f32x2(p.scale_log2, p.scale_log2);
          bool redo;
          if (i == 0) {
            // First tile: there is no running max yet, find it before any exponential.
            float mt = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              tmem_ld32(s_addr + c * 32, ra);
              tmem_wait_ld();
              mt = fmaxf(mt, chunk_max(ra, c * 32, valid));
            }
            m_run = mt;
            redo = true;
          } else {
            // Stream the tile against the current max; track the tile's own max on the side.
            const float nm = -m_run * p.scale_log2;
            const uint64_t neg_m2 = pack_f32x2(nm, nm);
            tmem_ld32(s_addr, ra);
            tmem_ld32(s_addr + 32, rb);
            tmem_wait_ld();
            softmax_chunk(ra, 0, valid, scale2, neg_m2, st, pk);
            // P_t of the previous tile must have been consumed before it is overwritten.
            mbar_wait(bar_pv_done(t), (i - 1) & 1, &abort_flag, p.status);
            tc_fence_after();
            tmem_st16(p_addr, pk);
            tmem_ld32(s_addr + 64, ra);
            softmax_chunk(rb, 32, valid, scale2, neg_m2, st, pk);
            tmem_st16(p_addr + 16, pk);
            tmem_ld32(s_addr + 96, rb);
            tmem_wait_ld();
            softmax_chunk(ra, 64, valid, scale2, neg_m2, st, pk);
            tmem_st16(p_addr + 32, pk);
            softmax_chunk(rb, 96, valid, scale2, neg_m2, st, pk);
            tmem_st16(p_addr + 48, pk);
            const float m_new = fmaxf(m_run, st.max());
            const bool need = (m_new - m_run) * p.scale_log2 > kRescaleThreshold;
            redo = __any_sync(0xffffffffu, need);
            if (redo) {
              // Rare: refresh the max of the rows that need it and rescale their O accumulator
              // (quiescent: the previous P V has completed) and running sum.
              const float alpha = need ? fast_exp2((m_run - m_new) * p.scale_log2) : 1.f;
              if (need) m_run = m_new;
              l_run *= alpha;
#pragma unroll 1
              for (int c = 0; c < 2; ++c) {
                tmem_ld32(o_addr + c * 32, ra);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 32; ++j) ra[j] = __float_as_uint(__uint_as_float(ra[j]) * alpha);
                tmem_st32(o_addr + c * 32, ra);
              }
            }
          }
          if (redo) {
            const float nm = -m_run * p.scale_log2;
            const uint64_t neg_m2 = pack_f32x2(nm, nm);
            st.reset();
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              tmem_ld32(s_addr + c * 32, ra);
              tmem_wait_ld();
              softmax_chunk(ra, c * 32, valid, scale2, neg_m2, st, pk);
              tmem_st16(p_addr + c * 16, pk);
            }
          }
          l_run += st.sum();
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(bar_p_full(t));
        }

        // Epilogue: O / l -> bf16, natural-log LSE.
        mbar_wait(bar_pv_done(t), (n_kv - 1) & 1, &abort_flag, p.status);
        tc_fence_after();
        const int row = q_row0 + t * kTile + row_in_tile;
        const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* optr =
            p.o + int64_t(bcoord) * p.o_sb + int64_t(q_begin + row) * p.o_st + int64_t(h) * p.o_sh;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t o[32];
          tmem_ld32(o_addr + c * 32, o);
          tmem_wait_ld();
          if (row < lq) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(o[8 * j + 0]) * inv_l, __uint_as_float(o[8 * j + 1]) * inv_l);
              v.y = pack_bf16(__uint_as_float(o[8 * j + 2]) * inv_l, __uint_as_float(o[8 * j + 3]) * inv_l);
              v.z = pack_bf16(__uint_as_float(o[8 * j + 4]) * inv_l, __uint_as_float(o[8 * j + 5]) * inv_l);
              v.w = pack_bf16(__uint_as_float(o[8 * j + 6]) * inv_l, __uint_as_float(o[8 * j + 7]) * inv_l);
              reinterpret_cast<uint4*>(optr)[c * 4 + j] = v;
            }
          }
        }
        if (row < lq) {
          const float lse = (m_run * p.scale_log2 + log2f(l_run)) * 0.6931471805599453f;
          const int64_t lse_idx = p.cu_q != nullptr ? int64_t(h) * p.total_q + q_begin + row
                                                    : (int64_t(b) * p.heads + h) * p.lq + row;
          p.lse[lse_idx] = lse;
        }
      }
    }
  } else if (warp < 8) {
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
  if (warp == 8) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kFwdTmemCols);
  }
}

}  // namespace nb
