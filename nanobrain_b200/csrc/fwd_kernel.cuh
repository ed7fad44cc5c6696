// Forward attention kernel: O = softmax(Q K^T * scale) V, bf16 in / bf16 out, fp32 softmax
// statistics and accumulation, head_dim 64, non-causal. One CTA owns one 128-row query tile of
// one (sequence, head) and walks the sequence's keys in 128-row tiles:
//
//   TMA (SWIZZLE_128B)  : Q tile once, K/V tiles double-buffered in shared memory
//   tcgen05.mma  S      : S[128x128] = Q K^T        (A, B from shared memory, D in tensor memory)
//   softmax             : thread r owns row r of S (tensor-memory lane r); online max / sum,
//                         exp2 with scale*log2(e) folded into one FFMA, P rounded to bf16 and
//                         written back to tensor memory
//   tcgen05.mma  PV     : Otile[128x64] = P V       (A = P from tensor memory, B = V from shared
//                         memory, MN-major)
//   accumulate          : O = O*alpha + Otile in registers
//
// Two CTAs fit on one SM (80 KB shared memory, 256 tensor-memory columns each), so one CTA's
// softmax overlaps the other's MMAs; inside a CTA the S MMA of tile i+1 is issued before the
// O accumulation of tile i.
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

constexpr int kFwdThreads = 128;
constexpr int kTile = 128;              // rows per Q tile and per K/V tile
constexpr int kHeadDim = 64;
constexpr int kTileBytes = kTile * kHeadDim * 2;  // 16 KB
constexpr int kFwdSmemBytes = 5 * kTileBytes + 1024;  // Q + 2x(K,V) + alignment slack
constexpr int kFwdTmemCols = 256;       // S: 0..127, P: 128..191, Otile: 192..255

__global__ void __launch_bounds__(kFwdThreads)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[5];  // q, kv0, kv1, s, o
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;

  // Sequence geometry. In varlen mode tokens are packed and the batch coordinate is 0.
  int q_begin = 0, k_begin = 0, lq = p.lq, lk = p.lk, bcoord = b;
  if (p.cu_q != nullptr) {
    q_begin = p.cu_q[b];
    lq = p.cu_q[b + 1] - q_begin;
    k_begin = p.cu_k[b];
    lk = p.cu_k[b + 1] - k_begin;
    bcoord = 0;
  }
  const int q_row0 = qt * kTile;
  if (q_row0 >= lq) return;  // this tile lies past the end of the sequence
  const int n_kv = (lk + kTile - 1) / kTile;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = smem_base;
  const uint32_t sK[2] = {smem_base + 1 * kTileBytes, smem_base + 3 * kTileBytes};
  const uint32_t sV[2] = {smem_base + 2 * kTileBytes, smem_base + 4 * kTileBytes};
  const uint32_t bar_q = smem_u32(&bars[0]);
  const uint32_t bar_kv[2] = {smem_u32(&bars[1]), smem_u32(&bars[2])};
  const uint32_t bar_s = smem_u32(&bars[3]);
  const uint32_t bar_o = smem_u32(&bars[4]);

  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < 5; ++i) mbar_init(smem_u32(&bars[i]), 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_base_slot), kFwdTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t tm_s = tmem_base;
  const uint32_t tm_p = tmem_base + 128;
  const uint32_t tm_o = tmem_base + 192;
  const uint32_t lane_off = uint32_t(warp * 32) << 16;

  constexpr uint32_t kIdescS = make_idesc(128, 128, 0, 0);
  constexpr uint32_t kIdescPV = make_idesc(128, 64, 0, 1);

  float o_acc[kHeadDim];
#pragma unroll
  for (int d = 0; d < kHeadDim; ++d) o_acc[d] = 0.f;
  float m_run = -INFINITY;  // running max of the raw (unscaled) scores
  float l_run = 0.f;        // running sum of exp

  if (n_kv > 0) {
    if (tid == 0) {
      mbar_arrive_expect_tx(bar_q, kTileBytes);
      tma_load_4d(sQ, &tmap_q, bar_q, 0, q_begin + q_row0, h, bcoord);
      mbar_arrive_expect_tx(bar_kv[0], 2 * kTileBytes);
      tma_load_4d(sK[0], &tmap_k, bar_kv[0], 0, k_begin, h, bcoord);
      tma_load_4d(sV[0], &tmap_v, bar_kv[0], 0, k_begin, h, bcoord);
      // First S = Q K^T.
      mbar_wait(bar_q, 0, &abort_flag, p.status);
      mbar_wait(bar_kv[0], 0, &abort_flag, p.status);
      tc_fence_after();
      const uint64_t a = make_sdesc(sQ, 16, 1024), bd = make_sdesc(sK[0], 16, 1024);
#pragma unroll
      for (int k = 0; k < 4; ++k) mma_ss(tm_s, a + 2 * k, bd + 2 * k, kIdescS, k > 0);
      tc_commit(bar_s);
    }
    __syncwarp();

    for (int i = 0; i < n_kv; ++i) {
      const int st = i & 1;
      // Prefetch the next K/V tile into the other stage (its last readers, the S MMA of tile
      // i-1... and the PV MMA of tile i-1, completed before the end of the previous iteration).
      if (tid == 0 && i + 1 < n_kv) {
        mbar_arrive_expect_tx(bar_kv[st ^ 1], 2 * kTileBytes);
        tma_load_4d(sK[st ^ 1], &tmap_k, bar_kv[st ^ 1], 0, k_begin + (i + 1) * kTile, h, bcoord);
        tma_load_4d(sV[st ^ 1], &tmap_v, bar_kv[st ^ 1], 0, k_begin + (i + 1) * kTile, h, bcoord);
      }
      __syncwarp();

      mbar_wait(bar_s, i & 1, &abort_flag, p.status);
      tc_fence_after();

      // Pass 1: row maximum over the valid key columns of this tile.
      const int valid = lk - i * kTile;  // columns >= valid are padding
      float m_tile = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tm_s + lane_off + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float s = __uint_as_float(r[j]);
          if (c * 32 + j >= valid) s = -INFINITY;
          m_tile = fmaxf(m_tile, s);
        }
      }
      const float m_new = fmaxf(m_run, m_tile);
      const float alpha = fast_exp2((m_run - m_new) * p.scale_log2);
      const float m_scaled = m_new * p.scale_log2;

      // Pass 2: P = exp2(S*scale_log2 - m), row sum, bf16 P into tensor memory.
      float l_tile = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tm_s + lane_off + c * 32, r);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float p0 = fast_exp2(fmaf(__uint_as_float(r[j]), p.scale_log2, -m_scaled));
          float p1 = fast_exp2(fmaf(__uint_as_float(r[j + 1]), p.scale_log2, -m_scaled));
          if (c * 32 + j >= valid) p0 = 0.f;
          if (c * 32 + j + 1 >= valid) p1 = 0.f;
          l_tile += p0 + p1;
          pk[j >> 1] = pack_bf16(p0, p1);
        }
        tmem_st16(tm_p + lane_off + c * 16, pk);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncthreads();  // P complete, S fully consumed, previous Otile fully consumed

      if (tid == 0) {
        tc_fence_after();
        const uint64_t vd = make_sdesc(sV[st], 1024, 1024);
#pragma unroll
        for (int k = 0; k < 8; ++k) mma_ts(tm_o, tm_p + 8 * k, vd + 128 * k, kIdescPV, k > 0);
        tc_commit(bar_o);
        if (i + 1 < n_kv) {
          mbar_wait(bar_kv[st ^ 1], ((i + 1) >> 1) & 1, &abort_flag, p.status);
          tc_fence_after();
          const uint64_t a = make_sdesc(sQ, 16, 1024), bd = make_sdesc(sK[st ^ 1], 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k) mma_ss(tm_s, a + 2 * k, bd + 2 * k, kIdescS, k > 0);
          tc_commit(bar_s);
        }
      }
      __syncwarp();

      // Rescale the running output while the PV MMA runs.
      l_run = l_run * alpha + l_tile;
      m_run = m_new;
#pragma unroll
      for (int d = 0; d < kHeadDim; ++d) o_acc[d] *= alpha;

      mbar_wait(bar_o, i & 1, &abort_flag, p.status);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32(tm_o + lane_off + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) o_acc[c * 32 + j] += __uint_as_float(r[j]);
      }
      tc_fence_before();
    }
  }

  // Epilogue: normalise, write O (bf16) and the natural-log LSE.
  const int row = q_row0 + tid;
  if (row < lq) {
    const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
    __nv_bfloat16* optr = p.o + int64_t(bcoord) * p.o_sb + int64_t(q_begin + row) * p.o_st + int64_t(h) * p.o_sh;
    uint4* o4 = reinterpret_cast<uint4*>(optr);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint4 v;
      v.x = pack_bf16(o_acc[c * 8 + 0] * inv_l, o_acc[c * 8 + 1] * inv_l);
      v.y = pack_bf16(o_acc[c * 8 + 2] * inv_l, o_acc[c * 8 + 3] * inv_l);
      v.z = pack_bf16(o_acc[c * 8 + 4] * inv_l, o_acc[c * 8 + 5] * inv_l);
      v.w = pack_bf16(o_acc[c * 8 + 6] * inv_l, o_acc[c * 8 + 7] * inv_l);
      o4[c] = v;
    }
    const float lse = l_run > 0.f ? (m_run * p.scale_log2 + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
    const int64_t lse_idx = p.cu_q != nullptr ? int64_t(h) * p.total_q + q_begin + row
                                              : (int64_t(b) * p.heads + h) * p.lq + row;
    p.lse[lse_idx] = lse;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kFwdTmemCols);
  }
}

}  // namespace nb
