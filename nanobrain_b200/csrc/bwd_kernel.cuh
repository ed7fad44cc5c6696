// Backward attention kernels (head_dim 64, bf16 tensors, fp32 accumulation):
//
//   attn_bwd_prologue_kernel : delta[row] = sum_d dO[row,d] * O[row,d] (warp-shuffle row dot) and
//                              clears the fp32 dQ accumulator. HBM-bound.
//   attn_bwd_kernel          : one CTA owns one 128-row K/V tile of one (sequence, head) and walks
//                              the sequence's queries in 128-row tiles. Everything is computed
//                              transposed so that thread r owns key row r (tensor-memory lane r):
//                                S^T  = K Q^T                       (tcgen05, smem x smem)
//                                dP^T = V dO^T                      (tcgen05, smem x smem)
//                                P^T  = exp2(S^T*scale_log2 - lse)  (recomputed from the saved LSE)
//                                dS^T = P^T o (dP^T - delta)
//                                dV  += P^T dO                      (A = P^T from tensor memory)
//                                dK  += dS^T Q                      (A = dS^T from shared memory)
//                                dQ   = dS K                        (same dS bytes read MN-major)
//                              dQ tiles are added into the fp32 accumulator with vector atomics
//                              because every K/V tile of a sequence contributes to every dQ row.
//   attn_bwd_epilogue_kernel : dQ = bf16(scale * accumulator). HBM-bound.
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
  int32_t batch, heads;
  int32_t lq, lk;
  int64_t total_q;
  float scale, scale_log2;
  int32_t* status;
};

// ----------------------------------------------------------------------------------------
// Prologue: one quarter-warp (8 lanes x 16 bytes) per (token, head) row.
// ----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) attn_bwd_prologue_kernel(const BwdParams p) {
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
constexpr int kBwdThreads = 128;
// K, V, 2x(Q, dO), dS (two 64-column halves) + LSE/delta stages + alignment slack
constexpr int kBwdSmemBytes = 8 * kTileBytes + 2 * 2 * kTile * 4 + 1024;
constexpr int kBwdTmemCols = 512;  // S^T 0, dP^T 128, P^T 256, dV 320, dK 384, dQ 448

__global__ void __launch_bounds__(kBwdThreads)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[6];  // kv, qdo0, qdo1, s, dp, dq
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int kt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;

  int q_begin = 0, k_begin = 0, lq = p.lq, lk = p.lk, bcoord = b;
  if (p.cu_q != nullptr) {
    q_begin = p.cu_q[b];
    lq = p.cu_q[b + 1] - q_begin;
    k_begin = p.cu_k[b];
    lk = p.cu_k[b + 1] - k_begin;
    bcoord = 0;
  }
  const int k_row0 = kt * kTile;
  if (k_row0 >= lk) return;
  const int n_q = (lq + kTile - 1) / kTile;

  uint8_t* smem_al = smem_raw + (((smem_u32(smem_raw) + 1023u) & ~1023u) - smem_u32(smem_raw));
  const uint32_t smem_base = smem_u32(smem_al);
  const uint32_t sK = smem_base;
  const uint32_t sV = smem_base + 1 * kTileBytes;
  const uint32_t sQ[2] = {smem_base + 2 * kTileBytes, smem_base + 4 * kTileBytes};
  const uint32_t sDO[2] = {smem_base + 3 * kTileBytes, smem_base + 5 * kTileBytes};
  const uint32_t sDS = smem_base + 6 * kTileBytes;  // 32 KB: q columns 0..63 | 64..127
  uint8_t* sDS_ptr = smem_al + 6 * kTileBytes;
  float* sLse = reinterpret_cast<float*>(smem_al + 8 * kTileBytes);  // [2][128], log2 domain
  float* sDelta = sLse + 2 * kTile;                                  // [2][128]

  const uint32_t bar_kv = smem_u32(&bars[0]);
  const uint32_t bar_qdo[2] = {smem_u32(&bars[1]), smem_u32(&bars[2])};
  const uint32_t bar_s = smem_u32(&bars[3]);
  const uint32_t bar_dp = smem_u32(&bars[4]);
  const uint32_t bar_dq = smem_u32(&bars[5]);

  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < 6; ++i) mbar_init(smem_u32(&bars[i]), 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_do);
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(smem_u32(&tmem_base_slot), kBwdTmemCols);
    tmem_relinquish();
  }

  // LSE (converted to the log2 domain) and delta of query tile `jt` into stage `stg`. Rows past
  // the end of the sequence get lse = +inf, which makes their P^T column exactly zero.
  const int64_t stat_base = p.cu_q != nullptr ? int64_t(h) * p.total_q + q_begin : (int64_t(b) * p.heads + h) * p.lq;
  auto load_stats = [&](int jt, int stg) {
    const int r = jt * kTile + tid;
    float l2 = INFINITY, dl = 0.f;
    if (r < lq) {
      l2 = p.lse[stat_base + r] * 1.4426950408889634f;
      dl = p.delta[stat_base + r];
    }
    sLse[stg * kTile + tid] = l2;
    sDelta[stg * kTile + tid] = dl;
  };
  if (n_q > 0) load_stats(0, 0);

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128, tm_pt = tmem_base + 256;
  const uint32_t tm_dv = tmem_base + 320, tm_dk = tmem_base + 384, tm_dq = tmem_base + 448;
  const uint32_t lane_off = uint32_t(warp * 32) << 16;

  constexpr uint32_t kIdescS = make_idesc(128, 128, 0, 0);     // K-major x K-major, N = 128
  constexpr uint32_t kIdescKN = make_idesc(128, 64, 0, 1);     // A K-major / tensor memory, B MN-major
  constexpr uint32_t kIdescNN = make_idesc(128, 64, 1, 1);     // A MN-major, B MN-major

  auto issue_s_dp = [&](int stg) {
    const uint64_t kd = make_sdesc(sK, 16, 1024), qd = make_sdesc(sQ[stg], 16, 1024);
    const uint64_t vd = make_sdesc(sV, 16, 1024), gd = make_sdesc(sDO[stg], 16, 1024);
#pragma unroll
    for (int k = 0; k < 4; ++k) mma_ss(tm_s, kd + 2 * k, qd + 2 * k, kIdescS, k > 0);
    tc_commit(bar_s);
#pragma unroll
    for (int k = 0; k < 4; ++k) mma_ss(tm_dp, vd + 2 * k, gd + 2 * k, kIdescS, k > 0);
    tc_commit(bar_dp);
  };

  if (n_q > 0) {
    if (tid == 0) {
      mbar_arrive_expect_tx(bar_kv, 2 * kTileBytes);
      tma_load_4d(sK, &tmap_k, bar_kv, 0, k_begin + k_row0, h, bcoord);
      tma_load_4d(sV, &tmap_v, bar_kv, 0, k_begin + k_row0, h, bcoord);
      mbar_arrive_expect_tx(bar_qdo[0], 2 * kTileBytes);
      tma_load_4d(sQ[0], &tmap_q, bar_qdo[0], 0, q_begin, h, bcoord);
      tma_load_4d(sDO[0], &tmap_do, bar_qdo[0], 0, q_begin, h, bcoord);
      mbar_wait(bar_kv, 0, &abort_flag, p.status);
      mbar_wait(bar_qdo[0], 0, &abort_flag, p.status);
      tc_fence_after();
      issue_s_dp(0);
    }
    __syncwarp();

    const bool row_valid = (k_row0 + tid) < lk;

    for (int j = 0; j < n_q; ++j) {
      const int st = j & 1;
      if (j + 1 < n_q) {
        if (tid == 0) {
          mbar_arrive_expect_tx(bar_qdo[st ^ 1], 2 * kTileBytes);
          tma_load_4d(sQ[st ^ 1], &tmap_q, bar_qdo[st ^ 1], 0, q_begin + (j + 1) * kTile, h, bcoord);
          tma_load_4d(sDO[st ^ 1], &tmap_do, bar_qdo[st ^ 1], 0, q_begin + (j + 1) * kTile, h, bcoord);
        }
        __syncwarp();
        load_stats(j + 1, st ^ 1);
      }

      mbar_wait(bar_s, j & 1, &abort_flag, p.status);
      tc_fence_after();
      const float* lse_s = sLse + st * kTile;
      const float* dl_s = sDelta + st * kTile;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        float pf[32];
        tmem_ld32(tm_s + lane_off + c * 32, r);
        tmem_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float pv = fast_exp2(fmaf(__uint_as_float(r[i]), p.scale_log2, -lse_s[c * 32 + i]));
          pf[i] = row_valid ? pv : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[i] = pack_bf16(pf[2 * i], pf[2 * i + 1]);
        tmem_st16(tm_pt + lane_off + c * 16, pk);

        if (c == 0) {
          mbar_wait(bar_dp, j & 1, &abort_flag, p.status);
          tc_fence_after();
        }
        tmem_ld32(tm_dp + lane_off + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float d0 = pf[2 * i] * (__uint_as_float(r[2 * i]) - dl_s[c * 32 + 2 * i]);
          const float d1 = pf[2 * i + 1] * (__uint_as_float(r[2 * i + 1]) - dl_s[c * 32 + 2 * i + 1]);
          pk[i] = pack_bf16(d0, d1);
        }
        // dS^T row `tid`, query columns [32c, 32c+32): four 16-byte chunks of the swizzled row.
        uint8_t* half = sDS_ptr + (c >> 1) * kTileBytes;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint4 v = make_uint4(pk[q4 * 4], pk[q4 * 4 + 1], pk[q4 * 4 + 2], pk[q4 * 4 + 3]);
          *reinterpret_cast<uint4*>(half + swz128(tid, (c & 1) * 4 + q4)) = v;
        }
      }
      tmem_wait_st();
      fence_proxy_async_smem();
      tc_fence_before();
      __syncthreads();

      if (tid == 0) {
        tc_fence_after();
        const uint64_t gd_mn = make_sdesc(sDO[st], 1024, 1024);
        const uint64_t qd_mn = make_sdesc(sQ[st], 1024, 1024);
        const uint64_t kd_mn = make_sdesc(sK, 1024, 1024);
        const uint64_t ds_mn = make_sdesc(sDS, kTileBytes, 1024);
        // dV += P^T dO
#pragma unroll
        for (int k = 0; k < 8; ++k) mma_ts(tm_dv, tm_pt + 8 * k, gd_mn + 128 * k, kIdescKN, (j > 0) || (k > 0));
        // dK += dS^T Q   (A: K-major view of the dS buffer; K step = 16 query columns)
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t ad = make_sdesc(sDS + (k >> 2) * kTileBytes, 16, 1024) + 2 * (k & 3);
          mma_ss(tm_dk, ad, qd_mn + 128 * k, kIdescKN, (j > 0) || (k > 0));
        }
        // dQ = dS K      (A: MN-major view of the same bytes; K step = 16 key rows)
#pragma unroll
        for (int k = 0; k < 8; ++k) mma_ss(tm_dq, ds_mn + 128 * k, kd_mn + 128 * k, kIdescNN, k > 0);
        tc_commit(bar_dq);
        if (j + 1 < n_q) {
          mbar_wait(bar_qdo[st ^ 1], ((j + 1) >> 1) & 1, &abort_flag, p.status);
          tc_fence_after();
          issue_s_dp(st ^ 1);
        }
      }
      __syncwarp();

      // dQ tile -> fp32 accumulator. Here thread r owns QUERY row r of tile j.
      mbar_wait(bar_dq, j & 1, &abort_flag, p.status);
      tc_fence_after();
      const int qrow = j * kTile + tid;
      float* acc_row = p.dq_accum + ((int64_t(p.cu_q != nullptr ? 0 : b) * p.lq + q_begin + qrow) * p.heads + h) * kHeadDim;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32(tm_dq + lane_off + c * 32, r);
        tmem_wait_ld();
        if (qrow < lq) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 v = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                         __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
            atomicAdd(reinterpret_cast<float4*>(acc_row + c * 32 + 4 * i), v);
          }
        }
      }
      tc_fence_before();
    }
  }

  // Epilogue: dK (scaled) and dV rows of this tile.
  const int krow = k_row0 + tid;
  __nv_bfloat16* dk_ptr = p.dk + int64_t(bcoord) * p.dk_sb + int64_t(k_begin + krow) * p.dk_st + int64_t(h) * p.dk_sh;
  __nv_bfloat16* dv_ptr = p.dv + int64_t(bcoord) * p.dv_sb + int64_t(k_begin + krow) * p.dv_st + int64_t(h) * p.dv_sh;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t rk[32], rv[32];
    if (n_q > 0) {
      tmem_ld32(tm_dk + lane_off + c * 32, rk);
      tmem_ld32(tm_dv + lane_off + c * 32, rv);
      tmem_wait_ld();
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) rk[i] = rv[i] = 0u;
    }
    if (krow < lk) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 a, g;
        a.x = pack_bf16(__uint_as_float(rk[8 * i + 0]) * p.scale, __uint_as_float(rk[8 * i + 1]) * p.scale);
        a.y = pack_bf16(__uint_as_float(rk[8 * i + 2]) * p.scale, __uint_as_float(rk[8 * i + 3]) * p.scale);
        a.z = pack_bf16(__uint_as_float(rk[8 * i + 4]) * p.scale, __uint_as_float(rk[8 * i + 5]) * p.scale);
        a.w = pack_bf16(__uint_as_float(rk[8 * i + 6]) * p.scale, __uint_as_float(rk[8 * i + 7]) * p.scale);
        g.x = pack_bf16(__uint_as_float(rv[8 * i + 0]), __uint_as_float(rv[8 * i + 1]));
        g.y = pack_bf16(__uint_as_float(rv[8 * i + 2]), __uint_as_float(rv[8 * i + 3]));
        g.z = pack_bf16(__uint_as_float(rv[8 * i + 4]), __uint_as_float(rv[8 * i + 5]));
        g.w = pack_bf16(__uint_as_float(rv[8 * i + 6]), __uint_as_float(rv[8 * i + 7]));
        reinterpret_cast<uint4*>(dk_ptr)[c * 4 + i] = a;
        reinterpret_cast<uint4*>(dv_ptr)[c * 4 + i] = g;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kBwdTmemCols);
  }
}

}  // namespace nb
