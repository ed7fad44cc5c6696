// Work list of the varlen tile scheduler.
//
// In packed (cu_seqlens) mode the attention kernels do not launch a rectangular grid of
// ceil(max_seqlen / 128) tiles per sequence and let the tiles past a short sequence's end exit;
// they work through a compact list of (sequence, tile) items, built on the device from cu_seqlens by
// the single-CTA kernel below with no host synchronisation (the forward launches one CTA per entry
// and head, the backward one persistent CTA per SM that takes the entries in order):
//
//   * an item is one 128-row tile on the list's "own" side (query tiles for the forward, key
//     tiles for the backward); its cost is the number of 128-row steps on the other side;
//   * items are ordered most expensive first (sequences bucketed by their step count), and the
//     ragged last tile of every sequence -- fewer live rows, trimmed inner work -- comes after all
//     full tiles. The hardware hands CTAs to SMs in list order, so the long items start first and
//     the short ones fill the last wave: ragged visible-token counts do not leave SMs idle;
//   * rows of the packed buffer past the last sequence (a caller may pack into a buffer of fixed
//     capacity to avoid a device-to-host sync) form one more pseudo-sequence, index `batch`, that
//     owns rows [cu_seqlens[batch], total) and has nothing on the other side: its items make the
//     kernels write zeros there, so every row of every output is defined;
//   * the list has a host-known capacity of floor(total / 128) + batch + 1 entries; unused entries
//     have seq = -1 and their CTAs exit at once;
//   * an entry carries the sequence's offsets and lengths on both sides, so a CTA learns all it
//     needs about its work from one 32-byte read instead of a chain of dependent loads.
//
// The same kernel validates the packing it reads: offsets non-negative and non-decreasing, every
// length <= max_seqlen (the caller's bound sizes tensor maps and grids), last offset <= total
// tokens. On a violation it writes kStatusBadSeqlens to the status word and leaves the whole list
// empty, so the attention kernel does nothing instead of reading out of bounds.
//
// The reference's ragged consumer that this serves is the per-image eval loop of
// src/nanobrain/model.py:254-270 and the per-sample visible counts of model.py:186-199.
#pragma once

#include "ptx.cuh"

namespace nb {

// One work item; mirrors nb_attn_sched_item in include/nb_attn.h.
struct __align__(16) SchedItem {
  int32_t seq;          // sequence index; `batch` = the rows past the last sequence; -1 = unused entry
  int32_t tile;         // 128-row tile on the own side
  int32_t own_begin;    // first packed row of the sequence on the own side
  int32_t own_len;      // its length there
  int32_t other_begin;  // the same on the side the item's inner loop walks
  int32_t other_len;
  int32_t reserved[2];
};
static_assert(sizeof(SchedItem) == 32, "two 16-byte loads");

// Reads one entry with two 16-byte loads (one memory round trip).
__device__ __forceinline__ SchedItem sched_load(const SchedItem* items, uint32_t idx) {
  const int4* src = reinterpret_cast<const int4*>(items + idx);
  const int4 a = src[0], b = src[1];
  SchedItem it;
  it.seq = a.x, it.tile = a.y, it.own_begin = a.z, it.own_len = a.w;
  it.other_begin = b.x, it.other_len = b.y, it.reserved[0] = 0, it.reserved[1] = 0;
  return it;
}

constexpr int kSchedThreads = 1024;
constexpr int kSchedBuckets = 1024;  // step counts >= kSchedBuckets - 1 share the first bucket
constexpr int kSchedTile = 128;

// Upper bound of the number of items of a packing with `total` tokens in `batch` sequences (plus
// the pseudo-sequence of the unused rows at the end).
__host__ __device__ inline int64_t sched_capacity(int64_t total, int32_t batch) {
  return total / kSchedTile + batch + 1;
}

struct SchedParams {
  const int32_t* cu_own;    // offsets on the side whose tiles become items
  const int32_t* cu_other;  // offsets on the side an item's inner loop walks
  int32_t batch;
  int32_t max_own, max_other;
  int64_t total_own, total_other;
  SchedItem* items;  // [n_items]
  int32_t n_items;  // capacity, >= sched_capacity(total_own, batch)
  int32_t* status;
};

// Exclusive prefix sum over one value per thread of a block of kThreads threads (returns the
// exclusive prefix and writes the grand total to *total). `scratch` holds 32 ints.
template <int kThreads>
__device__ __forceinline__ int block_exclusive_scan(int v, int* scratch, int* total) {
  static_assert(kThreads % 32 == 0 && kThreads <= 1024, "whole warps");
  constexpr int kWarps = kThreads / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += up;
  }
  if (lane == 31) scratch[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = lane < kWarps ? scratch[lane] : 0;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) w += up;
    }
    scratch[lane] = w;  // inclusive over warps
  }
  __syncthreads();
  const int warp_prefix = warp > 0 ? scratch[warp - 1] : 0;
  *total = scratch[31];
  __syncthreads();  // scratch may be reused
  return warp_prefix + incl - v;
}

// Does this kernel's part of one sequence: lengths, validity, bucket.
struct SchedSeq {
  int full;    // full tiles on the own side
  int ragged;  // 1 if a partial last tile exists
  int bucket;  // 0 = most expensive
  bool ok;
  int own_begin, own_len, other_begin, other_len;
};

__host__ __device__ inline SchedItem sched_item(const SchedSeq& s, int seq, int tile) {
  SchedItem it;
  it.seq = seq, it.tile = tile;
  it.own_begin = s.own_begin, it.own_len = s.own_len, it.other_begin = s.other_begin, it.other_len = s.other_len;
  it.reserved[0] = it.reserved[1] = 0;
  return it;
}

__host__ __device__ inline SchedItem sched_no_item() {
  SchedItem it;
  it.seq = -1, it.tile = 0, it.own_begin = it.own_len = it.other_begin = it.other_len = 0;
  it.reserved[0] = it.reserved[1] = 0;
  return it;
}

// i in [0, batch]: i == batch is the pseudo-sequence of the rows past the last sequence.
__host__ __device__ inline SchedSeq sched_classify(const SchedParams& p, int i) {
  SchedSeq s;
  int64_t len, steps_len;
  if (i == p.batch) {
    len = p.total_own - int64_t(p.cu_own[i]);
    steps_len = 0;
    s.ok = len >= 0;  // the last offset does not exceed the token count
    s.own_begin = p.cu_own[i];
    s.other_begin = 0;
  } else {
    const int64_t a = p.cu_own[i], b = p.cu_own[i + 1];
    const int64_t c = p.cu_other[i], d = p.cu_other[i + 1];
    len = b - a;
    steps_len = d - c;
    s.ok = a >= 0 && c >= 0 && len >= 0 && steps_len >= 0 && len <= p.max_own && steps_len <= p.max_other &&
           b <= p.total_own && d <= p.total_other;
    s.own_begin = int(a);
    s.other_begin = int(c);
  }
  s.own_len = int(len);
  s.other_len = int(steps_len);
  s.full = len > 0 ? int(len / kSchedTile) : 0;
  s.ragged = len > 0 && (len % kSchedTile) != 0;
  const int steps = steps_len > 0 ? int((steps_len + kSchedTile - 1) / kSchedTile) : 0;
  const int clipped = steps < kSchedBuckets - 1 ? steps : kSchedBuckets - 1;
  s.bucket = kSchedBuckets - 1 - clipped;
  return s;
}

// Shared-memory state of one list build.
struct SchedShared {
  int full_pos[kSchedBuckets];    // full tiles per bucket, then the bucket's write cursor
  int ragged_pos[kSchedBuckets];  // ragged tiles per bucket, then the bucket's write cursor
  int scratch[32];
  int bad;
};

// Builds the list with one block of kThreads threads (every thread of the block must call it).
template <int kThreads>
__device__ __forceinline__ void sched_build(const SchedParams& p, SchedShared& sm) {
  static_assert(kSchedBuckets % kThreads == 0, "each thread owns a run of consecutive buckets");
  constexpr int kPer = kSchedBuckets / kThreads;
  const int tid = threadIdx.x;
  for (int k = 0; k < kPer; ++k) {
    sm.full_pos[tid * kPer + k] = 0;
    sm.ragged_pos[tid * kPer + k] = 0;
  }
  if (tid == 0) sm.bad = 0;
  __syncthreads();

  for (int i = tid; i <= p.batch; i += kThreads) {
    const SchedSeq s = sched_classify(p, i);
    if (!s.ok) {
      sm.bad = 1;
    } else {
      if (s.full) atomicAdd(&sm.full_pos[s.bucket], s.full);
      if (s.ragged) atomicAdd(&sm.ragged_pos[s.bucket], 1);
    }
  }
  __syncthreads();
  int my_full = 0, my_ragged = 0;
  for (int k = 0; k < kPer; ++k) {
    my_full += sm.full_pos[tid * kPer + k];
    my_ragged += sm.ragged_pos[tid * kPer + k];
  }
  int total_full = 0, total_ragged = 0;
  int full_at = block_exclusive_scan<kThreads>(my_full, sm.scratch, &total_full);
  int ragged_at = block_exclusive_scan<kThreads>(my_ragged, sm.scratch, &total_ragged);
  const bool overflow = int64_t(total_full) + total_ragged > p.n_items;  // cannot happen for a valid packing
  if (sm.bad || overflow) {
    if (tid == 0 && p.status) atomicExch(p.status, (int)kStatusBadSeqlens);
    for (int i = tid; i < p.n_items; i += kThreads) p.items[i] = sched_no_item();
    return;
  }
  ragged_at += total_full;
  for (int k = 0; k < kPer; ++k) {
    const int nf = sm.full_pos[tid * kPer + k], nr = sm.ragged_pos[tid * kPer + k];
    sm.full_pos[tid * kPer + k] = full_at;
    sm.ragged_pos[tid * kPer + k] = ragged_at;
    full_at += nf;
    ragged_at += nr;
  }
  __syncthreads();

  for (int i = tid; i <= p.batch; i += kThreads) {
    const SchedSeq s = sched_classify(p, i);
    if (s.full) {
      const int at = atomicAdd(&sm.full_pos[s.bucket], s.full);
      for (int t = 0; t < s.full; ++t) p.items[at + t] = sched_item(s, i, t);
    }
    if (s.ragged) {
      const int at = atomicAdd(&sm.ragged_pos[s.bucket], 1);
      p.items[at] = sched_item(s, i, s.full);
    }
  }
  for (int i = total_full + total_ragged + tid; i < p.n_items; i += kThreads) p.items[i] = sched_no_item();
}

__global__ void __launch_bounds__(kSchedThreads) attn_sched_kernel(const SchedParams p) {
  __shared__ SchedShared sm;
  pdl_wait();  // cu_seqlens may come from the kernel right before this one
  pdl_launch_dependents();
  sched_build<kSchedThreads>(p, sm);
}

}  // namespace nb
