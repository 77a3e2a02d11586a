// Gate + per-query top-k on the tensor pipe, for 16-bit q.
//
// The pooled keys are rounded to the input dtype (MoonshotAI/MoBA moba/moba_efficient.py:335-340 rounds the
// mean with .type_as before widening it), and q is 16-bit, so every product of the gate's dot product is exact
// in fp32: a tcgen05 product with fp32 accumulation computes the same sum as the reference's fp32 einsum up to
// the order of the additions. One CTA per (128-token query tile, head):
//   Q tile [128 x 128] by TMA; the tile's candidate chunks' pooled keys converted fp32 -> 16 bit (exactly) into
//   a K-major shared-memory tile by all threads; scores[128 x n] = Q kmean^T by 8 UMMAs into TMEM (up to 256
//   candidates per round); thread = token row reads its scores back and keeps the best kk in registers.
// The fp32-FMA kernel in gate.cu stays for fp32 q (and for more than 4096 candidate chunks per sequence); it is
// bound by shared-memory broadcasts of the pooled keys (one 16-byte read per four FMAs) at ~20 % of the FMA rate.
// Output format is that of gate.cu (sel, sel_score, tile_cnt).
#include "attn_common.cuh"

#include <algorithm>
#include <stdlib.h>

namespace moba {
namespace {

constexpr int kGateThreads = 160;      // warps 0-3: token rows (TMEM lanes); warp 4: TMA + MMA issue
constexpr int kCandTile = 256;         // candidates per round (TMEM columns)

struct __align__(1024) GateSmem {
  uint8_t q[2][16384];                 // [d half][128 tokens x 64], 128-byte swizzle
  uint64_t bar_q, bar_mma;
  uint32_t tmem_base;
  int abort_flag;
};
// After it in dynamic shared memory: km[2][cand_rows x 128 B] ([d half][candidates x 64], 128-byte swizzle; 1024-
// aligned because cand_rows is a multiple of 16), then uint32_t bitmap[max_cand][4]. cand_rows = candidates per
// round = min(256, max_cand rounded up to 16); the CTA allocates that many TMEM columns (a power of two >= 32).
// Sized like this, three CTAs fit an SM (registers) when sequences have up to ~100 chunks, two when they have 256 or more.

template <bool kBf16>
__device__ __forceinline__ uint32_t pack16_exact(float a, float b) {
  return pack2<kBf16>(a, b);           // the values are representable, so the rounding is exact
}

template <bool kBf16, int KMAX>
__global__ void __launch_bounds__(kGateThreads, 3)
gate_topk_umma_kernel(const __grid_constant__ CUtensorMap map_q, int H, const float* __restrict__ kmean, int kv_rep,
                      PlanDev plan,
                      int32_t* __restrict__ sel, float* __restrict__ sel_score, int32_t* __restrict__ tile_cnt,
                      int* status, int cand_rows, int tmem_cols) {
  extern __shared__ uint8_t smem_raw[];
  GateSmem& sm = *reinterpret_cast<GateSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* km = reinterpret_cast<uint8_t*>(&sm) + sizeof(GateSmem);
  const uint32_t km_half = static_cast<uint32_t>(cand_rows) * 128u;       // bytes of one d half
  uint32_t* bitmap = reinterpret_cast<uint32_t*>(km + 2 * km_half);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  WaitCtx wctx{&sm.abort_flag, status};

  const int tile = blockIdx.x, h = blockIdx.y;
  const int chunk = plan.qtile_chunk[tile];
  const int c0 = plan.chunk_seq_first[chunk];
  const int ncand = chunk - c0;
  const int kk = plan.kk;
  const int tok0 = plan.qtile_start[tile];
  const int tok = tok0 + tid;
  const bool valid = tid < MOBA_TILE && tok < plan.chunk_start[chunk + 1];
  const int64_t slot0 = (static_cast<int64_t>(tok) * H + h) * kk;

  if (ncand == 0) {                    // first chunk of its sequence: nothing to choose from
    if (valid)
      for (int j = 0; j < kk; ++j) {
        sel[slot0 + j] = -1;
        if (sel_score) sel_score[slot0 + j] = -INFINITY;
      }
    return;
  }

  if (tid == 0) {
    sm.abort_flag = 0;
    mbar_init(&sm.bar_q, 1);
    mbar_init(&sm.bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc(&sm.tmem_base, tmem_cols);
    tmem_relinquish();
  }
  for (int i = tid; i < ncand * 4; i += kGateThreads) bitmap[i] = 0u;
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;

  if (warp == 4 && lane == 0) {
    mbar_arrive_expect_tx(&sm.bar_q, 32768);
    tma_load_3d(smem_u32(sm.q[0]), &map_q, &sm.bar_q, 0, h, tok0);
    tma_load_3d(smem_u32(sm.q[1]), &map_q, &sm.bar_q, 64, h, tok0);
  }

  float best[KMAX];
  int bidx[KMAX];
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    best[j] = -INFINITY;
    bidx[j] = -1;
  }

  // pooled keys are [chunk, H / kv_rep, 128]; query head h reads key head h / kv_rep
  const int64_t km_stride = static_cast<int64_t>(H / kv_rep) * MOBA_HEAD_DIM;
  const int64_t km_head = static_cast<int64_t>(h / kv_rep) * MOBA_HEAD_DIM;
  bool ok = true;
  int round = 0;
  for (int b0 = 0; b0 < ncand; b0 += cand_rows, ++round) {
    const int nb = min(cand_rows, ncand - b0);
    const int n16 = (nb + 15) & ~15;                     // UMMA N: a multiple of 16
    // pooled keys of candidates b0 .. b0 + nb (rows up to n16 zero) -> K-major swizzled tile; 16 pieces of 8
    // elements per row
    for (int i = tid; i < n16 * 16; i += kGateThreads) {
      const int r = i >> 4, j = i & 15;
      uint4 out = make_uint4(0, 0, 0, 0);
      if (r < nb) {
        const float4* src = reinterpret_cast<const float4*>(kmean + (c0 + b0 + r) * km_stride + km_head + j * 8);
        const float4 a = __ldg(src), b = __ldg(src + 1);
        out = make_uint4(pack16_exact<kBf16>(a.x, a.y), pack16_exact<kBf16>(a.z, a.w), pack16_exact<kBf16>(b.x, b.y),
                         pack16_exact<kBf16>(b.z, b.w));
      }
      *reinterpret_cast<uint4*>(km + (j >> 3) * km_half + sw128_offset(r, j & 7)) = out;
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();                                     // tile written; scores of the previous round read
    tc_fence_after_sync();

    if (warp == 4) {
      const uint32_t leader = elect_one();
      ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_q, 0, wctx));
      if (ok) {
        tc_fence_after_sync();
        const uint32_t idesc = umma_idesc(128, n16, kBf16, false, false);
        const uint64_t q_km = umma_smem_desc(smem_u32(sm.q[0]), 16, 1024);
        const uint64_t k_km = umma_smem_desc(smem_u32(km), 16, 1024);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss_w(leader, tmem, q_km + (((ks >> 2) * 16384u + (ks & 3) * 32u) >> 4),
                    k_km + (((ks >> 2) * km_half + (ks & 3) * 32u) >> 4), idesc, ks > 0);
        umma_commit_w(leader, &sm.bar_mma);
        // the next round rewrites the pooled-key tile: this warp, too, must know that the products have read it
        ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_mma, round & 1, wctx));
      }
    } else {
      // thread = token row: scores of this round, 32 columns at a time, into the running top-kk
      ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_mma, round & 1, wctx));
      if (ok) {
        tc_fence_after_sync();
        const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        for (int cb = 0; cb < nb; cb += 32) {
          uint32_t r[32];
          tmem_ld32(lane_addr + cb, r);
          tmem_wait_ld();
          if (valid) {
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const float s = __uint_as_float(r[c]);
              if (cb + c < nb && s > best[KMAX - 1]) {
                best[KMAX - 1] = s;
                bidx[KMAX - 1] = b0 + cb + c;
#pragma unroll
                for (int j = KMAX - 1; j > 0; --j) {
                  if (best[j] > best[j - 1]) {
                    const float tf = best[j]; best[j] = best[j - 1]; best[j - 1] = tf;
                    const int ti = bidx[j]; bidx[j] = bidx[j - 1]; bidx[j - 1] = ti;
                  }
                }
              }
            }
          }
        }
      }
    }
    // everyone is done with this round's scores (and agrees on whether a wait was abandoned)
    tc_fence_before_sync();
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    tc_fence_after_sync();
    if (!ok) break;
  }

  if (valid) {
    // A wait that ran out leaves the scores unknown: the tile's queries then select nothing (the status word
    // carries the error), so that the list kernels downstream never see an uninitialised chunk id.
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
      if (j < kk) {
        const int lc = ok ? bidx[j] : -1;
        sel[slot0 + j] = lc >= 0 ? c0 + lc : -1;
        if (sel_score) sel_score[slot0 + j] = ok ? best[j] : -INFINITY;
        if (lc >= 0) atomicOr(&bitmap[lc * 4 + warp], 1u << lane);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, tmem_cols);
  const int64_t cnt0 = (static_cast<int64_t>(plan.qtile_cand_off[tile]) * H) + static_cast<int64_t>(h) * ncand;
  for (int c = tid; c < ncand; c += kGateThreads)
    tile_cnt[cnt0 + c] = __popc(bitmap[c * 4]) + __popc(bitmap[c * 4 + 1]) + __popc(bitmap[c * 4 + 2]) +
                         __popc(bitmap[c * 4 + 3]);
}


// ---------------------------------------------------------------------------------------------------------------
// Streaming form of the same gate for sequences of at most 257 chunks (256 candidates: one round of the product):
// one persistent CTA per SM walks the (query tile, head) items i = blockIdx.x, blockIdx.x + gridDim.x, ... in
// head-major order. Per CTA, once: tensor memory (two score buffers), barriers, the query-tile ring. Per item:
//   control warp   keeps the Q tiles of the next two items in flight (three-stage TMA ring), extends the pooled-key
//                  operand tile in shared memory when the item's chunk has more candidates than the tile holds
//                  (tiles of a head come in ascending token order, so the tile only grows until the head or the
//                  sequence changes), issues the eight UMMAs of the item into score buffer (item & 1)
//   scan group     (item & 1): four warps, thread = token row, read the scores back and keep the best kk in
//                  registers while the control warp already works on the next item for the other group
// so the query read (the only HBM traffic that matters: S * H * 256 bytes) is never waited for and the fixed costs
// of a CTA are paid once per SM instead of once per 128 tokens. Output format as above.
constexpr int kStreamThreads = 288;    // warps 0-3 / 4-7: scan groups 0 / 1 (warp & 3 = TMEM lane quarter); warp 8: control
constexpr int kQStages = 3;

struct __align__(1024) StreamSmem {
  uint8_t q[kQStages][2][16384];       // [stage][d half][128 tokens x 64], 128-byte swizzle
  uint64_t bar_q_full[kQStages], bar_q_empty[kQStages], bar_mma[2], bar_free[2];
  uint32_t tmem_base;
  int abort_flag;
  int group_abort[2];
};
// After it in dynamic shared memory: km[2][cand_rows x 128 B] and uint32_t bitmap[2 groups][2][cand_rows][4].

template <bool kBf16, int KMAX>
__global__ void __launch_bounds__(kStreamThreads, 1)
gate_topk_stream_kernel(const __grid_constant__ CUtensorMap map_q, int H, const float* __restrict__ kmean, int kv_rep,
                        PlanDev plan, int32_t* __restrict__ sel, float* __restrict__ sel_score,
                        int32_t* __restrict__ tile_cnt, int* status, int cand_rows, int buf_cols) {
  extern __shared__ uint8_t smem_raw[];
  StreamSmem& sm = *reinterpret_cast<StreamSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* km = reinterpret_cast<uint8_t*>(&sm) + sizeof(StreamSmem);
  const uint32_t km_half = static_cast<uint32_t>(cand_rows) * 128u;       // bytes of one d half
  uint32_t* bitmaps = reinterpret_cast<uint32_t*>(km + 2 * km_half);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  WaitCtx wctx{&sm.abort_flag, status};
  const int kk = plan.kk;
  const int64_t n_items = static_cast<int64_t>(plan.n_qtiles) * H;

  if (tid == 0) {
    sm.abort_flag = 0;
    sm.group_abort[0] = sm.group_abort[1] = 0;
    for (int i = 0; i < kQStages; ++i) {
      mbar_init(&sm.bar_q_full[i], 1);
      mbar_init(&sm.bar_q_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.bar_mma[i], 1);
      mbar_init(&sm.bar_free[i], 128);
    }
    mbar_fence_init();
  }
  if (warp == 8) {
    tmem_alloc(&sm.tmem_base, 2 * buf_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  // items of this CTA: n = 0, 1, ... -> global item blockIdx.x + n * gridDim.x
  const int64_t first = blockIdx.x, stride = gridDim.x;
  const int n_mine = first < n_items ? static_cast<int>((n_items - first + stride - 1) / stride) : 0;

  if (warp == 8) {
    // ================= control warp =================
    const uint32_t leader = elect_one();
    const uint64_t k_km = umma_smem_desc(smem_u32(km), 16, 1024);
    const int64_t km_stride = static_cast<int64_t>(H / kv_rep) * MOBA_HEAD_DIM;
    int cur_hk = -1, cur_c0 = -1, n_loaded = 0;      // the pooled-key tile holds candidates [0, n_loaded) of this key
    int next_load = 0;
    bool ok = true;
    for (int n = 0; n < n_mine && ok; ++n) {
      // ---- keep the Q tiles of items n .. n + 2 in flight
      for (; next_load < n_mine && next_load <= n + 2; ++next_load) {
        const int m = next_load, s = m % kQStages;
        if (m >= kQStages) {
          ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_q_empty[s], ((m / kQStages) - 1) & 1, wctx));
          if (!ok) break;
        }
        if (lane == 0) {
          const int64_t i = first + m * stride;
          const int hh = static_cast<int>(i / plan.n_qtiles), tile = static_cast<int>(i - static_cast<int64_t>(hh) * plan.n_qtiles);
          const int tok0 = plan.qtile_start[tile];
          mbar_arrive_expect_tx(&sm.bar_q_full[s], 32768);
          tma_load_3d(smem_u32(sm.q[s][0]), &map_q, &sm.bar_q_full[s], 0, hh, tok0);
          tma_load_3d(smem_u32(sm.q[s][1]), &map_q, &sm.bar_q_full[s], 64, hh, tok0);
        }
      }
      if (!ok) break;
      const int64_t i = first + n * stride;
      const int h = static_cast<int>(i / plan.n_qtiles), tile = static_cast<int>(i - static_cast<int64_t>(h) * plan.n_qtiles);
      const int chunk = plan.qtile_chunk[tile];
      const int c0 = plan.chunk_seq_first[chunk];
      const int ncand = chunk - c0;
      const int n16 = (ncand + 15) & ~15;
      const int b = n & 1, s = n % kQStages;
      // ---- pooled keys of candidates [0, ncand) of (key head, sequence) in the operand tile. Rows from ncand up to
      // the product's width n16 may hold anything: their score columns are never read.
      const int hk = h / kv_rep;
      if (hk != cur_hk || c0 != cur_c0) {
        n_loaded = 0;
        cur_hk = hk;
        cur_c0 = c0;
      }
      if (ncand > n_loaded) {
        // the products of the two previous items may still be reading the tile
        if (n >= 1) ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_mma[(n - 1) & 1], ((n - 1) >> 1) & 1, wctx));
        if (ok && n >= 2) ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_mma[(n - 2) & 1], ((n - 2) >> 1) & 1, wctx));
        if (!ok) break;
        for (int idx = n_loaded * 16 + lane; idx < ncand * 16; idx += 32) {
          const int r = idx >> 4, j = idx & 15;
          const float4* src = reinterpret_cast<const float4*>(kmean + (c0 + r) * km_stride + static_cast<int64_t>(hk) * MOBA_HEAD_DIM + j * 8);
          const float4 x = __ldg(src), y = __ldg(src + 1);
          *reinterpret_cast<uint4*>(km + (j >> 3) * km_half + sw128_offset(r, j & 7)) =
              make_uint4(pack16_exact<kBf16>(x.x, x.y), pack16_exact<kBf16>(x.z, x.w), pack16_exact<kBf16>(y.x, y.y),
                         pack16_exact<kBf16>(y.z, y.w));
        }
        n_loaded = ncand;
        fence_proxy_async_smem();
        __syncwarp();
      }
      // ---- the item's product: scores[128 x n16] = Q kmean^T into buffer b
      const BarPhase need[2] = {{&sm.bar_q_full[s], static_cast<uint32_t>((n / kQStages) & 1)},
                                {n >= 2 ? &sm.bar_free[b] : &sm.bar_q_full[s],
                                 static_cast<uint32_t>(n >= 2 ? ((n >> 1) - 1) & 1 : (n / kQStages) & 1)}};
      ok = __all_sync(0xffffffffu, mbar_wait_all(need, wctx));
      if (!ok) break;
      tc_fence_after_sync();
      if (ncand > 0) {
        const uint32_t idesc = umma_idesc(128, n16, kBf16, false, false);
        const uint64_t q_km = umma_smem_desc(smem_u32(sm.q[s][0]), 16, 1024);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss_w(leader, tmem + b * buf_cols, q_km + (((ks >> 2) * 16384u + (ks & 3) * 32u) >> 4),
                    k_km + (((ks >> 2) * km_half + (ks & 3) * 32u) >> 4), idesc, ks > 0);
      }
      // with nothing issued the commits arrive at once: every item completes one phase of both barriers
      umma_commit_w(leader, &sm.bar_mma[b]);
      umma_commit_w(leader, &sm.bar_q_empty[s]);
    }
    if (!ok) __nanosleep(1000000);
  } else {
    // ================= scan groups: thread = token row =================
    const int g = warp >> 2, gt = tid & 127;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t gbar = 1 + g;                       // named barrier of the group's four warps
    for (int n = g; n < n_mine; n += 2) {
      const int64_t i = first + n * stride;
      const int h = static_cast<int>(i / plan.n_qtiles), tile = static_cast<int>(i - static_cast<int64_t>(h) * plan.n_qtiles);
      const int chunk = plan.qtile_chunk[tile];
      const int c0 = plan.chunk_seq_first[chunk];
      const int ncand = chunk - c0;
      const int tok = plan.qtile_start[tile] + gt;
      const bool valid = tok < plan.chunk_start[chunk + 1];
      const int64_t slot0 = (static_cast<int64_t>(tok) * H + h) * kk;
      uint32_t* bitmap = bitmaps + static_cast<size_t>(g * 2 + ((n >> 1) & 1)) * cand_rows * 4;
      for (int j = gt; j < ncand * 4; j += 128) bitmap[j] = 0u;
      const bool got = mbar_wait(&sm.bar_mma[n & 1], (n >> 1) & 1, wctx);
      if (!got) sm.group_abort[g] = 1;
      asm volatile("bar.sync %0, 128;" ::"r"(gbar) : "memory");     // bitmap cleared; one view of the abort flag
      if (*reinterpret_cast<volatile int*>(&sm.group_abort[g])) break;
      tc_fence_after_sync();
      float best[KMAX];
      int bidx[KMAX];
#pragma unroll
      for (int j = 0; j < KMAX; ++j) {
        best[j] = -INFINITY;
        bidx[j] = -1;
      }
      for (int cb = 0; cb < ncand; cb += 32) {
        uint32_t r[32];
        tmem_ld32(lane_addr + (n & 1) * buf_cols + cb, r);
        tmem_wait_ld();
        if (valid) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const float sc = __uint_as_float(r[c]);
            if (cb + c < ncand && sc > best[KMAX - 1]) {
              best[KMAX - 1] = sc;
              bidx[KMAX - 1] = cb + c;
#pragma unroll
              for (int j = KMAX - 1; j > 0; --j) {
                if (best[j] > best[j - 1]) {
                  const float tf = best[j]; best[j] = best[j - 1]; best[j - 1] = tf;
                  const int ti = bidx[j]; bidx[j] = bidx[j - 1]; bidx[j - 1] = ti;
                }
              }
            }
          }
        }
      }
      // the scores are in registers: the buffer may take the product of item n + 2
      tc_fence_before_sync();
      mbar_arrive(&sm.bar_free[n & 1]);
      if (valid) {
#pragma unroll
        for (int j = 0; j < KMAX; ++j) {
          if (j < kk) {
            const int lc = bidx[j];
            sel[slot0 + j] = lc >= 0 ? c0 + lc : -1;
            if (sel_score) sel_score[slot0 + j] = best[j];
            if (lc >= 0) atomicOr(&bitmap[lc * 4 + (warp & 3)], 1u << lane);
          }
        }
      }
      asm volatile("bar.sync %0, 128;" ::"r"(gbar) : "memory");
      const int64_t cnt0 = (static_cast<int64_t>(plan.qtile_cand_off[tile]) * H) + static_cast<int64_t>(h) * ncand;
      for (int c = gt; c < ncand; c += 128)
        tile_cnt[cnt0 + c] = __popc(bitmap[c * 4]) + __popc(bitmap[c * 4 + 1]) + __popc(bitmap[c * 4 + 2]) +
                             __popc(bitmap[c * 4 + 3]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, 2 * buf_cols);
}

}  // namespace

int launch_gate_umma(const void* q, int32_t dtype, int32_t H, int64_t stride_s, int64_t stride_h, const float* kmean,
                     int kv_rep, const moba_plan_info* info, const PlanDev& plan, int32_t* sel, float* sel_score,
                     int32_t* tile_cnt, int32_t* status, cudaStream_t st) {
  CUtensorMap mq;
  int rc = make_tensor_map_shd(&mq, q, dtype, info->total_tokens, H, stride_s, stride_h, MOBA_TILE);
  if (rc) return rc;
  const int max_cand = info->max_cand > 0 ? info->max_cand : 1;
  const bool bf16 = dtype == MOBA_DTYPE_BF16;
  if (max_cand <= kCandTile && !getenv("MOBA_GATE_PER_TILE")) {
    // streaming kernel: one persistent CTA per SM
    const int rows = (max_cand + 15) & ~15;
    int cols = 32;
    while (cols < rows) cols *= 2;
    const size_t smem_s = sizeof(StreamSmem) + 1024 + static_cast<size_t>(rows) * 256 + static_cast<size_t>(rows) * 64;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t items = static_cast<int64_t>(plan.n_qtiles) * H;
    const unsigned grid_s = static_cast<unsigned>(items < sms ? items : sms);
    auto run_s = [&](auto kern) -> int {
      MOBA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_s));
      kern<<<grid_s, kStreamThreads, smem_s, st>>>(mq, H, kmean, kv_rep, plan, sel, sel_score, tile_cnt, status, rows, cols);
      MOBA_CUDA_OK(cudaGetLastError());
      return 0;
    };
    if (plan.kk <= 2) return bf16 ? run_s(gate_topk_stream_kernel<true, 2>) : run_s(gate_topk_stream_kernel<false, 2>);
    if (plan.kk <= 4) return bf16 ? run_s(gate_topk_stream_kernel<true, 4>) : run_s(gate_topk_stream_kernel<false, 4>);
    if (plan.kk <= 8) return bf16 ? run_s(gate_topk_stream_kernel<true, 8>) : run_s(gate_topk_stream_kernel<false, 8>);
    if (plan.kk <= 12) return bf16 ? run_s(gate_topk_stream_kernel<true, 12>) : run_s(gate_topk_stream_kernel<false, 12>);
    if (plan.kk <= 16) return bf16 ? run_s(gate_topk_stream_kernel<true, 16>) : run_s(gate_topk_stream_kernel<false, 16>);
    return bf16 ? run_s(gate_topk_stream_kernel<true, 32>) : run_s(gate_topk_stream_kernel<false, 32>);
  }
  const int cand_rows = std::min(kCandTile, (max_cand + 15) & ~15);
  int tmem_cols = 32;
  while (tmem_cols < cand_rows) tmem_cols *= 2;
  const size_t smem = sizeof(GateSmem) + 1024 + static_cast<size_t>(cand_rows) * 256 + static_cast<size_t>(max_cand) * 16;
  dim3 grid(plan.n_qtiles, H);
  auto run = [&](auto kern) -> int {
    MOBA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kGateThreads, smem, st>>>(mq, H, kmean, kv_rep, plan, sel, sel_score, tile_cnt, status, cand_rows, tmem_cols);
    MOBA_CUDA_OK(cudaGetLastError());
    return 0;
  };
  if (plan.kk <= 4) return bf16 ? run(gate_topk_umma_kernel<true, 4>) : run(gate_topk_umma_kernel<false, 4>);
  if (plan.kk <= 8) return bf16 ? run(gate_topk_umma_kernel<true, 8>) : run(gate_topk_umma_kernel<false, 8>);
  if (plan.kk <= 16) return bf16 ? run(gate_topk_umma_kernel<true, 16>) : run(gate_topk_umma_kernel<false, 16>);
  return bf16 ? run(gate_topk_umma_kernel<true, 32>) : run(gate_topk_umma_kernel<false, 32>);
}

}  // namespace moba
