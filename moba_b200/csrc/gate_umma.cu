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
          tmem_wait_ld32(r);
          if (valid) {
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const float s = __uint_as_float(r[c]);
              if constexpr (KMAX == 2) {
                // two slots: the same insertion (strict >, the earlier candidate keeps a tie) as selects, no branch
                const bool in = cb + c < nb;
                const bool g0 = in && s > best[0], g1 = in && s > best[1];
                const int ci = b0 + cb + c;
                best[1] = g0 ? best[0] : (g1 ? s : best[1]);
                bidx[1] = g0 ? bidx[0] : (g1 ? ci : bidx[1]);
                best[0] = g0 ? s : best[0];
                bidx[0] = g0 ? ci : bidx[0];
              } else if (cb + c < nb && s > best[KMAX - 1]) {
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
// head-major order. Per CTA, once: tensor memory (NG score buffers), barriers, the query-tile ring. Per item:
//   control warp   keeps the Q tiles of the next NG items in flight (TMA ring of NG + 1 stages), extends the
//                  pooled-key operand tile in shared memory when the item's chunk has more candidates than the tile
//                  holds (tiles of a head come in ascending token order, so the tile only grows until the head or the
//                  sequence changes), issues the eight UMMAs of the item into score buffer (item % NG)
//   scan group     (item % NG): four warps, thread = token row, select the best kk of the row's scores while the
//                  control warp already works on the next items for the other groups
// so the query read (the only HBM traffic that matters: S * H * 256 bytes) is never waited for and the fixed costs
// of a CTA are paid once per SM instead of once per 128 tokens. NG = 4 buffers of up to 128 candidates, or 2 of
// up to 256.
//
// Selection without data-dependent branches (a warp whose 32 rows insert at different candidates pays for every
// insertion): pass 1 keeps the kk largest VALUES sorted in registers -- inserting s is v[j] = max(min(v[j-1], s),
// v[j]) for all j, independent operations -- which yields the kk-th largest value t; pass 2 re-reads the scores
// from tensor memory and emits the candidates with score > t in ascending chunk order, then (only if a row still
// lacks entries: an exact tie at t) those with score == t, lowest chunk first. The chosen SET is that of a full
// sort; sel lists it in ascending chunk order.
// Items are handed out in blocks of kBlockTiles consecutive query tiles of one head (block gb = blockIdx.x,
// blockIdx.x + gridDim.x, ...): inside a block the candidate set grows by at most one chunk per tile, so the
// pooled-key tile is extended a row at a time, and the blocks of a head are spread over all CTAs, which evens out
// the work (late tiles of a sequence have more candidates than early ones). The last block of a head is padded with
// empty items, so item n of a CTA is tile n % kBlockTiles of its block n / kBlockTiles.
// What an item needs from the plan tables (tile -> chunk -> first chunk of the sequence, token range) is looked
// up 32 items at a time, one item per lane of the control warp, into a ring in shared memory: the chains of
// dependent loads then overlap instead of standing in every item's way.
constexpr int kBlockTiles = 16;
constexpr int kStreamMaxCand = 32;     // the streaming kernel is launched up to this many candidate chunks per sequence
constexpr int kMetaRing = 128;         // entries; filled in batches of 32, one batch ahead
struct ItemMeta {
  int h, tile, c0, ncand, tok0, tok_end, cand_off, empty;
};

template <int NG>
struct __align__(1024) StreamSmem {
  uint8_t q[NG + 1][2][16384];         // [stage][d half][128 tokens x 64], 128-byte swizzle
  ItemMeta meta[kMetaRing];
  uint64_t bar_q_full[NG + 1], bar_q_empty[NG + 1], bar_mma[NG], bar_free[NG], bar_meta[kMetaRing / 32];
  uint32_t tmem_base;
  int abort_flag;
  int group_abort[NG];
};
// After it in dynamic shared memory: km[2][cand_rows x 128 B] and uint32_t bitmap[NG groups][2][cand_rows][4].

template <bool kBf16, int KMAX, int NG>
__global__ void __launch_bounds__(NG * 128 + 32, 1)
gate_topk_stream_kernel(const __grid_constant__ CUtensorMap map_q, int H, const float* __restrict__ kmean, int kv_rep,
                        PlanDev plan, int32_t* __restrict__ sel, float* __restrict__ sel_score,
                        int32_t* __restrict__ tile_cnt, int* status, int cand_rows, int buf_cols) {
  constexpr int kStagesQ = NG + 1;
  constexpr int kCtl = NG * 4;          // index of the control warp
  extern __shared__ uint8_t smem_raw[];
  using Smem = StreamSmem<NG>;
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* km = reinterpret_cast<uint8_t*>(&sm) + sizeof(Smem);
  const uint32_t km_half = static_cast<uint32_t>(cand_rows) * 128u;       // bytes of one d half
  uint32_t* bitmaps = reinterpret_cast<uint32_t*>(km + 2 * km_half);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  WaitCtx wctx{&sm.abort_flag, status};
  const int kk = plan.kk;

  if (tid == 0) {
    sm.abort_flag = 0;
    for (int i = 0; i < kStagesQ; ++i) {
      mbar_init(&sm.bar_q_full[i], 1);
      mbar_init(&sm.bar_q_empty[i], 1);
    }
    for (int i = 0; i < NG; ++i) {
      sm.group_abort[i] = 0;
      mbar_init(&sm.bar_mma[i], 1);
      mbar_init(&sm.bar_free[i], 128);
    }
    for (int i = 0; i < kMetaRing / 32; ++i) mbar_init(&sm.bar_meta[i], 1);
    mbar_fence_init();
  }
  if (warp == kCtl) {
    tmem_alloc(&sm.tmem_base, NG * buf_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  // blocks gb = first + m * stride of this CTA; its items n = 0 .. n_mine - 1
  const int nb_per_head = (plan.n_qtiles + kBlockTiles - 1) / kBlockTiles;
  const int64_t n_blocks = static_cast<int64_t>(nb_per_head) * H;
  const int64_t first = blockIdx.x, stride = gridDim.x;
  const int n_mine = first < n_blocks ? static_cast<int>((n_blocks - first + stride - 1) / stride) * kBlockTiles : 0;

  if (warp == kCtl) {
    // ================= control warp =================
    const uint32_t leader = elect_one();
    const uint64_t k_km = umma_smem_desc(smem_u32(km), 16, 1024);
    const int64_t km_stride = static_cast<int64_t>(H / kv_rep) * MOBA_HEAD_DIM;
    int cur_hk = -1, cur_c0 = -1, n_loaded = 0;      // the pooled-key tile holds candidates [0, n_loaded) of this key
    int next_load = 0;
    bool ok = true;
    // batch k = items [32 k, 32 k + 32): one item per lane
    auto fill_meta = [&](int batch) {
      const int n = batch * 32 + lane;
      ItemMeta e;
      e.empty = 1;
      e.h = 0; e.tile = 0; e.c0 = 0; e.ncand = 0; e.tok0 = 0; e.tok_end = 0; e.cand_off = 0;
      if (n < n_mine) {
        const int64_t gb = first + static_cast<int64_t>(n / kBlockTiles) * stride;
        e.h = static_cast<int>(gb / nb_per_head);
        e.tile = static_cast<int>(gb % nb_per_head) * kBlockTiles + n % kBlockTiles;
        if (e.tile < plan.n_qtiles) {
          const int chunk = plan.qtile_chunk[e.tile];
          e.c0 = plan.chunk_seq_first[chunk];
          e.ncand = chunk - e.c0;
          e.tok0 = plan.qtile_start[e.tile];
          e.tok_end = plan.chunk_start[chunk + 1];
          e.cand_off = plan.qtile_cand_off[e.tile];
          e.empty = 0;
        } else {
          e.tile = plan.n_qtiles - 1;                 // padding item: loads a tile, selects nothing
          e.tok0 = plan.qtile_start[e.tile];
        }
      }
      sm.meta[n & (kMetaRing - 1)] = e;
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.bar_meta[batch & (kMetaRing / 32 - 1)]);
    };
    if (n_mine > 0) fill_meta(0);
    for (int n = 0; n < n_mine && ok; ++n) {
      if ((n & 31) == 0 && n + 32 < n_mine) fill_meta(n / 32 + 1);
      // ---- keep the Q tiles of items n .. n + NG in flight
      for (; next_load < n_mine && next_load <= n + NG; ++next_load) {
        const int m = next_load, s = m % kStagesQ;
        if (m >= kStagesQ) {
          ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_q_empty[s], ((m / kStagesQ) - 1) & 1, wctx));
          if (!ok) break;
        }
        if (lane == 0) {
          const ItemMeta& e = sm.meta[m & (kMetaRing - 1)];
          mbar_arrive_expect_tx(&sm.bar_q_full[s], 32768);
          tma_load_3d(smem_u32(sm.q[s][0]), &map_q, &sm.bar_q_full[s], 0, e.h, e.tok0);
          tma_load_3d(smem_u32(sm.q[s][1]), &map_q, &sm.bar_q_full[s], 64, e.h, e.tok0);
        }
      }
      if (!ok) break;
      const ItemMeta e = sm.meta[n & (kMetaRing - 1)];
      const int h = e.h, c0 = e.c0, ncand = e.ncand;
      const int n16 = (ncand + 15) & ~15;
      const int b = n % NG, s = n % kStagesQ;
      // ---- pooled keys of candidates [0, ncand) of (key head, sequence) in the operand tile. Rows from ncand up to
      // the product's width n16 may hold anything: their score columns are never read. For the same reason rows
      // can be appended while earlier products are still running (they read those rows as padding at most); only
      // a new (key head, sequence) rewrites rows in use and has to wait for the products in flight.
      const int hk = h / kv_rep;
      if (ncand > 0 && (hk != cur_hk || c0 != cur_c0)) {
        for (int p = 1; p <= NG && p <= n && ok; ++p)
          ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_mma[(n - p) % NG], ((n - p) / NG) & 1, wctx));
        if (!ok) break;
        n_loaded = 0;
        cur_hk = hk;
        cur_c0 = c0;
      }
      if (ncand > n_loaded) {
        // 16-byte pieces (8 values) of the new rows, four per lane and round so that eight loads are in flight
        const int p0 = n_loaded * 16, p1 = ncand * 16;
        for (int base = p0; base < p1; base += 128) {
          float4 x[4], y[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int idx = base + u * 32 + lane;
            if (idx < p1) {
              const int r = idx >> 4, j = idx & 15;
              const float4* src = reinterpret_cast<const float4*>(kmean + (c0 + r) * km_stride + static_cast<int64_t>(hk) * MOBA_HEAD_DIM + j * 8);
              x[u] = __ldg(src);
              y[u] = __ldg(src + 1);
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int idx = base + u * 32 + lane;
            if (idx < p1) {
              const int r = idx >> 4, j = idx & 15;
              *reinterpret_cast<uint4*>(km + (j >> 3) * km_half + sw128_offset(r, j & 7)) =
                  make_uint4(pack16_exact<kBf16>(x[u].x, x[u].y), pack16_exact<kBf16>(x[u].z, x[u].w),
                             pack16_exact<kBf16>(y[u].x, y[u].y), pack16_exact<kBf16>(y[u].z, y[u].w));
            }
          }
        }
        n_loaded = ncand;
        fence_proxy_async_smem();
        __syncwarp();
      }
      // ---- the item's product: scores[128 x n16] = Q kmean^T into buffer b
      const BarPhase need[2] = {{&sm.bar_q_full[s], static_cast<uint32_t>((n / kStagesQ) & 1)},
                                {n >= NG ? &sm.bar_free[b] : &sm.bar_q_full[s],
                                 static_cast<uint32_t>(n >= NG ? ((n / NG) - 1) & 1 : (n / kStagesQ) & 1)}};
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
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + g * buf_cols;
    const uint32_t gbar = 1 + g;                       // named barrier of the group's four warps
    for (int n = g; n < n_mine; n += NG) {
      // the item's plan data (written by the control warp a batch ahead)
      const int batch = n >> 5;
      bool got = mbar_wait(&sm.bar_meta[batch & (kMetaRing / 32 - 1)], (batch / (kMetaRing / 32)) & 1, wctx);
      const ItemMeta e = sm.meta[n & (kMetaRing - 1)];
      const int h = e.h, c0 = e.c0, ncand = got ? e.ncand : 0;
      const int tok = e.tok0 + gt;
      const bool valid = got && !e.empty && tok < e.tok_end;
      const int64_t slot0 = (static_cast<int64_t>(tok) * H + h) * kk;
      uint32_t* bitmap = bitmaps + static_cast<size_t>(g * 2 + ((n / NG) & 1)) * cand_rows * 4;
      for (int j = gt; j < ncand * 4; j += 128) bitmap[j] = 0u;
      got = got && mbar_wait(&sm.bar_mma[g], (n / NG) & 1, wctx);
      if (!got) sm.group_abort[g] = 1;
      asm volatile("bar.sync %0, 128;" ::"r"(gbar) : "memory");     // bitmap cleared; one view of the abort flag
      if (*reinterpret_cast<volatile int*>(&sm.group_abort[g])) break;
      tc_fence_after_sync();
      // ---- pass 1: the kk largest values, sorted, without branches
      float v[KMAX];
#pragma unroll
      for (int j = 0; j < KMAX; ++j) v[j] = -INFINITY;
      for (int cb = 0; cb < ncand; cb += 32) {
        uint32_t r[32];
        tmem_ld32(lane_addr + cb, r);
        tmem_wait_ld32(r);
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float sc = cb + c < ncand ? __uint_as_float(r[c]) : -INFINITY;
#pragma unroll
          for (int j = KMAX - 1; j > 0; --j) v[j] = fmaxf(fminf(v[j - 1], sc), v[j]);
          v[0] = fmaxf(v[0], sc);
        }
      }
      float thr = v[KMAX - 1];
#pragma unroll
      for (int j = 0; j < KMAX; ++j)
        if (j == kk - 1) thr = v[j];
      const int want = min(kk, ncand);
      // ---- pass 2: the candidates above the kk-th largest value, ascending; then ties at that value if a row
      // still lacks entries
      int cnt = 0;
      for (int pass = 0; pass < 2; ++pass) {
        if (pass == 1 && !__any_sync(0xffffffffu, valid && cnt < want)) break;
        for (int cb = 0; cb < ncand; cb += 32) {
          uint32_t r[32];
          tmem_ld32(lane_addr + cb, r);
          tmem_wait_ld32(r);
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const float sc = __uint_as_float(r[c]);
            const bool take = cb + c < ncand && cnt < want && (pass == 0 ? sc > thr : sc == thr);
            if (take) {
              if (valid) {
                sel[slot0 + cnt] = c0 + cb + c;
                if (sel_score) sel_score[slot0 + cnt] = sc;
                atomicOr(&bitmap[(cb + c) * 4 + (warp & 3)], 1u << lane);
              }
              ++cnt;
            }
          }
        }
      }
      // the scores are no longer needed: the buffer may take the product of item n + NG
      tc_fence_before_sync();
      mbar_arrive(&sm.bar_free[g]);
      if (valid)
        for (int j = cnt; j < kk; ++j) {
          sel[slot0 + j] = -1;
          if (sel_score) sel_score[slot0 + j] = -INFINITY;
        }
      asm volatile("bar.sync %0, 128;" ::"r"(gbar) : "memory");
      if (!e.empty) {
        const int64_t cnt0 = (static_cast<int64_t>(e.cand_off) * H) + static_cast<int64_t>(h) * ncand;
        for (int c = gt; c < ncand; c += 128)
          tile_cnt[cnt0 + c] = __popc(bitmap[c * 4]) + __popc(bitmap[c * 4 + 1]) + __popc(bitmap[c * 4 + 2]) +
                               __popc(bitmap[c * 4 + 3]);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kCtl) tmem_dealloc(tmem, NG * buf_cols);
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
  // The streaming kernel wins where a query row has few candidates (measured: 0.80 vs 1.23 ms at 31 candidates,
  // top-k 12); with a hundred or more candidates per row both kernels are bound by the instructions of the
  // thread-per-row scan, and the per-tile kernel's many small CTAs hide its latencies slightly better (3.6 vs 3.8 ms
  // at 125 candidates, 3.9 vs 4.6 ms at 255).
  if (max_cand <= kStreamMaxCand) {
    // streaming kernel: one persistent CTA per SM; four score buffers when they fit tensor memory (<= 128 columns each)
    const int rows = (max_cand + 15) & ~15;
    int cols = 32;
    while (cols < rows) cols *= 2;
    auto smem_for = [&](int groups) {
      return (groups == 4 ? sizeof(StreamSmem<4>) : sizeof(StreamSmem<2>)) + 1024 + static_cast<size_t>(rows) * 256 +
             static_cast<size_t>(rows) * 32 * groups;
    };
    constexpr size_t kSmemMax = 232448;
    int ng = cols <= 128 ? 4 : 2;
    if (smem_for(ng) > kSmemMax) ng = 2;
    const size_t smem_s = smem_for(ng);
    if (smem_s <= kSmemMax) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t blocks = static_cast<int64_t>((plan.n_qtiles + kBlockTiles - 1) / kBlockTiles) * H;
    const unsigned grid_s = static_cast<unsigned>(blocks < sms ? blocks : sms);
    auto run_s = [&](auto kern) -> int {
      MOBA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_s));
      kern<<<grid_s, ng * 128 + 32, smem_s, st>>>(mq, H, kmean, kv_rep, plan, sel, sel_score, tile_cnt, status, rows, cols);
      MOBA_CUDA_OK(cudaGetLastError());
      return 0;
    };
#define MOBA_GATE_STREAM(K)                                                                                  \
  return ng == 4 ? (bf16 ? run_s(gate_topk_stream_kernel<true, K, 4>) : run_s(gate_topk_stream_kernel<false, K, 4>)) \
                 : (bf16 ? run_s(gate_topk_stream_kernel<true, K, 2>) : run_s(gate_topk_stream_kernel<false, K, 2>))
    if (plan.kk <= 2) MOBA_GATE_STREAM(2);
    if (plan.kk <= 4) MOBA_GATE_STREAM(4);
    if (plan.kk <= 8) MOBA_GATE_STREAM(8);
    if (plan.kk <= 12) MOBA_GATE_STREAM(12);
    if (plan.kk <= 16) MOBA_GATE_STREAM(16);
    MOBA_GATE_STREAM(32);
#undef MOBA_GATE_STREAM
    }
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
  if (plan.kk <= 2) return bf16 ? run(gate_topk_umma_kernel<true, 2>) : run(gate_topk_umma_kernel<false, 2>);
  if (plan.kk <= 4) return bf16 ? run(gate_topk_umma_kernel<true, 4>) : run(gate_topk_umma_kernel<false, 4>);
  if (plan.kk <= 8) return bf16 ? run(gate_topk_umma_kernel<true, 8>) : run(gate_topk_umma_kernel<false, 8>);
  if (plan.kk <= 16) return bf16 ? run(gate_topk_umma_kernel<true, 16>) : run(gate_topk_umma_kernel<false, 16>);
  return bf16 ? run(gate_topk_umma_kernel<true, 32>) : run(gate_topk_umma_kernel<false, 32>);
}

}  // namespace moba
