// Backward, query side, for sm_100a (tcgen05 / TMEM). No atomics.
//
// One CTA per 128-row query tile (own-chunk tile or (chunk, head) list tile). The Q and dO tiles stay in shared
// memory; the CTA walks the keys of the chunk in tiles of 128 keys (j = 0, 1, ...; S buffer b = j & 1):
//   S_b = Q K_j^T, dP = dO V_j^T              operands in shared memory (K-major), 8 x UMMA 128x128x16 each
//   dS = exp2(S_b c - lse) (dP - delta) * scale               written over S_b as 16-bit pairs
//   dQ += dS K_j                               A from TMEM, B = the K tile read MN-major
// -> fp32 rows: dq_self [S,H,D] for own-chunk rows, part_dq [R*H, D] for list rows; the per-query sum and the
// single rounding to 16 bit happen in the merge kernel. Replaces the dq halves of both flash backward calls of
// MoonshotAI/MoBA moba/moba_efficient.py:208-264; lse / delta are the merged statistics, as there.
//
// Full-width (N = 128) products run at the tensor pipe's full rate, 64-wide ones at 2/3 of it (issue rate), so
// the tile is 128 keys wide: 1536 tensor clocks per tile instead of 2048. TMEM then holds two S buffers, ONE dP
// buffer and dQ (4 x 128 columns). The single dP buffer is enough because the compute warps copy S and dP of a
// tile into registers first and release dP at once (bar_dp_free); dP of the next tile is computed while the
// exponentials of this one run.
// Each kind of product has its own issuing warp (a warp with tcgen05.mma instructions queued does not see an
// mbarrier change until they have left the queue, measured on B200), and every wait of a round is polled
// together before the round's products. The tensor pipe may interleave the warps' instructions, so every
// dependency between them goes through an mbarrier.
// Warp roles (640 threads): 0-15 compute (warp & 3 = TMEM lane quarter, so thread = query row; warp >> 2 = which
// 32 of the tile's 128 key columns), 16 = MMA issue of S, 17 = of dP, 18 = of dQ, 19 = TMA producer (Q / dO tiles,
// then K through three slots and V through two: K_j is needed from S_j until dQ += dS_j K_j).
// TMEM columns: [0,128) S_0 / dS_0   [128,256) S_1 / dS_1   [256,384) dP   [384,512) dQ.
#include "attn_common.cuh"

namespace moba {
namespace {

constexpr int kDqThreads = 640;
constexpr int kComputeWarps = 16;
constexpr int kWarpS = 16, kWarpDp = 17, kWarpDq = 18, kTmaWarp = 19;
constexpr int kKSlots = 3, kVSlots = 2;


struct __align__(1024) DqSmem {
  uint8_t q[2][16384];              // [d half][128 rows x 64], 128-byte swizzle
  uint8_t d_o[2][16384];
  uint8_t k[kKSlots][2][16384];     // [slot][d half][128 keys x 64]
  uint8_t v[kVSlots][2][16384];
  uint64_t bar_qdo_full, bar_k_full[kKSlots], bar_k_empty[kKSlots], bar_v_full[kVSlots], bar_v_empty[kVSlots],
      bar_s_ready[2], bar_dp_ready, bar_dp_free, bar_ds_ready[2], bar_buf_free[2], bar_all_done;
  uint32_t tmem_base;
  int abort_flag;
  int work[8];
};

// One key tile of a compute warp (thread = query row, 32 of the tile's 128 key columns), shared by both forms of
// the kernel: wait for S and dP of the tile, take them into registers (dP's buffer is released at once), form
// dS = exp2(S c - lse) (dP - delta) * scale and write it over the S buffer as 16-bit pairs. `ncol` = how many of the
// tile's key columns exist for this row. Returns false when the wait was abandoned.
template <bool kBf16>
__device__ __forceinline__ bool dq_compute_tile(uint64_t* bar_s, uint32_t phase_s, uint64_t* bar_dp, uint32_t phase_dp,
                                                uint64_t* bar_dp_free, uint64_t* bar_ds, uint32_t t_s, uint32_t t_dp,
                                                int ci, int ncol, float lse2, float dlt, float sc, float scale,
                                                uint32_t quad_bar, const WaitCtx& wctx) {
  const BarPhase need[2] = {{bar_s, phase_s}, {bar_dp, phase_dp}};
  if (!__all_sync(0xffffffffu, mbar_wait_all(need, wctx))) {
    // warps of the lane quarter that saw the barriers complete may be waiting at the quarter's barrier: release them
    asm volatile("bar.arrive %0, 128;" ::"r"(quad_bar) : "memory");
    return false;
  }
  tc_fence_after_sync();
  const bool full = __all_sync(0xffffffffu, ncol >= 32 * ci + 32);
  uint32_t rs[32], rd[32];
  tmem_ld32(t_s + ci * 32, rs);
  tmem_ld32(t_dp + ci * 32, rd);
  tmem_wait_ld32(rs);
  tmem_wait_ld32(rd);
  // dP is in registers: the next tile's dP may overwrite the buffer
  tc_fence_before_sync();
  mbar_arrive(bar_dp_free);
  uint32_t pd[16];
  if (full) {
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      const float p0 = ex2_approx(fmaf(__uint_as_float(rs[2 * c]), sc, -lse2));
      const float p1 = ex2_approx(fmaf(__uint_as_float(rs[2 * c + 1]), sc, -lse2));
      pd[c] = pack2<kBf16>(p0 * fmaf(__uint_as_float(rd[2 * c]), scale, -dlt),
                           p1 * fmaf(__uint_as_float(rd[2 * c + 1]), scale, -dlt));
    }
  } else {
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      const int c0 = ci * 32 + 2 * c;
      float p0 = ex2_approx(fmaf(__uint_as_float(rs[2 * c]), sc, -lse2));
      float p1 = ex2_approx(fmaf(__uint_as_float(rs[2 * c + 1]), sc, -lse2));
      if (c0 >= ncol) p0 = 0.f;
      if (c0 + 1 >= ncol) p1 = 0.f;
      pd[c] = pack2<kBf16>(p0 * fmaf(__uint_as_float(rd[2 * c]), scale, -dlt),
                           p1 * fmaf(__uint_as_float(rd[2 * c + 1]), scale, -dlt));
    }
  }
  // the 16-bit results land on TMEM columns [0, 64) of the S buffer, which other warps of the lane quarter read
  // their fp32 inputs from: all four must have their inputs in registers first
  asm volatile("bar.sync %0, 128;" ::"r"(quad_bar) : "memory");
  tmem_st16(t_s + ci * 16, pd);
  tmem_wait_st();
  tc_fence_before_sync();
  mbar_arrive(bar_ds);
  return true;
}


template <bool kBf16, bool kGathered>
__global__ void __launch_bounds__(kDqThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                   const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                   const BwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  DqSmem& sm = *reinterpret_cast<DqSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  WaitCtx wctx{&sm.abort_flag, a.status};

  // ---- prologue: work item (warp 0), barriers (warp 1) and tensor memory (warp A0) in parallel --------------
  if (warp == 0) {
    int chunk = 0, head = 0, first = 0, n_rows = 0, key0 = 0, nkeys = 0, active = 1;
    if constexpr (kGathered) {
      const int w = blockIdx.x;
      const int E = a.n_experts;
      if (a.tile_rec) {
        // the tile's record: one 32-byte load (lanes 0-7) instead of the search below
        const int val = lane < 8 ? __ldg(&a.tile_rec[8 * static_cast<size_t>(w) + lane]) : 0;
        head = __shfl_sync(0xffffffffu, val, 0);
        first = __shfl_sync(0xffffffffu, val, 1);
        n_rows = __shfl_sync(0xffffffffu, val, 2);
        key0 = __shfl_sync(0xffffffffu, val, 3);
        nkeys = __shfl_sync(0xffffffffu, val, 4);
        active = n_rows > 0;
      } else if (w >= a.work_off[E]) {
        active = 0;
      } else {
        // which (chunk, head) list owns work tile w: the last e with work_off[e] <= w. A 32-way search, every
        // lane probing one entry per round (two dependent loads for up to 1024 lists instead of ten).
        int lo = 0, hi = E;
        while (hi - lo > 1) {
          const int step = (hi - lo + 31) / 32;
          const int idx = lo + (lane + 1) * step;
          const bool le = idx < hi && a.work_off[idx] <= w;
          const int n_le = __popc(__ballot_sync(0xffffffffu, le));     // the probes are ascending
          const int nlo = lo + n_le * step;
          hi = min(nlo + step, hi);
          lo = nlo;
        }
        const int e = lo;
        chunk = e / a.H;
        head = e - chunk * a.H;
        // four independent loads by four lanes
        int val = 0;
        if (lane == 0) val = a.list_off[e];
        else if (lane == 1) val = a.list_off[e + 1];
        else if (lane == 2) val = a.plan.chunk_start[chunk];
        else if (lane == 3) val = a.plan.chunk_start[chunk + 1];
        else if (lane == 4) val = a.work_off[e];
        const int l0 = __shfl_sync(0xffffffffu, val, 0), l1 = __shfl_sync(0xffffffffu, val, 1);
        const int c0 = __shfl_sync(0xffffffffu, val, 2), c1 = __shfl_sync(0xffffffffu, val, 3);
        const int w0 = __shfl_sync(0xffffffffu, val, 4);
        first = l0 + (w - w0) * MOBA_TILE;
        n_rows = min(MOBA_TILE, l1 - first);
        key0 = c0;
        nkeys = c1 - c0;
      }
    } else {
      const int t = blockIdx.x;
      head = blockIdx.y;
      chunk = a.plan.qtile_chunk[t];
      first = a.plan.qtile_start[t];
      key0 = a.plan.chunk_start[chunk];
      n_rows = min(MOBA_TILE, a.plan.chunk_start[chunk + 1] - first);
      nkeys = first + n_rows - key0;                 // causal: keys up to the last row of the tile
    }
    if (lane == 0) {
      sm.abort_flag = 0;
      sm.work[0] = chunk; sm.work[1] = head; sm.work[2] = first; sm.work[3] = n_rows;
      sm.work[5] = key0; sm.work[6] = nkeys; sm.work[7] = active;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int i = 0; i < kKSlots; ++i) {
        mbar_init(&sm.bar_k_full[i], 1);
        mbar_init(&sm.bar_k_empty[i], 1);
      }
      for (int i = 0; i < kVSlots; ++i) {
        mbar_init(&sm.bar_v_full[i], 1);
        mbar_init(&sm.bar_v_empty[i], 1);
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(&sm.bar_s_ready[i], 1);
        mbar_init(&sm.bar_ds_ready[i], kComputeWarps * 32);
        mbar_init(&sm.bar_buf_free[i], 1);
      }
      mbar_init(&sm.bar_dp_ready, 1);
      mbar_init(&sm.bar_dp_free, kComputeWarps * 32);
      mbar_init(&sm.bar_all_done, 1);
      mbar_init(&sm.bar_qdo_full, 1);
      mbar_fence_init();
    }
  } else if (warp == kWarpS) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (!sm.work[7]) {
    // no work for this CTA (the grid covers the largest possible number of list tiles)
    if (warp == kWarpS) tmem_dealloc(sm.tmem_base, 512);
    return;
  }
  const int head = sm.work[1], first = sm.work[2], n_rows = sm.work[3], key0 = sm.work[5], nkeys = sm.work[6];
  const int nkv = (nkeys + MOBA_TILE - 1) / MOBA_TILE;      // key tiles
  const uint32_t tmem = sm.tmem_base;
  const uint32_t tm_dp = tmem + 256, tm_dq = tmem + 384;

  float lse2 = INFINITY, dlt = 0.f;                  // padding rows: exp2(-inf) = 0
  const int row = tid & 127, ci = (warp >> 2) & 3;   // query row of a compute thread; its 32-column slice
  if (warp < kComputeWarps && row < n_rows) {
    // list tiles read the list-ordered copies (one coalesced load per warp), own-chunk tiles the [S,H] arrays
    if constexpr (kGathered) {
      lse2 = a.lse_g[first + row] * kLog2e;
      dlt = a.delta_g[first + row] * a.scale;
    } else {
      const size_t i = static_cast<size_t>(first + row) * a.H + head;
      lse2 = a.lse[i] * kLog2e;
      dlt = a.delta[i] * a.scale;
    }
  }

  if (warp == kTmaWarp) {
    // ================= TMA producer =================
    if (lane == 0) {
      // The Q and dO tiles: 128 consecutive rows of q / d_out (own-chunk tile) or of their list-ordered copies
      // (list tile). Rows past the end of the tile hold other rows' data or zeros and are neutralised by
      // lse = +inf (P = 0).
      const int hq = kGathered ? 0 : head;
      mbar_arrive_expect_tx(&sm.bar_qdo_full, 65536);
      tma_load_3d(smem_u32(sm.q[0]), &map_q, &sm.bar_qdo_full, 0, hq, first);
      tma_load_3d(smem_u32(sm.q[1]), &map_q, &sm.bar_qdo_full, 64, hq, first);
      tma_load_3d(smem_u32(sm.d_o[0]), &map_do, &sm.bar_qdo_full, 0, hq, first);
      tma_load_3d(smem_u32(sm.d_o[1]), &map_do, &sm.bar_qdo_full, 64, hq, first);
      const int head_kv = head / a.kv_rep;          // key/value head of this query head
      for (int j = 0; j < nkv; ++j) {
        const int t0 = key0 + j * MOBA_TILE;
        const int sk = j % kKSlots, sv = j % kVSlots;
        if (j >= kKSlots && !mbar_wait(&sm.bar_k_empty[sk], (j / kKSlots - 1) & 1, wctx)) break;
        mbar_arrive_expect_tx(&sm.bar_k_full[sk], 32768);
        tma_load_3d(smem_u32(sm.k[sk][0]), &map_k, &sm.bar_k_full[sk], 0, head_kv, t0);
        tma_load_3d(smem_u32(sm.k[sk][1]), &map_k, &sm.bar_k_full[sk], 64, head_kv, t0);
        if (j >= kVSlots && !mbar_wait(&sm.bar_v_empty[sv], (j / kVSlots - 1) & 1, wctx)) break;
        mbar_arrive_expect_tx(&sm.bar_v_full[sv], 32768);
        tma_load_3d(smem_u32(sm.v[sv][0]), &map_v, &sm.bar_v_full[sv], 0, head_kv, t0);
        tma_load_3d(smem_u32(sm.v[sv][1]), &map_v, &sm.bar_v_full[sv], 64, head_kv, t0);
      }
    }
  } else if (warp == kWarpS) {
    // ================= MMA issue: S_b = Q K_j^T =================
    const uint32_t leader = elect_one();
    constexpr uint32_t idesc = umma_idesc(128, 128, kBf16, false, false);
    const uint64_t q_km = umma_smem_desc(smem_u32(sm.q[0]), 16, 1024);
    const uint64_t k_km0 = umma_smem_desc(smem_u32(sm.k[0][0]), 16, 1024);
    bool ok = true;
    for (int j = 0; j < nkv && ok; ++j) {
      const int b = j & 1, sk = j % kKSlots;
      const BarPhase need[3] = {
          {&sm.bar_k_full[sk], static_cast<uint32_t>((j / kKSlots) & 1)},
          {&sm.bar_qdo_full, 0u},
          // S_b is free once dQ += dS_(j-2) K_(j-2) has read dS out of it
          {j >= 2 ? &sm.bar_buf_free[b] : &sm.bar_qdo_full, static_cast<uint32_t>(j >= 2 ? ((j >> 1) - 1) & 1 : 0)}};
      ok = __all_sync(0xffffffffu, mbar_wait_all(need, wctx));
      if (!ok) break;
      tc_fence_after_sync();
      const uint64_t k_km = k_km0 + static_cast<uint32_t>(sk) * (32768u >> 4);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t off = ((ks >> 2) * 16384u + (ks & 3) * 32u) >> 4;
        umma_ss_w(leader, tmem + b * 128u, q_km + off, k_km + off, idesc, ks > 0);
      }
      umma_commit_w(leader, &sm.bar_s_ready[b]);
    }
    if (!ok) __nanosleep(1000000);
  } else if (warp == kWarpDp) {
    // ================= MMA issue: dP = dO V_j^T =================
    const uint32_t leader = elect_one();
    constexpr uint32_t idesc = umma_idesc(128, 128, kBf16, false, false);
    const uint64_t do_km = umma_smem_desc(smem_u32(sm.d_o[0]), 16, 1024);
    const uint64_t v_km0 = umma_smem_desc(smem_u32(sm.v[0][0]), 16, 1024);
    bool ok = true;
    for (int j = 0; j < nkv && ok; ++j) {
      const int sv = j % kVSlots;
      const BarPhase need[3] = {
          {&sm.bar_v_full[sv], static_cast<uint32_t>((j / kVSlots) & 1)},
          {&sm.bar_qdo_full, 0u},
          // the one dP buffer is free once every compute thread holds dP_(j-1) in registers
          {j >= 1 ? &sm.bar_dp_free : &sm.bar_qdo_full, static_cast<uint32_t>(j >= 1 ? (j - 1) & 1 : 0)}};
      ok = __all_sync(0xffffffffu, mbar_wait_all(need, wctx));
      if (!ok) break;
      tc_fence_after_sync();
      const uint64_t v_km = v_km0 + static_cast<uint32_t>(sv) * (32768u >> 4);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t off = ((ks >> 2) * 16384u + (ks & 3) * 32u) >> 4;
        umma_ss_w(leader, tm_dp, do_km + off, v_km + off, idesc, ks > 0);
      }
      umma_commit_w(leader, &sm.bar_dp_ready);
      umma_commit_w(leader, &sm.bar_v_empty[sv]);
    }
    if (!ok) __nanosleep(1000000);
  } else if (warp == kWarpDq) {
    // ================= MMA issue: dQ += dS_b K_j =================
    const uint32_t leader = elect_one();
    constexpr uint32_t idesc = umma_idesc(128, 128, kBf16, false, true);
    const uint64_t k_mn0 = umma_smem_desc(smem_u32(sm.k[0][0]), 16384, 1024);    // K tile read MN-major
    bool ok = true;
    for (int j = 0; j < nkv && ok; ++j) {
      const int b = j & 1, sk = j % kKSlots;
      ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_ds_ready[b], (j >> 1) & 1, wctx));
      if (!ok) break;
      tc_fence_after_sync();
      const uint64_t k_mn = k_mn0 + static_cast<uint32_t>(sk) * (32768u >> 4);
      const uint32_t a_ds = tmem + b * 128u;
      const uint32_t acc = j > 0;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) umma_ts_w(leader, tm_dq, a_ds + ks * 8, k_mn + ((ks * 2048u) >> 4), idesc, ks > 0 ? 1u : acc);
      umma_commit_w(leader, &sm.bar_k_empty[sk]);      // S_j finished before dS_j existed
      umma_commit_w(leader, &sm.bar_buf_free[b]);
    }
    // dQ is complete when this warp's products are; all others precede the last of them through the barriers
    if (ok) umma_commit_w(leader, &sm.bar_all_done);
    else __nanosleep(1000000);
  } else {
    // ================= compute warps: thread = query row, 32 key columns =================
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t quad_bar = 1 + (warp & 3);      // named barrier shared by the four warps of a lane quarter
    const float sc = a.scale * kLog2e, scale = a.scale;
    bool ok = true;
    for (int j = 0; j < nkv && ok; ++j) {
      const int b = j & 1;
      int ncol = nkeys - j * MOBA_TILE;                            // keys of this tile that exist
      if constexpr (!kGathered) ncol = min(ncol, first + row - key0 - j * MOBA_TILE + 1);   // causal: key <= query
      ok = dq_compute_tile<kBf16>(&sm.bar_s_ready[b], (j >> 1) & 1, &sm.bar_dp_ready, j & 1, &sm.bar_dp_free,
                                  &sm.bar_ds_ready[b], tmem + lane_base + b * 128u, tm_dp + lane_base, ci, ncol, lse2,
                                  dlt, sc, scale, quad_bar, wctx);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_all_done, 0, wctx));
    // ---- epilogue: dQ rows -> global memory through shared memory, so that a warp writes whole 512-byte rows
    // (thread = row straight from TMEM writes 16 bytes per row and instruction: measured 6500 clocks per tile).
    // The K/V ring is idle by now; the staging rows are padded to 132 floats against bank conflicts.
    if (!ok) sm.abort_flag = 1;
    float* stage = reinterpret_cast<float*>(sm.k[0][0]);
    constexpr int kPitch = MOBA_HEAD_DIM + 4;
    static_assert(sizeof(sm.k) >= MOBA_TILE * kPitch * sizeof(float), "staging tile does not fit the K ring");
    if (ok) {
      tc_fence_after_sync();
      uint32_t r[32];
      tmem_ld32(tm_dq + lane_base + ci * 32, r);      // each of the four threads of a row: 32 of its 128 columns
      tmem_wait_ld32(r);
      uint4* d = reinterpret_cast<uint4*>(stage + row * kPitch + ci * 32);
#pragma unroll
      for (int i = 0; i < 8; ++i) d[i] = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
    }
    asm volatile("bar.sync 5, %0;" ::"n"(kComputeWarps * 32) : "memory");      // the sixteen compute warps
    if (*reinterpret_cast<volatile int*>(&sm.abort_flag) == 0) {
#pragma unroll
      for (int i = 0; i < MOBA_TILE / kComputeWarps; ++i) {
        const int r_out = warp * (MOBA_TILE / kComputeWarps) + i;
        if (r_out < n_rows) {
          size_t off;
          if constexpr (kGathered) off = static_cast<size_t>(first + r_out) * MOBA_HEAD_DIM;
          else off = (static_cast<size_t>(first + r_out) * a.H + head) * MOBA_HEAD_DIM;
          const uint4 val = *reinterpret_cast<const uint4*>(stage + r_out * kPitch + lane * 4);
          *reinterpret_cast<uint4*>(a.dq_f32 + off + lane * 4) = val;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kWarpS) tmem_dealloc(tmem, 512);
}


// ---------------------------------------------------------------------------------------------------------
// The same pipeline as a persistent kernel: one CTA per SM walks its share of the query tiles, and nothing of a
// tile's set-up or tear-down stands between two tiles any more. Tensor memory, barriers and the K / V rings are
// set up once and run through; the producer warp looks up the next tile's parameters (list search, offsets) ahead
// of everyone and publishes them in a small ring in shared memory; the Q / dO tiles of the next query tile are
// loaded as soon as the last S and dP products of the current one have read theirs; the finished dQ tile leaves
// tensor memory straight from the compute warps' registers with 32-byte stores (a thread's 32 columns are 128
// contiguous bytes of the fp32 row, whole sectors), so that no shared-memory staging tile is needed while the K / V
// ring already carries the next tile, and the next tile's first dQ product waits only for those registers.
// Round r of the walk gives CTA b the tile r * G + (b + r) mod G (G CTAs): every CTA meets every length of the
// causal own-chunk tiles equally often.
constexpr int kItemSlots = 4;

struct __align__(1024) DqPersistSmem {
  uint8_t q[2][16384];              // [d half][128 rows x 64], 128-byte swizzle
  uint8_t d_o[2][16384];
  uint8_t k[kKSlots][2][16384];     // [slot][d half][128 keys x 64]
  uint8_t v[kVSlots][2][16384];
  uint64_t bar_qdo_full, bar_qdo_free, bar_k_full[kKSlots], bar_k_empty[kKSlots], bar_v_full[kVSlots],
      bar_v_empty[kVSlots], bar_s_ready[2], bar_dp_ready, bar_dp_free, bar_ds_ready[2], bar_buf_free[2],
      bar_all_done, bar_dq_free, bar_item_full[kItemSlots], bar_item_empty[kItemSlots];
  TileItem item[kItemSlots];
  uint32_t tmem_base;
  int abort_flag;
};

template <bool kBf16, bool kGathered>
__global__ void __launch_bounds__(kDqThreads, 1)
attn_bwd_dq_persist_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                           const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                           const BwdArgs a, const int n_items_host) {
  extern __shared__ uint8_t smem_raw[];
  DqPersistSmem& sm = *reinterpret_cast<DqPersistSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  WaitCtx wctx{&sm.abort_flag, a.status};
  const int G = gridDim.x, cta = blockIdx.x;
  // list tiles: the number of work tiles is known on the device only
  const int n_items = kGathered ? __ldg(&a.work_off[a.n_experts]) : n_items_host;
  const int n_rounds = (n_items + G - 1) / G;
  auto item_of_round = [&](int r) { return r * G + (cta + r) % G; };     // >= n_items: none (last round only)

  if (warp == 1) {
    if (lane == 0) {
      sm.abort_flag = 0;
      for (int i = 0; i < kKSlots; ++i) {
        mbar_init(&sm.bar_k_full[i], 1);
        mbar_init(&sm.bar_k_empty[i], 1);
      }
      for (int i = 0; i < kVSlots; ++i) {
        mbar_init(&sm.bar_v_full[i], 1);
        mbar_init(&sm.bar_v_empty[i], 1);
      }
      for (int i = 0; i < 2; ++i) {
        mbar_init(&sm.bar_s_ready[i], 1);
        mbar_init(&sm.bar_ds_ready[i], kComputeWarps * 32);
        mbar_init(&sm.bar_buf_free[i], 1);
      }
      for (int i = 0; i < kItemSlots; ++i) {
        mbar_init(&sm.bar_item_full[i], 1);
        mbar_init(&sm.bar_item_empty[i], kComputeWarps + 3);     // one arrival per consuming warp
      }
      mbar_init(&sm.bar_dp_ready, 1);
      mbar_init(&sm.bar_dp_free, kComputeWarps * 32);
      mbar_init(&sm.bar_all_done, 1);
      mbar_init(&sm.bar_dq_free, kComputeWarps * 32);
      mbar_init(&sm.bar_qdo_full, 1);
      mbar_init(&sm.bar_qdo_free, 2);                             // the S and the dP issuing warps
      mbar_fence_init();
    }
  } else if (warp == kWarpS) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t tm_dp = tmem + 256, tm_dq = tmem + 384;

  // a consuming warp's copy of the parameters of round r (published by the producer warp)
  auto take_item = [&](int r, TileItem& it) -> bool {
    const int slot = r & (kItemSlots - 1);
    if (!__all_sync(0xffffffffu, mbar_wait(&sm.bar_item_full[slot], static_cast<uint32_t>((r / kItemSlots) & 1), wctx)))
      return false;
    it = sm.item[slot];
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.bar_item_empty[slot]);
    return true;
  };

  if (warp == kTmaWarp) {
    // ================= producer: tile parameters, then the tile's Q / dO and its K / V tiles =================
    int e_hint = 0, T = 0;
    bool ok = true;
    for (int r = 0; r < n_rounds && ok; ++r) {
      const int w = item_of_round(r);
      if (w >= n_items) break;
      const int slot = r & (kItemSlots - 1);
      if (r >= kItemSlots)
        ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_item_empty[slot], static_cast<uint32_t>((r / kItemSlots - 1) & 1), wctx));
      if (!ok) break;
      const TileItem it = lookup_tile<kGathered>(a, w, lane, e_hint);
      const int nkv = (it.nkeys + MOBA_TILE - 1) / MOBA_TILE;
      if (lane == 0) {
        sm.item[slot] = it;
        mbar_arrive(&sm.bar_item_full[slot]);
        const int hq = kGathered ? 0 : it.head;
        if (r > 0) {
          // the tiles are on their way into L2 while the buffers are still in use
          tma_prefetch_3d(&map_q, 0, hq, it.first);
          tma_prefetch_3d(&map_q, 64, hq, it.first);
          tma_prefetch_3d(&map_do, 0, hq, it.first);
          tma_prefetch_3d(&map_do, 64, hq, it.first);
        }
        const int head_kv = it.head / a.kv_rep;
        auto load_kv = [&](int j) -> bool {
          const int Tj = T + j, t0 = it.key0 + j * MOBA_TILE;
          const int sk = Tj % kKSlots, sv = Tj % kVSlots;
          if (Tj >= kKSlots && !mbar_wait(&sm.bar_k_empty[sk], (Tj / kKSlots - 1) & 1, wctx)) return false;
          mbar_arrive_expect_tx(&sm.bar_k_full[sk], 32768);
          tma_load_3d(smem_u32(sm.k[sk][0]), &map_k, &sm.bar_k_full[sk], 0, head_kv, t0);
          tma_load_3d(smem_u32(sm.k[sk][1]), &map_k, &sm.bar_k_full[sk], 64, head_kv, t0);
          if (Tj >= kVSlots && !mbar_wait(&sm.bar_v_empty[sv], (Tj / kVSlots - 1) & 1, wctx)) return false;
          mbar_arrive_expect_tx(&sm.bar_v_full[sv], 32768);
          tma_load_3d(smem_u32(sm.v[sv][0]), &map_v, &sm.bar_v_full[sv], 0, head_kv, t0);
          tma_load_3d(smem_u32(sm.v[sv][1]), &map_v, &sm.bar_v_full[sv], 64, head_kv, t0);
          return true;
        };
        // Q / dO first: the buffers are free once the previous tile's last S and dP products are done, which is
        // earlier than the ring slots of this tile's first K / V tiles are
        if (r > 0) ok = mbar_wait(&sm.bar_qdo_free, static_cast<uint32_t>((r - 1) & 1), wctx);
        if (ok) {
          mbar_arrive_expect_tx(&sm.bar_qdo_full, 65536);
          tma_load_3d(smem_u32(sm.q[0]), &map_q, &sm.bar_qdo_full, 0, hq, it.first);
          tma_load_3d(smem_u32(sm.q[1]), &map_q, &sm.bar_qdo_full, 64, hq, it.first);
          tma_load_3d(smem_u32(sm.d_o[0]), &map_do, &sm.bar_qdo_full, 0, hq, it.first);
          tma_load_3d(smem_u32(sm.d_o[1]), &map_do, &sm.bar_qdo_full, 64, hq, it.first);
        }
        for (int j = 0; j < nkv && ok; ++j) ok = load_kv(j);
      }
      ok = __all_sync(0xffffffffu, ok);
      T += nkv;
    }
    if (!ok) __nanosleep(1000000);     // let copies already in flight land before the CTA retires
  } else if (warp == kWarpS) {
    // ================= MMA issue: S_b = Q K_j^T =================
    const uint32_t leader = elect_one();
    constexpr uint32_t idesc = umma_idesc(128, 128, kBf16, false, false);
    const uint64_t q_km = umma_smem_desc(smem_u32(sm.q[0]), 16, 1024);
    const uint64_t k_km0 = umma_smem_desc(smem_u32(sm.k[0][0]), 16, 1024);
    bool ok = true;
    int T = 0;
    for (int r = 0; r < n_rounds && ok; ++r) {
      if (item_of_round(r) >= n_items) break;
      TileItem it;
      ok = take_item(r, it);
      if (!ok) break;
      const int nkv = (it.nkeys + MOBA_TILE - 1) / MOBA_TILE;
      for (int j = 0; j < nkv && ok; ++j) {
        const int Tj = T + j, b = Tj & 1, sk = Tj % kKSlots;
        const BarPhase need[3] = {
            {&sm.bar_k_full[sk], static_cast<uint32_t>((Tj / kKSlots) & 1)},
            {&sm.bar_qdo_full, static_cast<uint32_t>(r & 1)},
            // S_b is free once dQ += dS K of two tiles ago has read dS out of it
            {Tj >= 2 ? &sm.bar_buf_free[b] : &sm.bar_k_full[sk],
             static_cast<uint32_t>(Tj >= 2 ? ((Tj >> 1) - 1) & 1 : (Tj / kKSlots) & 1)}};
        ok = __all_sync(0xffffffffu, mbar_wait_all(need, wctx));
        if (!ok) break;
        tc_fence_after_sync();
        const uint64_t k_km = k_km0 + static_cast<uint32_t>(sk) * (32768u >> 4);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = ((ks >> 2) * 16384u + (ks & 3) * 32u) >> 4;
          umma_ss_w(leader, tmem + b * 128u, q_km + off, k_km + off, idesc, ks > 0);
        }
        umma_commit_w(leader, &sm.bar_s_ready[b]);
        if (j == nkv - 1) umma_commit_w(leader, &sm.bar_qdo_free);     // Q has been read for the last time
      }
      T += nkv;
    }
    if (!ok) __nanosleep(1000000);
  } else if (warp == kWarpDp) {
    // ================= MMA issue: dP = dO V_j^T =================
    const uint32_t leader = elect_one();
    constexpr uint32_t idesc = umma_idesc(128, 128, kBf16, false, false);
    const uint64_t do_km = umma_smem_desc(smem_u32(sm.d_o[0]), 16, 1024);
    const uint64_t v_km0 = umma_smem_desc(smem_u32(sm.v[0][0]), 16, 1024);
    bool ok = true;
    int T = 0;
    for (int r = 0; r < n_rounds && ok; ++r) {
      if (item_of_round(r) >= n_items) break;
      TileItem it;
      ok = take_item(r, it);
      if (!ok) break;
      const int nkv = (it.nkeys + MOBA_TILE - 1) / MOBA_TILE;
      for (int j = 0; j < nkv && ok; ++j) {
        const int Tj = T + j, sv = Tj % kVSlots;
        const BarPhase need[3] = {
            {&sm.bar_v_full[sv], static_cast<uint32_t>((Tj / kVSlots) & 1)},
            {&sm.bar_qdo_full, static_cast<uint32_t>(r & 1)},
            // the one dP buffer is free once every compute thread holds the previous dP in registers
            {Tj >= 1 ? &sm.bar_dp_free : &sm.bar_v_full[sv],
             static_cast<uint32_t>(Tj >= 1 ? (Tj - 1) & 1 : (Tj / kVSlots) & 1)}};
        ok = __all_sync(0xffffffffu, mbar_wait_all(need, wctx));
        if (!ok) break;
        tc_fence_after_sync();
        const uint64_t v_km = v_km0 + static_cast<uint32_t>(sv) * (32768u >> 4);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = ((ks >> 2) * 16384u + (ks & 3) * 32u) >> 4;
          umma_ss_w(leader, tm_dp, do_km + off, v_km + off, idesc, ks > 0);
        }
        umma_commit_w(leader, &sm.bar_dp_ready);
        umma_commit_w(leader, &sm.bar_v_empty[sv]);
        if (j == nkv - 1) umma_commit_w(leader, &sm.bar_qdo_free);     // dO has been read for the last time
      }
      T += nkv;
    }
    if (!ok) __nanosleep(1000000);
  } else if (warp == kWarpDq) {
    // ================= MMA issue: dQ += dS_b K_j =================
    const uint32_t leader = elect_one();
    constexpr uint32_t idesc = umma_idesc(128, 128, kBf16, false, true);
    const uint64_t k_mn0 = umma_smem_desc(smem_u32(sm.k[0][0]), 16384, 1024);    // K tile read MN-major
    bool ok = true;
    int T = 0;
    for (int r = 0; r < n_rounds && ok; ++r) {
      if (item_of_round(r) >= n_items) break;
      TileItem it;
      ok = take_item(r, it);
      if (!ok) break;
      const int nkv = (it.nkeys + MOBA_TILE - 1) / MOBA_TILE;
      for (int j = 0; j < nkv && ok; ++j) {
        const int Tj = T + j, b = Tj & 1, sk = Tj % kKSlots;
        const bool fresh = j == 0 && r > 0;     // a new dQ tile: the previous one must have left tensor memory
        const BarPhase need[2] = {
            {&sm.bar_ds_ready[b], static_cast<uint32_t>((Tj >> 1) & 1)},
            {fresh ? &sm.bar_dq_free : &sm.bar_ds_ready[b],
             static_cast<uint32_t>(fresh ? (r - 1) & 1 : (Tj >> 1) & 1)}};
        ok = __all_sync(0xffffffffu, mbar_wait_all(need, wctx));
        if (!ok) break;
        tc_fence_after_sync();
        const uint64_t k_mn = k_mn0 + static_cast<uint32_t>(sk) * (32768u >> 4);
        const uint32_t a_ds = tmem + b * 128u;
        const uint32_t acc = j > 0;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ts_w(leader, tm_dq, a_ds + ks * 8, k_mn + ((ks * 2048u) >> 4), idesc, ks > 0 ? 1u : acc);
        umma_commit_w(leader, &sm.bar_k_empty[sk]);      // S_j finished before dS_j existed
        umma_commit_w(leader, &sm.bar_buf_free[b]);
      }
      // the tile's dQ is complete when this warp's products are
      if (ok) umma_commit_w(leader, &sm.bar_all_done);
      T += nkv;
    }
    if (!ok) __nanosleep(1000000);
  } else {
    // ================= compute warps: thread = query row, 32 key columns =================
    // A tile's parameters stay in their slot of the ring until its dQ has been written (the warp's arrival on
    // the slot's "empty" barrier comes last), so they are read from shared memory where needed instead of living
    // in registers across the key-tile loop.
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t quad_bar = 1 + (warp & 3);      // named barrier shared by the four warps of a lane quarter
    const float sc = a.scale * kLog2e, scale = a.scale;
    const int row = tid & 127, ci = (warp >> 2) & 3;   // query row of the thread; its 32-column slice
    // rounds in which this CTA has a tile: all of them, except possibly the last
    const int my_rounds = n_rounds - ((n_rounds > 0 && item_of_round(n_rounds - 1) >= n_items) ? 1 : 0);
    auto wait_item = [&](int r) -> bool {
      return __all_sync(0xffffffffu, mbar_wait(&sm.bar_item_full[r & (kItemSlots - 1)],
                                               static_cast<uint32_t>((r / kItemSlots) & 1), wctx));
    };
    // log-sum-exp (log2 units) and delta * scale of the thread's row in the tile of round r; padding rows: exp2(-inf) = 0
    auto row_stats = [&](int r, float& lse2, float& dlt) {
      const TileItem& it = sm.item[r & (kItemSlots - 1)];
      lse2 = INFINITY;
      dlt = 0.f;
      if (row < it.n_rows) {
        if constexpr (kGathered) {
          lse2 = __ldg(&a.lse_g[it.first + row]) * kLog2e;
          dlt = __ldg(&a.delta_g[it.first + row]) * a.scale;
        } else {
          const size_t i = static_cast<size_t>(it.first + row) * a.H + it.head;
          lse2 = __ldg(&a.lse[i]) * kLog2e;
          dlt = __ldg(&a.delta[i]) * a.scale;
        }
      }
    };
    // dQ of round r: tensor memory -> registers -> global memory, then the tile's slot of the ring is released.
    auto drain = [&](int r) -> bool {
      if (!__all_sync(0xffffffffu, mbar_wait(&sm.bar_all_done, static_cast<uint32_t>(r & 1), wctx))) return false;
      tc_fence_after_sync();
      uint32_t rq[32];
      tmem_ld32(tm_dq + lane_base + ci * 32, rq);
      tmem_wait_ld32(rq);
      tc_fence_before_sync();
      mbar_arrive(&sm.bar_dq_free);          // the accumulator may be overwritten by the next tile's first product
      const TileItem& it = sm.item[r & (kItemSlots - 1)];
      const int n_rows = it.n_rows;
      const int row0 = (row & ~3);             // first row of the quad
      size_t off, pitch;
      if constexpr (kGathered) {
        off = static_cast<size_t>(it.first + row0) * MOBA_HEAD_DIM;
        pitch = MOBA_HEAD_DIM;
      } else {
        off = (static_cast<size_t>(it.first + row0) * a.H + it.head) * MOBA_HEAD_DIM;
        pitch = static_cast<size_t>(a.H) * MOBA_HEAD_DIM;
      }
      // A thread holds 32 consecutive columns (four 32-byte pieces) of its row; the four lanes of a quad swap pieces
      // so that each store instruction writes whole 128-byte lines instead of 32 bytes to each of 32 lines.
      quad_transpose_pieces(rq, lane);
      store_quad_rows(a.dq_f32 + off + ci * 32 + (lane & 3) * 8, pitch, n_rows - row0, rq);
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.bar_item_empty[r & (kItemSlots - 1)]);
      return true;
    };
    bool ok = true;
    int T = 0;
    float lse2 = INFINITY, dlt = 0.f, lse2_n = INFINITY, dlt_n = 0.f;
    if (my_rounds > 0) {
      ok = wait_item(0);
      if (ok) row_stats(0, lse2, dlt);
    }
    for (int r = 0; r < my_rounds && ok; ++r) {
      const int nkeys = sm.item[r & (kItemSlots - 1)].nkeys;
      const int nkv = (nkeys + MOBA_TILE - 1) / MOBA_TILE;
      int causal_off = 0;                      // own-chunk tiles: query position relative to the chunk's first key
      if constexpr (!kGathered) causal_off = sm.item[r & (kItemSlots - 1)].first + row - sm.item[r & (kItemSlots - 1)].key0 + 1;
      // one key tile; false when a wait was abandoned
      auto key_tile = [&](const int j) -> bool {
        if (j == nkv - 1 && r + 1 < my_rounds) {
          // the next tile's row statistics are fetched under this tile's last key tile
          ok = wait_item(r + 1);
          if (!ok) {
            asm volatile("bar.arrive %0, 128;" ::"r"(quad_bar) : "memory");
            return false;
          }
          row_stats(r + 1, lse2_n, dlt_n);
        }
        const int Tj = T + j, b = Tj & 1;
        int ncol = nkeys - j * MOBA_TILE;                            // keys of this tile that exist
        if constexpr (!kGathered) ncol = min(ncol, causal_off - j * MOBA_TILE);   // causal: key <= query
        if (!dq_compute_tile<kBf16>(&sm.bar_s_ready[b], (Tj >> 1) & 1, &sm.bar_dp_ready, Tj & 1, &sm.bar_dp_free,
                                    &sm.bar_ds_ready[b], tmem + lane_base + b * 128u, tm_dp + lane_base, ci, ncol,
                                    lse2, dlt, sc, scale, quad_bar, wctx))
          return false;
        return true;
      };
      // The first key tile stands apart from the loop over the others: after it the previous query tile's dQ
      // leaves (its last product runs meanwhile, and the tensor pipe has S and dP of the next key tiles to do
      // while the rows are written), and the loop itself stays small.
      ok = key_tile(0);
      if (ok && r > 0) ok = drain(r - 1);
      for (int j = 1; j < nkv && ok; ++j) ok = key_tile(j);
      if (!ok) break;
      T += nkv;
      lse2 = lse2_n;
      dlt = dlt_n;
    }
    if (ok && my_rounds > 0) drain(my_rounds - 1);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kWarpS) tmem_dealloc(tmem, 512);
}

}  // namespace
}  // namespace moba


extern "C" int moba_attn_bwd_dq(const void* q, const void* k, const void* v, const void* d_out, int32_t dtype,
                                int32_t H, int64_t stride_s, int64_t stride_h, const moba_kv_layout* kv,
                                const moba_plan_info* info, const int32_t* meta_dev, const int32_t* list_off,
                                const int32_t* work_off, const int32_t* list_tok, const int32_t* tile_rec, const void* qg, const void* dog, const float* lse_g,
                                const float* delta_g, const float* lse, const float* delta, float* dq,
                                float* part_dq, int32_t parts, float softmax_scale, int32_t* status, int32_t device,
                                void* stream) {
  using namespace moba;
  const int32_t form = parts & (MOBA_DQ_FORM_TILE | MOBA_DQ_FORM_PERSISTENT);
  parts &= ~(MOBA_DQ_FORM_TILE | MOBA_DQ_FORM_PERSISTENT);
  MOBA_REQUIRE(parts >= 1 && parts <= 3, MOBA_ERR_ARG, "parts=%d must be 1 (own chunk), 2 (lists) or 3 (both)", parts);
  MOBA_REQUIRE(form != (MOBA_DQ_FORM_TILE | MOBA_DQ_FORM_PERSISTENT), MOBA_ERR_ARG, "two kernel forms named in parts");
  int rc = check_bwd_args(q, k, v, d_out, dtype, H, stride_s, stride_h, info, meta_dev, lse, delta, status);
  if (rc) return rc;
  MOBA_REQUIRE(dq || !(parts & 1), MOBA_ERR_ARG, "null pointer argument");
  if (info->kk > 0 && (parts & 2)) MOBA_REQUIRE(list_off && work_off && list_tok && part_dq, MOBA_ERR_ARG, "null list / partial buffers");
  MOBA_SET_DEVICE(device);
  if (info->n_qtiles == 0) return 0;
  CUtensorMap mk, mv;   // 128-key boxes
  BwdArgs a;
  rc = make_kv_maps(&mk, &mv, k, v, dtype, H, stride_s, stride_h, kv, info, &a.kv_rep);
  if (rc) return rc;
  // 128-row boxes of Q / dO: own-chunk tiles from q / d_out, list tiles from the list-ordered copies
  const bool lists = (parts & 2) && info->kk > 0 && info->max_work_tiles_per_head > 0;
  CUtensorMap mq, mdo, mqg, mdog;
  const int64_t q_rows = (parts & 1) ? info->total_tokens : 1;
  rc = make_tensor_map_shd(&mq, q, dtype, q_rows, H, stride_s, stride_h, MOBA_TILE);
  if (rc) return rc;
  rc = make_tensor_map_shd(&mdo, d_out, dtype, q_rows, H, stride_s, stride_h, MOBA_TILE);
  if (rc) return rc;
  mqg = mq;
  mdog = mdo;
  if (lists) {
    MOBA_REQUIRE(qg && dog && lse_g && delta_g, MOBA_ERR_ARG, "null list-ordered buffers");
    const int64_t n_list_rows = info->rows_per_head * H;
    rc = make_tensor_map_shd(&mqg, qg, dtype, n_list_rows, 1, MOBA_HEAD_DIM, MOBA_HEAD_DIM, MOBA_TILE);
    if (rc) return rc;
    rc = make_tensor_map_shd(&mdog, dog, dtype, n_list_rows, 1, MOBA_HEAD_DIM, MOBA_HEAD_DIM, MOBA_TILE);
    if (rc) return rc;
  }
  a.q = static_cast<const uint16_t*>(q);
  a.d_out = static_cast<const uint16_t*>(d_out);
  a.stride_s = stride_s; a.stride_h = stride_h; a.H = H; a.lse_g = lse_g; a.delta_g = delta_g; a.parts = parts;
  a.scale = softmax_scale_or_default(softmax_scale);
  a.plan = make_plan_dev(info, meta_dev);
  a.list_off = list_off; a.work_off = work_off; a.list_tok = list_tok; a.tile_rec = tile_rec;
  a.lse = lse; a.delta = delta;
  a.o0 = nullptr; a.o1 = nullptr; a.dq_f32 = dq;
  a.status = status;
  a.n_experts = info->n_chunks * H;
  BwdArgs g = a;
  g.dq_f32 = part_dq;
  const size_t smem = sizeof(DqSmem) + 1024;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto run = [&](auto k_self, auto k_gath) -> int {
    MOBA_CUDA_OK(cudaFuncSetAttribute(k_self, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MOBA_CUDA_OK(cudaFuncSetAttribute(k_gath, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (lists) {
      const int64_t nw = info->max_work_tiles_per_head * H;
      MOBA_REQUIRE(nw < (1ll << 31), MOBA_ERR_LIMIT, "too many gathered tiles");
      k_gath<<<static_cast<unsigned>(nw), kDqThreads, smem, st>>>(mk, mv, mqg, mdog, g);
      MOBA_CUDA_OK(cudaGetLastError());
    }
    if (parts & 1) {
      dim3 grid(info->n_qtiles, H);
      k_self<<<grid, kDqThreads, smem, st>>>(mk, mv, mq, mdo, a);
      MOBA_CUDA_OK(cudaGetLastError());
    }
    return 0;
  };
  // Query tiles with few key tiles go through the persistent kernel (the per-tile set-up is what they spend their
  // time on); long ones through the one-tile-per-CTA kernel, whose steady state is a few percent faster.
  const bool persist = form ? form == MOBA_DQ_FORM_PERSISTENT : info->chunk_size <= 16 * MOBA_TILE;
  if (persist) {
    int n_sm = 0;
    MOBA_CUDA_OK(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, device));
    const size_t smem_p = sizeof(DqPersistSmem) + 1024;
    auto run_p = [&](auto k_self, auto k_gath) -> int {
      MOBA_CUDA_OK(cudaFuncSetAttribute(k_self, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_p));
      MOBA_CUDA_OK(cudaFuncSetAttribute(k_gath, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_p));
      if (lists) {
        const int64_t nw = info->max_work_tiles_per_head * H;       // upper bound; the kernel reads the exact count
        MOBA_REQUIRE(nw < (1ll << 31), MOBA_ERR_LIMIT, "too many gathered tiles");
        const unsigned grid = static_cast<unsigned>(nw < n_sm ? nw : n_sm);
        k_gath<<<grid, kDqThreads, smem_p, st>>>(mk, mv, mqg, mdog, g, -1);
        MOBA_CUDA_OK(cudaGetLastError());
      }
      if (parts & 1) {
        const int64_t n_items = static_cast<int64_t>(info->n_qtiles) * H;
        MOBA_REQUIRE(n_items < (1ll << 31), MOBA_ERR_LIMIT, "too many query tiles");
        const unsigned grid = static_cast<unsigned>(n_items < n_sm ? n_items : n_sm);
        k_self<<<grid, kDqThreads, smem_p, st>>>(mk, mv, mq, mdo, a, static_cast<int>(n_items));
        MOBA_CUDA_OK(cudaGetLastError());
      }
      return 0;
    };
    if (dtype == MOBA_DTYPE_BF16)
      return run_p(attn_bwd_dq_persist_kernel<true, false>, attn_bwd_dq_persist_kernel<true, true>);
    return run_p(attn_bwd_dq_persist_kernel<false, false>, attn_bwd_dq_persist_kernel<false, true>);
  }
  if (dtype == MOBA_DTYPE_BF16) return run(attn_bwd_dq_kernel<true, false>, attn_bwd_dq_kernel<true, true>);
  return run(attn_bwd_dq_kernel<false, false>, attn_bwd_dq_kernel<false, true>);
}


