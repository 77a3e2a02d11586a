// Forward attention tiles for sm_100a: tcgen05 MMA with accumulators in tensor memory, K/V tiles fed by TMA,
// online softmax in registers.
//
// One CTA computes one 128-row query tile against a run of 128-key tiles:
//   self mode      rows = 128 consecutive tokens of a chunk, keys = the chunk up to the diagonal (causal)
//                  -> out [S,H,D], lse [S,H]      (MoonshotAI/MoBA moba/moba_efficient.py:89-102)
//   gathered mode  rows = 128 entries of one (chunk, head) query list, keys = the whole chunk
//                  -> part_o [R*H, D], part_lse   (moba/moba_efficient.py:105-116; the Q gather of :381-386 and
//                  the KV regrouping of :406-414 happen here by index instead of through copies)
//
// Per key tile j:
//   S = Q K_j^T          8 x UMMA 128x128x16, operands in shared memory (K-major), fp32 result in TMEM
//   P = exp2(S c - m) rounded to 16 bit, written back over S (two values per column)
//   O += P V_j           8 x UMMA, A from TMEM, B = V tile read MN-major
// A CTA is deliberately half an SM: 256 TMEM columns, < 113 KB of shared memory, 320 threads, so that two CTAs
// are resident per SM. Within a CTA the steps of a tile depend on one another (S -> softmax -> P V -> next S) and
// use the tensor pipe and the exp2 unit in turns (each needs ~1024 clocks per tile); the second CTA fills the
// other half of both, and the prologue and epilogue of one CTA (TMEM allocation, Q gather, first loads, final
// store: a quarter of a work item's time when CTAs ran one per SM) overlap with the steady state of the other.
// The probabilities are computed in the same pass as the row maximum, against the maximum in use; that one is
// only raised when the true maximum exceeds it by more than 8 (log2 units; rare after the first tiles), and only
// then are the tile's probabilities computed again and O rescaled. The row sum uses the same stale maximum, so
// the result is exact.
//
// A warp with tcgen05.mma instructions queued does not see an mbarrier change until they have left the queue
// (measured on B200), so the MMA warp waits for P_j, V_j and K_(j+1) in one round of overlapping try_waits and then
// issues P V_j and Q K_(j+1)^T back to back.
//
// Warp roles (320 threads): 0-7 softmax (warp & 3 = TMEM lane quarter, so thread = query row; warp >> 2 = which
// 64 of the tile's 128 key columns, handled in two passes of 32; the two threads of a row exchange their maxima
// through shared memory), 8 = MMA issue (warp-converged, one elected lane), 9 = TMA producer (one K slot, one V
// slot: K_(j+1) is fetched while the softmax of tile j runs, V_(j+1) while S_(j+1) is computed).
// TMEM columns: [0,128) S / P   [128,256) O.
#include "attn_common.cuh"

namespace moba {
namespace {

constexpr int kFwdThreads = 320;
constexpr int kSoftmaxWarps = 8;
constexpr int kMmaWarp = 8, kTmaWarp = 9;
constexpr int kTmemCols = 256;
constexpr float kRescaleThreshold = 8.0f;


struct __align__(1024) FwdSmem {
  uint8_t q[2][16384];              // [128 rows x 64] sub-tiles, 128-byte swizzle (d 0..63 | d 64..127)
  uint8_t k[2][16384];              // the K tile in use / in flight
  uint8_t v[2][16384];              // the V tile in use / in flight
  float xchg[2][128];               // [column half][row]: row maxima, then row sums, of the two threads of a row
  uint64_t bar_k_full, bar_k_empty, bar_v_full, bar_v_empty, bar_s_ready, bar_p_ready, bar_pv_done, bar_all_done;
  uint32_t tmem_base;
  int abort_flag;
  int work[8];           // chunk, head, first row / token, n_rows, nkv, key token start, keys in chunk, active
};

struct FwdArgs {
  const uint16_t* q;
  int64_t stride_s, stride_h;
  int H;
  PlanDev plan;
  const int32_t* list_off;
  const int32_t* work_off;
  const int32_t* list_tok;
  const int32_t* tile_rec;   // work-tile records (moba_tile_records), or null: search work_off
  uint16_t* out;        // self: [S,H,D] contiguous; gathered: part_o [R*H, D]
  float* lse;           // self: [S,H]; gathered: part_lse [R*H]
  int* status;
  int n_experts;
  float scale_log2;     // softmax scale * log2(e)
  int kv_rep;           // query heads per key/value head
};

template <bool kBf16, bool kGathered>
__global__ void __launch_bounds__(kFwdThreads, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                const FwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  FwdSmem& sm = *reinterpret_cast<FwdSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  WaitCtx wctx{&sm.abort_flag, a.status};

  // ---- prologue: work item (warp 0), barriers (warp 1) and tensor memory (MMA warp) in parallel ---------------
  if (warp == 0) {
    int chunk = 0, head = 0, first = 0, n_rows = 0, nkv = 0, key0 = 0, nkeys = 0, active = 1;
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
        nkv = (nkeys + MOBA_TILE - 1) / MOBA_TILE;
        active = n_rows > 0;
      } else if (w >= a.work_off[E]) {
        active = 0;
      } else {
        // which (chunk, head) list owns work tile w: the last e with work_off[e] <= w. A 32-way search, every
        // lane probing one entry per round (three dependent loads for 30000 lists instead of fifteen).
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
        int val = 0;                                    // five independent loads by five lanes
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
        nkv = (nkeys + MOBA_TILE - 1) / MOBA_TILE;
      }
    } else {
      const int t = blockIdx.x;
      head = blockIdx.y;
      chunk = a.plan.qtile_chunk[t];
      first = a.plan.qtile_start[t];
      key0 = a.plan.chunk_start[chunk];
      n_rows = min(MOBA_TILE, a.plan.chunk_start[chunk + 1] - first);
      nkeys = first + n_rows - key0;                 // causal: keys up to the last row of the tile
      nkv = (nkeys + MOBA_TILE - 1) / MOBA_TILE;
    }
    if (lane == 0) {
      sm.abort_flag = 0;
      sm.work[0] = chunk; sm.work[1] = head; sm.work[2] = first; sm.work[3] = n_rows;
      sm.work[4] = nkv; sm.work[5] = key0; sm.work[6] = nkeys; sm.work[7] = active;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      mbar_init(&sm.bar_k_full, 1);
      mbar_init(&sm.bar_k_empty, 1);
      mbar_init(&sm.bar_v_full, 1);
      mbar_init(&sm.bar_v_empty, 1);
      mbar_init(&sm.bar_s_ready, 1);
      mbar_init(&sm.bar_p_ready, kSoftmaxWarps * 32);
      mbar_init(&sm.bar_pv_done, 1);
      mbar_init(&sm.bar_all_done, 1);
      mbar_fence_init();
    }
  } else if (warp == kMmaWarp) {
    tmem_alloc(&sm.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (!sm.work[7]) {
    // no work for this CTA (the grid covers the largest possible number of list tiles)
    if (warp == kMmaWarp) tmem_dealloc(sm.tmem_base, kTmemCols);
    return;
  }
  const int head = sm.work[1], first = sm.work[2], n_rows = sm.work[3], nkv = sm.work[4], key0 = sm.work[5],
            nkeys = sm.work[6];
  const int head_kv = head / a.kv_rep;               // key/value head of this query head
  const int row = tid & 127, ch = (warp >> 2) & 1;   // query row of a softmax thread; its 64-column half

  if (warp == kTmaWarp && lane == 0) {
    // the first K and V tiles travel while the Q rows are gathered
    mbar_arrive_expect_tx(&sm.bar_k_full, 32768);
    tma_load_3d(smem_u32(sm.k[0]), &map_k, &sm.bar_k_full, 0, head_kv, key0);
    tma_load_3d(smem_u32(sm.k[1]), &map_k, &sm.bar_k_full, 64, head_kv, key0);
    mbar_arrive_expect_tx(&sm.bar_v_full, 32768);
    tma_load_3d(smem_u32(sm.v[0]), &map_v, &sm.bar_v_full, 0, head_kv, key0);
    tma_load_3d(smem_u32(sm.v[1]), &map_v, &sm.bar_v_full, 64, head_kv, key0);
  }

  // ---- Q tile: rows gathered by token index into the swizzled K-major layout (256 threads: 16 per row, eight rows
  // each; a thread reads the tokens of its eight rows itself, all eight loads in flight together) -----------
  if (warp < 8) {
    const int c16 = tid & 15, r0 = tid >> 4;
    int toks[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = r0 + 16 * i;
      toks[i] = r < n_rows ? (kGathered ? __ldg(&a.list_tok[first + r]) : first + r) : -1;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = r0 + 16 * i;
      const uint32_t d = smem_u32(sm.q[0]) + (c16 >> 3) * 16384u + sw128_offset(r, c16 & 7);
      if (toks[i] >= 0) {
        cp_async16(d, a.q + static_cast<int64_t>(toks[i]) * a.stride_s + static_cast<int64_t>(head) * a.stride_h + c16 * 8);
      } else {
        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(d), "r"(0u) : "memory");   // rows past the tile's end
      }
    }
    cp_async_wait_all();
    fence_proxy_async_smem();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t tmem_o = tmem + 128;

  if (warp == kTmaWarp) {
    // ================= TMA producer: K_1, V_1, K_2, V_2, ... through one slot each (K_0, V_0 are on their way)
    if (lane == 0) {
      for (int j = 1; j < nkv; ++j) {
        const int t0 = key0 + j * MOBA_TILE;
        if (!mbar_wait(&sm.bar_k_empty, (j - 1) & 1, wctx)) break;
        mbar_arrive_expect_tx(&sm.bar_k_full, 32768);
        tma_load_3d(smem_u32(sm.k[0]), &map_k, &sm.bar_k_full, 0, head_kv, t0);
        tma_load_3d(smem_u32(sm.k[1]), &map_k, &sm.bar_k_full, 64, head_kv, t0);
        if (!mbar_wait(&sm.bar_v_empty, (j - 1) & 1, wctx)) break;
        mbar_arrive_expect_tx(&sm.bar_v_full, 32768);
        tma_load_3d(smem_u32(sm.v[0]), &map_v, &sm.bar_v_full, 0, head_kv, t0);
        tma_load_3d(smem_u32(sm.v[1]), &map_v, &sm.bar_v_full, 64, head_kv, t0);
      }
    }
  } else if (warp == kMmaWarp) {
    // ================= MMA issue =================
    const uint32_t leader = elect_one();
    constexpr uint32_t idesc_s = umma_idesc(128, 128, kBf16, false, false);
    constexpr uint32_t idesc_o = umma_idesc(128, 128, kBf16, false, true);
    const uint64_t q_km = umma_smem_desc(smem_u32(sm.q[0]), 16, 1024);
    const uint64_t k_km = umma_smem_desc(smem_u32(sm.k[0]), 16, 1024);       // K tile: K-major
    const uint64_t v_mn = umma_smem_desc(smem_u32(sm.v[0]), 16384, 1024);    // V tile: MN-major
    auto issue_s = [&]() {        // S = Q K_j^T
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t off = ((ks >> 2) * 16384u + (ks & 3) * 32u) >> 4;
        umma_ss_w(leader, tmem, q_km + off, k_km + off, idesc_s, ks > 0);
      }
      umma_commit_w(leader, &sm.bar_s_ready);
      umma_commit_w(leader, &sm.bar_k_empty);
    };
    bool ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_k_full, 0, wctx));
    if (ok) {
      tc_fence_after_sync();
      issue_s();
    }
    for (int j = 0; j < nkv && ok; ++j) {
      // every wait comes before the products of this round: P_j, V_j and K_(j+1)
      const bool more = j + 1 < nkv;
      const BarPhase need[3] = {
          {&sm.bar_p_ready, static_cast<uint32_t>(j & 1)},
          {&sm.bar_v_full, static_cast<uint32_t>(j & 1)},
          // no next tile: name the V barrier again
          {more ? &sm.bar_k_full : &sm.bar_v_full, static_cast<uint32_t>(more ? (j + 1) & 1 : j & 1)}};
      ok = __all_sync(0xffffffffu, mbar_wait_all(need, wctx));
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t acc = j > 0;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) umma_ts_w(leader, tmem_o, tmem + ks * 8, v_mn + ((ks * 2048u) >> 4), idesc_o, ks > 0 ? 1u : acc);
      umma_commit_w(leader, &sm.bar_pv_done);
      umma_commit_w(leader, &sm.bar_v_empty);
      if (more) issue_s();
      else umma_commit_w(leader, &sm.bar_all_done);
    }
    if (!ok) __nanosleep(1000000);   // let copies already in flight land before the CTA retires
  } else {
    // ================= softmax threads: two per query row, 64 key columns each =================
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t pair_bar = 1 + (warp & 3);          // named barrier of the two warps that share rows
    const float sc = a.scale_log2;
    const uint32_t t_s = tmem + lane_base, t_o = tmem_o + lane_base;
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < nkv; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_s_ready, j & 1, wctx));
      if (!ok) {
        // the partner warp may have seen the barrier complete and be waiting at the pair barrier: release it
        asm volatile("bar.arrive %0, 64;" ::"r"(pair_bar) : "memory");
        break;
      }
      tc_fence_after_sync();
      const bool last = j == nkv - 1;
      int ncol = nkeys - j * MOBA_TILE;                       // keys of this tile that exist
      if constexpr (!kGathered) {
        if (last) ncol = min(ncol, row + 1);                  // diagonal tile: key <= query
      }
      ncol -= ch * 64;                                        // relative to this thread's 64 columns
      // One pass over the values: the row maximum and, speculatively, the probabilities against the maximum
      // in use (two sub-passes of 32 columns to bound the registers).
      uint32_t pk[32];
      float mx = -INFINITY, ls0 = 0.f, ls1 = 0.f;
      auto probabilities = [&](const bool with_max, const bool with_exp) {
        ls0 = 0.f;
        ls1 = 0.f;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t s[32];
          tmem_ld32(t_s + ch * 64 + h * 32, s);
          tmem_wait_ld32(s);
          if (!last) {
#pragma unroll
            for (int c = 0; c < 16; ++c) {
              const float s0 = __uint_as_float(s[2 * c]), s1 = __uint_as_float(s[2 * c + 1]);
              if (with_max) mx = fmaxf(mx, fmaxf(s0, s1));
              if (with_exp) {
                const float p0 = ex2_approx(fmaf(s0, sc, -m_used));
                const float p1 = ex2_approx(fmaf(s1, sc, -m_used));
                ls0 += p0;
                ls1 += p1;
                pk[h * 16 + c] = pack2<kBf16>(p0, p1);
              }
            }
          } else {
#pragma unroll
            for (int c = 0; c < 16; ++c) {
              const float s0 = __uint_as_float(s[2 * c]), s1 = __uint_as_float(s[2 * c + 1]);
              const int c0 = h * 32 + 2 * c;
              if (with_max) {
                if (c0 < ncol) mx = fmaxf(mx, s0);
                if (c0 + 1 < ncol) mx = fmaxf(mx, s1);
              }
              if (with_exp) {
                float p0 = ex2_approx(fmaf(s0, sc, -m_used));
                float p1 = ex2_approx(fmaf(s1, sc, -m_used));
                if (c0 >= ncol) p0 = 0.f;
                if (c0 + 1 >= ncol) p1 = 0.f;
                ls0 += p0;
                ls1 += p1;
                pk[h * 16 + c] = pack2<kBf16>(p0, p1);
              }
            }
          }
        }
      };
      // The first key tile has no maximum in use yet: only the row maximum is taken in the first pass (the
      // probabilities follow below, once, against it). Later tiles compute them in the same pass, speculatively.
      if (j == 0) probabilities(true, false);
      else probabilities(true, true);
      sm.xchg[ch][row] = mx;
      // also orders the in-place write of P below after every S load of the row's two threads
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      mx = fmaxf(mx, sm.xchg[ch ^ 1][row]);
      const float m_new = fmaxf(m_used, mx * sc);
      // (xchg is not written again before the partner has read it: the next S needs the partner's P first)
      if (__any_sync(0xffffffffu, m_new > m_used + kRescaleThreshold)) {
        const float alpha = ex2_approx(m_used - m_new);       // 0 on the first tile (m_used = -inf)
        l_sum *= alpha;
        if (j > 0) {
          // O may still be accumulating P V of the previous tile
          ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_pv_done, (j - 1) & 1, wctx));
          if (!ok) {
            // the partner warp may have seen the barrier complete and be waiting at the pair barrier: release it
            asm volatile("bar.arrive %0, 64;" ::"r"(pair_bar) : "memory");
            break;
          }
          tc_fence_after_sync();
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            uint32_t r[32];
            tmem_ld32(t_o + ch * 64 + i * 32, r);
            tmem_wait_ld32(r);
#pragma unroll
            for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
            tmem_st32(t_o + ch * 64 + i * 32, r);
          }
        }
        m_used = m_new;
        probabilities(false, true);      // S is still intact: P has not been written yet
        // the partner may already write P over columns this thread has just read again
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      }
      l_sum += ls0 + ls1;
      tmem_st32(t_s + ch * 32, pk);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&sm.bar_p_ready);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_all_done, 0, wctx));
    // ---- epilogue: O / l rows -> global memory through shared memory, so that a warp writes whole 256-byte rows
    // (thread = row straight from TMEM would write 16 bytes per row and instruction). The K and V slots are idle
    // by now; the staging rows are padded to 272 bytes against bank conflicts.
    if (!ok) sm.abort_flag = 1;
    uint8_t* stage = sm.k[0];
    constexpr int kPitch = MOBA_HEAD_DIM * 2 + 16;
    static_assert(sizeof(sm.k) + sizeof(sm.v) >= MOBA_TILE * kPitch, "staging tile does not fit the K and V slots");
    if (ok) {
      tc_fence_after_sync();
      sm.xchg[ch][row] = l_sum;
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      l_sum += sm.xchg[ch ^ 1][row];
      const float inv_l = 1.0f / l_sum;
      if (row < n_rows && ch == 0) {
        size_t lse_idx;
        if constexpr (kGathered) lse_idx = static_cast<size_t>(first + row);
        else lse_idx = static_cast<size_t>(first + row) * a.H + head;
        a.lse[lse_idx] = (m_used + __log2f(l_sum)) * kLn2;
      }
      uint4* d = reinterpret_cast<uint4*>(stage + row * kPitch + ch * 128);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        uint32_t r[32];
        tmem_ld32(t_o + ch * 64 + i * 32, r);
        tmem_wait_ld32(r);
        uint32_t pk[16];
#pragma unroll
        for (int c = 0; c < 16; ++c)
          pk[c] = pack2<kBf16>(__uint_as_float(r[2 * c]) * inv_l, __uint_as_float(r[2 * c + 1]) * inv_l);
#pragma unroll
        for (int g = 0; g < 4; ++g) d[i * 4 + g] = make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
      }
    }
    asm volatile("bar.sync 5, %0;" ::"n"(kSoftmaxWarps * 32) : "memory");        // the eight softmax warps
    if (*reinterpret_cast<volatile int*>(&sm.abort_flag) == 0) {
      // a warp moves two rows per step: lanes 0-15 the 16-byte pieces of one row, lanes 16-31 those of the next
#pragma unroll
      for (int i = 0; i < MOBA_TILE / (2 * kSoftmaxWarps); ++i) {
        const int r_out = warp * (MOBA_TILE / kSoftmaxWarps) + 2 * i + (lane >> 4);
        if (r_out < n_rows) {
          size_t row_off;
          if constexpr (kGathered) row_off = static_cast<size_t>(first + r_out) * MOBA_HEAD_DIM;
          else row_off = (static_cast<size_t>(first + r_out) * a.H + head) * MOBA_HEAD_DIM;
          const uint4 val = *reinterpret_cast<const uint4*>(stage + r_out * kPitch + (lane & 15) * 16);
          *reinterpret_cast<uint4*>(a.out + row_off + (lane & 15) * 8) = val;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tmem, kTmemCols);
}


template <bool kBf16>
int launch_fwd(const CUtensorMap& mk, const CUtensorMap& mv, FwdArgs args, const FwdArgs& gargs,
               const moba_plan_info* info, int parts, cudaStream_t st) {
  const size_t smem = sizeof(FwdSmem) + 1024;
  auto k_self = attn_fwd_kernel<kBf16, false>;
  auto k_gath = attn_fwd_kernel<kBf16, true>;
  MOBA_CUDA_OK(cudaFuncSetAttribute(k_self, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  MOBA_CUDA_OK(cudaFuncSetAttribute(k_gath, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  if ((parts & 2) && info->kk > 0 && info->max_work_tiles_per_head > 0) {
    const int64_t nw = info->max_work_tiles_per_head * args.H;
    MOBA_REQUIRE(nw < (1ll << 31), MOBA_ERR_LIMIT, "too many gathered tiles");
    k_gath<<<static_cast<unsigned>(nw), kFwdThreads, smem, st>>>(mk, mv, gargs);
    MOBA_CUDA_OK(cudaGetLastError());
  }
  if (parts & 1) {
    dim3 grid(info->n_qtiles, args.H);
    k_self<<<grid, kFwdThreads, smem, st>>>(mk, mv, args);
    MOBA_CUDA_OK(cudaGetLastError());
  }
  return 0;
}

}  // namespace
}  // namespace moba

extern "C" int moba_attn_fwd(const void* q, const void* k, const void* v, int32_t dtype, int32_t H,
                             int64_t stride_s, int64_t stride_h, const moba_kv_layout* kv,
                             const moba_plan_info* info, const int32_t* meta_dev, const int32_t* list_off,
                             const int32_t* work_off, const int32_t* list_tok, const int32_t* tile_rec, void* out,
                             float* lse, void* part_o, float* part_lse, int32_t parts, float softmax_scale,
                             int32_t* status, int32_t device, void* stream) {
  using namespace moba;
  int rc = check_common(q, H, stride_s, stride_h, info, meta_dev);
  if (rc) return rc;
  MOBA_REQUIRE(parts >= 1 && parts <= 3, MOBA_ERR_ARG, "parts=%d must be 1 (own chunk), 2 (lists) or 3 (both)", parts);
  MOBA_REQUIRE(k && v && status && ((out && lse) || !(parts & 1)), MOBA_ERR_ARG, "null pointer argument");
  MOBA_REQUIRE(dtype == MOBA_DTYPE_BF16 || dtype == MOBA_DTYPE_F16, MOBA_ERR_ARG,
               "attention kernels take bf16 or f16 tensors (dtype=%d)", dtype);
  if (info->kk > 0 && (parts & 2))
    MOBA_REQUIRE(list_off && work_off && list_tok && part_o && part_lse, MOBA_ERR_ARG, "null list / partial buffers");
  MOBA_SET_DEVICE(device);
  if (info->n_qtiles == 0) return 0;
  CUtensorMap mk, mv;
  FwdArgs a;
  rc = make_kv_maps(&mk, &mv, k, v, dtype, H, stride_s, stride_h, kv, info, &a.kv_rep);
  if (rc) return rc;
  a.q = static_cast<const uint16_t*>(q);
  a.stride_s = stride_s;
  a.stride_h = stride_h;
  a.H = H;
  a.plan = make_plan_dev(info, meta_dev);
  a.list_off = list_off;
  a.work_off = work_off;
  a.list_tok = list_tok;
  a.tile_rec = tile_rec;
  a.out = static_cast<uint16_t*>(out);
  a.lse = lse;
  a.status = status;
  a.n_experts = info->n_chunks * H;
  a.scale_log2 = softmax_scale_or_default(softmax_scale) * kLog2e;
  FwdArgs g = a;
  g.out = static_cast<uint16_t*>(part_o);
  g.lse = part_lse;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == MOBA_DTYPE_BF16) return launch_fwd<true>(mk, mv, a, g, info, parts, st);
  return launch_fwd<false>(mk, mv, a, g, info, parts, st);
}
