// Backward, key/value side, for sm_100a (tcgen05 / TMEM). No atomics.
//
// One CTA per (chunk, key/value head, 128-key tile). The K and V tiles stay in shared memory; for every query
// head that shares the key/value head (one without grouped-query K / V) the CTA walks the chunk's own query
// tiles from the diagonal on (causal) and then the 128-row tiles of the (chunk, head) query list, so self and
// gathered contributions of the whole group meet in tensor memory and dk / dv are written once. Replaces the dk/dv
// halves of both flash backward calls of MoonshotAI/MoBA moba/moba_efficient.py:208-264 and the autograd
// scatter through the KV regrouping (:406-414).
//
// Per query tile, keys on TMEM lanes and queries on columns, in two 64-query halves h = 0, 1:
//   S^T_h = K Q_h^T, dP^T_h = V dO_h^T          operands in shared memory (K-major), N = 64
//   P^T_h = exp2(S^T_h c - lse), dS^T_h = P^T_h (dP^T_h - delta) * scale      written back as 16-bit pairs
//   dV += P^T_h dO_h, dK += dS^T_h Q_h          A from TMEM, B = the same dO / Q rows read MN-major, K = 64
// lse / delta are the merged log-sum-exp and rowsum(dO * O), so P is the global softmax restricted to the
// block. The two halves ping-pong: while the compute warps turn half h into P^T / dS^T, the tensor pipe works
// on the other half (and on the next tile's S^T / dP^T).
//
// Warp roles (384 threads): 0-7 compute (warp & 3 = TMEM lane quarter, so thread = key row; warp >> 2 = which
// 32 of a half tile's 64 query columns), 8 / 9 = MMA issue for the even / odd half tiles (warp-converged, one
// elected lane; warp 8 also fetches K and V), 10-11 = loaders feeding a four-stage ring; a stage holds one half
// tile (64 query rows of Q and of dO plus the lse / delta operands of those rows: with keys on the TMEM lanes,
// lse and delta vary along the columns, so they are added by the tensor pipe as a ninth k-step of the S^T / dP^T
// products, ones[key] x (-lse / scale)[query], instead of being re-read from shared memory by every compute
// warp). List rows are read from list-ordered copies (moba_gather_rows), so every half tile is four TMA tile
// loads.
// TMEM columns: [0,64) S^T_0  [64,128) dP^T_0  [128,192) S^T_1  [192,256) dP^T_1  [256,384) dV  [384,512) dK.
#include "attn_common.cuh"

namespace moba {
namespace {

constexpr int kDkdvThreads = 384;
constexpr int kMmaWarp0 = 8, kLoaderWarp0 = 10;      // 8, 9: MMA issue for the even / odd half tiles; 10, 11: loaders

constexpr int kStages = 4;

struct __align__(1024) DkdvSmem {
  uint8_t k[2][16384];
  uint8_t v[2][16384];
  uint8_t q[kStages][2][8192];      // [stage][d half][64 rows x 64], 128-byte swizzle
  uint8_t d_o[kStages][2][8192];
  // lse / delta enter through the tensor pipe: a ninth k-step adds ones[key][0..1] * x[query][0..1] to S^T / dP^T,
  // where x holds -lse / scale (resp. -delta) of the query row split into two 16-bit halves. K-major tiles of 16
  // columns without swizzle (nosw_offset).
  uint8_t ones[4096];               // [128 keys x 16]: columns 0, 1 = 1.0 (bf16) or 256.0 (f16), the rest 0
  uint8_t lse_b[kStages][2048];     // [64 query rows x 16]: columns 0, 1 = hi, lo of -lse / scale, the rest 0
  uint8_t dlt_b[kStages][2048];     // the same for -delta
  uint64_t bar_kv_full, bar_q_full[kStages], bar_q_empty[kStages], bar_s_ready[2], bar_p_ready[2], bar_acc_done,
      bar_all_done;
  uint32_t tmem_base;
  int abort_flag;
  // per query head of the group: first half tile, first list row and list length; seg_start[kv_rep] = n_half
  int seg_start[MOBA_MAX_KV_REP + 1], seg_list0[MOBA_MAX_KV_REP], seg_len[MOBA_MAX_KV_REP];
};

template <bool kBf16>
__global__ void __launch_bounds__(kDkdvThreads, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                     const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                     const __grid_constant__ CUtensorMap map_qg, const __grid_constant__ CUtensorMap map_dog,
                     const BwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  DkdvSmem& sm = *reinterpret_cast<DkdvSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  WaitCtx wctx{&sm.abort_flag, a.status};

  // One CTA per (key tile, key/value head). Its query-side work is, for each of the kv_rep query heads of the
  // group in turn, the own-chunk tiles from the diagonal on and then that head's list of the chunk: one sequence
  // of half tiles g = 0 .. n_half - 1 cut into kv_rep segments (seg_start), all accumulated into the same dK / dV.
  const int t = blockIdx.x, head_kv = blockIdx.y;
  const int rep = a.kv_rep, head0 = head_kv * rep, H_kv = a.H / rep;
  const int chunk = a.plan.qtile_chunk[t];
  const int kv0 = a.plan.qtile_start[t];
  const int chunk_end = a.plan.chunk_start[chunk + 1];
  const int n_keys = min(MOBA_TILE, chunk_end - kv0);
  // own-chunk query tiles from the diagonal on (none when the caller asked for the list part only)
  const int n_self = (a.parts & 1) ? a.plan.chunk_qtile_first[chunk + 1] - t : 0;
  if (warp == 1) {
    // lists of the group's heads are neighbours in the expert order e = chunk * H + head
    const bool lists = a.plan.kk > 0 && (a.parts & 2);
    const int e0 = chunk * a.H + head0;
    const int lo = (lists && lane <= rep) ? a.list_off[e0 + lane] : 0;
    const int len = __shfl_down_sync(0xffffffffu, lo, 1) - lo;
    int halves = lane < rep ? 2 * (n_self + (len + MOBA_TILE - 1) / MOBA_TILE) : 0;
    int incl = halves;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += up;
    }
    if (lane < rep) {
      sm.seg_start[lane] = incl - halves;
      sm.seg_list0[lane] = lo;
      sm.seg_len[lane] = lists ? len : 0;
    }
    if (lane == rep) sm.seg_start[rep] = incl;       // lanes >= rep add nothing: the total
  }

  if (tid == 0) {
    sm.abort_flag = 0;
    mbar_init(&sm.bar_kv_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&sm.bar_q_full[i], 1);
      mbar_init(&sm.bar_q_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.bar_s_ready[i], 1);
      mbar_init(&sm.bar_p_ready[i], 256);
    }
    mbar_init(&sm.bar_all_done, 1);
    mbar_init(&sm.bar_acc_done, 1);
    mbar_fence_init();
  }
  if (warp == kMmaWarp0) {
    tmem_alloc(&sm.tmem_base, 512);
    tmem_relinquish();
  }
  {
    // constant parts of the ninth-k-step operands (columns 2..15 stay zero for the whole kernel)
    // bf16: 1.0; f16: 256.0, with the query-side values divided by 256, so that -lse / scale up to 1.6e7 stays
    // inside the f16 range (the product is exact either way)
    constexpr uint32_t kOne = kBf16 ? 0x3F80u : 0x5C00u;
    if (tid < 128) {
      *reinterpret_cast<uint4*>(sm.ones + nosw_offset(tid, 0)) = make_uint4(kOne | (kOne << 16), 0, 0, 0);
      *reinterpret_cast<uint4*>(sm.ones + nosw_offset(tid, 1)) = make_uint4(0, 0, 0, 0);
    }
    for (int i = tid; i < kStages * 64; i += kDkdvThreads) {
      *reinterpret_cast<uint4*>(sm.lse_b[i >> 6] + nosw_offset(i & 63, 1)) = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(sm.dlt_b[i >> 6] + nosw_offset(i & 63, 1)) = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async_smem();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t tm_dv = tmem + 256, tm_dk = tmem + 384;
  const int n_half = sm.seg_start[rep];                         // half tiles of 64 query rows

  if (warp >= kLoaderWarp0) {
    // ================= loader warps: warp 9 the first half of every query tile, warp 10 the second ==========
    // Own-chunk half tiles come straight from q / d_out (64 consecutive tokens), list half tiles from the
    // list-ordered copies qg / dog; either way four TMA tile loads by one lane. lse / delta of the 64 rows are
    // read by the lanes (two rows each). Rows past the end of the chunk / list hold other rows' data and are
    // neutralised by lse = +inf (P = 0).
    int seg = 0;
    for (int g = warp - kLoaderWarp0; g < n_half; g += 2) {
      while (g >= sm.seg_start[seg + 1]) ++seg;                  // segments hold an even number of half tiles
      const int head = head0 + seg, list0 = sm.seg_list0[seg], list_len = sm.seg_len[seg];
      const int st = g & (kStages - 1);
      const int it = (g - sm.seg_start[seg]) >> 1, r_half = (g & 1) * 64;
      const bool self_tile = it < n_self;
      // x = -lse / scale and -delta of this lane's two rows; rows that do not exist get a value that makes P = 0
      float l_a = 0.f, l_b = 0.f, d_a = 0.f, d_b = 0.f;
      bool ok_a = false, ok_b = false;
      int row0;                                                  // first row of the half tile in its source
      if (self_tile) {
        row0 = kv0 + it * MOBA_TILE + r_half;                    // token; tiles of a chunk are contiguous
        ok_a = row0 + lane < chunk_end;
        ok_b = row0 + lane + 32 < chunk_end;
        if (ok_a) {
          const size_t i = static_cast<size_t>(row0 + lane) * a.H + head;
          l_a = a.lse[i];
          d_a = a.delta[i];
        }
        if (ok_b) {
          const size_t i = static_cast<size_t>(row0 + lane + 32) * a.H + head;
          l_b = a.lse[i];
          d_b = a.delta[i];
        }
      } else {
        const int idx = (it - n_self) * MOBA_TILE + r_half;      // position inside the list
        row0 = list0 + idx;
        ok_a = idx + lane < list_len;
        ok_b = idx + lane + 32 < list_len;
        if (ok_a) {
          l_a = a.lse_g[row0 + lane];
          d_a = a.delta_g[row0 + lane];
        }
        if (ok_b) {
          l_b = a.lse_g[row0 + lane + 32];
          d_b = a.delta_g[row0 + lane + 32];
        }
      }
      constexpr float kInvOne = kBf16 ? 1.0f : 1.0f / 256.0f;      // the ones tile holds 1 (bf16) or 256 (f16)
      const uint32_t xl_a = ok_a ? split16<kBf16>(l_a * (-kInvOne / a.scale)) : kMaskedPair<kBf16>;
      const uint32_t xl_b = ok_b ? split16<kBf16>(l_b * (-kInvOne / a.scale)) : kMaskedPair<kBf16>;
      const uint32_t xd_a = split16<kBf16>(-kInvOne * d_a), xd_b = split16<kBf16>(-kInvOne * d_b);
      int go = 1;
      if (g >= kStages) {
        if (lane == 0) go = mbar_wait(&sm.bar_q_empty[st], ((g >> 2) - 1) & 1, wctx) ? 1 : 0;
        go = __shfl_sync(0xffffffffu, go, 0);
      }
      if (!go) break;
      *reinterpret_cast<uint4*>(sm.lse_b[st] + nosw_offset(lane, 0)) = make_uint4(xl_a, 0, 0, 0);
      *reinterpret_cast<uint4*>(sm.lse_b[st] + nosw_offset(lane + 32, 0)) = make_uint4(xl_b, 0, 0, 0);
      *reinterpret_cast<uint4*>(sm.dlt_b[st] + nosw_offset(lane, 0)) = make_uint4(xd_a, 0, 0, 0);
      *reinterpret_cast<uint4*>(sm.dlt_b[st] + nosw_offset(lane + 32, 0)) = make_uint4(xd_b, 0, 0, 0);
      fence_proxy_async_smem();          // the tensor pipe reads these through the async proxy
      __syncwarp();
      if (lane == 0) {
        const uint32_t q_dst = smem_u32(sm.q[st][0]), do_dst = smem_u32(sm.d_o[st][0]);
        mbar_arrive_expect_tx(&sm.bar_q_full[st], 32768);
        if (self_tile) {
          tma_load_3d(q_dst, &map_q, &sm.bar_q_full[st], 0, head, row0);
          tma_load_3d(q_dst + 8192, &map_q, &sm.bar_q_full[st], 64, head, row0);
          tma_load_3d(do_dst, &map_do, &sm.bar_q_full[st], 0, head, row0);
          tma_load_3d(do_dst + 8192, &map_do, &sm.bar_q_full[st], 64, head, row0);
        } else {
          tma_load_3d(q_dst, &map_qg, &sm.bar_q_full[st], 0, 0, row0);
          tma_load_3d(q_dst + 8192, &map_qg, &sm.bar_q_full[st], 64, 0, row0);
          tma_load_3d(do_dst, &map_dog, &sm.bar_q_full[st], 0, 0, row0);
          tma_load_3d(do_dst + 8192, &map_dog, &sm.bar_q_full[st], 64, 0, row0);
        }
      }
    }
  } else if (warp >= kMmaWarp0) {
    // ================= K/V load + MMA issue: warp M_b owns S^T / dP^T buffer b and the half tiles g = b, b + 2, ...
    // A warp with tcgen05.mma instructions queued does not see an mbarrier change until they have left the queue
    // (measured on B200): with one issuing warp the accumulations of half tile g + 1 had to wait for S^T / dP^T of
    // half tile g + 2 to drain. Each warp now polls everything its round needs together, then issues the
    // accumulations of half tile g and S^T / dP^T of half tile g + 2 back to back; by the time these have drained
    // its next P^T / dS^T are still being computed. dV and dK are shared by the two warps, so the accumulations
    // of half tile g wait for those of g - 1 to have completed (bar_acc_done).
    {
      // The whole warp runs this loop converged; one elected lane issues the tcgen05 instructions.
      const uint32_t leader = elect_one();
      constexpr uint32_t idesc_sdp = umma_idesc(128, 64, kBf16, false, false);    // both operands K-major
      constexpr uint32_t idesc_acc = umma_idesc(128, 128, kBf16, false, true);    // B read MN-major
      const uint32_t k_addr = smem_u32(sm.k[0]), v_addr = smem_u32(sm.v[0]);
      const int mb = warp - kMmaWarp0;
      if (lane == 0 && mb == 0) {
        mbar_arrive_expect_tx(&sm.bar_kv_full, 65536);
        tma_load_3d(k_addr, &map_k, &sm.bar_kv_full, 0, head_kv, kv0);
        tma_load_3d(k_addr + 16384, &map_k, &sm.bar_kv_full, 64, head_kv, kv0);
        tma_load_3d(v_addr, &map_v, &sm.bar_kv_full, 0, head_kv, kv0);
        tma_load_3d(v_addr + 16384, &map_v, &sm.bar_kv_full, 64, head_kv, kv0);
      }
      __syncwarp();

      // Descriptors are built once; issuing an MMA then costs a couple of integer adds. Offsets are in 16-byte
      // units: a stage is 16384 B (two [64 x 64] sub-tiles), a K-major k-step is 32 B inside a 128-byte row,
      // an MN-major k-step is 16 rows = 2048 B.
      const uint64_t k_km = umma_smem_desc(k_addr, 16, 1024), v_km = umma_smem_desc(v_addr, 16, 1024);
      const uint64_t q_km0 = umma_smem_desc(smem_u32(sm.q[0][0]), 16, 1024);
      const uint64_t do_km0 = umma_smem_desc(smem_u32(sm.d_o[0][0]), 16, 1024);
      const uint64_t q_mn0 = umma_smem_desc(smem_u32(sm.q[0][0]), 8192, 1024);
      const uint64_t do_mn0 = umma_smem_desc(smem_u32(sm.d_o[0][0]), 8192, 1024);
      const uint64_t ones_d = umma_smem_desc_nosw(smem_u32(sm.ones), 128, 256);
      const uint64_t lse_d0 = umma_smem_desc_nosw(smem_u32(sm.lse_b[0]), 128, 256);
      const uint64_t dlt_d0 = umma_smem_desc_nosw(smem_u32(sm.dlt_b[0]), 128, 256);
      // S^T_h = K Q_h^T and dP^T_h = V dO_h^T for half tile g (h = g & 1), operands of stage g & 3
      auto issue_sdp = [&](int g) {
        const uint32_t st_off = static_cast<uint32_t>(g & (kStages - 1)) * (16384u >> 4);
        const uint64_t q_km = q_km0 + st_off, do_km = do_km0 + st_off;
        const uint32_t d_s = tmem + (g & 1) * 128u, d_dp = d_s + 64u;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss_w(leader, d_s, k_km + (((ks >> 2) * 16384u + (ks & 3) * 32u) >> 4), q_km + (((ks >> 2) * 8192u + (ks & 3) * 32u) >> 4),
                  idesc_sdp, ks > 0);
        umma_ss_w(leader, d_s, ones_d, lse_d0 + static_cast<uint32_t>(g & (kStages - 1)) * (2048u >> 4), idesc_sdp, 1);   // - lse / scale
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss_w(leader, d_dp, v_km + (((ks >> 2) * 16384u + (ks & 3) * 32u) >> 4), do_km + (((ks >> 2) * 8192u + (ks & 3) * 32u) >> 4),
                  idesc_sdp, ks > 0);
        umma_ss_w(leader, d_dp, ones_d, dlt_d0 + static_cast<uint32_t>(g & (kStages - 1)) * (2048u >> 4), idesc_sdp, 1);  // - delta
        umma_commit_w(leader, &sm.bar_s_ready[g & 1]);
      };
      // dV += P^T_h dO_h, dK += dS^T_h Q_h  (K = 64 query rows)
      auto issue_acc = [&](int g) {
        const int st = g & (kStages - 1);
        const uint32_t st_off = static_cast<uint32_t>(st) * (16384u >> 4);
        const uint64_t q_mn = q_mn0 + st_off, do_mn = do_mn0 + st_off;
        const uint32_t a_p = tmem + (g & 1) * 128u, a_ds = a_p + 64u;
        const uint32_t acc = g > 0;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) umma_ts_w(leader, tm_dv, a_p + ks * 8, do_mn + ((ks * 2048u) >> 4), idesc_acc, ks > 0 ? 1u : acc);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) umma_ts_w(leader, tm_dk, a_ds + ks * 8, q_mn + ((ks * 2048u) >> 4), idesc_acc, ks > 0 ? 1u : acc);
        umma_commit_w(leader, &sm.bar_q_empty[st]);          // the stage may be refilled once these have read it
        umma_commit_w(leader, &sm.bar_acc_done);
      };

      bool ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_kv_full, 0, wctx));
      if (ok && mb < n_half) {
        ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_q_full[mb], 0, wctx));
        if (ok) {
          tc_fence_after_sync();
          issue_sdp(mb);
        }
      }
      for (int g = mb; g < n_half && ok; g += 2) {
        const bool more = g + 2 < n_half;
        const BarPhase need[3] = {
            {&sm.bar_p_ready[mb], static_cast<uint32_t>((g >> 1) & 1)},
            // no next half tile / no previous one: name the first barrier again
            {more ? &sm.bar_q_full[(g + 2) & (kStages - 1)] : &sm.bar_p_ready[mb],
             static_cast<uint32_t>(more ? ((g + 2) >> 2) & 1 : (g >> 1) & 1)},
            {g > 0 ? &sm.bar_acc_done : &sm.bar_p_ready[mb], static_cast<uint32_t>(g > 0 ? (g - 1) & 1 : (g >> 1) & 1)}};
        ok = __all_sync(0xffffffffu, mbar_wait_all(need, wctx));
        if (!ok) break;
        tc_fence_after_sync();
        issue_acc(g);
        if (more) issue_sdp(g + 2);
        if (g == n_half - 1) umma_commit_w(leader, &sm.bar_all_done);     // follows every other product
      }
      if (!ok) __nanosleep(1000000);
    }
  } else {
    // ================= compute warps: thread = key row =================
    const int row = tid & 127, ci = warp >> 2;     // key row; which 32 of the 64 query columns of a half tile
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t pair_bar = 1 + (warp & 3);      // named barrier shared by warps w and w + 4 (same rows)
    const float sc = a.scale * kLog2e, scale = a.scale;
    bool ok = true;
    int seg = 0;
    for (int g = 0; g < n_half; ++g) {
      while (g >= sm.seg_start[seg + 1]) ++seg;
      const int st = g & (kStages - 1), h = g & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_q_full[st], (g >> 2) & 1, wctx) && mbar_wait(&sm.bar_s_ready[h], (g >> 1) & 1, wctx));
      if (!ok) {
        // the partner warp may have seen the barrier complete and be waiting at the pair barrier: release it
        asm volatile("bar.arrive %0, 64;" ::"r"(pair_bar) : "memory");
        break;
      }
      tc_fence_after_sync();
      // the first own-chunk tile of every head's segment is the diagonal one: key <= query
      const bool diag = n_self > 0 && g - sm.seg_start[seg] < 2;
      const uint32_t t_s = tmem + lane_base + h * 128u, t_dp = t_s + 64u;
      {
        const int i = ci;
        uint32_t rs[32], rd[32];
        tmem_ld32(t_s + i * 32, rs);
        tmem_ld32(t_dp + i * 32, rd);
        tmem_wait_ld32(rs);
        tmem_wait_ld32(rd);
        uint32_t pp[16], pd[16];
        // S^T and dP^T arrive with - lse / scale and - delta already added (ninth k-step of their products)
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float p0 = ex2_approx(__uint_as_float(rs[4 * c]) * sc);
          float p1 = ex2_approx(__uint_as_float(rs[4 * c + 1]) * sc);
          float p2 = ex2_approx(__uint_as_float(rs[4 * c + 2]) * sc);
          float p3 = ex2_approx(__uint_as_float(rs[4 * c + 3]) * sc);
          if (diag) {
            const int col = h * 64 + i * 32 + 4 * c;
            if (row > col) p0 = 0.f;
            if (row > col + 1) p1 = 0.f;
            if (row > col + 2) p2 = 0.f;
            if (row > col + 3) p3 = 0.f;
          }
          const float e0 = p0 * (__uint_as_float(rd[4 * c]) * scale);
          const float e1 = p1 * (__uint_as_float(rd[4 * c + 1]) * scale);
          const float e2 = p2 * (__uint_as_float(rd[4 * c + 2]) * scale);
          const float e3 = p3 * (__uint_as_float(rd[4 * c + 3]) * scale);
          pp[2 * c] = pack2<kBf16>(p0, p1);
          pp[2 * c + 1] = pack2<kBf16>(p2, p3);
          pd[2 * c] = pack2<kBf16>(e0, e1);
          pd[2 * c + 1] = pack2<kBf16>(e2, e3);
        }
        // the 16-bit results of columns [32, 64) land on TMEM columns the partner warp reads its fp32 inputs
        // from: both warps of a row must have their inputs in registers first
        asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
        tmem_st16(t_s + i * 16, pp);
        tmem_st16(t_dp + i * 16, pd);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&sm.bar_p_ready[h]);
    }
    if (n_half == 0) {
      // no query attends these keys (list part only, empty list): the gradients are zero
      if (row < n_keys) {
        uint4* d = reinterpret_cast<uint4*>((ci == 0 ? a.o0 : a.o1) + (static_cast<size_t>(kv0 + row) * H_kv + head_kv) * MOBA_HEAD_DIM);
#pragma unroll
        for (int i = 0; i < 16; ++i) d[i] = make_uint4(0, 0, 0, 0);
      }
      ok = false;
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_all_done, 0, wctx));
    if (ok) {
      tc_fence_after_sync();
      // warps 0-3 write dK, warps 4-7 dV: thread = key row, whole 128-byte lines per quad of rows
      const int row0 = row & ~3;
      const size_t off = (static_cast<size_t>(kv0 + row0) * H_kv + head_kv) * MOBA_HEAD_DIM;
      const size_t pitch = static_cast<size_t>(H_kv) * MOBA_HEAD_DIM;
      if (ci == 0) store_rows_from_tmem<kBf16>(tm_dk + lane_base, a.o0 + off, pitch, n_keys - row0, lane);
      else store_rows_from_tmem<kBf16>(tm_dv + lane_base, a.o1 + off, pitch, n_keys - row0, lane);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp0) tmem_dealloc(tmem, 512);
}

}  // namespace
}  // namespace moba


extern "C" int moba_attn_bwd_dkdv(const void* q, const void* k, const void* v, const void* d_out, int32_t dtype,
                                  int32_t H, int64_t stride_s, int64_t stride_h, const moba_kv_layout* kv,
                                  const moba_plan_info* info, const int32_t* meta_dev, const int32_t* list_off,
                                  const void* qg, const void* dog,
                                  const float* lse_g, const float* delta_g, const float* lse, const float* delta,
                                  void* dk, void* dv, int32_t parts, float softmax_scale, int32_t* status,
                                  int32_t device, void* stream) {
  using namespace moba;
  MOBA_REQUIRE(parts >= 1 && parts <= 3, MOBA_ERR_ARG, "parts=%d must be 1 (own chunk), 2 (lists) or 3 (both)", parts);
  int rc = check_bwd_args(q, k, v, d_out, dtype, H, stride_s, stride_h, info, meta_dev, lse, delta, status);
  if (rc) return rc;
  MOBA_REQUIRE(dk && dv, MOBA_ERR_ARG, "null pointer argument");
  if (info->kk > 0 && (parts & 2)) MOBA_REQUIRE(list_off, MOBA_ERR_ARG, "null list buffers");
  MOBA_SET_DEVICE(device);
  if (info->n_qtiles == 0) return 0;
  CUtensorMap mk, mv;
  BwdArgs a;
  rc = make_kv_maps(&mk, &mv, k, v, dtype, H, stride_s, stride_h, kv, info, &a.kv_rep);
  if (rc) return rc;
  // 64-row boxes: own-chunk half tiles from q / d_out, list half tiles from the list-ordered copies
  CUtensorMap mq, mdo, mqg, mdog;
  const int64_t n_list_rows = (info->kk > 0 && (parts & 2)) ? info->rows_per_head * H : 0;
  // a list-only call never loads through the q / d_out maps; describe no more rows than q is known to hold
  const int64_t q_rows = (parts & 1) ? info->total_tokens : (n_list_rows > 0 ? n_list_rows / H : 1);
  rc = make_tensor_map_shd(&mq, q, dtype, q_rows, H, stride_s, stride_h, 64);
  if (rc) return rc;
  rc = make_tensor_map_shd(&mdo, d_out, dtype, q_rows, H, stride_s, stride_h, 64);
  if (rc) return rc;
  if (n_list_rows > 0) {
    MOBA_REQUIRE(qg && dog && lse_g && delta_g, MOBA_ERR_ARG, "null list-ordered buffers");
    rc = make_tensor_map_shd(&mqg, qg, dtype, n_list_rows, 1, MOBA_HEAD_DIM, MOBA_HEAD_DIM, 64);
    if (rc) return rc;
    rc = make_tensor_map_shd(&mdog, dog, dtype, n_list_rows, 1, MOBA_HEAD_DIM, MOBA_HEAD_DIM, 64);
    if (rc) return rc;
  } else {
    mqg = mq;
    mdog = mdo;
  }
  a.lse_g = lse_g;
  a.delta_g = delta_g;
  a.q = static_cast<const uint16_t*>(q);
  a.d_out = static_cast<const uint16_t*>(d_out);
  a.stride_s = stride_s; a.stride_h = stride_h; a.H = H;
  a.plan = make_plan_dev(info, meta_dev);
  a.list_off = list_off; a.work_off = nullptr; a.list_tok = nullptr; a.tile_rec = nullptr;
  a.lse = lse; a.delta = delta;
  a.o0 = static_cast<uint16_t*>(dk); a.o1 = static_cast<uint16_t*>(dv); a.dq_f32 = nullptr;
  a.status = status;
  a.n_experts = info->n_chunks * H;
  a.parts = parts;
  a.scale = softmax_scale_or_default(softmax_scale);
  const size_t smem = sizeof(DkdvSmem) + 1024;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(info->n_qtiles, H / a.kv_rep);
  if (dtype == MOBA_DTYPE_BF16) {
    MOBA_CUDA_OK(cudaFuncSetAttribute(attn_bwd_dkdv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attn_bwd_dkdv_kernel<true><<<grid, kDkdvThreads, smem, st>>>(mk, mv, mq, mdo, mqg, mdog, a);
  } else {
    MOBA_CUDA_OK(cudaFuncSetAttribute(attn_bwd_dkdv_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attn_bwd_dkdv_kernel<false><<<grid, kDkdvThreads, smem, st>>>(mk, mv, mq, mdo, mqg, mdog, a);
  }
  MOBA_CUDA_OK(cudaGetLastError());
  return 0;
}
