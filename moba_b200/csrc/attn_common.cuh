// Device helpers shared by the attention tile kernels (forward, dK/dV, dQ).
#pragma once
#include "common.cuh"
#include "ptx.cuh"

namespace moba {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kSoftmaxScale = 0.08838834764831845f;   // 128^-0.5 (MoonshotAI/MoBA moba/moba_efficient.py:86), the default
// The scale the caller asked for: a value <= 0 means the default. Tensors of a smaller head dim reach the kernels
// zero-padded to 128 columns (the products are unchanged) with their own head_dim^-0.5.
inline float softmax_scale_or_default(float s) { return s > 0.f ? s : kSoftmaxScale; }

struct BwdArgs {
  const uint16_t* q;
  const uint16_t* d_out;
  int64_t stride_s, stride_h;
  int H;
  PlanDev plan;
  const int32_t* list_off;
  const int32_t* work_off;
  const int32_t* list_tok;
  const int32_t* tile_rec;   // work-tile records (moba_tile_records), or null: search work_off
  const float* lse;      // [S,H] merged log-sum-exp (natural log)
  const float* delta;    // [S,H] rowsum(dO * O)
  const float* lse_g;    // dkdv: lse / delta of the list rows, in list order [R*H]
  const float* delta_g;
  uint16_t* o0;          // dkdv: dk [S,H,D]
  uint16_t* o1;          // dkdv: dv
  float* dq_f32;         // dq kernel: fp32 rows, [S,H,D] for own-chunk tiles or [R*H, D] for list tiles
  int* status;
  int n_experts;
  int parts;             // bit 0: own-chunk (causal) tiles, bit 1: list tiles
  int kv_rep;            // query heads per key/value head (1 without grouped-query K / V)
  float scale;           // softmax scale (head_dim^-0.5 of the caller's head dim)
};

// One 128-row query tile of a persistent kernel's walk: a (chunk, head) list tile or an own-chunk tile.
struct TileItem {
  int head, first, n_rows, key0, nkeys;
};

// Parameters of work tile w, looked up by one full warp. `e_hint` carries the list found last time (the walk only
// moves forward), so the search is one window of 32 offsets in the common case.
template <bool kGathered, typename Args>
__device__ __forceinline__ TileItem lookup_tile(const Args& a, int w, int lane, int& e_hint) {
  TileItem it;
  if constexpr (kGathered) {
    if (a.tile_rec) {
      const int val = lane < 8 ? __ldg(&a.tile_rec[8 * static_cast<size_t>(w) + lane]) : 0;
      it.head = __shfl_sync(0xffffffffu, val, 0);
      it.first = __shfl_sync(0xffffffffu, val, 1);
      it.n_rows = __shfl_sync(0xffffffffu, val, 2);
      it.key0 = __shfl_sync(0xffffffffu, val, 3);
      it.nkeys = __shfl_sync(0xffffffffu, val, 4);
      return it;
    }
    const int E = a.n_experts;
    int e = e_hint;
    while (true) {                                    // last e with work_off[e] <= w, scanning forward from the hint
      const int idx = e + 1 + lane;
      const bool le = idx <= E - 1 && __ldg(&a.work_off[idx]) <= w;
      const int n_le = __popc(__ballot_sync(0xffffffffu, le));     // work_off ascends: the true lanes are a prefix
      e += n_le;
      if (n_le < 32) break;
    }
    e_hint = e;
    const int chunk = e / a.H;
    int val = 0;                                      // five independent loads by five lanes
    if (lane == 0) val = __ldg(&a.list_off[e]);
    else if (lane == 1) val = __ldg(&a.list_off[e + 1]);
    else if (lane == 2) val = __ldg(&a.plan.chunk_start[chunk]);
    else if (lane == 3) val = __ldg(&a.plan.chunk_start[chunk + 1]);
    else if (lane == 4) val = __ldg(&a.work_off[e]);
    const int l0 = __shfl_sync(0xffffffffu, val, 0), l1 = __shfl_sync(0xffffffffu, val, 1);
    const int c0 = __shfl_sync(0xffffffffu, val, 2), c1 = __shfl_sync(0xffffffffu, val, 3);
    const int w0 = __shfl_sync(0xffffffffu, val, 4);
    it.head = e - chunk * a.H;
    it.first = l0 + (w - w0) * MOBA_TILE;
    it.n_rows = min(MOBA_TILE, l1 - it.first);
    it.key0 = c0;
    it.nkeys = c1 - c0;
  } else {
    const int nq = a.plan.n_qtiles;
    const int t = w % nq;
    it.head = w / nq;
    const int chunk = __ldg(&a.plan.qtile_chunk[t]);
    it.first = __ldg(&a.plan.qtile_start[t]);
    it.key0 = __ldg(&a.plan.chunk_start[chunk]);
    it.n_rows = min(MOBA_TILE, __ldg(&a.plan.chunk_start[chunk + 1]) - it.first);
    it.nkeys = it.first + it.n_rows - it.key0;       // causal: keys up to the last row of the tile
  }
  return it;
}

// Four 32-byte pieces per lane (r[8 p .. 8 p + 7] = piece p of the lane's row) are swapped inside each quad of
// lanes, so that afterwards lane a holds piece a of the quad's row i in slot i: a store of slot i then writes whole
// 128-byte lines (four lanes x 32 bytes of one row) instead of 32 bytes to each of 32 lines.
__device__ __forceinline__ void quad_transpose_pieces(uint32_t (&r)[32], int lane) {
#pragma unroll
  for (int bit = 1; bit <= 2; bit <<= 1) {
    const bool up = (lane & bit) != 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      if (c & bit) continue;               // pieces c (bit clear) and c | bit (bit set) form a pair
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        const uint32_t lo = r[8 * c + x], hi = r[8 * (c | bit) + x];
        const uint32_t got = __shfl_xor_sync(0xffffffffu, up ? lo : hi, bit);
        r[8 * c + x] = up ? got : lo;
        r[8 * (c | bit) + x] = up ? hi : got;
      }
    }
  }
}
// Slot i of every lane (after quad_transpose_pieces) -> row i of the quad: dst = the lane's 32-byte piece of the
// quad's first row, pitch = elements of T between consecutive rows, n_valid = rows of the quad that exist.
template <typename T>
__device__ __forceinline__ void store_quad_rows(T* dst, size_t pitch, int n_valid, const uint32_t (&r)[32]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (i < n_valid)
      asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + i * pitch), "r"(r[8 * i]),
                   "r"(r[8 * i + 1]), "r"(r[8 * i + 2]), "r"(r[8 * i + 3]), "r"(r[8 * i + 4]), "r"(r[8 * i + 5]),
                   "r"(r[8 * i + 6]), "r"(r[8 * i + 7])
                   : "memory");
  }
}

// The 128 TMEM lanes of a tile (thread = row, 128 fp32 columns starting at taddr) -> 16-bit rows in global memory,
// written as whole 128-byte lines. `quad_dst` = column 0 of the first row of this lane's quad, `pitch` = elements
// between consecutive rows, `n_valid` = rows of the quad that exist (<= 0: none). Warp-collective.
template <bool kBf16>
__device__ __forceinline__ void store_rows_from_tmem(uint32_t taddr, uint16_t* quad_dst, size_t pitch, int n_valid,
                                                     int lane) {
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    uint32_t pk[32];                       // 64 columns as 16-bit pairs: four 32-byte pieces
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t r[32];
      tmem_ld32(taddr + half * 64 + i * 32, r);
      tmem_wait_ld32(r);
#pragma unroll
      for (int c = 0; c < 16; ++c) pk[i * 16 + c] = pack2<kBf16>(__uint_as_float(r[2 * c]), __uint_as_float(r[2 * c + 1]));
    }
    quad_transpose_pieces(pk, lane);
    store_quad_rows(quad_dst + half * 64 + (lane & 3) * 16, pitch, n_valid, pk);
  }
}

// K / V tensor maps; *kv_rep receives the number of query heads per key/value head. `kv` may be null (K / V laid
// out like q).
inline int make_kv_maps(CUtensorMap* mk, CUtensorMap* mv, const void* k, const void* v, int32_t dtype, int32_t H,
                        int64_t stride_s, int64_t stride_h, const moba_kv_layout* kv, const moba_plan_info* info,
                        int* kv_rep) {
  int32_t kv_heads = H;
  if (kv) {
    kv_heads = kv->kv_heads;
    stride_s = kv->stride_s;
    stride_h = kv->stride_h;
    MOBA_REQUIRE(kv_heads > 0 && H % kv_heads == 0, MOBA_ERR_ARG, "kv_heads=%d must divide H=%d", kv_heads, H);
    MOBA_REQUIRE(H / kv_heads <= MOBA_MAX_KV_REP, MOBA_ERR_LIMIT, "at most %d query heads per key/value head",
                 MOBA_MAX_KV_REP);
  }
  *kv_rep = H / kv_heads;
  int rc = make_tensor_map_shd(mk, k, dtype, info->total_tokens, kv_heads, stride_s, stride_h, MOBA_TILE);
  if (rc) return rc;
  return make_tensor_map_shd(mv, v, dtype, info->total_tokens, kv_heads, stride_s, stride_h, MOBA_TILE);
}

inline int check_bwd_args(const void* q, const void* k, const void* v, const void* d_out, int32_t dtype,
                          int32_t H, int64_t stride_s, int64_t stride_h, const moba_plan_info* info,
                          const int32_t* meta_dev, const float* lse, const float* delta,
                          const int32_t* status) {
  int rc = check_common(q, H, stride_s, stride_h, info, meta_dev);
  if (rc) return rc;
  MOBA_REQUIRE(k && v && d_out && lse && delta && status, MOBA_ERR_ARG, "null pointer argument");
  MOBA_REQUIRE(dtype == MOBA_DTYPE_BF16 || dtype == MOBA_DTYPE_F16, MOBA_ERR_ARG,
               "attention kernels take bf16 or f16 tensors (dtype=%d)", dtype);
  return 0;
}

}  // namespace moba
