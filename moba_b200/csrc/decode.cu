// Dense causal attention for the decode phase (few query positions against a long key/value cache), sm_100a.
//
// Replaces the flash_attn_func(query, key, value, dropout, scaling, True) call of MoonshotAI/MoBA
// moba/wrapper.py:76-82 (the reference has no MoBA decode; its decode step is dense attention with the causal mask
// aligned to the end of the keys). The work is reading K and V once: 2 * kv_len * 128 * 2 bytes per (batch,
// key/value head) against 4 * rows * kv_len * 128 flops for the rows = q_len * (query heads per key/value head)
// query rows that share them, i.e. bound by HBM for every realistic row count. So the kernel is built around the
// memory stream, not the tensor pipe:
//   * the keys of one (batch, key/value head) are cut into `splits` ranges so that the grid fills the GPU; a CTA
//     streams its range as 64-key tiles of K and V through a three-stage ring of TMA loads (128-byte swizzle,
//     32 KB per stage, two CTAs per SM = 192 KB in flight per SM) issued by a producer warp;
//   * four consumer warps take 16 keys of every tile each and keep their own online softmax (running maximum, sum
//     and a 16 x 128 fp32 output accumulator in registers) for a block of 16 query rows: S = Q K^T and O += P V as
//     m16n8k16 warp MMAs fed by ldmatrix from the swizzled tiles, P staying in registers between the two;
//   * the four warps' results are merged through shared memory, every CTA writes (max, sum, unnormalised output)
//     of its range to a workspace, and a second small kernel merges the ranges and writes the output.
// All query heads of a group read the K / V tiles once (the rows of a block are q_len x group heads).
#include "common.cuh"
#include "ptx.cuh"

namespace moba {
namespace {

constexpr int kDecStages = 3;
constexpr int kDecWarps = 4;                          // consumer warps
constexpr int kDecThreads = (kDecWarps + 1) * 32;     // + the producer warp
constexpr int kKeyTile = 64;
constexpr int kRowBlock = 16;
constexpr int kPartFloats = 2 * kRowBlock + kRowBlock * MOBA_HEAD_DIM;   // m[16], l[16], o[16][128]
constexpr float kNegBig = -1.0e30f;                   // "no key seen yet": finite, so differences stay finite

struct __align__(1024) DecSmem {
  uint8_t k[kDecStages][2][8192];   // [stage][d half][64 keys x 64], 128-byte swizzle
  uint8_t v[kDecStages][2][8192];
  uint64_t bar_full[kDecStages], bar_empty[kDecStages];
  int abort_flag;
};
static_assert(sizeof(DecSmem::k) >= kDecWarps * kPartFloats * sizeof(float), "warp merge reuses the K ring");

struct DecArgs {
  const uint16_t* q;
  int64_t q_stride_b, q_stride_h, q_stride_l;
  int Hq, Hkv, Lq, Lk, rep, rows, row_blocks, splits, tiles_per_split, n_tiles;
  float scale_log2;
  float* ws;
  int* status;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <bool kBf16>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (kBf16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(kDecThreads, 2)
decode_attn_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                   const DecArgs a) {
  extern __shared__ uint8_t smem_raw[];
  DecSmem& sm = *reinterpret_cast<DecSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  WaitCtx wctx{&sm.abort_flag, a.status};

  int idx = blockIdx.x;
  const int split = idx % a.splits;
  idx /= a.splits;
  const int rb = idx % a.row_blocks;
  const int bh = idx / a.row_blocks;                 // batch * Hkv + key/value head
  const int b = bh / a.Hkv, hkv = bh - b * a.Hkv;
  const int t_begin = split * a.tiles_per_split;
  const int t_end = min(t_begin + a.tiles_per_split, a.n_tiles);
  const int n_local = t_end - t_begin;

  if (tid == 0) {
    sm.abort_flag = 0;
    for (int i = 0; i < kDecStages; ++i) {
      mbar_init(&sm.bar_full[i], 1);
      mbar_init(&sm.bar_empty[i], kDecWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kDecWarps) {
    // ================= producer: K and V tiles of the range through the ring =================
    if (lane == 0) {
      for (int n = 0; n < n_local; ++n) {
        const int st = n % kDecStages;
        if (n >= kDecStages && !mbar_wait(&sm.bar_empty[st], (n / kDecStages - 1) & 1, wctx)) break;
        const int key0 = (t_begin + n) * kKeyTile;      // rows past kv_len are filled with zeros
        mbar_arrive_expect_tx(&sm.bar_full[st], 32768);
        tma_load_3d(smem_u32(sm.k[st][0]), &map_k, &sm.bar_full[st], 0, bh, key0);
        tma_load_3d(smem_u32(sm.k[st][1]), &map_k, &sm.bar_full[st], 64, bh, key0);
        tma_load_3d(smem_u32(sm.v[st][0]), &map_v, &sm.bar_full[st], 0, bh, key0);
        tma_load_3d(smem_u32(sm.v[st][1]), &map_v, &sm.bar_full[st], 64, bh, key0);
      }
    }
    return;
  }

  // ================= consumers: warp w owns keys [16 w, 16 w + 16) of every tile =================
  const int g = lane >> 2, t = lane & 3;
  // query rows of this thread: r0 = block row g, r1 = g + 8; row r = (head in group) * q_len + position
  int lim[2];
  uint32_t qa[8][4];
  {
    const uint16_t* ptr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = rb * kRowBlock + g + 8 * h;
      if (r < a.rows) {
        const int j = r / a.Lq, i = r - j * a.Lq;
        ptr[h] = a.q + b * a.q_stride_b + static_cast<int64_t>(hkv * a.rep + j) * a.q_stride_h + i * a.q_stride_l;
        lim[h] = a.Lk - a.Lq + i;                     // last key this query position may see
      } else {
        ptr[h] = nullptr;
        lim[h] = -1;
      }
    }
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int d = ks * 16 + 2 * t;
      qa[ks][0] = ptr[0] ? *reinterpret_cast<const uint32_t*>(ptr[0] + d) : 0u;
      qa[ks][1] = ptr[1] ? *reinterpret_cast<const uint32_t*>(ptr[1] + d) : 0u;
      qa[ks][2] = ptr[0] ? *reinterpret_cast<const uint32_t*>(ptr[0] + d + 8) : 0u;
      qa[ks][3] = ptr[1] ? *reinterpret_cast<const uint32_t*>(ptr[1] + d + 8) : 0u;
    }
  }
  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {kNegBig, kNegBig}, l_run[2] = {0.f, 0.f};

  // per-lane ldmatrix row: matrix = lane / 8, row inside it = lane % 8
  const int mat = lane >> 3, rr = lane & 7;
  const int k_row = warp * 16 + (mat >> 1) * 8 + rr, k_chunk = mat & 1;      // K: matrices (keys lo|hi) x (d lo|hi)
  const int v_row = warp * 16 + (mat & 1) * 8 + rr, v_chunk = mat >> 1;      // V (transposed): (d lo|hi) x (keys lo|hi)

  bool ok = true;
  for (int n = 0; n < n_local; ++n) {
    const int st = n % kDecStages;
    ok = __all_sync(0xffffffffu, mbar_wait(&sm.bar_full[st], (n / kDecStages) & 1, wctx));
    if (!ok) break;
    const uint32_t k_base = smem_u32(sm.k[st][0]), v_base = smem_u32(sm.v[st][0]);
    const int key0 = (t_begin + n) * kKeyTile + warp * 16;

    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int chunk = ks * 2 + k_chunk;
      uint32_t bk[4];
      ldmatrix_x4(k_base + (chunk >> 3) * 8192u + sw128_offset(k_row, chunk & 7), bk);
      mma_16816<kBf16>(s[0], qa[ks], bk[0], bk[1]);
      mma_16816<kBf16>(s[1], qa[ks], bk[2], bk[3]);
    }
    // causal mask aligned to the end of the keys, scale, online softmax (log2 domain)
    float mx[2] = {kNegBig, kNegBig};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = key0 + nt * 8 + 2 * t + (c & 1);
        const int h = c >> 1;
        s[nt][c] = key <= lim[h] ? s[nt][c] * a.scale_log2 : -INFINITY;
        mx[h] = fmaxf(mx[h], s[nt][c]);
      }
    float corr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      corr[h] = ex2_approx(m_run[h] - m_new);
      m_run[h] = m_new;
      l_run[h] *= corr[h];
    }
    uint32_t pa[4];
    {
      float p[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          p[nt][c] = ex2_approx(s[nt][c] - m_run[c >> 1]);
          l_run[c >> 1] += p[nt][c];
        }
      pa[0] = pack2<kBf16>(p[0][0], p[0][1]);
      pa[1] = pack2<kBf16>(p[0][2], p[0][3]);
      pa[2] = pack2<kBf16>(p[1][0], p[1][1]);
      pa[3] = pack2<kBf16>(p[1][2], p[1][3]);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o[i][0] *= corr[0];
      o[i][1] *= corr[0];
      o[i][2] *= corr[1];
      o[i][3] *= corr[1];
    }
#pragma unroll
    for (int dn = 0; dn < 8; ++dn) {
      const int chunk = dn * 2 + v_chunk;
      uint32_t bv[4];
      ldmatrix_x4_trans(v_base + (chunk >> 3) * 8192u + sw128_offset(v_row, chunk & 7), bv);
      mma_16816<kBf16>(o[2 * dn], pa, bv[0], bv[1]);
      mma_16816<kBf16>(o[2 * dn + 1], pa, bv[2], bv[3]);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.bar_empty[st]);      // the stage may be refilled
  }

  // ---- merge the four warps (each saw a quarter of the keys) and write this range's partial result ----------
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  float* part = reinterpret_cast<float*>(&sm.k[0][0][0]);         // every load of the ring has been consumed
  asm volatile("bar.sync 1, %0;" ::"n"(kDecWarps * 32) : "memory");   // ... by all four warps
  {
    float* wp = part + warp * kPartFloats;
    if (t == 0) {
      wp[g] = m_run[0];
      wp[g + 8] = m_run[1];
      wp[kRowBlock + g] = l_run[0];
      wp[kRowBlock + g + 8] = l_run[1];
    }
    float* wo = wp + 2 * kRowBlock;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      *reinterpret_cast<float2*>(wo + g * MOBA_HEAD_DIM + i * 8 + 2 * t) = make_float2(o[i][0], o[i][1]);
      *reinterpret_cast<float2*>(wo + (g + 8) * MOBA_HEAD_DIM + i * 8 + 2 * t) = make_float2(o[i][2], o[i][3]);
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kDecWarps * 32) : "memory");
  {
    float* dst = a.ws + (static_cast<size_t>(bh * a.row_blocks + rb) * a.splits + split) * kPartFloats;
    const int d = tid;                                  // 128 consumer threads = 128 output columns
    for (int row = 0; row < kRowBlock; ++row) {
      float mw[kDecWarps], M = kNegBig;
#pragma unroll
      for (int w = 0; w < kDecWarps; ++w) {
        mw[w] = part[w * kPartFloats + row];
        M = fmaxf(M, mw[w]);
      }
      float num = 0.f, den = 0.f;
#pragma unroll
      for (int w = 0; w < kDecWarps; ++w) {
        const float f = ex2_approx(mw[w] - M);
        num += f * part[w * kPartFloats + 2 * kRowBlock + row * MOBA_HEAD_DIM + d];
        den += f * part[w * kPartFloats + kRowBlock + row];
      }
      if (!ok) num = den = 0.f;                         // a wait expired: the status word says so
      dst[2 * kRowBlock + row * MOBA_HEAD_DIM + d] = num;
      if (d == 0) {
        dst[row] = M;
        dst[kRowBlock + row] = den;
      }
    }
  }
}

// out[b, i, head, :] = sum over ranges of o * 2^(m - M) / sum over ranges of l * 2^(m - M). One CTA per query row:
// the weights of all ranges are computed once into shared memory (a block reduction for M and the denominator),
// then thread d sums column d over the ranges with independent loads (a serial walk over the ranges would pay one
// memory latency per range).
constexpr int kMaxSplits = 1024;

template <bool kBf16>
__global__ void __launch_bounds__(128)
decode_merge_kernel(const DecArgs a, uint16_t* __restrict__ out) {
  __shared__ float w_s[kMaxSplits];
  __shared__ float red[8];
  const int row = blockIdx.y, rb = blockIdx.x % a.row_blocks, bh = blockIdx.x / a.row_blocks;
  const int r = rb * kRowBlock + row;
  if (r >= a.rows) return;
  const int b = bh / a.Hkv, hkv = bh - b * a.Hkv;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* src = a.ws + static_cast<size_t>(bh * a.row_blocks + rb) * a.splits * kPartFloats;
  float m_loc = kNegBig;
  for (int s = tid; s < a.splits; s += 128) {
    const float m = src[s * kPartFloats + row];
    w_s[s] = m;
    m_loc = fmaxf(m_loc, m);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) m_loc = fmaxf(m_loc, __shfl_xor_sync(0xffffffffu, m_loc, d));
  if (lane == 0) red[warp] = m_loc;
  __syncthreads();
  const float M = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  float den = 0.f;
  for (int s = tid; s < a.splits; s += 128) {
    const float f = ex2_approx(w_s[s] - M);
    w_s[s] = f;
    den += f * src[s * kPartFloats + kRowBlock + row];
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) den += __shfl_xor_sync(0xffffffffu, den, d);
  if (lane == 0) red[4 + warp] = den;
  __syncthreads();
  den = (red[4] + red[5]) + (red[6] + red[7]);
  const float* col = src + 2 * kRowBlock + row * MOBA_HEAD_DIM + tid;
  float num = 0.f;
  int s = 0;
  for (; s + 8 <= a.splits; s += 8) {
    float x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) x[u] = col[static_cast<size_t>(s + u) * kPartFloats];
#pragma unroll
    for (int u = 0; u < 8; ++u) num += w_s[s + u] * x[u];
  }
  for (; s < a.splits; ++s) num += w_s[s] * col[static_cast<size_t>(s) * kPartFloats];
  const int j = r / a.Lq, i = r - j * a.Lq;
  const float val = den > 0.f ? num / den : 0.f;
  const size_t off = ((static_cast<size_t>(b) * a.Lq + i) * a.Hq + hkv * a.rep + j) * MOBA_HEAD_DIM + tid;
  const float other = __shfl_down_sync(0xffffffffu, val, 1);
  if ((tid & 1) == 0) *reinterpret_cast<uint32_t*>(out + off) = pack2<kBf16>(val, other);
}

// How the keys of one (batch, key/value head, row block) are cut: enough CTAs for two full waves where the length
// allows, never less than four tiles (256 keys) per range.
void choose_splits(int64_t base_ctas, int n_tiles, int* splits, int* tiles_per_split) {
  int64_t want = (4 * 148 + base_ctas - 1) / base_ctas;
  int64_t most = n_tiles / 4 > 0 ? n_tiles / 4 : 1;
  int64_t s = want < most ? want : most;
  if (s < 1) s = 1;
  if (s > kMaxSplits) s = kMaxSplits;
  const int tps = static_cast<int>((n_tiles + s - 1) / s);
  *tiles_per_split = tps;
  *splits = (n_tiles + tps - 1) / tps;
}

}  // namespace
}  // namespace moba

extern "C" int64_t moba_decode_ws_floats(int32_t batch, int32_t q_heads, int32_t kv_heads, int32_t q_len,
                                         int32_t kv_len) {
  using namespace moba;
  if (batch < 1 || kv_heads < 1 || q_heads < kv_heads || q_heads % kv_heads || q_len < 1 || kv_len < q_len) return 0;
  const int rows = q_len * (q_heads / kv_heads);
  const int row_blocks = (rows + kRowBlock - 1) / kRowBlock;
  const int n_tiles = (kv_len + kKeyTile - 1) / kKeyTile;
  int splits, tps;
  choose_splits(static_cast<int64_t>(batch) * kv_heads * row_blocks, n_tiles, &splits, &tps);
  return static_cast<int64_t>(batch) * kv_heads * row_blocks * splits * kPartFloats;
}

extern "C" int moba_decode_attn(const void* q, const void* k, const void* v, int32_t dtype, int32_t batch,
                                int32_t q_heads, int32_t kv_heads, int32_t q_len, int32_t kv_len,
                                int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_l, int64_t kv_stride_h,
                                int64_t kv_stride_l, float scale, void* out, float* ws, int32_t* status,
                                int32_t device, void* stream) {
  using namespace moba;
  MOBA_REQUIRE(q && k && v && out && ws && status, MOBA_ERR_ARG, "null pointer argument");
  MOBA_REQUIRE(dtype == MOBA_DTYPE_BF16 || dtype == MOBA_DTYPE_F16, MOBA_ERR_ARG,
               "decode attention takes bf16 or f16 tensors (dtype=%d)", dtype);
  MOBA_REQUIRE(batch >= 1 && kv_heads >= 1 && q_heads >= kv_heads && q_heads % kv_heads == 0, MOBA_ERR_ARG,
               "batch=%d, q_heads=%d, kv_heads=%d: kv_heads must divide q_heads", batch, q_heads, kv_heads);
  MOBA_REQUIRE(q_len >= 1 && kv_len >= q_len, MOBA_ERR_ARG, "q_len=%d, kv_len=%d: need 1 <= q_len <= kv_len", q_len,
               kv_len);
  MOBA_REQUIRE(q_stride_b % 8 == 0 && q_stride_h % 8 == 0 && q_stride_l % 8 == 0 && kv_stride_h % 8 == 0 &&
                   kv_stride_l % 8 == 0 && kv_stride_l >= MOBA_HEAD_DIM,
               MOBA_ERR_ARG, "strides must be multiples of 8 elements (16-byte rows)");
  MOBA_REQUIRE((reinterpret_cast<uintptr_t>(q) & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 3) == 0, MOBA_ERR_ARG,
               "q / out not 4-byte aligned");
  const int64_t n_bh = static_cast<int64_t>(batch) * kv_heads;
  DecArgs a;
  a.q = static_cast<const uint16_t*>(q);
  a.q_stride_b = q_stride_b; a.q_stride_h = q_stride_h; a.q_stride_l = q_stride_l;
  a.Hq = q_heads; a.Hkv = kv_heads; a.Lq = q_len; a.Lk = kv_len;
  a.rep = q_heads / kv_heads;
  a.rows = q_len * a.rep;
  a.row_blocks = (a.rows + kRowBlock - 1) / kRowBlock;
  a.n_tiles = (kv_len + kKeyTile - 1) / kKeyTile;
  choose_splits(n_bh * a.row_blocks, a.n_tiles, &a.splits, &a.tiles_per_split);
  a.scale_log2 = scale * 1.4426950408889634f;
  a.ws = ws;
  a.status = status;
  const int64_t n_ctas = n_bh * a.row_blocks * a.splits;
  MOBA_REQUIRE(n_ctas < (1ll << 31) && n_bh < (1ll << 31), MOBA_ERR_LIMIT, "too many (batch, head, row block, range) items");
  MOBA_SET_DEVICE(device);
  // K / V as [batch * kv_heads] "heads" of kv_len tokens: one 3-D tensor map each (64-key boxes)
  CUtensorMap mk, mv;
  int rc = make_tensor_map_shd(&mk, k, dtype, kv_len, static_cast<int32_t>(n_bh), kv_stride_l, kv_stride_h, kKeyTile);
  if (rc) return rc;
  rc = make_tensor_map_shd(&mv, v, dtype, kv_len, static_cast<int32_t>(n_bh), kv_stride_l, kv_stride_h, kKeyTile);
  if (rc) return rc;
  const size_t smem = sizeof(DecSmem) + 1024;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(static_cast<unsigned>(n_ctas)), mgrid(static_cast<unsigned>(n_bh * a.row_blocks), kRowBlock);
  if (dtype == MOBA_DTYPE_BF16) {
    MOBA_CUDA_OK(cudaFuncSetAttribute(decode_attn_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    decode_attn_kernel<true><<<grid, kDecThreads, smem, st>>>(mk, mv, a);
    MOBA_CUDA_OK(cudaGetLastError());
    decode_merge_kernel<true><<<mgrid, 128, 0, st>>>(a, static_cast<uint16_t*>(out));
  } else {
    MOBA_CUDA_OK(cudaFuncSetAttribute(decode_attn_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    decode_attn_kernel<false><<<grid, kDecThreads, smem, st>>>(mk, mv, a);
    MOBA_CUDA_OK(cudaGetLastError());
    decode_merge_kernel<false><<<mgrid, 128, 0, st>>>(a, static_cast<uint16_t*>(out));
  }
  MOBA_CUDA_OK(cudaGetLastError());
  return 0;
}
