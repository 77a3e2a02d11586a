// HBM-bound row kernels around the attention tiles: log-sum-exp merge of partial results, the backward row
// term delta = rowsum(dO * O), and the sum of dq partials. A warp works on one (token, head) row of 128 elements
// at a time, each lane owns 4 consecutive elements (8 bytes), partial rows are fetched by index (no atomics, fixed
// summation order).
#include "common.cuh"

namespace moba {
namespace {

template <bool kBf16>
__device__ __forceinline__ void unpack4(uint2 u, float (&f)[4]) {
  if constexpr (kBf16) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  } else {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
    const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  }
}
template <bool kBf16>
__device__ __forceinline__ uint2 pack4(const float (&f)[4]) {
  uint2 u;
  if constexpr (kBf16) {
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
  } else {
    __half2 a = __floats2half2_rn(f[0], f[1]), b = __floats2half2_rn(f[2], f[3]);
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
  }
  return u;
}

// All three row kernels run a fixed number of warps that stride over the rows. What the next row needs first (its
// row_of entries, its own row) is requested one iteration ahead and the partial rows of a row are requested
// together, so a warp keeps several independent loads in flight even when a row has only two or three partials
// (one warp per row with a row_of -> partial-row chain left too little in flight to fill the memory pipe).
constexpr int kRowWarps = 8;             // warps per CTA

// As many CTAs as are resident at once (or fewer when there are fewer rows): the warps stride over the rows, so a
// grid larger than one wave would only add a ragged last wave.
template <typename Kernel>
unsigned row_grid(int64_t n_rows, Kernel kern) {
  int dev = 0, sms = 148, per_sm = 1;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kRowWarps * 32, 0) != cudaSuccess || per_sm < 1)
    per_sm = 1;
  const int64_t want = (n_rows + kRowWarps - 1) / kRowWarps;
  const int64_t cap = static_cast<int64_t>(sms) * per_sm;
  return static_cast<unsigned>(want < cap ? want : cap);
}

// Restates MoonshotAI/MoBA moba/moba_efficient.py:118-168: m = max of the partial LSEs, se = sum of
// exp(lse - m), L = log(se) + m, out = sum_j out_j * exp(lse_j - L). In place on out / lse (the self result).
// KB = partial rows requested together (a row with more slots takes several rounds).
template <bool kBf16, int KB>
__global__ void __launch_bounds__(kRowWarps * 32)
merge_fwd_kernel(uint16_t* __restrict__ out, float* __restrict__ lse, int64_t n_rows, int kk,
                 const uint16_t* __restrict__ part_o, const float* __restrict__ part_lse,
                 const int32_t* __restrict__ row_of) {
  const int lane = threadIdx.x & 31;
  const int64_t n_warps = static_cast<int64_t>(gridDim.x) * kRowWarps;
  int64_t idx = static_cast<int64_t>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5);
  if (idx >= n_rows) return;
  int r_next = lane < kk ? __ldg(row_of + idx * kk + lane) : -1;
  for (; idx < n_rows; idx += n_warps) {
    const int r = r_next;
    const int64_t nxt = idx + n_warps;
    if (nxt < n_rows) r_next = lane < kk ? __ldg(row_of + nxt * kk + lane) : -1;
    const float lj = r >= 0 ? __ldg(part_lse + r) : -INFINITY;
    // the first KB partial rows need only r: requested together with the partial log-sum-exps
    uint2 bits[KB];
#pragma unroll
    for (int j = 0; j < KB; ++j) {
      const int rj = __shfl_sync(0xffffffffu, r, j);
      bits[j] = (j < kk && rj >= 0)
                    ? __ldg(reinterpret_cast<const uint2*>(part_o + static_cast<int64_t>(rj) * MOBA_HEAD_DIM) + lane)
                    : make_uint2(0u, 0u);
    }
    uint2* orow = reinterpret_cast<uint2*>(out + idx * MOBA_HEAD_DIM) + lane;
    const uint2 self_bits = *orow;
    const float ls = lse[idx];
    float m = fmaxf(ls, lj);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float wj = (r >= 0) ? __expf(lj - m) : 0.f;
    const float ws = __expf(ls - m);
    float se = wj;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) se += __shfl_xor_sync(0xffffffffu, se, o);
    se += ws;
    const float inv = 1.0f / se;
    float acc[4], f[4];
    unpack4<kBf16>(self_bits, f);
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = f[i] * ws;
    for (int j0 = 0; j0 < kk; j0 += KB) {
      if (j0 > 0) {
#pragma unroll
        for (int j = 0; j < KB; ++j) {
          const int rj = __shfl_sync(0xffffffffu, r, (j0 + j) & 31);
          bits[j] = (j0 + j < kk && rj >= 0)
                        ? __ldg(reinterpret_cast<const uint2*>(part_o + static_cast<int64_t>(rj) * MOBA_HEAD_DIM) + lane)
                        : make_uint2(0u, 0u);
        }
      }
#pragma unroll
      for (int j = 0; j < KB; ++j) {
        // an empty slot has weight 0 and zero bits
        const float w = __shfl_sync(0xffffffffu, wj, (j0 + j) & 31);
        unpack4<kBf16>(bits[j], f);
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] = fmaf(f[i], (j0 + j < kk) ? w : 0.f, acc[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] *= inv;
    *orow = pack4<kBf16>(acc);
    if (lane == 0) lse[idx] = m + __logf(se);
  }
}

// merge_fwd for rows with at most two partials (kk <= 2): a warp takes two rows per iteration, one per half warp
// for the row_of / log-sum-exp part, so that six row loads are in flight instead of three. The arithmetic per row
// is that of merge_fwd_kernel in the same order (the sums have at most two non-zero terms), so the bits are the same.
template <bool kBf16>
__global__ void __launch_bounds__(kRowWarps * 32)
merge_fwd_pair_kernel(uint16_t* __restrict__ out, float* __restrict__ lse, int64_t n_rows, int kk,
                      const uint16_t* __restrict__ part_o, const float* __restrict__ part_lse,
                      const int32_t* __restrict__ row_of) {
  const int lane = threadIdx.x & 31, half = lane >> 4, slot = lane & 15;
  const int64_t step = static_cast<int64_t>(gridDim.x) * kRowWarps * 2;
  int64_t base = (static_cast<int64_t>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5)) * 2;
  if (base >= n_rows) return;
  auto slot_row = [&](int64_t b) {          // lanes 0.. of each half: the partial rows of row b + half
    const int64_t row = b + half;
    return (slot < kk && row < n_rows) ? __ldg(row_of + row * kk + slot) : -1;
  };
  int r_next = slot_row(base);
  for (; base < n_rows; base += step) {
    const int r = r_next;
    if (base + step < n_rows) r_next = slot_row(base + step);
    const float lj = r >= 0 ? __ldg(part_lse + r) : -INFINITY;
    uint2 bits[2][2], self_bits[2];
    float ls[2];
    uint2* orow[2];
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      const bool live = base + x < n_rows;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int rj = __shfl_sync(0xffffffffu, r, 16 * x + j);
        bits[x][j] = (j < kk && rj >= 0)
                         ? __ldg(reinterpret_cast<const uint2*>(part_o + static_cast<int64_t>(rj) * MOBA_HEAD_DIM) + lane)
                         : make_uint2(0u, 0u);
      }
      orow[x] = reinterpret_cast<uint2*>(out + (base + (live ? x : 0)) * MOBA_HEAD_DIM) + lane;
      self_bits[x] = *orow[x];
      ls[x] = lse[base + (live ? x : 0)];
    }
    // per half warp: m and se of its row
    const float ls_mine = half ? ls[1] : ls[0];
    float m = fmaxf(ls_mine, lj);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float wj = (r >= 0) ? __expf(lj - m) : 0.f;
    const float ws_mine = __expf(ls_mine - m);
    float se = wj;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) se += __shfl_xor_sync(0xffffffffu, se, o);
    se += ws_mine;
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      const float m_x = __shfl_sync(0xffffffffu, m, 16 * x), se_x = __shfl_sync(0xffffffffu, se, 16 * x);
      const float ws = __shfl_sync(0xffffffffu, ws_mine, 16 * x);
      const float inv = 1.0f / se_x;
      float acc[4], f[4];
      unpack4<kBf16>(self_bits[x], f);
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = f[i] * ws;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float w = __shfl_sync(0xffffffffu, wj, 16 * x + j);
        unpack4<kBf16>(bits[x][j], f);
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] = fmaf(f[i], (j < kk) ? w : 0.f, acc[i]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] *= inv;
      if (base + x < n_rows) {
        *orow[x] = pack4<kBf16>(acc);
        if (lane == 0) lse[base + x] = m_x + __logf(se_x);
      }
    }
  }
}

template <bool kBf16>
__global__ void __launch_bounds__(kRowWarps * 32)
delta_kernel(const uint16_t* __restrict__ out, const uint16_t* __restrict__ d_out, int64_t n_rows,
             float* __restrict__ delta) {
  const int lane = threadIdx.x & 31;
  const int64_t n_warps = static_cast<int64_t>(gridDim.x) * kRowWarps;
  // four rows per warp and iteration: eight independent 256-byte loads in flight
  for (int64_t base = (static_cast<int64_t>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5)) * 4; base < n_rows;
       base += n_warps * 4) {
    uint2 a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t idx = base + i < n_rows ? base + i : n_rows - 1;
      a[i] = __ldg(reinterpret_cast<const uint2*>(out + idx * MOBA_HEAD_DIM) + lane);
      b[i] = __ldg(reinterpret_cast<const uint2*>(d_out + idx * MOBA_HEAD_DIM) + lane);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float x[4], y[4];
      unpack4<kBf16>(a[i], x);
      unpack4<kBf16>(b[i], y);
      float s = x[0] * y[0] + x[1] * y[1] + x[2] * y[2] + x[3] * y[3];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0 && base + i < n_rows) delta[base + i] = s;
    }
  }
}

template <bool kBf16, int KB>
__global__ void __launch_bounds__(kRowWarps * 32)
merge_dq_kernel(uint16_t* __restrict__ dq, const float* __restrict__ dq_self, int64_t n_rows, int kk,
                const float* __restrict__ part_dq, const int32_t* __restrict__ row_of) {
  const int lane = threadIdx.x & 31;
  const int64_t n_warps = static_cast<int64_t>(gridDim.x) * kRowWarps;
  int64_t idx = static_cast<int64_t>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5);
  if (idx >= n_rows) return;
  int r_next = (kk > 0 && lane < kk) ? __ldg(row_of + idx * kk + lane) : -1;
  for (; idx < n_rows; idx += n_warps) {
    const int r = r_next;
    const int64_t nxt = idx + n_warps;
    if (nxt < n_rows) r_next = (kk > 0 && lane < kk) ? __ldg(row_of + nxt * kk + lane) : -1;
    const float4 s4 = __ldg(reinterpret_cast<const float4*>(dq_self + idx * MOBA_HEAD_DIM) + lane);
    float acc[4] = {s4.x, s4.y, s4.z, s4.w};
    for (int j0 = 0; j0 < kk; j0 += KB) {
      float4 f[KB];
#pragma unroll
      for (int j = 0; j < KB; ++j) {
        const int rj = __shfl_sync(0xffffffffu, r, (j0 + j) & 31);
        f[j] = (j0 + j < kk && rj >= 0)
                   ? __ldg(reinterpret_cast<const float4*>(part_dq + static_cast<int64_t>(rj) * MOBA_HEAD_DIM) + lane)
                   : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      // summed in slot order (an empty slot adds zero), so the result does not depend on how rows are batched
#pragma unroll
      for (int j = 0; j < KB; ++j) {
        acc[0] += f[j].x; acc[1] += f[j].y; acc[2] += f[j].z; acc[3] += f[j].w;
      }
    }
    *(reinterpret_cast<uint2*>(dq + idx * MOBA_HEAD_DIM) + lane) = pack4<kBf16>(acc);
  }
}

// Copies the rows every (chunk, head) list names into list order: qg / dog [R*H, 128] and lse_g / delta_g
// [R*H]. One CTA per 128-row list tile (its record from moba_tile_records, else a binary search in work_off); a
// warp moves one row per step, 8 bytes per lane and tensor. The dK/dV kernel re-reads every list 128-key-tile
// many times, so it takes contiguous tiles by TMA instead of gathering rows itself.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ d_out, const float* __restrict__ lse,
                   const float* __restrict__ delta, int H, int64_t stride_s, int64_t stride_h, int n_experts,
                   const int32_t* __restrict__ list_off, const int32_t* __restrict__ work_off,
                   const int32_t* __restrict__ list_tok, const int32_t* __restrict__ tile_rec,
                   uint16_t* __restrict__ qg, uint16_t* __restrict__ dog, float* __restrict__ lse_g,
                   float* __restrict__ delta_g) {
  __shared__ int s_work[3];
  if (threadIdx.x == 0) {
    const int w = blockIdx.x;
    if (tile_rec) {
      // the tile's record (moba_tile_records) instead of the search below
      const int4 rec = __ldg(reinterpret_cast<const int4*>(tile_rec) + 2 * static_cast<size_t>(w));
      s_work[0] = rec.x;
      s_work[1] = rec.y;
      s_work[2] = rec.z;
    } else if (w >= work_off[n_experts]) {
      s_work[2] = 0;
    } else {
      int lo = 0, hi = n_experts;          // last e with work_off[e] <= w
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (work_off[mid] <= w) lo = mid; else hi = mid;
      }
      const int first = list_off[lo] + (w - work_off[lo]) * MOBA_TILE;
      s_work[0] = lo % H;
      s_work[1] = first;
      s_work[2] = min(MOBA_TILE, list_off[lo + 1] - first);
    }
  }
  __syncthreads();
  const int head = s_work[0], first = s_work[1], n_rows = s_work[2];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < n_rows; r += 8) {
    const int64_t row = first + r;
    const int tok = list_tok[row];
    const int64_t src = static_cast<int64_t>(tok) * stride_s + static_cast<int64_t>(head) * stride_h;
    const uint2 a = __ldg(reinterpret_cast<const uint2*>(q + src) + lane);
    const uint2 b = __ldg(reinterpret_cast<const uint2*>(d_out + src) + lane);
    reinterpret_cast<uint2*>(qg + row * MOBA_HEAD_DIM)[lane] = a;
    reinterpret_cast<uint2*>(dog + row * MOBA_HEAD_DIM)[lane] = b;
    if (lane == 0) {
      const int64_t i = static_cast<int64_t>(tok) * H + head;
      lse_g[row] = lse[i];
      delta_g[row] = delta[i];
    }
  }
}

inline int check16(int32_t dtype) {
  MOBA_REQUIRE(dtype == MOBA_DTYPE_BF16 || dtype == MOBA_DTYPE_F16, MOBA_ERR_ARG,
               "row kernels take bf16 or f16 tensors (dtype=%d)", dtype);
  return 0;
}

}  // namespace
}  // namespace moba

extern "C" int moba_merge_fwd(void* out, float* lse, int32_t dtype, int32_t H, const moba_plan_info* info,
                              const void* part_o, const float* part_lse, const int32_t* row_of,
                              int32_t device, void* stream) {
  using namespace moba;
  MOBA_REQUIRE(out && lse && info && part_o && part_lse && row_of, MOBA_ERR_ARG, "null pointer argument");
  MOBA_REQUIRE(H >= 1, MOBA_ERR_ARG, "H=%d must be >= 1", H);
  MOBA_REQUIRE(info->kk >= 1 && info->kk <= 32, MOBA_ERR_ARG, "kk=%d outside [1, 32]", info->kk);
  if (int rc = check16(dtype)) return rc;
  MOBA_SET_DEVICE(device);
  const int64_t n = static_cast<int64_t>(info->total_tokens) * H;
  if (n == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto run = [&](auto kern) {
    kern<<<row_grid(n, kern), kRowWarps * 32, 0, st>>>(static_cast<uint16_t*>(out), lse, n, info->kk,
                                          static_cast<const uint16_t*>(part_o), part_lse, row_of);
  };
  const bool bf16 = dtype == MOBA_DTYPE_BF16;
  auto run_pairs = [&](auto kern) {
    kern<<<row_grid((n + 1) / 2, kern), kRowWarps * 32, 0, st>>>(static_cast<uint16_t*>(out), lse, n, info->kk,
                                                static_cast<const uint16_t*>(part_o), part_lse, row_of);
  };
  if (info->kk <= 2) bf16 ? run_pairs(merge_fwd_pair_kernel<true>) : run_pairs(merge_fwd_pair_kernel<false>);
  else bf16 ? run(merge_fwd_kernel<true, 4>) : run(merge_fwd_kernel<false, 4>);
  MOBA_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int moba_bwd_delta(const void* out, const void* d_out, int32_t dtype, int32_t H, int64_t n_tokens,
                              float* delta, int32_t device, void* stream) {
  using namespace moba;
  MOBA_REQUIRE(out && d_out && delta, MOBA_ERR_ARG, "null pointer argument");
  MOBA_REQUIRE(H >= 1 && n_tokens >= 0, MOBA_ERR_ARG, "bad sizes");
  if (int rc = check16(dtype)) return rc;
  MOBA_SET_DEVICE(device);
  const int64_t n = n_tokens * H;
  if (n == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == MOBA_DTYPE_BF16)
    delta_kernel<true><<<row_grid((n + 3) / 4, delta_kernel<true>), kRowWarps * 32, 0, st>>>(
        static_cast<const uint16_t*>(out), static_cast<const uint16_t*>(d_out), n, delta);
  else
    delta_kernel<false><<<row_grid((n + 3) / 4, delta_kernel<false>), kRowWarps * 32, 0, st>>>(
        static_cast<const uint16_t*>(out), static_cast<const uint16_t*>(d_out), n, delta);
  MOBA_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int moba_merge_dq(void* dq, int32_t dtype, int32_t H, const moba_plan_info* info,
                             const float* dq_self, const float* part_dq, const int32_t* row_of,
                             int32_t device, void* stream) {
  using namespace moba;
  MOBA_REQUIRE(dq && info && dq_self, MOBA_ERR_ARG, "null pointer argument");
  MOBA_REQUIRE(H >= 1, MOBA_ERR_ARG, "H=%d must be >= 1", H);
  MOBA_REQUIRE(info->kk >= 0 && info->kk <= 32, MOBA_ERR_ARG, "kk=%d outside [0, 32]", info->kk);
  if (info->kk > 0) MOBA_REQUIRE(part_dq && row_of, MOBA_ERR_ARG, "null partial buffers");
  if (int rc = check16(dtype)) return rc;
  MOBA_SET_DEVICE(device);
  const int64_t n = static_cast<int64_t>(info->total_tokens) * H;
  if (n == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto run = [&](auto kern) {
    kern<<<row_grid(n, kern), kRowWarps * 32, 0, st>>>(static_cast<uint16_t*>(dq), dq_self, n, info->kk, part_dq, row_of);
  };
  const bool bf16 = dtype == MOBA_DTYPE_BF16;
  if (info->kk <= 2) bf16 ? run(merge_dq_kernel<true, 2>) : run(merge_dq_kernel<false, 2>);
  else bf16 ? run(merge_dq_kernel<true, 4>) : run(merge_dq_kernel<false, 4>);
  MOBA_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int moba_gather_rows(const void* q, const void* d_out, const float* lse, const float* delta,
                                int32_t dtype, int32_t H, int64_t stride_s, int64_t stride_h,
                                const moba_plan_info* info, const int32_t* list_off, const int32_t* work_off,
                                const int32_t* list_tok, const int32_t* tile_rec, void* qg, void* dog, float* lse_g,
                                float* delta_g, int32_t device, void* stream) {
  using namespace moba;
  MOBA_REQUIRE(q && d_out && lse && delta && info && list_off && work_off && list_tok && qg && dog && lse_g && delta_g,
               MOBA_ERR_ARG, "null pointer argument");
  MOBA_REQUIRE(H >= 1, MOBA_ERR_ARG, "H=%d must be >= 1", H);
  if (int rc = check16(dtype)) return rc;
  MOBA_SET_DEVICE(device);
  const int64_t nw = info->max_work_tiles_per_head * H;
  if (info->kk == 0 || nw == 0) return 0;
  MOBA_REQUIRE(nw < (1ll << 31), MOBA_ERR_LIMIT, "too many gathered tiles");
  gather_rows_kernel<<<static_cast<unsigned>(nw), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(q), static_cast<const uint16_t*>(d_out), lse, delta, H, stride_s, stride_h,
      info->n_chunks * H, list_off, work_off, list_tok, tile_rec, static_cast<uint16_t*>(qg),
      static_cast<uint16_t*>(dog), lse_g, delta_g);
  MOBA_CUDA_OK(cudaGetLastError());
  return 0;
}
