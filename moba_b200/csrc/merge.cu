// HBM-bound row kernels around the attention tiles: log-sum-exp merge of partial results, the backward row
// term delta = rowsum(dO * O), and the sum of dq partials. One warp per (token, head) row of 128 elements,
// each lane owns 4 consecutive elements (8 bytes), partial rows are fetched by index (no atomics, fixed
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

// Restates MoonshotAI/MoBA moba/moba_efficient.py:118-168: m = max of the partial LSEs, se = sum of
// exp(lse - m), L = log(se) + m, out = sum_j out_j * exp(lse_j - L). In place on out / lse (the self result).
template <bool kBf16>
__global__ void __launch_bounds__(256)
merge_fwd_kernel(uint16_t* __restrict__ out, float* __restrict__ lse, int64_t n_rows, int kk,
                 const uint16_t* __restrict__ part_o, const float* __restrict__ part_lse,
                 const int32_t* __restrict__ row_of) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (idx >= n_rows) return;
  const float ls = lse[idx];
  int r = -1;
  float lj = -INFINITY;
  if (lane < kk) {
    r = row_of[idx * kk + lane];
    if (r >= 0) lj = part_lse[r];
  }
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

  uint2* orow = reinterpret_cast<uint2*>(out + idx * MOBA_HEAD_DIM) + lane;
  float acc[4], f[4];
  unpack4<kBf16>(*orow, f);
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = f[i] * ws;
  for (int j = 0; j < kk; ++j) {
    const int rj = __shfl_sync(0xffffffffu, r, j);
    const float w = __shfl_sync(0xffffffffu, wj, j);
    if (rj >= 0) {
      unpack4<kBf16>(__ldg(reinterpret_cast<const uint2*>(part_o + static_cast<int64_t>(rj) * MOBA_HEAD_DIM) + lane), f);
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = fmaf(f[i], w, acc[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] *= inv;
  *orow = pack4<kBf16>(acc);
  if (lane == 0) lse[idx] = m + __logf(se);
}

template <bool kBf16>
__global__ void __launch_bounds__(256)
delta_kernel(const uint16_t* __restrict__ out, const uint16_t* __restrict__ d_out, int64_t n_rows,
             float* __restrict__ delta) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (idx >= n_rows) return;
  float a[4], b[4];
  unpack4<kBf16>(__ldg(reinterpret_cast<const uint2*>(out + idx * MOBA_HEAD_DIM) + lane), a);
  unpack4<kBf16>(__ldg(reinterpret_cast<const uint2*>(d_out + idx * MOBA_HEAD_DIM) + lane), b);
  float s = a[0] * b[0] + a[1] * b[1] + a[2] * b[2] + a[3] * b[3];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) delta[idx] = s;
}

template <bool kBf16>
__global__ void __launch_bounds__(256)
merge_dq_kernel(uint16_t* __restrict__ dq, const float* __restrict__ dq_self, int64_t n_rows, int kk,
                const float* __restrict__ part_dq, const int32_t* __restrict__ row_of) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (idx >= n_rows) return;
  int r = -1;
  if (kk > 0 && lane < kk) r = row_of[idx * kk + lane];
  const float4 s4 = __ldg(reinterpret_cast<const float4*>(dq_self + idx * MOBA_HEAD_DIM) + lane);
  float acc[4] = {s4.x, s4.y, s4.z, s4.w};
  for (int j = 0; j < kk; ++j) {
    const int rj = __shfl_sync(0xffffffffu, r, j);
    if (rj >= 0) {
      const float4 f = __ldg(reinterpret_cast<const float4*>(part_dq + static_cast<int64_t>(rj) * MOBA_HEAD_DIM) + lane);
      acc[0] += f.x; acc[1] += f.y; acc[2] += f.z; acc[3] += f.w;
    }
  }
  *(reinterpret_cast<uint2*>(dq + idx * MOBA_HEAD_DIM) + lane) = pack4<kBf16>(acc);
}

// Copies the rows every (chunk, head) list names into list order: qg / dog [R*H, 128] and lse_g / delta_g
// [R*H]. One CTA per 128-row list tile (found by binary search in work_off, like the attention kernels); a
// warp moves one row per step, 8 bytes per lane and tensor. The dK/dV kernel re-reads every list 128-key-tile
// many times, so it takes contiguous tiles by TMA instead of gathering rows itself.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ d_out, const float* __restrict__ lse,
                   const float* __restrict__ delta, int H, int64_t stride_s, int64_t stride_h, int n_experts,
                   const int32_t* __restrict__ list_off, const int32_t* __restrict__ work_off,
                   const int32_t* __restrict__ list_tok, uint16_t* __restrict__ qg, uint16_t* __restrict__ dog,
                   float* __restrict__ lse_g, float* __restrict__ delta_g) {
  __shared__ int s_work[3];
  if (threadIdx.x == 0) {
    const int w = blockIdx.x;
    if (w >= work_off[n_experts]) {
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
  const unsigned grid = static_cast<unsigned>((n + 7) / 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == MOBA_DTYPE_BF16)
    merge_fwd_kernel<true><<<grid, 256, 0, st>>>(static_cast<uint16_t*>(out), lse, n, info->kk,
                                                 static_cast<const uint16_t*>(part_o), part_lse, row_of);
  else
    merge_fwd_kernel<false><<<grid, 256, 0, st>>>(static_cast<uint16_t*>(out), lse, n, info->kk,
                                                  static_cast<const uint16_t*>(part_o), part_lse, row_of);
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
  const unsigned grid = static_cast<unsigned>((n + 7) / 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == MOBA_DTYPE_BF16)
    delta_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(out), static_cast<const uint16_t*>(d_out), n, delta);
  else
    delta_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(out), static_cast<const uint16_t*>(d_out), n, delta);
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
  const unsigned grid = static_cast<unsigned>((n + 7) / 8);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == MOBA_DTYPE_BF16)
    merge_dq_kernel<true><<<grid, 256, 0, st>>>(static_cast<uint16_t*>(dq), dq_self, n, info->kk, part_dq, row_of);
  else
    merge_dq_kernel<false><<<grid, 256, 0, st>>>(static_cast<uint16_t*>(dq), dq_self, n, info->kk, part_dq, row_of);
  MOBA_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int moba_gather_rows(const void* q, const void* d_out, const float* lse, const float* delta,
                                int32_t dtype, int32_t H, int64_t stride_s, int64_t stride_h,
                                const moba_plan_info* info, const int32_t* list_off, const int32_t* work_off,
                                const int32_t* list_tok, void* qg, void* dog, float* lse_g, float* delta_g,
                                int32_t device, void* stream) {
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
      info->n_chunks * H, list_off, work_off, list_tok, static_cast<uint16_t*>(qg), static_cast<uint16_t*>(dog),
      lse_g, delta_g);
  MOBA_CUDA_OK(cudaGetLastError());
  return 0;
}
