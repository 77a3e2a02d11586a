// Key mean-pooling over varlen chunks (HBM-bound): one coalesced pass over K.
// Follows MoonshotAI/MoBA moba/moba_efficient.py:335-340: fp32 sum, times 1/len, rounded to the input dtype,
// then widened to fp32 for the gate. Two steps so that large chunks spread over many CTAs and the summation
// order stays fixed: (1) per 128-token tile partial sums, (2) per chunk sum of its tiles in tile order.
#include "common.cuh"

#include <mutex>

namespace moba {
namespace {

template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = __bfloat1622float2(h[i]);
      f[2 * i] = v.x;
      f[2 * i + 1] = v.y;
    }
  }
  static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};
template <> struct Vec8<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&f)[8]) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = __half22float2(h[i]);
      f[2 * i] = v.x;
      f[2 * i + 1] = v.y;
    }
  }
  static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  static __device__ __forceinline__ float round(float x) { return x; }
};

// grid: (n_qtiles, ceil(H*16 / blockDim.x)); thread = one group of 8 consecutive head-dim elements
template <typename T>
__global__ void __launch_bounds__(128)
pool_partial_kernel(const T* __restrict__ k, int H, int64_t stride_s, int64_t stride_h, PlanDev plan,
                    float* __restrict__ ws) {
  const int tile = blockIdx.x;
  const int col8 = blockIdx.y * blockDim.x + threadIdx.x;
  if (col8 >= H * 16) return;
  const int h = col8 >> 4, d8 = col8 & 15;
  const int chunk = plan.qtile_chunk[tile];
  const int t0 = plan.qtile_start[tile];
  const int t1 = min(t0 + MOBA_TILE, plan.chunk_start[chunk + 1]);
  const T* p = k + static_cast<int64_t>(t0) * stride_s + static_cast<int64_t>(h) * stride_h + d8 * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  int t = t0;
  for (; t + 8 <= t1; t += 8) {
    float f[8][8];
#pragma unroll
    for (int u = 0; u < 8; ++u) Vec8<T>::load(p + static_cast<int64_t>(u) * stride_s, f[u]);
#pragma unroll
    for (int u = 0; u < 8; ++u)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[u][i];
    p += 8 * stride_s;
  }
  for (; t < t1; ++t) {
    float f[8];
    Vec8<T>::load(p, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += f[i];
    p += stride_s;
  }
  float4* o = reinterpret_cast<float4*>(ws + (static_cast<int64_t>(tile) * H * 16 + col8) * 8);
  o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
  o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

// grid: (n_chunks, ceil(H*128 / blockDim.x)); thread = one (head, d) column of one chunk
template <typename T>
__global__ void __launch_bounds__(256)
pool_finalize_kernel(const float* __restrict__ ws, int H, PlanDev plan, float* __restrict__ kmean) {
  const int chunk = blockIdx.x;
  const int col = blockIdx.y * blockDim.x + threadIdx.x;
  const int ncol = H * MOBA_HEAD_DIM;
  if (col >= ncol) return;
  const int tile0 = plan.chunk_qtile_first[chunk], tile1 = plan.chunk_qtile_first[chunk + 1];
  const int len = plan.chunk_start[chunk + 1] - plan.chunk_start[chunk];
  float acc = 0.f;
  for (int t = tile0; t < tile1; ++t) acc += ws[static_cast<int64_t>(t) * ncol + col];
  const float mean = acc * (1.0f / static_cast<float>(len));
  kmean[static_cast<int64_t>(chunk) * ncol + col] = Vec8<T>::round(mean);
}

template <typename T>
int launch_pool(const void* k, int32_t H, int64_t stride_s, int64_t stride_h, const PlanDev& plan,
                float* ws, float* kmean, cudaStream_t st) {
  if (plan.n_qtiles == 0) return 0;
  dim3 g1(plan.n_qtiles, (H * 16 + 127) / 128);
  pool_partial_kernel<T><<<g1, 128, 0, st>>>(static_cast<const T*>(k), H, stride_s, stride_h, plan, ws);
  MOBA_CUDA_OK(cudaGetLastError());
  dim3 g2(plan.n_chunks, (H * MOBA_HEAD_DIM + 255) / 256);
  pool_finalize_kernel<T><<<g2, 256, 0, st>>>(ws, H, plan, kmean);
  MOBA_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace
}  // namespace moba

extern "C" int64_t moba_pool_ws_floats(const moba_plan_info* info, int32_t H) {
  if (!info || H < 1) return 0;
  return static_cast<int64_t>(info->n_qtiles) * H * MOBA_HEAD_DIM;
}

extern "C" int moba_pool_keys(const void* k, int32_t dtype, int32_t H, int64_t stride_s, int64_t stride_h,
                              const moba_plan_info* info, const int32_t* meta_dev, float* pool_ws,
                              float* kmean, int32_t device, void* stream) {
  using namespace moba;
  int rc = check_common(k, H, stride_s, stride_h, info, meta_dev);
  if (rc) return rc;
  MOBA_REQUIRE(pool_ws && kmean, MOBA_ERR_ARG, "null pointer argument");
  MOBA_REQUIRE(info->n_qtiles <= 2147483647 && (H * 16 + 127) / 128 <= 65535, MOBA_ERR_LIMIT, "grid too large");
  MOBA_SET_DEVICE(device);
  const PlanDev plan = make_plan_dev(info, meta_dev);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case MOBA_DTYPE_BF16: return launch_pool<__nv_bfloat16>(k, H, stride_s, stride_h, plan, pool_ws, kmean, st);
    case MOBA_DTYPE_F16: return launch_pool<__half>(k, H, stride_s, stride_h, plan, pool_ws, kmean, st);
    case MOBA_DTYPE_F32: return launch_pool<float>(k, H, stride_s, stride_h, plan, pool_ws, kmean, st);
    default: return set_error(MOBA_ERR_ARG, "unsupported dtype %d", dtype);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Allocation-free variant of moba_pool_keys.
//
// Some callers of this library cannot hand it scratch memory: a serving process that gave every free byte of
// the device to its own arena at start-up (a later cudaMalloc would fail, and cudaMalloc / cudaFree also stall
// the whole device), or a host binding written in a language that has no device allocator of its own. For
// them the per-tile partial sums live in the fixed array below instead of a caller-provided workspace.
//
// The array is part of the library image: every GPU that loads libmoba_b200.so carries these 16 MiB until the
// process exits. All calls on a device share it and it keeps whatever the previous call left there. Nothing
// has to be cleared, because a call writes every partial sum before it reads it; but two calls whose kernels
// overlap on the GPU (different streams) race on it, so keep calls on one device in stream order.
constexpr int64_t kPoolStaticFloats = 4ll * 1024 * 1024;    // 16 MiB: e.g. 131072 tokens x 32 heads x 128
static __device__ __align__(256) float g_pool_scratch[kPoolStaticFloats];

namespace moba {
namespace {

constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
float* g_scratch_ptr[kMaxDevices] = {nullptr};

// In host code `g_pool_scratch` is only a handle for the symbol, not a device address. The address differs
// per device, so it is looked up once per device (with that device current) and remembered.
int pool_scratch_address(int device, float** out) {
  MOBA_REQUIRE(device >= 0 && device < kMaxDevices, MOBA_ERR_ARG, "device ordinal %d out of range", device);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_ptr[device]) {
    MOBA_SET_DEVICE(device);
    void* p = nullptr;
    MOBA_CUDA_OK(cudaGetSymbolAddress(&p, g_pool_scratch));
    g_scratch_ptr[device] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[device];
  return 0;
}

}  // namespace
}  // namespace moba

extern "C" int64_t moba_pool_keys_static_max_floats(void) { return kPoolStaticFloats; }

extern "C" int moba_pool_keys_static(const void* k, int32_t dtype, int32_t H, int64_t stride_s, int64_t stride_h,
                                     const moba_plan_info* info, const int32_t* meta_dev, float* kmean,
                                     int32_t device, void* stream) {
  using namespace moba;
  int rc = check_common(k, H, stride_s, stride_h, info, meta_dev);
  if (rc) return rc;
  MOBA_REQUIRE(kmean, MOBA_ERR_ARG, "null pointer argument");
  const int64_t need = moba_pool_ws_floats(info, H);
  MOBA_REQUIRE(need <= kPoolStaticFloats, MOBA_ERR_LIMIT,
               "moba_pool_keys_static: %lld query tiles x %d heads need %lld scratch floats, the built-in scratch "
               "holds %lld; use moba_pool_keys with a caller-provided workspace",
               (long long)info->n_qtiles, H, (long long)need, (long long)kPoolStaticFloats);
  MOBA_REQUIRE((H * 16 + 127) / 128 <= 65535, MOBA_ERR_LIMIT, "grid too large");
  float* ws = nullptr;
  rc = pool_scratch_address(device, &ws);     // first call on a device: symbol lookup (do it before any capture)
  if (rc) return rc;
  MOBA_SET_DEVICE(device);
  const PlanDev plan = make_plan_dev(info, meta_dev);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case MOBA_DTYPE_BF16: return launch_pool<__nv_bfloat16>(k, H, stride_s, stride_h, plan, ws, kmean, st);
    case MOBA_DTYPE_F16: return launch_pool<__half>(k, H, stride_s, stride_h, plan, ws, kmean, st);
    case MOBA_DTYPE_F32: return launch_pool<float>(k, H, stride_s, stride_h, plan, ws, kmean, st);
    default: return set_error(MOBA_ERR_ARG, "unsupported dtype %d", dtype);
  }
}
