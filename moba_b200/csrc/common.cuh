// Host-side helpers shared by all translation units of libmoba_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/moba_b200.h"

namespace moba {

// thread-local message for moba_last_error_string()
char* last_error_buf();
int set_error(int code, const char* fmt, ...);

#define MOBA_CUDA_OK(expr)                                                                     \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess) {                                                                   \
      return moba::set_error(static_cast<int>(_e), "%s failed: %s (%s:%d)", #expr,           \
                             cudaGetErrorString(_e), __FILE__, __LINE__);                      \
    }                                                                                          \
  } while (0)

// Makes `device` current for the rest of the calling function and restores the caller's device on every return
// path: the library shares the thread's CUDA context with its caller (torch), which must not find its current
// device changed by a call that was handed tensors of another GPU.
struct DeviceGuard {
  int prev = -1;
  bool changed = false;
  cudaError_t set(int device) {
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return e;
    if (prev == device) return cudaSuccess;
    e = cudaSetDevice(device);
    changed = e == cudaSuccess;
    return e;
  }
  ~DeviceGuard() {
    if (changed) cudaSetDevice(prev);
  }
};
#define MOBA_SET_DEVICE(device)  \
  moba::DeviceGuard _moba_device_guard; \
  MOBA_CUDA_OK(_moba_device_guard.set(device))

#define MOBA_REQUIRE(cond, code, ...)                     \
  do {                                                    \
    if (!(cond)) return moba::set_error((code), __VA_ARGS__); \
  } while (0)

// Device-side view of the plan tables.
struct PlanDev {
  const int32_t* chunk_start;
  const int32_t* chunk_seq_first;
  const int32_t* chunk_seq_last;
  const int32_t* qtile_chunk;
  const int32_t* qtile_start;
  const int32_t* qtile_cand_off;
  const int32_t* chunk_qtile_first;
  int32_t n_chunks, n_qtiles, kk, chunk_size, total_tokens;
};

inline PlanDev make_plan_dev(const moba_plan_info* info, const int32_t* meta_dev) {
  PlanDev p;
  p.chunk_start = meta_dev + info->off_chunk_start;
  p.chunk_seq_first = meta_dev + info->off_chunk_seq_first;
  p.chunk_seq_last = meta_dev + info->off_chunk_seq_last;
  p.qtile_chunk = meta_dev + info->off_qtile_chunk;
  p.qtile_start = meta_dev + info->off_qtile_start;
  p.qtile_cand_off = meta_dev + info->off_qtile_cand_off;
  p.chunk_qtile_first = meta_dev + info->off_chunk_qtile_first;
  p.n_chunks = info->n_chunks;
  p.n_qtiles = info->n_qtiles;
  p.kk = info->kk;
  p.chunk_size = info->chunk_size;
  p.total_tokens = info->total_tokens;
  return p;
}

// 3-D tensor map over a [S, H, 128] 16-bit tensor: dims (d, h, s), box (64, 1, box_rows), 128-byte
// swizzle. One box is a [box_rows x 64] sub-tile; a 128-wide tile is two boxes (x = 0 and x = 64).
int make_tensor_map_shd(CUtensorMap* map, const void* base, int32_t dtype, int64_t S, int32_t H,
                        int64_t stride_s, int64_t stride_h, int32_t box_rows);

// 2-D tensor map for row gathers (tile::gather4) over the same [S, H, 128] tensor viewed as [S*H, 128] rows:
// dims (d, row), box (64, 1), 128-byte swizzle. Needs stride_s == H * stride_h (rows evenly spaced).
int make_tensor_map_rows(CUtensorMap* map, const void* base, int32_t dtype, int64_t n_rows, int64_t row_stride);

// Tensor-pipe gate for 16-bit q (gate_umma.cu); same outputs as the fp32-FMA gate in gate.cu.
int launch_gate_umma(const void* q, int32_t dtype, int32_t H, int64_t stride_s, int64_t stride_h, const float* kmean,
                     int kv_rep, const moba_plan_info* info, const PlanDev& plan, int32_t* sel, float* sel_score,
                     int32_t* tile_cnt, int32_t* status, cudaStream_t st);

inline int check_common(const void* q, int32_t H, int64_t stride_s, int64_t stride_h,
                        const moba_plan_info* info, const int32_t* meta_dev) {
  MOBA_REQUIRE(q && info && meta_dev, MOBA_ERR_ARG, "null pointer argument");
  MOBA_REQUIRE(H >= 1 && H <= 65535, MOBA_ERR_ARG, "H=%d out of range [1, 65535]", H);
  MOBA_REQUIRE(stride_h >= MOBA_HEAD_DIM && stride_s >= (int64_t)H * 0 + MOBA_HEAD_DIM, MOBA_ERR_ARG,
               "strides (%lld, %lld) smaller than head_dim", (long long)stride_s, (long long)stride_h);
  MOBA_REQUIRE(stride_s % 8 == 0 && stride_h % 8 == 0, MOBA_ERR_ARG,
               "strides must be multiples of 8 elements (16-byte rows)");
  return 0;
}

}  // namespace moba
