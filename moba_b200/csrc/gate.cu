// Parameter-less gate, causal top-k and the per-(chunk, head) query lists.
// Semantics (MoonshotAI/MoBA moba/moba_efficient.py:341-386, moba/moba_naive.py:53-73): a query in the c-th
// chunk of its sequence scores the c earlier chunks of the same sequence with an fp32 dot product between
// the query and the chunk's pooled key, and keeps the min(c, topk-1) best. No dense [chunks, H, S] tensor is
// formed: scores live in registers, the selection goes straight into compact index lists.
//
// Kernels:
//   gate_topk_kernel   one CTA per (128-token query tile, head); thread = token
//   expert_scan_kernel one warp per (chunk, head): exclusive prefix of that expert's per-tile counts
//   offsets_kernel     one CTA: exclusive prefix over experts of list lengths and of 128-row tile counts
//   fill_lists_kernel  one CTA per (query tile, head): rows are placed in ascending token order
#include "common.cuh"

namespace moba {
namespace {

constexpr int kCandBatch = 32;   // pooled keys staged in shared memory per step

template <typename T>
__device__ __forceinline__ void load_row128(const T* p, float (&f)[128]);

template <>
__device__ __forceinline__ void load_row128<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[128]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(p) + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 v = __bfloat1622float2(h[j]);
      f[i * 8 + 2 * j] = v.x;
      f[i * 8 + 2 * j + 1] = v.y;
    }
  }
}
template <>
__device__ __forceinline__ void load_row128<__half>(const __half* p, float (&f)[128]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(p) + i);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 v = __half22float2(h[j]);
      f[i * 8 + 2 * j] = v.x;
      f[i * 8 + 2 * j + 1] = v.y;
    }
  }
}
template <>
__device__ __forceinline__ void load_row128<float>(const float* p, float (&f)[128]) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(p) + i);
    f[4 * i] = v.x; f[4 * i + 1] = v.y; f[4 * i + 2] = v.z; f[4 * i + 3] = v.w;
  }
}

// dynamic shared memory: float kmean_s[kCandBatch][128]; uint32_t bitmap[ncand][4]
template <typename T, int KMAX>
__global__ void __launch_bounds__(128)
gate_topk_kernel(const T* __restrict__ q, int H, int64_t stride_s, int64_t stride_h,
                 const float* __restrict__ kmean, int kv_rep, PlanDev plan, int32_t* __restrict__ sel,
                 float* __restrict__ sel_score, int32_t* __restrict__ tile_cnt) {
  extern __shared__ __align__(16) uint8_t gate_smem[];
  float* km = reinterpret_cast<float*>(gate_smem);
  uint32_t* bitmap = reinterpret_cast<uint32_t*>(gate_smem + kCandBatch * 128 * sizeof(float));

  const int tile = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int chunk = plan.qtile_chunk[tile];
  const int c0 = plan.chunk_seq_first[chunk];
  const int ncand = chunk - c0;
  const int kk = plan.kk;
  const int tok = plan.qtile_start[tile] + tid;
  const bool valid = tok < plan.chunk_start[chunk + 1];
  const int64_t slot0 = (static_cast<int64_t>(tok) * H + h) * kk;

  if (ncand == 0) {
    if (valid)
      for (int j = 0; j < kk; ++j) {
        sel[slot0 + j] = -1;
        if (sel_score) sel_score[slot0 + j] = -INFINITY;
      }
    return;
  }

  float qf[128];
  if (valid) {
    load_row128<T>(q + static_cast<int64_t>(tok) * stride_s + static_cast<int64_t>(h) * stride_h, qf);
  } else {
#pragma unroll
    for (int i = 0; i < 128; ++i) qf[i] = 0.f;
  }

  float best[KMAX];
  int bidx[KMAX];
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    best[j] = -INFINITY;
    bidx[j] = -1;
  }

  for (int i = tid; i < ncand * 4; i += 128) bitmap[i] = 0u;

  // pooled keys are [chunk, H / kv_rep, 128]; query head h reads key head h / kv_rep
  const int64_t km_stride = static_cast<int64_t>(H / kv_rep) * MOBA_HEAD_DIM;
  const int64_t km_head = static_cast<int64_t>(h / kv_rep) * MOBA_HEAD_DIM;
  for (int b0 = 0; b0 < ncand; b0 += kCandBatch) {
    const int nb = min(kCandBatch, ncand - b0);
    __syncthreads();
    for (int i = tid; i < nb * 32; i += 128) {
      const int ci = i >> 5, d4 = i & 31;
      reinterpret_cast<float4*>(km)[ci * 32 + d4] = __ldg(
          reinterpret_cast<const float4*>(kmean + (c0 + b0 + ci) * km_stride + km_head) + d4);
    }
    __syncthreads();
    for (int ci = 0; ci < nb; ++ci) {
      const float4* kr = reinterpret_cast<const float4*>(km) + ci * 32;
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
      for (int d4 = 0; d4 < 32; ++d4) {
        const float4 kv = kr[d4];
        a0 = fmaf(qf[4 * d4], kv.x, a0);
        a1 = fmaf(qf[4 * d4 + 1], kv.y, a1);
        a2 = fmaf(qf[4 * d4 + 2], kv.z, a2);
        a3 = fmaf(qf[4 * d4 + 3], kv.w, a3);
      }
      const float s = (a0 + a1) + (a2 + a3);
      if (s > best[KMAX - 1]) {
        best[KMAX - 1] = s;
        bidx[KMAX - 1] = b0 + ci;
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

  if (valid) {
    const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
      if (j < kk) {
        const int lc = bidx[j];
        sel[slot0 + j] = lc >= 0 ? c0 + lc : -1;
        if (sel_score) sel_score[slot0 + j] = best[j];
        if (lc >= 0) atomicOr(&bitmap[lc * 4 + warp], 1u << lane);
      }
    }
  }
  __syncthreads();
  const int64_t cnt0 = (static_cast<int64_t>(plan.qtile_cand_off[tile]) * H) + static_cast<int64_t>(h) * ncand;
  for (int c = tid; c < ncand; c += 128)
    tile_cnt[cnt0 + c] = __popc(bitmap[c * 4]) + __popc(bitmap[c * 4 + 1]) + __popc(bitmap[c * 4 + 2]) +
                         __popc(bitmap[c * 4 + 3]);
}

// One warp per expert (chunk, head): walk the query tiles of the later chunks of the same sequence in token
// order and turn the per-tile counts into exclusive prefixes; the total is the expert's list length.
__global__ void __launch_bounds__(256)
expert_scan_kernel(int H, PlanDev plan, int32_t* __restrict__ tile_cnt, int32_t* __restrict__ expert_len) {
  const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (e >= plan.n_chunks * H) return;
  const int c = e / H, h = e - c * H;
  const int c0 = plan.chunk_seq_first[c], clast = plan.chunk_seq_last[c];
  const int j = c - c0;
  const int tbeg = plan.chunk_qtile_first[c + 1], tend = plan.chunk_qtile_first[clast + 1];
  int running = 0;
  for (int base = tbeg; base < tend; base += 32) {
    const int t = base + lane;
    int v = 0;
    int64_t idx = 0;
    if (t < tend) {
      const int nc = plan.qtile_chunk[t] - c0;
      idx = static_cast<int64_t>(plan.qtile_cand_off[t]) * H + static_cast<int64_t>(h) * nc + j;
      v = tile_cnt[idx];
    }
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    if (t < tend) tile_cnt[idx] = running + incl - v;
    running += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) expert_len[e] = running;
}

// Single CTA: list_off (in: lengths, out: exclusive prefix, E+1 entries) and work_off (prefix of
// ceil(len/128)).
__global__ void __launch_bounds__(1024)
offsets_kernel(int E, int32_t* __restrict__ list_off, int32_t* __restrict__ work_off) {
  __shared__ int s_len[1024];
  __shared__ int s_til[1024];
  const int tid = threadIdx.x;
  const int per = (E + 1023) / 1024;
  const int b = tid * per, e_end = min(b + per, E);
  int sl = 0, stl = 0;
  for (int i = b; i < e_end; ++i) {
    const int l = list_off[i];
    sl += l;
    stl += (l + MOBA_TILE - 1) / MOBA_TILE;
  }
  s_len[tid] = sl;
  s_til[tid] = stl;
  __syncthreads();
  // Hillis-Steele inclusive scan over 1024 partials
  for (int o = 1; o < 1024; o <<= 1) {
    int a = 0, c = 0;
    if (tid >= o) { a = s_len[tid - o]; c = s_til[tid - o]; }
    __syncthreads();
    s_len[tid] += a;
    s_til[tid] += c;
    __syncthreads();
  }
  int rl = s_len[tid] - sl, rt = s_til[tid] - stl;
  for (int i = b; i < e_end; ++i) {
    const int l = list_off[i];
    list_off[i] = rl;
    work_off[i] = rt;
    rl += l;
    rt += (l + MOBA_TILE - 1) / MOBA_TILE;
  }
  if (tid == 1023) {
    list_off[E] = s_len[1023];
    work_off[E] = s_til[1023];
  }
}

// dynamic shared memory: uint32_t bitmap[ncand][4]
__global__ void __launch_bounds__(128)
fill_lists_kernel(int H, PlanDev plan, const int32_t* __restrict__ sel, const int32_t* __restrict__ tile_cnt,
                  const int32_t* __restrict__ list_off, int32_t* __restrict__ list_tok,
                  int32_t* __restrict__ row_of, int* status, int n_rows_total) {
  extern __shared__ __align__(16) uint8_t fill_smem[];
  uint32_t* bitmap = reinterpret_cast<uint32_t*>(fill_smem);
  const int tile = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int chunk = plan.qtile_chunk[tile];
  const int c0 = plan.chunk_seq_first[chunk];
  const int ncand = chunk - c0;
  const int kk = plan.kk;
  const int tok = plan.qtile_start[tile] + tid;
  const bool valid = tok < plan.chunk_start[chunk + 1];
  const int64_t slot0 = (static_cast<int64_t>(tok) * H + h) * kk;
  if (ncand == 0) {
    if (valid)
      for (int j = 0; j < kk; ++j) row_of[slot0 + j] = -1;
    return;
  }
  for (int i = tid; i < ncand * 4; i += 128) bitmap[i] = 0u;
  __syncthreads();
  // a chunk id outside the candidates of this tile (a caller's buffer that the gate did not write) is treated
  // as an empty slot and reported through the status word; it must not index the bitmap or the lists
  if (valid)
    for (int j = 0; j < kk; ++j) {
      const int g = sel[slot0 + j];
      if (g >= c0 && g < chunk) atomicOr(&bitmap[(g - c0) * 4 + warp], 1u << lane);
      else if (g >= 0 && status) atomicCAS(status, 0, 2);
    }
  __syncthreads();
  if (!valid) return;
  const int64_t cnt0 = (static_cast<int64_t>(plan.qtile_cand_off[tile]) * H) + static_cast<int64_t>(h) * ncand;
  const uint32_t lt = (1u << lane) - 1u;
  for (int j = 0; j < kk; ++j) {
    const int g = sel[slot0 + j];
    int r = -1;
    if (g >= c0 && g < chunk) {
      const int lc = g - c0;
      int rank = __popc(bitmap[lc * 4 + warp] & lt);
      for (int w = 0; w < warp; ++w) rank += __popc(bitmap[lc * 4 + w]);
      r = list_off[g * H + h] + tile_cnt[cnt0 + lc] + rank;
      // counts that do not belong to this selection (a gate launch that was cut short) must not become an address
      if (r < 0 || r >= n_rows_total) {
        if (status) atomicCAS(status, 0, 2);
        r = -1;
      } else {
        list_tok[r] = tok;
      }
    }
    row_of[slot0 + j] = r;
  }
}

template <typename T>
int launch_gate(const void* q, int32_t H, int64_t stride_s, int64_t stride_h, const float* kmean, int kv_rep,
                const PlanDev& plan, int32_t max_cand, int32_t* sel, float* sel_score, int32_t* tile_cnt,
                cudaStream_t st) {
  const size_t smem = kCandBatch * 128 * sizeof(float) + static_cast<size_t>(max_cand > 0 ? max_cand : 1) * 16;
  dim3 grid(plan.n_qtiles, H);
  auto run = [&](auto kern) -> int {
    MOBA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, 128, smem, st>>>(static_cast<const T*>(q), H, stride_s, stride_h, kmean, kv_rep, plan, sel, sel_score,
                                  tile_cnt);
    MOBA_CUDA_OK(cudaGetLastError());
    return 0;
  };
  if (plan.kk <= 4) return run(gate_topk_kernel<T, 4>);
  if (plan.kk <= 8) return run(gate_topk_kernel<T, 8>);
  if (plan.kk <= 16) return run(gate_topk_kernel<T, 16>);
  return run(gate_topk_kernel<T, 32>);
}

}  // namespace
}  // namespace moba

extern "C" int moba_gate_topk(const void* q, int32_t dtype, int32_t H, int64_t stride_s, int64_t stride_h,
                              const float* kmean, int32_t kv_heads, const moba_plan_info* info,
                              const int32_t* meta_dev, int32_t* sel, float* sel_score, int32_t* tile_cnt,
                              int32_t* status, int32_t device, void* stream) {
  using namespace moba;
  int rc = check_common(q, H, stride_s, stride_h, info, meta_dev);
  if (rc) return rc;
  if (kv_heads == 0) kv_heads = H;
  MOBA_REQUIRE(kv_heads > 0 && H % kv_heads == 0, MOBA_ERR_ARG, "kv_heads=%d must divide H=%d", kv_heads, H);
  const int kv_rep = H / kv_heads;
  MOBA_REQUIRE(kmean && sel && tile_cnt, MOBA_ERR_ARG, "null pointer argument");
  MOBA_REQUIRE(info->kk >= 1, MOBA_ERR_ARG, "no selection slots (kk=0): the gate is not needed");
  MOBA_REQUIRE(info->kk <= 32, MOBA_ERR_LIMIT, "moba_topk-1=%d exceeds the supported 32", info->kk);
  MOBA_REQUIRE(info->max_cand <= 11000, MOBA_ERR_LIMIT,
               "a sequence has %d chunks; at most 11001 are supported", info->max_cand + 1);
  MOBA_REQUIRE(info->cand_per_head * H < (1ll << 31), MOBA_ERR_LIMIT, "candidate table exceeds 2^31 entries");
  MOBA_SET_DEVICE(device);
  if (info->n_qtiles == 0) return 0;
  const PlanDev plan = make_plan_dev(info, meta_dev);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // 16-bit q: scores on the tensor pipe (exact products, fp32 accumulation). It needs the status word for its
  // bounded waits; without one, for fp32 q, and for sequences of more than 4097 chunks the FMA kernel runs.
  if (status && (dtype == MOBA_DTYPE_BF16 || dtype == MOBA_DTYPE_F16) && info->max_cand <= 4096)
    return launch_gate_umma(q, dtype, H, stride_s, stride_h, kmean, kv_rep, info, plan, sel, sel_score, tile_cnt, status, st);
  switch (dtype) {
    case MOBA_DTYPE_BF16:
      return launch_gate<__nv_bfloat16>(q, H, stride_s, stride_h, kmean, kv_rep, plan, info->max_cand, sel, sel_score, tile_cnt, st);
    case MOBA_DTYPE_F16:
      return launch_gate<__half>(q, H, stride_s, stride_h, kmean, kv_rep, plan, info->max_cand, sel, sel_score, tile_cnt, st);
    case MOBA_DTYPE_F32:
      return launch_gate<float>(q, H, stride_s, stride_h, kmean, kv_rep, plan, info->max_cand, sel, sel_score, tile_cnt, st);
    default: return set_error(MOBA_ERR_ARG, "unsupported dtype %d", dtype);
  }
}

namespace moba {
namespace {
// One record per work tile: the list that owns it (last e with work_off[e] <= w), the tile's first row and row count,
// the key range of the list's chunk. Tiles past the last one get zero rows.
__global__ void __launch_bounds__(256)
tile_records_kernel(int H, PlanDev plan, int n_experts, int n_tiles, const int32_t* __restrict__ list_off,
                    const int32_t* __restrict__ work_off, int32_t* __restrict__ tile_rec) {
  const int w = blockIdx.x * blockDim.x + threadIdx.x;
  if (w >= n_tiles) return;
  int4 lo4 = make_int4(0, 0, 0, 0), hi4 = make_int4(0, 0, 0, 0);
  if (w < work_off[n_experts]) {
    int lo = 0, hi = n_experts;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (work_off[mid] <= w) lo = mid; else hi = mid;
    }
    const int chunk = lo / H;
    const int first = list_off[lo] + (w - work_off[lo]) * MOBA_TILE;
    const int key0 = plan.chunk_start[chunk];
    lo4 = make_int4(lo - chunk * H, first, min(MOBA_TILE, list_off[lo + 1] - first), key0);
    hi4 = make_int4(plan.chunk_start[chunk + 1] - key0, 0, 0, 0);
  }
  reinterpret_cast<int4*>(tile_rec)[2 * w] = lo4;
  reinterpret_cast<int4*>(tile_rec)[2 * w + 1] = hi4;
}
}  // namespace
}  // namespace moba

extern "C" int moba_tile_records(int32_t H, const moba_plan_info* info, const int32_t* meta_dev,
                                 const int32_t* list_off, const int32_t* work_off, int32_t* tile_rec, int32_t device,
                                 void* stream) {
  using namespace moba;
  MOBA_REQUIRE(info && meta_dev && list_off && work_off && tile_rec, MOBA_ERR_ARG, "null pointer argument");
  MOBA_REQUIRE(H >= 1 && H <= 65535, MOBA_ERR_ARG, "H=%d out of range", H);
  const int64_t nw = info->max_work_tiles_per_head * H;
  MOBA_REQUIRE(nw < (1ll << 28), MOBA_ERR_LIMIT, "too many gathered tiles");
  MOBA_SET_DEVICE(device);
  if (info->kk == 0 || nw == 0) return 0;
  const PlanDev plan = make_plan_dev(info, meta_dev);
  tile_records_kernel<<<static_cast<unsigned>((nw + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      H, plan, info->n_chunks * H, static_cast<int>(nw), list_off, work_off, tile_rec);
  MOBA_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" int moba_build_lists(int32_t H, const moba_plan_info* info, const int32_t* meta_dev,
                                const int32_t* sel, int32_t* tile_cnt, int32_t* list_off, int32_t* work_off,
                                int32_t* list_tok, int32_t* row_of, int32_t* status, int32_t device,
                                void* stream) {
  using namespace moba;
  MOBA_REQUIRE(info && meta_dev && sel && tile_cnt && list_off && work_off && list_tok && row_of, MOBA_ERR_ARG,
               "null pointer argument");
  MOBA_REQUIRE(H >= 1 && H <= 65535, MOBA_ERR_ARG, "H=%d out of range", H);
  MOBA_REQUIRE(info->kk >= 1, MOBA_ERR_ARG, "no selection slots (kk=0)");
  MOBA_REQUIRE(info->rows_per_head * H < (1ll << 31), MOBA_ERR_LIMIT, "row space exceeds 2^31");
  MOBA_REQUIRE(static_cast<int64_t>(info->n_chunks) * H < (1ll << 30), MOBA_ERR_LIMIT, "too many experts");
  MOBA_SET_DEVICE(device);
  if (info->n_qtiles == 0) return 0;
  const PlanDev plan = make_plan_dev(info, meta_dev);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int E = info->n_chunks * H;
  expert_scan_kernel<<<(E + 7) / 8, 256, 0, st>>>(H, plan, tile_cnt, list_off);
  MOBA_CUDA_OK(cudaGetLastError());
  offsets_kernel<<<1, 1024, 0, st>>>(E, list_off, work_off);
  MOBA_CUDA_OK(cudaGetLastError());
  const size_t smem = static_cast<size_t>(info->max_cand > 0 ? info->max_cand : 1) * 16;
  MOBA_CUDA_OK(cudaFuncSetAttribute(fill_lists_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(plan.n_qtiles, H);
  fill_lists_kernel<<<grid, 128, smem, st>>>(H, plan, sel, tile_cnt, list_off, list_tok, row_of, status,
                                             static_cast<int>(info->rows_per_head * H));
  MOBA_CUDA_OK(cudaGetLastError());
  return 0;
}
