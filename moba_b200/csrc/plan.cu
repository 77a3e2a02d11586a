// Host side of the library: error strings, the chunk plan (integer tables derived from cu_seqlens) and
// tensor-map creation. The plan restates calc_chunks (MoonshotAI/MoBA moba/moba_efficient.py:14-64):
// chunks are aligned per sequence, the last chunk of a sequence may be short, and a chunk is a candidate
// only for queries of later chunks of the same sequence.
#include "common.cuh"

#include <mutex>
#include <vector>
#include <string.h>

namespace moba {

char* last_error_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct PlanTables {
  std::vector<int32_t> chunk_start, chunk_seq_first, chunk_seq_last, qtile_chunk, qtile_start, qtile_cand_off,
      chunk_qtile_first;
};

int build_plan(const int32_t* cu, int32_t batch, int32_t B, int32_t topk, moba_plan_info* info,
               PlanTables* tab) {
  MOBA_REQUIRE(cu && info, MOBA_ERR_ARG, "null pointer argument");
  MOBA_REQUIRE(batch >= 1, MOBA_ERR_ARG, "batch=%d must be >= 1", batch);
  MOBA_REQUIRE(B >= 1, MOBA_ERR_ARG, "moba_chunk_size=%d must be >= 1", B);
  MOBA_REQUIRE(topk >= 1, MOBA_ERR_ARG, "moba_topk=%d must be >= 1", topk);
  MOBA_REQUIRE(cu[0] == 0, MOBA_ERR_SEQLENS, "cu_seqlens[0]=%d must be 0", cu[0]);
  for (int b = 0; b < batch; ++b)
    MOBA_REQUIRE(cu[b + 1] >= cu[b], MOBA_ERR_SEQLENS, "cu_seqlens decreases at index %d", b + 1);

  memset(info, 0, sizeof(*info));
  info->batch = batch;
  info->chunk_size = B;
  info->topk = topk;
  info->total_tokens = cu[batch];

  int64_t n_chunks = 0, n_qtiles = 0, cand = 0, rows = 0, work = 0;
  int32_t max_seq_chunks = 0, n_filtered = 0;
  for (int b = 0; b < batch; ++b) {
    const int64_t len = cu[b + 1] - cu[b];
    const int64_t nb = (len + B - 1) / B;
    if (nb > max_seq_chunks) max_seq_chunks = static_cast<int32_t>(nb);
    if (nb > 0) n_filtered += static_cast<int32_t>(nb - 1);
    n_chunks += nb;
  }
  const int32_t kk_raw = topk - 1;
  const int32_t max_cand = max_seq_chunks > 0 ? max_seq_chunks - 1 : 0;
  const int32_t kk = kk_raw < max_cand ? kk_raw : max_cand;
  MOBA_REQUIRE(n_chunks < (1 << 24), MOBA_ERR_LIMIT, "too many chunks (%lld)", (long long)n_chunks);

  if (tab) {
    tab->chunk_start.reserve(n_chunks + 1);
  }
  int32_t c_global = 0;
  for (int b = 0; b < batch; ++b) {
    const int64_t t0 = cu[b], len = cu[b + 1] - cu[b];
    const int32_t nb = static_cast<int32_t>((len + B - 1) / B);
    const int32_t first = c_global;
    for (int32_t c = 0; c < nb; ++c) {
      const int64_t cs = (c + 1 < nb) ? B : (len - static_cast<int64_t>(c) * B);
      const int64_t tiles = (cs + MOBA_TILE - 1) / MOBA_TILE;
      const int32_t picks = c < kk ? c : kk;
      rows += cs * picks;
      // gathered tiles of this chunk's expert: at most floor(len/128)+1, bounded later via rows.
      if (tab) {
        tab->chunk_start.push_back(static_cast<int32_t>(t0 + static_cast<int64_t>(c) * B));
        tab->chunk_seq_first.push_back(first);
        tab->chunk_seq_last.push_back(first + nb - 1);
        tab->chunk_qtile_first.push_back(static_cast<int32_t>(n_qtiles));
        for (int64_t t = 0; t < tiles; ++t) {
          tab->qtile_chunk.push_back(c_global);
          tab->qtile_start.push_back(static_cast<int32_t>(t0 + static_cast<int64_t>(c) * B + t * MOBA_TILE));
          tab->qtile_cand_off.push_back(static_cast<int32_t>(cand + t * c));
        }
      }
      n_qtiles += tiles;
      cand += tiles * c;
      ++c_global;
    }
  }
  if (tab) {
    tab->chunk_start.push_back(cu[batch]);
    tab->chunk_qtile_first.push_back(static_cast<int32_t>(n_qtiles));
    tab->qtile_cand_off.push_back(static_cast<int32_t>(cand));
  }
  work = rows / MOBA_TILE + n_filtered;
  MOBA_REQUIRE(cand < (1ll << 31), MOBA_ERR_LIMIT, "candidate table too large (%lld entries per head)",
               (long long)cand);
  MOBA_REQUIRE(n_qtiles < (1ll << 31), MOBA_ERR_LIMIT, "too many query tiles");

  info->kk = kk;
  info->n_chunks = static_cast<int32_t>(n_chunks);
  info->n_filtered = n_filtered;
  info->n_qtiles = static_cast<int32_t>(n_qtiles);
  info->max_cand = max_cand;
  info->max_seq_chunks = max_seq_chunks;
  info->rows_per_head = kk > 0 ? rows : 0;
  info->cand_per_head = cand;
  info->max_work_tiles_per_head = kk > 0 ? work : 0;
  int32_t off = 0;
  info->off_chunk_start = off;        off += info->n_chunks + 1;
  info->off_chunk_seq_first = off;    off += info->n_chunks;
  info->off_chunk_seq_last = off;     off += info->n_chunks;
  info->off_qtile_chunk = off;        off += info->n_qtiles;
  info->off_qtile_start = off;        off += info->n_qtiles;
  info->off_qtile_cand_off = off;     off += info->n_qtiles + 1;
  info->off_chunk_qtile_first = off;  off += info->n_chunks + 1;
  info->meta_ints = off;
  return 0;
}

}  // namespace

int make_tensor_map_shd(CUtensorMap* map, const void* base, int32_t dtype, int64_t S, int32_t H,
                        int64_t stride_s, int64_t stride_h, int32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  MOBA_REQUIRE(fn != nullptr, MOBA_ERR_DRIVER, "cuTensorMapEncodeTiled entry point not available");
  MOBA_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, MOBA_ERR_ARG, "tensor base not 16-byte aligned");
  MOBA_REQUIRE(dtype == MOBA_DTYPE_BF16 || dtype == MOBA_DTYPE_F16, MOBA_ERR_ARG,
               "tensor maps are built for 16-bit tensors only");
  cuuint64_t dims[3] = {MOBA_HEAD_DIM, static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(S)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(stride_h) * 2, static_cast<cuuint64_t>(stride_s) * 2};
  cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dtype == MOBA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MOBA_REQUIRE(r == CUDA_SUCCESS, MOBA_ERR_DRIVER, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

int make_tensor_map_rows(CUtensorMap* map, const void* base, int32_t dtype, int64_t n_rows, int64_t row_stride) {
  EncodeTiledFn fn = get_encode_fn();
  MOBA_REQUIRE(fn != nullptr, MOBA_ERR_DRIVER, "cuTensorMapEncodeTiled entry point not available");
  MOBA_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, MOBA_ERR_ARG, "tensor base not 16-byte aligned");
  MOBA_REQUIRE(dtype == MOBA_DTYPE_BF16 || dtype == MOBA_DTYPE_F16, MOBA_ERR_ARG,
               "tensor maps are built for 16-bit tensors only");
  cuuint64_t dims[2] = {MOBA_HEAD_DIM, static_cast<cuuint64_t>(n_rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_stride) * 2};
  cuuint32_t box[2] = {64, 1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dtype == MOBA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  MOBA_REQUIRE(r == CUDA_SUCCESS, MOBA_ERR_DRIVER, "cuTensorMapEncodeTiled (row map) failed with CUresult %d", (int)r);
  return 0;
}

}  // namespace moba

extern "C" {

int moba_version(void) { return 100; }

const char* moba_last_error_string(void) { return moba::last_error_buf(); }

int moba_plan_sizes(const int32_t* cu_seqlens_host, int32_t batch, int32_t chunk_size, int32_t topk,
                    moba_plan_info* info) {
  return moba::build_plan(cu_seqlens_host, batch, chunk_size, topk, info, nullptr);
}

int moba_plan_fill(const int32_t* cu_seqlens_host, int32_t batch, int32_t chunk_size, int32_t topk,
                   const moba_plan_info* info, int32_t* meta_host) {
  MOBA_REQUIRE(info && meta_host, MOBA_ERR_ARG, "null pointer argument");
  moba_plan_info chk;
  moba::PlanTables tab;
  int rc = moba::build_plan(cu_seqlens_host, batch, chunk_size, topk, &chk, &tab);
  if (rc) return rc;
  MOBA_REQUIRE(chk.meta_ints == info->meta_ints && chk.n_chunks == info->n_chunks &&
                   chk.n_qtiles == info->n_qtiles,
               MOBA_ERR_ARG, "plan info does not match the arguments");
  auto put = [&](int32_t off, const std::vector<int32_t>& v) {
    if (!v.empty()) memcpy(meta_host + off, v.data(), v.size() * sizeof(int32_t));
  };
  put(info->off_chunk_start, tab.chunk_start);
  put(info->off_chunk_seq_first, tab.chunk_seq_first);
  put(info->off_chunk_seq_last, tab.chunk_seq_last);
  put(info->off_qtile_chunk, tab.qtile_chunk);
  put(info->off_qtile_start, tab.qtile_start);
  put(info->off_qtile_cand_off, tab.qtile_cand_off);
  put(info->off_chunk_qtile_first, tab.chunk_qtile_first);
  return 0;
}

int moba_check_status(const int32_t* status_dev, int32_t device, void* stream) {
  MOBA_REQUIRE(status_dev, MOBA_ERR_ARG, "null pointer argument");
  MOBA_SET_DEVICE(device);
  int32_t h = 0;
  MOBA_CUDA_OK(cudaMemcpyAsync(&h, status_dev, sizeof(h), cudaMemcpyDeviceToHost,
                               static_cast<cudaStream_t>(stream)));
  MOBA_CUDA_OK(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  MOBA_REQUIRE(h == 0, MOBA_ERR_DEVICE, "kernel status word = %d (1 = bounded wait expired, 2 = bad index)", h);
  return 0;
}

}  // extern "C"
