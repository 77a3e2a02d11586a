/*
 * moba_b200.h -- C ABI of libmoba_b200.so: the MoBA efficient-attention path as sm_100a kernels.
 *
 * This is test-and-product surface: the Python package `moba_b200` binds exactly these symbols with
 * ctypes, and nothing else crosses the boundary. Plain pointers and sizes only; the caller (torch) owns
 * every buffer. Every device entry point takes the CUDA device ordinal and a stream and is stream-ordered
 * (no host synchronisation inside). Return value: 0 = ok, negative = bad argument (see
 * moba_last_error_string), positive = a cudaError_t.
 *
 * Reference citations are file:line inside the MoonshotAI/MoBA repository.
 *
 * Tensor conventions (as in the reference, moba/moba_efficient.py:281-287): q, k, v, out, d_out, dq, dk,
 * dv are [S, H, D] with D == 128, innermost stride 1, row strides given in elements. Tokens of all
 * sequences are packed along S; cu_seqlens has batch+1 entries, starts at 0 and ends at S.
 */
#ifndef MOBA_B200_H_
#define MOBA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOBA_HEAD_DIM 128
#define MOBA_TILE 128          /* query rows / key rows per tensor-core tile */
#define MOBA_MAX_KV_REP 16    /* most query heads that may share one key/value head (moba_kv_layout) */

/* element types of q/k/v */
enum { MOBA_DTYPE_BF16 = 0, MOBA_DTYPE_F16 = 1, MOBA_DTYPE_F32 = 2 };

/* bad-argument codes */
enum {
  MOBA_OK = 0,
  MOBA_ERR_ARG = -1,       /* null pointer, non-positive size, unsupported dtype/head_dim */
  MOBA_ERR_SEQLENS = -2,   /* cu_seqlens not starting at 0 / not non-decreasing */
  MOBA_ERR_LIMIT = -3,     /* a size exceeds what the kernels index with (see message) */
  MOBA_ERR_DEVICE = -4,    /* a kernel reported a non-zero status word (bounded wait expired, bad index) */
  MOBA_ERR_DRIVER = -5     /* cuTensorMapEncodeTiled not obtainable / failed */
};

/*
 * Chunk plan: everything that depends only on cu_seqlens, the chunk size and top-k.
 * Replaces calc_chunks (moba/moba_efficient.py:14-64) and the size bookkeeping of
 * moba_attn_varlen (moba/moba_efficient.py:306-316, 392-423). Computed on the host from a host copy of
 * cu_seqlens; the integer tables are then uploaded once ("meta" buffer) and shared by all kernels.
 *
 * Offsets off_* index int32 words of the meta buffer:
 *   chunk_start[n_chunks+1]      token offset of every chunk (the reference's cu_chunk)
 *   chunk_seq_first[n_chunks]    global index of the first chunk of the chunk's sequence
 *   chunk_seq_last[n_chunks]     global index of the last chunk of the chunk's sequence
 *   qtile_chunk[n_qtiles]        chunk that a 128-token query tile lies in (tiles never straddle chunks)
 *   qtile_start[n_qtiles]        first token of the tile
 *   qtile_cand_off[n_qtiles+1]   prefix sum over tiles of the tile's candidate-chunk count
 *   chunk_qtile_first[n_chunks+1] index of the first query tile of every chunk
 */
typedef struct moba_plan_info {
  int32_t batch;
  int32_t chunk_size;
  int32_t topk;            /* as passed by the caller */
  int32_t kk;              /* selection slots per query = min(topk-1, max chunks per sequence - 1) */
  int32_t total_tokens;    /* S */
  int32_t n_chunks;        /* n */
  int32_t n_filtered;      /* F = n - batch' (chunks that are not the last of their sequence) */
  int32_t n_qtiles;        /* T */
  int32_t max_cand;        /* largest candidate count of any query = max chunks per sequence - 1 */
  int32_t max_seq_chunks;
  int64_t rows_per_head;   /* R: number of (query, selected chunk) pairs per head; data independent */
  int64_t cand_per_head;   /* qtile_cand_off[T] */
  int64_t max_work_tiles_per_head; /* upper bound on gathered 128-row tiles per head */
  int32_t off_chunk_start, off_chunk_seq_first, off_chunk_seq_last;
  int32_t off_qtile_chunk, off_qtile_start, off_qtile_cand_off, off_chunk_qtile_first;
  int32_t meta_ints;       /* size of the meta buffer in int32 words */
} moba_plan_info;

int moba_version(void);
/* Message for the last non-zero return on the calling thread. */
const char* moba_last_error_string(void);

/* Host only. Fills *info. cu_seqlens_host: batch+1 int32 on the host. */
int moba_plan_sizes(const int32_t* cu_seqlens_host, int32_t batch, int32_t chunk_size, int32_t topk,
                    moba_plan_info* info);
/* Host only. Writes info->meta_ints int32 words into meta_host (same arguments as moba_plan_sizes). */
int moba_plan_fill(const int32_t* cu_seqlens_host, int32_t batch, int32_t chunk_size, int32_t topk,
                   const moba_plan_info* info, int32_t* meta_host);

/*
 * Key mean-pooling: kmean[c, h, :] = round_to_dtype(mean over the tokens of chunk c of k[:, h, :]), stored
 * as fp32. Replaces the stack / index_select / view / mean / float sequence of
 * moba/moba_efficient.py:299, 326-340 (the mean is rounded to the input dtype there too, :335-340).
 * pool_ws: fp32 scratch of moba_pool_ws_floats(info, H) elements.
 */
int64_t moba_pool_ws_floats(const moba_plan_info* info, int32_t H);
int moba_pool_keys(const void* k, int32_t dtype, int32_t H, int64_t stride_s, int64_t stride_h,
                   const moba_plan_info* info, const int32_t* meta_dev, float* pool_ws, float* kmean,
                   int32_t device, void* stream);

/*
 * moba_pool_keys without a workspace argument, for callers that cannot allocate device memory: processes that
 * handed all free device memory to their own arena at start-up, and host bindings without a device allocator.
 * It has no counterpart in the reference. The partial sums go to a 16 MiB array built into the library
 * (moba_pool_keys_static_max_floats() floats; every GPU that loads the library holds it until exit), so
 * n_qtiles * H * 128 must not exceed that many floats, else MOBA_ERR_LIMIT. Calls no cudaMalloc / cudaFree. The
 * first call on a device looks up the array's device address (make that call before any stream capture). All
 * calls on a device share the array: nothing needs clearing between calls, but calls whose kernels overlap on
 * the GPU race on it. Result identical to moba_pool_keys.
 */
int64_t moba_pool_keys_static_max_floats(void);
int moba_pool_keys_static(const void* k, int32_t dtype, int32_t H, int64_t stride_s, int64_t stride_h,
                          const moba_plan_info* info, const int32_t* meta_dev, float* kmean, int32_t device,
                          void* stream);

/*
 * Grouped-query layout of K and V (an extension: the reference expands K / V to the query head count before
 * the call, moba/wrapper.py:59-61). kv_heads divides H; query head h reads key / value head
 * h / (H / kv_heads). Strides in elements. Wherever a `const moba_kv_layout*` is accepted, NULL means
 * kv_heads == H with the strides of q.
 */
typedef struct moba_kv_layout {
  int32_t kv_heads;
  int32_t reserved;
  int64_t stride_s;
  int64_t stride_h;
} moba_kv_layout;

/*
 * Gate: fp32 score q . kmean for every causal candidate chunk of the query's own sequence, top-kk per
 * (token, head). Replaces the einsum, masks and torch.topk of moba/moba_efficient.py:341-371 without the
 * dense [F, H, S] tensors.
 *   sel      [S, H, kk] int32: global chunk ids chosen (in ascending chunk order from the tensor-pipe kernel for
 *            sequences of up to 257 chunks, best first otherwise), then -1 where a query has fewer candidates
 *   sel_score[S, H, kk] fp32 (may be NULL): their scores
 *   tile_cnt [cand_per_head * H] int32: per (query tile, head, candidate) selection counts (input of
 *            moba_build_lists)
 *   status   device status word as for the attention kernels, or NULL. With a status word and bf16 / f16 q the
 *            scores are computed on the tensor pipe (q and the pooled keys are 16-bit values, so every product
 *            is exact and only the order of the fp32 additions differs); otherwise by fp32 FMAs.
 *   kv_heads head count of kmean ([n_chunks, kv_heads, 128]); 0 means H. Query head h is scored against the
 *            pooled keys of head h / (H / kv_heads).
 */
int moba_gate_topk(const void* q, int32_t dtype, int32_t H, int64_t stride_s, int64_t stride_h,
                   const float* kmean, int32_t kv_heads, const moba_plan_info* info, const int32_t* meta_dev,
                   int32_t* sel, float* sel_score, int32_t* tile_cnt, int32_t* status, int32_t device,
                   void* stream);

/*
 * Index lists: for every (chunk, head) "expert" e = chunk*H + head the ascending list of query tokens that
 * selected it. Replaces nonzero / sum / index_select / expert pruning of moba/moba_efficient.py:375-423.
 *   tile_cnt   in: counts from moba_gate_topk; out: exclusive prefix inside each expert (in place)
 *   list_off   [n_chunks*H + 1] int32: start row of every expert's list (row space is [0, R*H))
 *   work_off   [n_chunks*H + 1] int32: prefix sum of ceil(len/128) = first gathered tile of every expert
 *   list_tok   [R*H] int32: token of every row
 *   row_of     [S, H, kk] int32: row that slot j of (token, head) occupies, -1 if the slot is empty
 *   status     device status word or NULL: a chunk id in sel that is not a candidate of its query (only a sel
 *              buffer that moba_gate_topk did not write can hold one) is skipped like an empty slot and sets
 *              the word to 2 (bad index)
 */
int moba_build_lists(int32_t H, const moba_plan_info* info, const int32_t* meta_dev, const int32_t* sel,
                     int32_t* tile_cnt, int32_t* list_off, int32_t* work_off, int32_t* list_tok,
                     int32_t* row_of, int32_t* status, int32_t device, void* stream);

/*
 * One record per 128-row work tile w of the list part (w < max_work_tiles_per_head * H, the grid the list kernels
 * run on): tile_rec[8 w ..] = {head, first list row, rows (0: no such tile), first key token of the chunk, keys in
 * the chunk, 0, 0, 0}, from list_off / work_off of moba_build_lists. Part of the list building (the reference's
 * index_select / split bookkeeping, moba/moba_efficient.py:375-423): the tile kernels that receive the records
 * start from one 32-byte load instead of a search through work_off. tile_rec: [max_work_tiles_per_head * H, 8] int32.
 */
int moba_tile_records(int32_t H, const moba_plan_info* info, const int32_t* meta_dev, const int32_t* list_off,
                      const int32_t* work_off, int32_t* tile_rec, int32_t device, void* stream);

/*
 * Forward attention tiles (tcgen05 / TMEM, TMA-fed K and V, online softmax). Replaces the two
 * _flash_attn_varlen_forward calls of MixedAttention.forward (moba/moba_efficient.py:89-116) and the Q / KV
 * regrouping that feeds them (:381-386, :406-414).
 *  - self part: causal attention inside every chunk -> out [S,H,D] (dtype of q), lse [S,H] fp32 (natural log)
 *  - gathered part: every list row against all keys of its chunk -> part_o [R*H, D] (dtype of q),
 *    part_lse [R*H] fp32
 * q/k/v: bf16 or f16. status: one int32 device word, zeroed by the caller; non-zero after the launch means
 * a bounded wait expired (see MOBA_ERR_DEVICE; read it with moba_check_status).
 * softmax_scale (here and in the two backward tile entry points): the scale of the scores; <= 0 means 128^-0.5
 * (moba/moba_efficient.py:86 uses head_dim^-0.5). Tensors of a head dim below 128 are passed zero-padded to 128
 * columns with their own head_dim^-0.5: the padding changes no product.
 * parts (here and in the two backward tile entry points): 3 = both parts (the normal call), 1 = own-chunk part
 * only, 2 = list part only -- the two halves MixedAttention (moba/moba_efficient.py:67-267) runs as separate
 * flash calls; buffers of a part that is not requested may be NULL.
 * tile_rec (here, in moba_gather_rows and in moba_attn_bwd_dq): the work-tile records of moba_tile_records, or NULL
 * (the kernels then find a tile's list by searching work_off).
 */
int moba_attn_fwd(const void* q, const void* k, const void* v, int32_t dtype, int32_t H, int64_t stride_s,
                  int64_t stride_h, const moba_kv_layout* kv, const moba_plan_info* info, const int32_t* meta_dev,
                  const int32_t* list_off, const int32_t* work_off, const int32_t* list_tok,
                  const int32_t* tile_rec, void* out, float* lse, void* part_o, float* part_lse, int32_t parts,
                  float softmax_scale, int32_t* status, int32_t device, void* stream);

/*
 * Log-sum-exp merge of the self result with the <= kk gathered partial results of every (token, head),
 * in place on out / lse. Replaces moba/moba_efficient.py:118-168 (gather-based, no atomics).
 */
int moba_merge_fwd(void* out, float* lse, int32_t dtype, int32_t H, const moba_plan_info* info,
                   const void* part_o, const float* part_lse, const int32_t* row_of, int32_t device,
                   void* stream);

/* delta[s,h] = sum_d d_out[s,h,d] * out[s,h,d] (fp32): the row term flash backward needs. */
int moba_bwd_delta(const void* out, const void* d_out, int32_t dtype, int32_t H, int64_t n_tokens,
                   float* delta, int32_t device, void* stream);

/*
 * List-ordered copies for the key/value-side backward: qg / dog [R*H, 128] (dtype of q) hold q / d_out of
 * every list row, lse_g / delta_g [R*H] the merged lse and delta of those rows. This is the one place a
 * gathered copy of Q is materialised (the reference builds moba_q the same way, moba/moba_efficient.py:381-386
 * and gathers d_out / lse per row in backward, :231-241); the forward and query-side kernels read rows in place.
 */
int moba_gather_rows(const void* q, const void* d_out, const float* lse, const float* delta, int32_t dtype,
                     int32_t H, int64_t stride_s, int64_t stride_h, const moba_plan_info* info,
                     const int32_t* list_off, const int32_t* work_off, const int32_t* list_tok,
                     const int32_t* tile_rec, void* qg, void* dog, float* lse_g, float* delta_g, int32_t device,
                     void* stream);

/*
 * Backward, key/value side: dk, dv [S, kv_heads, D] (dtype of q; kv_heads == H without a kv layout). One CTA
 * per (chunk, key/value head, 128-key tile) walks, for every query head of the group, the chunk's own causal
 * queries and then the expert's list rows (from qg / dog / lse_g / delta_g, see moba_gather_rows; may be NULL
 * when info->kk == 0), so self and gathered contributions of the whole group are summed in TMEM and written
 * once. Replaces the dk/dv halves of both _flash_attn_varlen_backward calls
 * (moba/moba_efficient.py:208-264) and the autograd scatter through the KV regrouping.
 */
int moba_attn_bwd_dkdv(const void* q, const void* k, const void* v, const void* d_out, int32_t dtype,
                       int32_t H, int64_t stride_s, int64_t stride_h, const moba_kv_layout* kv,
                       const moba_plan_info* info, const int32_t* meta_dev, const int32_t* list_off, const void* qg, const void* dog,
                       const float* lse_g, const float* delta_g, const float* lse, const float* delta, void* dk,
                       void* dv, int32_t parts, float softmax_scale, int32_t* status, int32_t device, void* stream);

/*
 * Backward, query side, unrounded: dq of the self part -> dq_self [S,H,D] fp32; dq of every gathered row ->
 * part_dq [R*H, D] fp32. List tiles read their query-side rows from the list-ordered copies qg / dog / lse_g /
 * delta_g (moba_gather_rows; may be NULL when no list part is requested), own-chunk tiles from q / d_out / lse /
 * delta. Replaces the dq halves of moba/moba_efficient.py:208-264.
 * parts: bit 0 = own-chunk tiles, bit 1 = list tiles. The kernel has two forms with bit-identical results -- one
 * query tile per CTA, and a persistent CTA per SM that walks its share of the tiles -- chosen by chunk size (the
 * persistent form up to 2048 keys); MOBA_DQ_FORM_TILE or MOBA_DQ_FORM_PERSISTENT or'ed into parts names one.
 */
#define MOBA_DQ_FORM_TILE 0x10
#define MOBA_DQ_FORM_PERSISTENT 0x20
int moba_attn_bwd_dq(const void* q, const void* k, const void* v, const void* d_out, int32_t dtype,
                     int32_t H, int64_t stride_s, int64_t stride_h, const moba_kv_layout* kv,
                     const moba_plan_info* info, const int32_t* meta_dev, const int32_t* list_off, const int32_t* work_off,
                     const int32_t* list_tok, const int32_t* tile_rec, const void* qg, const void* dog,
                     const float* lse_g, const float* delta_g, const float* lse, const float* delta, float* dq_self,
                     float* part_dq, int32_t parts, float softmax_scale, int32_t* status, int32_t device,
                     void* stream);

/* dq[s,h,:] = round(dq_self[s,h,:] + sum_j part_dq[row_of[s,h,j], :]) (fp32 sum in slot order, one rounding
 * to `dtype`). Replaces the index_select backward (index_add) autograd runs for moba_q
 * (moba/moba_efficient.py:381-386). With info->kk == 0 it only rounds dq_self. */
int moba_merge_dq(void* dq, int32_t dtype, int32_t H, const moba_plan_info* info, const float* dq_self,
                  const float* part_dq, const int32_t* row_of, int32_t device, void* stream);

/*
 * Dense causal attention for the decode phase: q_len query positions (usually 1) against a key/value cache of
 * kv_len >= q_len positions, the causal mask aligned to the end of the keys (query position i sees keys
 * 0 .. kv_len - q_len + i). Replaces flash_attn_func(query, key, value, dropout, scaling, True) of
 * moba/wrapper.py:76-82 (the reference's decode step is dense; it has no MoBA decode).
 *   q      [batch, q_heads, q_len, 128] 16-bit with element strides (q_stride_b, q_stride_h, q_stride_l)
 *   k, v   [batch, kv_heads, kv_len, 128] 16-bit, strides (kv_heads * kv_stride_h, kv_stride_h, kv_stride_l): the
 *          (batch, head) pairs must be evenly spaced; kv_heads divides q_heads (query head h reads head
 *          h / (q_heads / kv_heads))
 *   scale  softmax scale (128^-0.5 in the reference's models)
 *   out    [batch, q_len, q_heads, 128] contiguous, dtype of q (the layout the reference returns)
 *   ws     moba_decode_ws_floats(...) floats of scratch (partial results of the key ranges)
 *   status zeroed device status word, as for the attention kernels
 * K and V are read once (TMA ring, all query heads of a group share the tiles): the kernel is bound by HBM.
 */
int64_t moba_decode_ws_floats(int32_t batch, int32_t q_heads, int32_t kv_heads, int32_t q_len, int32_t kv_len);
int moba_decode_attn(const void* q, const void* k, const void* v, int32_t dtype, int32_t batch, int32_t q_heads,
                     int32_t kv_heads, int32_t q_len, int32_t kv_len, int64_t q_stride_b, int64_t q_stride_h,
                     int64_t q_stride_l, int64_t kv_stride_h, int64_t kv_stride_l, float scale, void* out, float* ws,
                     int32_t* status, int32_t device, void* stream);

/* Copies the device status word to the host (synchronises the stream) and maps non-zero to
 * MOBA_ERR_DEVICE. */
int moba_check_status(const int32_t* status_dev, int32_t device, void* stream);

/*
 * Pitched host <-> device copy on `stream` (cudaMemcpy2DAsync): rows of width_bytes, dst_pitch / src_pitch bytes
 * apart; to_device != 0 copies host -> device, else device -> host. The host side should be pinned. Used by the
 * host entry point (moba_b200/host_io.py) to move one head group of a [tokens, heads, 128] tensor; the reference
 * has no counterpart (its tensors start on the device).
 */
int moba_memcpy_2d(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int64_t width_bytes,
                   int64_t rows, int32_t to_device, int32_t device, void* stream);

/*
 * Building-block self test (not on any product path): one 128x128x128 tile product through the same TMA,
 * descriptor and tcgen05 helpers the attention kernels use.
 *   mode 0: C = A * B^T   A [128,128] and B [128,128] row-major (both K-major operands in shared memory)
 *   mode 1: C = A * B     A from tensor memory (packed 16-bit pairs), B [128(K),128(N)] row-major (MN-major)
 *   mode 2: C = A * B     A written to shared memory by threads with the 128-byte swizzle, B as in mode 1
 *   mode 4: C = A * B^T + A[:, :16] * B[:, :16]^T   mode 0 plus a ninth k-step from thread-written K-major tiles
 *           without swizzle (the way the dK/dV kernel folds lse / delta into its products)
 *   mode 5: C[:, :64] = A^T * B[:, :64]   both operands MN-major (A [128(K),128(M)] row-major by TMA, B's first 64
 *           columns written by threads with the 128-byte swizzle), N = 64
 * a, b: bf16 (dtype 0) or f16 (dtype 1) device buffers of 128*128 elements; c: 128*128 fp32.
 */
int moba_selftest_umma(int32_t mode, const void* a, const void* b, float* c, int32_t dtype, int32_t* status,
                       int32_t device, void* stream);

/* Same self test with mode 3 added: the 128 rows of A are fetched by index (row_idx[128], device) from a
 * [a_rows, 128] matrix with TMA row gathers; C = A[row_idx] * B^T. Modes 0-2 ignore row_idx. */
int moba_selftest_umma_gather(int32_t mode, const void* a, int32_t a_rows, const int32_t* row_idx,
                              const void* b, float* c, int32_t dtype, int32_t* status, int32_t device,
                              void* stream);

/* CTA-pair self test (no counterpart in the reference): S = Q K^T for q [256,128] and k [128,128], O = (S / 16
 * rounded to 16 bit) V for v [128,128], computed by two CTAs of one cluster with 256-row tcgen05 instructions
 * (cta_group::2): s_out, o_out [256,128] fp32. Used by the tests to pin the operand split between the two CTAs. */
int moba_selftest_umma_pair(const void* q, const void* k, const void* v, float* s_out, float* o_out, int32_t dtype,
                            int32_t* status, int32_t device, void* stream);

/*
 * Failure-path self test (not on any product path): n_ctas CTAs allocate tensor memory and wait on an mbarrier that
 * nothing arrives on, for at most limit_ns nanoseconds (1e3 .. 1e8). The waits run out, the kernel sets *status to
 * 1, releases its tensor memory and returns; moba_check_status then reports MOBA_ERR_DEVICE and the context stays
 * usable. This is how every bounded wait of the product kernels ends when its limit (2 s there) is reached.
 */
int moba_selftest_wait_timeout(int64_t limit_ns, int32_t n_ctas, int32_t* status, int32_t device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOBA_B200_H_ */
