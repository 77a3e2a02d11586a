// One 128x128x128 tile product through the same TMA / descriptor / tcgen05 helpers the attention kernels
// use. Exists so that the operand-layout conventions (K-major and MN-major shared-memory operands, an A
// operand held in tensor memory, thread-written swizzled tiles) can each be checked against a plain matrix
// product in isolation.
#include "common.cuh"
#include "ptx.cuh"

namespace moba {
namespace {

struct __align__(1024) SelftestSmem {
  uint8_t a[2][16384];   // two [128 x 64] sub-tiles, 128-byte swizzle
  uint8_t b[2][16384];
  uint8_t x[2][4096];    // mode 4: [128 x 16] K-major tiles without swizzle (A part, B part)
  uint64_t bar_load;
  uint64_t bar_mma;
  uint32_t tmem_base;
  int abort_flag;
};

template <bool kBf16>
__global__ void __launch_bounds__(128, 1)
selftest_kernel(int mode, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_rows, const int* __restrict__ row_idx,
                const uint16_t* __restrict__ a_gmem, const uint16_t* __restrict__ b_gmem, float* __restrict__ c,
                int* status) {
  extern __shared__ uint8_t smem_raw[];
  SelftestSmem& sm = *reinterpret_cast<SelftestSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5;
  WaitCtx wctx{&sm.abort_flag, status};

  if (tid == 0) {
    sm.abort_flag = 0;
    mbar_init(&sm.bar_load, 1);
    mbar_init(&sm.bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&sm.tmem_base, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);

  if (tid == 0) {
    // TMA brings A in modes 0, 3, 4, 5 and B in every mode but 5 (threads write it there)
    const uint32_t bytes = ((mode == 0 || mode == 3 || mode == 4) ? 4u : 2u) * 16384u;
    mbar_arrive_expect_tx(&sm.bar_load, bytes);
    if (mode == 3) {
      // A rows fetched by index, four rows per instruction, into the same swizzled K-major tile layout
      for (int r = 0; r < 128; r += 4) {
        const int i0 = row_idx[r], i1 = row_idx[r + 1], i2 = row_idx[r + 2], i3 = row_idx[r + 3];
        tma_gather4_2d(smem_u32(sm.a[0]) + r * 128, &map_rows, &sm.bar_load, 0, i0, i1, i2, i3);
        tma_gather4_2d(smem_u32(sm.a[1]) + r * 128, &map_rows, &sm.bar_load, 64, i0, i1, i2, i3);
      }
    }
    if (mode == 0 || mode == 4 || mode == 5) {
      tma_load_3d(smem_u32(sm.a[0]), &map_a, &sm.bar_load, 0, 0, 0);
      tma_load_3d(smem_u32(sm.a[1]), &map_a, &sm.bar_load, 64, 0, 0);
    }
    if (mode != 5) {
      tma_load_3d(smem_u32(sm.b[0]), &map_b, &sm.bar_load, 0, 0, 0);
      tma_load_3d(smem_u32(sm.b[1]), &map_b, &sm.bar_load, 64, 0, 0);
    }
  }

  if (mode == 1) {
    // thread = row; 128 x 16-bit = 64 packed words into tensor-memory columns [128, 192)
    const uint32_t* row = reinterpret_cast<const uint32_t*>(a_gmem + static_cast<size_t>(tid) * 128);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t r[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) r[j] = row[i * 16 + j];
      tmem_st16(lane_addr + 128 + i * 16, r);
    }
    tmem_wait_st();
  } else if (mode == 4) {
    // thread = row: the first 16 elements of row `tid` of A and of B, as two 16-byte chunks each
    const uint4* ra = reinterpret_cast<const uint4*>(a_gmem + static_cast<size_t>(tid) * 128);
    const uint4* rb = reinterpret_cast<const uint4*>(b_gmem + static_cast<size_t>(tid) * 128);
#pragma unroll
    for (int ch = 0; ch < 2; ++ch) {
      *reinterpret_cast<uint4*>(sm.x[0] + nosw_offset(tid, ch)) = ra[ch];
      *reinterpret_cast<uint4*>(sm.x[1] + nosw_offset(tid, ch)) = rb[ch];
    }
    fence_proxy_async_smem();
  } else if (mode == 5) {
    // thread = row k of B: its first 64 elements as eight 16-byte chunks of one swizzled 128-byte row
    const uint4* rb = reinterpret_cast<const uint4*>(b_gmem + static_cast<size_t>(tid) * 128);
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(sm.b[0] + sw128_offset(tid, ch)) = rb[ch];
    fence_proxy_async_smem();
  } else if (mode == 2) {
    // 16 consecutive threads copy the 16 16-byte chunks of one row; 8 rows per pass
    for (int pass = 0; pass < 16; ++pass) {
      const int row = pass * 8 + (tid >> 4), c16 = tid & 15;
      const uint32_t dst = smem_u32(sm.a[c16 >> 3]) + sw128_offset(row, c16 & 7);
      cp_async16(dst, a_gmem + static_cast<size_t>(row) * 128 + c16 * 8);
    }
    cp_async_wait_all();
    fence_proxy_async_smem();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  if (tid == 0) {
    bool ok = mbar_wait(&sm.bar_load, 0, wctx);
    if (ok) {
      tc_fence_after_sync();
      if (mode == 0 || mode == 3 || mode == 4) {
        constexpr uint32_t idesc = umma_idesc(128, 128, kBf16, false, false);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = (ks >> 2) * 16384u + (ks & 3) * 32u;
          umma_ss(tmem, umma_smem_desc(smem_u32(sm.a[0]) + off, 16, 1024),
                  umma_smem_desc(smem_u32(sm.b[0]) + off, 16, 1024), idesc, ks > 0);
        }
        // mode 4: a ninth k-step from the unswizzled tiles, accumulated into the same result
        if (mode == 4)
          umma_ss(tmem, umma_smem_desc_nosw(smem_u32(sm.x[0]), 128, 256), umma_smem_desc_nosw(smem_u32(sm.x[1]), 128, 256),
                  idesc, 1);
      } else if (mode == 5) {
        // both operands MN-major, N = 64: C[m, n] = sum_k A[k, m] B[k, n]
        constexpr uint32_t idesc = umma_idesc(128, 64, kBf16, true, true);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss(tmem, umma_smem_desc(smem_u32(sm.a[0]) + ks * 2048u, 16384, 1024),
                  umma_smem_desc(smem_u32(sm.b[0]) + ks * 2048u, 16384, 1024), idesc, ks > 0);
      } else if (mode == 1) {
        constexpr uint32_t idesc = umma_idesc(128, 128, kBf16, false, true);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ts(tmem, tmem + 128 + ks * 8, umma_smem_desc(smem_u32(sm.b[0]) + ks * 2048u, 16384, 1024), idesc,
                  ks > 0);
      } else {
        constexpr uint32_t idesc = umma_idesc(128, 128, kBf16, false, true);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t aoff = (ks >> 2) * 16384u + (ks & 3) * 32u;
          umma_ss(tmem, umma_smem_desc(smem_u32(sm.a[0]) + aoff, 16, 1024),
                  umma_smem_desc(smem_u32(sm.b[0]) + ks * 2048u, 16384, 1024), idesc, ks > 0);
        }
      }
      umma_commit(&sm.bar_mma);
    }
  }
  const bool done = mbar_wait(&sm.bar_mma, 0, wctx);
  tc_fence_after_sync();
  if (done) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t r[32];
      tmem_ld32(lane_addr + i * 32, r);
      tmem_wait_ld32(r);
      // mode 5 produces 64 columns; the rest of its rows is reported as zero
#pragma unroll
      for (int j = 0; j < 32; ++j)
        c[static_cast<size_t>(tid) * 128 + i * 32 + j] = (mode == 5 && i >= 2) ? 0.f : __uint_as_float(r[j]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

}  // namespace
}  // namespace moba

extern "C" int moba_selftest_umma(int32_t mode, const void* a, const void* b, float* c, int32_t dtype,
                                  int32_t* status, int32_t device, void* stream) {
  return moba_selftest_umma_gather(mode, a, 128, nullptr, b, c, dtype, status, device, stream);
}

extern "C" int moba_selftest_umma_gather(int32_t mode, const void* a, int32_t a_rows, const int32_t* row_idx,
                                         const void* b, float* c, int32_t dtype, int32_t* status,
                                         int32_t device, void* stream) {
  using namespace moba;
  MOBA_REQUIRE(a && b && c && status, MOBA_ERR_ARG, "null pointer argument");
  MOBA_REQUIRE(mode >= 0 && mode <= 5, MOBA_ERR_ARG, "mode=%d out of range", mode);
  MOBA_REQUIRE(a_rows >= 128 && (mode != 3 || row_idx), MOBA_ERR_ARG, "mode 3 needs row_idx and a_rows >= 128");
  MOBA_REQUIRE(dtype == MOBA_DTYPE_BF16 || dtype == MOBA_DTYPE_F16, MOBA_ERR_ARG, "dtype must be bf16 or f16");
  MOBA_SET_DEVICE(device);
  CUtensorMap ma, mb;
  int rc = make_tensor_map_shd(&ma, a, dtype, 128, 1, 128, 128, 128);
  if (rc) return rc;
  rc = make_tensor_map_shd(&mb, b, dtype, 128, 1, 128, 128, 128);
  if (rc) return rc;
  CUtensorMap mr;
  rc = make_tensor_map_rows(&mr, a, dtype, a_rows, 128);
  if (rc) return rc;
  const size_t smem = sizeof(SelftestSmem) + 1024;
  auto kern = dtype == MOBA_DTYPE_BF16 ? selftest_kernel<true> : selftest_kernel<false>;
  MOBA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(mode, ma, mb, mr, row_idx,
                                                           static_cast<const uint16_t*>(a),
                                                           static_cast<const uint16_t*>(b), c, status);
  MOBA_CUDA_OK(cudaGetLastError());
  return 0;
}

// ---------------------------------------------------------------------------------------------------
// CTA-pair self test: two CTAs of one cluster compute S = Q K^T for 256 query rows x 128 keys with one
// 256-row MMA per k-step (operands in shared memory, each CTA holding its 128 rows of Q and 64 of the 128 keys),
// hand S / 16 back as 16-bit values in tensor memory and compute O = (S / 16) V with the A operand read from tensor
// memory (each CTA holding 64 of V's 128 columns). Checks the operand split between the CTAs, the loads that
// signal the even CTA's barrier from both CTAs, arrivals across the pair and the commit that reaches both.
namespace moba {
namespace {

struct __align__(1024) PairSmem {
  uint8_t q[2][16384];     // own 128 rows: [128 x 64] sub-tiles (d 0..63 | d 64..127), 128-byte swizzle
  uint8_t k[2][8192];      // own 64 keys: [64 x 64] sub-tiles
  uint8_t v[16384];        // 128 keys x own 64 columns
  uint64_t bar_load, bar_s, bar_p, bar_o;
  uint32_t tmem_base;
  int abort_flag;
};

template <bool kBf16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1)
selftest_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, float* __restrict__ s_out,
                     float* __restrict__ o_out, int* status) {
  extern __shared__ uint8_t smem_raw[];
  PairSmem& sm = *reinterpret_cast<PairSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t rank = cluster_ctarank();
  WaitCtx wctx{&sm.abort_flag, status, 200000000ull};

  if (tid == 0) {
    sm.abort_flag = 0;
    mbar_init(&sm.bar_load, 1);
    mbar_init(&sm.bar_s, 1);
    mbar_init(&sm.bar_p, 256);          // every thread of both CTAs
    mbar_init(&sm.bar_o, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc_pair(&sm.tmem_base, 256);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  cluster_sync_all();                    // barriers of both CTAs exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t lane_addr = tmem + (static_cast<uint32_t>(warp * 32) << 16);
  const uint32_t load_bar0 = cluster_map_shared(smem_u32(&sm.bar_load), 0);
  const uint32_t p_bar0 = cluster_map_shared(smem_u32(&sm.bar_p), 0);

  if (tid == 0) {
    if (rank == 0) mbar_arrive_expect_tx(&sm.bar_load, 2u * (32768u + 16384u + 16384u));
    tma_load_3d_pair(smem_u32(sm.q[0]), &map_q, load_bar0, 0, 0, static_cast<int>(rank) * 128);
    tma_load_3d_pair(smem_u32(sm.q[1]), &map_q, load_bar0, 64, 0, static_cast<int>(rank) * 128);
    tma_load_3d_pair(smem_u32(sm.k[0]), &map_k, load_bar0, 0, 0, static_cast<int>(rank) * 64);
    tma_load_3d_pair(smem_u32(sm.k[1]), &map_k, load_bar0, 64, 0, static_cast<int>(rank) * 64);
    tma_load_3d_pair(smem_u32(sm.v), &map_v, load_bar0, static_cast<int>(rank) * 64, 0, 0);
  }
  bool ok = true;
  if (warp == 0 && rank == 0) {
    const uint32_t leader = elect_one();
    ok = __all_sync(0xffffffffu, mbar_wait_cluster(&sm.bar_load, 0, wctx));
    if (ok) {
      tc_fence_after_sync();
      constexpr uint32_t idesc = umma_idesc(256, 128, kBf16, false, false);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t qoff = ((ks >> 2) * 16384u + (ks & 3) * 32u) >> 4;
        const uint32_t koff = ((ks >> 2) * 8192u + (ks & 3) * 32u) >> 4;
        umma_ss_pair_w(leader, tmem, umma_smem_desc(smem_u32(sm.q[0]), 16, 1024) + qoff,
                       umma_smem_desc(smem_u32(sm.k[0]), 16, 1024) + koff, idesc, ks > 0);
      }
      umma_commit_pair_w(leader, &sm.bar_s);
    }
  }
  ok = mbar_wait(&sm.bar_s, 0, wctx);
  tc_fence_after_sync();
  if (ok) {
    const size_t row = static_cast<size_t>(rank) * 128 + tid;
    uint32_t pk[64];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t r[32];
      tmem_ld32(lane_addr + i * 32, r);
      tmem_wait_ld32(r);
#pragma unroll
      for (int j = 0; j < 32; ++j) s_out[row * 128 + i * 32 + j] = __uint_as_float(r[j]);
#pragma unroll
      for (int j = 0; j < 16; ++j)
        pk[i * 16 + j] = pack2<kBf16>(__uint_as_float(r[2 * j]) * 0.0625f, __uint_as_float(r[2 * j + 1]) * 0.0625f);
    }
    // every load of the row is complete (tmem_wait_ld) before the packed values go over its first 64 columns
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t r[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = pk[i * 32 + j];
      tmem_st32(lane_addr + i * 32, r);
    }
    tmem_wait_st();
    tc_fence_before_sync();
    mbar_arrive_cluster(p_bar0);
  }
  if (warp == 0 && rank == 0) {
    const uint32_t leader = elect_one();
    ok = __all_sync(0xffffffffu, mbar_wait_cluster(&sm.bar_p, 0, wctx));
    if (ok) {
      tc_fence_after_sync();
      constexpr uint32_t idesc = umma_idesc(256, 128, kBf16, false, true);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        umma_ts_pair_w(leader, tmem + 128, tmem + ks * 8, umma_smem_desc(smem_u32(sm.v), 16384, 1024) + ((ks * 2048u) >> 4),
                       idesc, ks > 0);
      umma_commit_pair_w(leader, &sm.bar_o);
    }
  }
  ok = mbar_wait(&sm.bar_o, 0, wctx);
  tc_fence_after_sync();
  if (ok) {
    const size_t row = static_cast<size_t>(rank) * 128 + tid;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t r[32];
      tmem_ld32(lane_addr + 128 + i * 32, r);
      tmem_wait_ld32(r);
#pragma unroll
      for (int j = 0; j < 32; ++j) o_out[row * 128 + i * 32 + j] = __uint_as_float(r[j]);
    }
  }
  tc_fence_before_sync();
  cluster_sync_all();                    // neither CTA leaves while the other may still signal or read it
  if (warp == 0) tmem_dealloc_pair(tmem, 256);
}

}  // namespace
}  // namespace moba

extern "C" int moba_selftest_umma_pair(const void* q, const void* k, const void* v, float* s_out, float* o_out,
                                       int32_t dtype, int32_t* status, int32_t device, void* stream) {
  using namespace moba;
  MOBA_REQUIRE(q && k && v && s_out && o_out && status, MOBA_ERR_ARG, "null pointer argument");
  MOBA_REQUIRE(dtype == MOBA_DTYPE_BF16 || dtype == MOBA_DTYPE_F16, MOBA_ERR_ARG, "dtype must be bf16 or f16");
  MOBA_SET_DEVICE(device);
  CUtensorMap mq, mk, mv;
  int rc = make_tensor_map_shd(&mq, q, dtype, 256, 1, 128, 128, 128);
  if (rc) return rc;
  rc = make_tensor_map_shd(&mk, k, dtype, 128, 1, 128, 128, 64);
  if (rc) return rc;
  rc = make_tensor_map_shd(&mv, v, dtype, 128, 1, 128, 128, 128);
  if (rc) return rc;
  const size_t smem = sizeof(PairSmem) + 1024;
  auto kern = dtype == MOBA_DTYPE_BF16 ? selftest_pair_kernel<true> : selftest_pair_kernel<false>;
  MOBA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<2, 128, smem, static_cast<cudaStream_t>(stream)>>>(mq, mk, mv, s_out, o_out, status);
  MOBA_CUDA_OK(cudaGetLastError());
  return 0;
}

// ---------------------------------------------------------------------------------------------------
// Failure-path self test: a CTA allocates tensor memory and waits on an mbarrier that nothing arrives on, with
// the wait limit given by the caller. The wait must run out, set the status word to 1 (kStatusWaitTimeout),
// and the CTA must still release its tensor memory and return, leaving the context usable.
namespace moba {
namespace {

__global__ void __launch_bounds__(128, 1) wait_timeout_kernel(unsigned long long limit_ns, int* status) {
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base, 32);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  WaitCtx wctx{&abort_flag, status, limit_ns};
  // every thread waits; the first whose limit runs out raises the CTA's abort flag, the others follow it
  mbar_wait(&bar, 0, wctx);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 32);
}

}  // namespace
}  // namespace moba

extern "C" int moba_selftest_wait_timeout(int64_t limit_ns, int32_t n_ctas, int32_t* status, int32_t device,
                                          void* stream) {
  using namespace moba;
  MOBA_REQUIRE(status, MOBA_ERR_ARG, "null pointer argument");
  MOBA_REQUIRE(limit_ns >= 1000 && limit_ns <= 100000000ll, MOBA_ERR_ARG, "limit_ns=%lld outside [1e3, 1e8]",
               (long long)limit_ns);
  MOBA_REQUIRE(n_ctas >= 1 && n_ctas <= 1024, MOBA_ERR_ARG, "n_ctas=%d outside [1, 1024]", n_ctas);
  MOBA_SET_DEVICE(device);
  wait_timeout_kernel<<<n_ctas, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<unsigned long long>(limit_ns), status);
  MOBA_CUDA_OK(cudaGetLastError());
  return 0;
}
