// Strided host <-> device copies for the host entry point: one head group of a [tokens, heads, 128] tensor is a
// pitched 2-D region (row = the group's heads of one token). cudaMemcpy2DAsync moves it with the copy engines
// straight from / to pinned memory; a framework-level strided copy would first pack it on the CPU.
#include "common.cuh"

extern "C" int moba_memcpy_2d(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int64_t width_bytes,
                              int64_t rows, int32_t to_device, int32_t device, void* stream) {
  using namespace moba;
  MOBA_REQUIRE(dst && src, MOBA_ERR_ARG, "null pointer argument");
  MOBA_REQUIRE(width_bytes > 0 && rows >= 0 && dst_pitch >= width_bytes && src_pitch >= width_bytes, MOBA_ERR_ARG,
               "bad 2-D copy geometry (width %lld, rows %lld, pitches %lld / %lld)", (long long)width_bytes,
               (long long)rows, (long long)dst_pitch, (long long)src_pitch);
  if (rows == 0) return 0;
  MOBA_SET_DEVICE(device);
  MOBA_CUDA_OK(cudaMemcpy2DAsync(dst, static_cast<size_t>(dst_pitch), src, static_cast<size_t>(src_pitch),
                                 static_cast<size_t>(width_bytes), static_cast<size_t>(rows),
                                 to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost,
                                 static_cast<cudaStream_t>(stream)));
  return 0;
}
