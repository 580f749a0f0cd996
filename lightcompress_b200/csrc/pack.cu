// Export layouts for 4-bit codes.
//
//   lc_pack_int4_awq   AutoAWQ GEMM layout: codes (out x in, one byte each) -> qweight (in x out/8)
//                      int32, eight consecutive OUT columns per word in nibble order 0,2,4,6,1,3,5,7.
//                      The same routine packs the zero points ((out x n_groups) -> (n_groups x out/8)).
// The compressed-tensors "pack-quantized" layout (eight consecutive IN columns per int32, first
// one in the lowest nibble, stored as q + 8) is LC_CODES_PACK4 of lc_rtn_int_quant viewed as int32.
#include "lc_common.cuh"

namespace lc {
namespace {

__global__ void __launch_bounds__(256) pack_awq_kernel(const uint8_t* codes, int64_t rows, int64_t cols, int32_t* out) {
  // thread -> (k = input column, c = block of eight output rows); k fastest so that the eight
  // byte reads of a warp are contiguous along the input dimension
  const int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t c = blockIdx.y;
  if (k >= cols) return;
  const int order[8] = {0, 2, 4, 6, 1, 3, 5, 7};
  uint32_t w = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) w |= (uint32_t)(codes[(c * 8 + order[i]) * cols + k] & 0xf) << (4 * i);
  out[k * (rows / 8) + c] = (int32_t)w;
}

}  // namespace
}  // namespace lc

extern "C" LC_API int lc_pack_int4_awq(const uint8_t* codes, int64_t rows, int64_t cols, int32_t* out,
                                       lc_stream_t stream) {
  if (!codes || !out || rows <= 0 || cols <= 0) return LC_ERR_ARG;
  if (rows % 8 != 0) return LC_ERR_SHAPE;
  if (rows / 8 > 65535) return LC_ERR_SHAPE;
  dim3 grid((unsigned)((cols + 255) / 256), (unsigned)(rows / 8));
  lc::pack_awq_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(codes, rows, cols, out);
  LC_LAUNCH_CHECK();
  return LC_OK;
}
