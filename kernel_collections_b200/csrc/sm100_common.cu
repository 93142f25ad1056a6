// Host-side pieces shared by the sm_100a kernels: the tensor-map encoder and the status clear.
#include "sm100_common.cuh"

namespace xkv {
namespace sm100 {

__global__ void clear_status_kernel(int* status) {
  if (threadIdx.x < 64) status[threadIdx.x] = 0;
}

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (tried) return fn;
  tried = true;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess)
    fn = reinterpret_cast<EncodeTiledFn>(p);
  else
    cudaGetLastError();
  return fn;
}

bool encode_tiled_16bit(CUtensorMap* m, int dtype, int rank, const void* ptr, const cuuint64_t* dims,
                        const cuuint64_t* strides, const cuuint32_t* box) {
  EncodeTiledFn fn = get_encode();
  if (!fn) return false;
  cuuint32_t es[5] = {1, 1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == XKV_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return fn(m, dt, (cuuint32_t)rank, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace sm100
}  // namespace xkv
