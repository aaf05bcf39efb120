// Host-side TMA descriptor encoding through the driver entry point (no link against libcuda).
#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>

#include "sm100_common.cuh"

namespace vafa {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

}  // namespace

int encode_tmap_rows(CUtensorMap* m, const void* base, int dtype, long long rows, int heads, int dim, int box_rows,
                     int box_heads) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return fail(VAFA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if (dtype != VAFA_BF16 && dtype != VAFA_F16) return fail(VAFA_ERR_UNSUPPORTED, "tensor maps are built for 16-bit types only");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return fail(VAFA_ERR_INVALID, "tensor base must be 16-byte aligned");
  // the row width need not fill the last 64-column box: columns past it read as zero
  if (dim < 8 || dim % 8 != 0 || box_rows < 1 || box_rows > 256 || box_heads < 1 || box_heads > heads || box_heads * box_rows > 256)
    return fail(VAFA_ERR_INVALID, "bad tensor map shape");
  cuuint64_t dims[3] = {(cuuint64_t)dim, (cuuint64_t)heads, (cuuint64_t)(rows > 0 ? rows : 1)};
  cuuint64_t strides[2] = {(cuuint64_t)dim * 2, (cuuint64_t)heads * dim * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_heads, (cuuint32_t)box_rows};
  cuuint32_t es[3] = {1, 1, 1};
  const CUtensorMapDataType dt = dtype == VAFA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = enc(m, dt, 3, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(VAFA_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return 0;
}

int encode_tmap_fold(CUtensorMap* m, const void* base, int dtype, long long rows, int heads) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return fail(VAFA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if (dtype != VAFA_BF16 && dtype != VAFA_F16) return fail(VAFA_ERR_UNSUPPORTED, "tensor maps are built for 16-bit types only");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return fail(VAFA_ERR_INVALID, "tensor base must be 16-byte aligned");
  cuuint64_t dims[3] = {32, (cuuint64_t)heads, (cuuint64_t)(rows > 0 ? rows : 1)};
  cuuint64_t strides[2] = {64, (cuuint64_t)heads * 64};
  cuuint32_t box[3] = {16, 1, 128};
  cuuint32_t es[3] = {1, 1, 1};
  const CUtensorMapDataType dt = dtype == VAFA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = enc(m, dt, 3, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(VAFA_ERR_CUDA, "cuTensorMapEncodeTiled (fold) failed with %d", (int)r);
  return 0;
}

}  // namespace vafa
