// Host-side tensor-map encoding.  The library links the static CUDA runtime only, so the
// driver's cuTensorMapEncodeTiled is looked up at run time through the runtime's
// driver-entry-point query.
#include <cudaTypedefs.h>

#include "d2d_tmap.cuh"

namespace d2d {
namespace {

PFN_cuTensorMapEncodeTiled_v12000 lookup_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
  if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault,
                                       &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
}

}  // namespace

int encode_tmap_2d_b16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer,
                       uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer,
                       bool swizzle128) {
  static const PFN_cuTensorMapEncodeTiled_v12000 encode = lookup_encode();   // thread-safe init
  if (!encode) return D2D_ERR_NO_DEVICE;
  if (!base || (reinterpret_cast<uintptr_t>(base) & 15) || (pitch_bytes & 15) || inner == 0 ||
      outer == 0 || box_inner == 0 || box_inner > 256 || box_outer == 0 || box_outer > 256 ||
      ((box_inner * 2) & 15) || (swizzle128 && box_inner * 2 > 128))
    return D2D_ERR_BAD_ARG;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult rc =
      encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
             estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? D2D_OK : D2D_ERR_BAD_ARG;
}

}  // namespace d2d
