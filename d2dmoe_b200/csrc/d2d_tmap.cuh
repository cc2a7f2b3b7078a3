// Tensor-map (TMA descriptor) helpers: host-side encoding through the driver entry point
// and the device-side load instructions that take a tensor map.
#pragma once
#include <cuda.h>

#include "d2d_common.cuh"

namespace d2d {

// 2-D row-major tensor [outer, inner] of 2-byte elements starting at `base` (16-byte
// aligned; row pitch a multiple of 16 bytes), traversed in boxes of box_outer rows x
// box_inner elements; with swizzle128 the 16-byte pieces of every 128-byte box row land
// XOR-swizzled by the row's position inside its 8-row group, which is the K-major
// 128-byte-swizzled tile layout the MMA descriptors describe.  Returns D2D_OK,
// D2D_ERR_NO_DEVICE (no driver entry point) or D2D_ERR_BAD_ARG (the driver refused).
int encode_tmap_2d_b16(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer,
                       uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer,
                       bool swizzle128);

#ifdef __CUDACC__
namespace umma {
// rows r0..r3 (any four rows of the tensor), box_inner elements from column c0 each, to four
// consecutive 128-byte rows at dst; completes 4 * box_inner * 2 bytes on the barrier
__device__ __forceinline__ void tma_gather4(uint32_t dst, const CUtensorMap* map, int c0, int r0,
                                            int r1, int r2, int r3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(bar)
      : "memory");
}
// one box at (column c0, row r0); rows past the tensor's end arrive as zeros
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int r0,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(r0), "r"(bar)
      : "memory");
}
}  // namespace umma
#endif

}  // namespace d2d
