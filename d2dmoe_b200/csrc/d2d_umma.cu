#include "d2d_umma_api.cuh"
namespace d2d {
bool umma_experts_supported(int, int, int, bool, int) { return false; }
size_t umma_experts_packed_bytes(int, int, int, bool) { return 0; }
int launch_prepack_experts(const void*, const void*, const void*, const void*, void*, int, int, int, cudaStream_t) { return D2D_ERR_UNSUPPORTED; }
int launch_experts_umma(const void*, const int32_t*, const int32_t*, const void*, void*, int64_t, int, int, int, bool, int, int*, cudaStream_t) { return D2D_ERR_UNSUPPORTED; }
bool umma_router_supported(int, int, int, int) { return false; }
size_t umma_router_packed_bytes(int, int, int) { return 0; }
int launch_prepack_router(const void*, const void*, void*, int, int, int, cudaStream_t) { return D2D_ERR_UNSUPPORTED; }
int launch_router_mask_umma(const void*, const void*, float, uint32_t*, void*, const void*, int, void*, int64_t, int, int, int, int*, cudaStream_t) { return D2D_ERR_UNSUPPORTED; }
}
