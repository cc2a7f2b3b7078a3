// Host-side interface of the tcgen05 (bf16) kernels, used by d2d_abi.cu.
#pragma once
#include "d2d_common.cuh"

namespace d2d {

bool umma_experts_supported(int d, int E, int H, bool glu, int dtype);
size_t umma_experts_packed_bytes(int d, int E, int H, bool glu);
int launch_prepack_experts(const void* w1, const void* b1, const void* w_up, const void* w2,
                           void* packed, int d, int E, int H, cudaStream_t s);
int launch_experts_umma(const void* x, const int32_t* token_idx, const int32_t* offsets,
                        const void* packed, void* out, int64_t N, int d, int E, int H, bool glu,
                        int act, int* dev_status, cudaStream_t s,
                        NormCapture nc = NormCapture());

bool umma_router_supported(int d, int R, int E, int dtype);
size_t umma_router_packed_bytes(int d, int R, int E);
int launch_prepack_router(const void* wa, const void* wb, void* packed, int d, int R, int E,
                          cudaStream_t s);
int launch_router_mask_umma(const void* x, const void* packed, float mult, uint32_t* mask_bits,
                            void* scores, void* rt_out, const void* last_bias, int add_residual,
                            void* out_init, int32_t* tile_counts, int64_t N, int d, int R, int E,
                            int* dev_status, cudaStream_t s);

// test hook: how the expert kernel gathers its token rows: 0/1 = 16-byte cp.async
// (default), 2 = TMA tile::gather4
void umma_debug_select_experts_kernel(int which);

// test hooks: poll limit of the bounded device waits (2^log2, out of range = default) and
// a flag that makes CTA 0 of the next launches skip its first weight tile
void umma_debug_configure(int wait_limit_log2, int withhold_weight_tile);

}  // namespace d2d
