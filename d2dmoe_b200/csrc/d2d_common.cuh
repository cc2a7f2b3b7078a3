// Shared device helpers for the D2DMoE sm_100a kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/d2dmoe.h"

namespace d2d {

using bf16 = __nv_bfloat16;

// ---- dtype traits --------------------------------------------------------
template <typename T> struct DT;
template <> struct DT<float> {
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
  // value after being materialised as a tensor of this dtype
  static __device__ __forceinline__ float round(float v) { return v; }
};
template <> struct DT<bf16> {
  static __device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ bf16 from_f(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float round(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
  }
};

// four consecutive elements as floats (16-byte load for float, 8-byte for bf16)
__device__ __forceinline__ float4 load4(const float* p) {
  return __ldg(reinterpret_cast<const float4*>(p));
}
__device__ __forceinline__ float4 load4(const bf16* p) {
  const uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}

// ---- programmatic dependent launch ----------------------------------------
// A kernel launched with launch_pdl may start while the previous kernel of the stream is
// still running; it must call grid_dependency_wait() before it touches memory written by
// earlier kernels.  grid_launch_dependents() lets the next such kernel be scheduled early.
// Both are no-ops for kernels launched the ordinary way.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                      cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...) == cudaSuccess) return D2D_OK;
  cudaGetLastError();
  return D2D_ERR_LAUNCH;
}

// ---- device status word ---------------------------------------------------
// First error wins; kernels return early after reporting, they never trap.
__device__ __forceinline__ void report(int* dev_status, int code) {
  if (dev_status) atomicCAS(dev_status, 0, code);
}

// ---- activations ----------------------------------------------------------
// relu, exact-erf gelu, tanh, leaky relu (slope 0.01), tanh-form gelu.
__device__ __forceinline__ float activate(float h, int act) {
  switch (act) {
    case D2D_RELU: return fmaxf(h, 0.0f);
    case D2D_GELU: return h * 0.5f * (1.0f + erff(h * 0.70710678118654752440f));
    case D2D_TANH: return tanhf(h);
    case D2D_LEAKY_RELU: return h >= 0.0f ? h : 0.01f * h;
    case D2D_GELU_TANH: {
      const float k = 0.79788456080286535588f;
      return 0.5f * h * (1.0f + tanhf(k * (h + 0.044715f * h * h * h)));
    }
    default: return h;
  }
}

// ---- vector reductions into global memory ---------------------------------
// fp32: one 16-byte red per 4 values.  bf16: packed pairs, 8 or 16 bytes per red.
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void red_add_v4(bf16* p, float a, float b, float c, float d) {
  uint32_t lo = pack_bf16x2(a, b), hi = pack_bf16x2(c, d);
  asm volatile("red.global.add.noftz.v2.bf16x2 [%0], {%1, %2};" ::"l"(p), "r"(lo), "r"(hi)
               : "memory");
}
__device__ __forceinline__ void red_add_bf16x8(bf16* p, uint32_t a, uint32_t b, uint32_t c,
                                               uint32_t d) {
  asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b),
               "r"(c), "r"(d)
               : "memory");
}
__device__ __forceinline__ void red_add_1(float* p, float a) { atomicAdd(p, a); }
__device__ __forceinline__ void red_add_1(bf16* p, float a) { atomicAdd(p, __float2bfloat16_rn(a)); }

__host__ __device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ __forceinline__ int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace d2d

// ---- internal launch interface (host side, used by d2d_abi.cu) -------------
namespace d2d {

// Optional by-product of the expert kernels: per (expert, token) vector norms over the last
// dimension of what the expert computes for that token, norms[e * N + token] in the tensor
// dtype (the labels router training captures with forward hooks upstream, utils.py:353-369).
struct NormCapture {
  void* norms = nullptr;   // [E, N]; entries of pairs outside the token lists are left alone
  int layer = 0;           // 0 none, D2D_NORM_OF_INTERMEDIATE, D2D_NORM_OF_OUTPUT
  int ord = 2;             // 1 (sum of magnitudes) or 2 (Euclidean)
};

int launch_router_mask_simt(const void* x, const void* wa, const void* wb, float mult,
                            uint32_t* mask_bits, void* scores, const void* last_bias,
                            int add_residual, void* out_init, int64_t N, int d, int R, int E,
                            int dtype, int* dev_status, cudaStream_t s, void* rt_out = nullptr);
int launch_gate_rule(const void* scores, int rule, int k, float tau, uint32_t* mask_bits,
                     int64_t N, int E, int dtype, cudaStream_t s);
int launch_mask_from_scores(const void* scores, float mult, uint32_t* mask_bits, int64_t N, int E,
                            int dtype, int* dev_status, cudaStream_t s);
int launch_gate_scores_fused(const void* scores, float mult, uint32_t* mask_bits, void* rt,
                             int32_t* tile_counts, const void* x, const void* last_bias,
                             int add_residual, void* out, int64_t N, int d, int E, int dtype,
                             cudaStream_t s);
int launch_init_out(const void* x, const void* last_bias, int add_residual, void* out, int64_t N,
                    int d, int dtype, cudaStream_t s);
int launch_prenorm_init(const void* x, const void* gamma, const void* beta, float eps, int kind,
                        float gamma_offset, const void* last_bias, void* xn, void* out, int64_t N,
                        int d, int dtype, cudaStream_t s);
int launch_expand_mask(const uint32_t* mask_bits, void* rt, int64_t N, int E, int dtype,
                       cudaStream_t s);
int launch_pack_mask(const void* rt, uint32_t* mask_bits, int64_t N, int E, int dtype,
                     cudaStream_t s);
size_t compact_workspace_bytes(int64_t n_max, int E);
int compact_row_cells(int E);      // cells (bytes) per row of the compaction's counts table
// counts_ready: the byte table counts_ws[tile of 128 tokens][compact_row_cells(E)] is already
// filled (by the router kernel); otherwise a count kernel fills it first
int launch_compact(const uint32_t* mask_bits, int32_t* token_idx, int32_t* offsets, int64_t N,
                   int E, int32_t* counts_ws, int* dev_status, cudaStream_t s,
                   bool counts_ready);
int launch_experts_simt(const void* x, const int32_t* token_idx, const int32_t* offsets,
                        const void* w1, const void* b1, const void* w_up, const void* w2,
                        void* out, int64_t N, int d, int E, int H, int act, int dtype,
                        int* dev_status, cudaStream_t s, NormCapture nc = NormCapture());

}  // namespace d2d
