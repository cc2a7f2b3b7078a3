// Pre-norm fused with the block's residual: the pass in front of the MoE-FFN layer.
//
// An upstream transformer block runs   y = ln_2(x);  y = mlp(y);  return x + y
// (architectures/moe/moe_models.py:69-76 ViT, :91-100 GPT, :148-156 Gemma with RMSNorm), i.e.
// a normalisation pass over [N, d] before the layer and a residual-add pass after it.  Here
// ONE pass reads x once and writes both
//     xn[t,:]  = T(norm(x[t,:]))                       the layer's input (router and expert gather)
//     out[t,:] = T(x[t,:] + last_bias)                 the layer output's initial value,
// after which the layer only adds the expert contributions to `out`
// (d2d_moe_forward with add_residual = D2D_OUT_PREINITIALISED): the separate residual pass and the
// router's initial-value writes disappear.
//
//   kind 0  LayerNorm: (x - mean) * rsqrt(var + eps) * gamma + beta   (biased variance)
//   kind 1  RMSNorm:   x * rsqrt(mean(x^2) + eps) * (gamma_offset + gamma)
//           (gamma_offset = 1 for the Gemma form, transformers GemmaRMSNorm; 0 for the plain form)
// Statistics and the affine map are evaluated in fp32, one rounding to T at the end, like the
// framework kernels they replace.  One warp per row; the row stays in registers between the
// statistics and the output (x is read once).
#include "d2d_common.cuh"

namespace d2d {
namespace {

constexpr int NT = 256;
constexpr int MAXV = 16;      // 16-byte vectors per lane: d <= 32 * 16 * (16 / sizeof(T))

// MAXV_ = vectors a lane holds (the register footprint, hence the number of resident warps and
// the bytes in flight per SM, follows the row length instead of the longest row supported).
template <typename T, int MAXV_>
__global__ void __launch_bounds__(NT)
prenorm_init_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                    const T* __restrict__ beta, float eps, int kind, float gamma_offset,
                    const T* __restrict__ last_bias, T* __restrict__ xn, T* __restrict__ out,
                    int64_t N, int d) {
  constexpr int V = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int dv = d / V;                       // vectors per row
  const int nv = (dv + 31) / 32;              // vectors per lane (<= MAXV)
  const int64_t warps = (int64_t)gridDim.x * (NT / 32);
  // Short rows (<= 4 vectors per lane) keep the NEXT row's loads in flight while the current
  // row is reduced and written: one row per warp at a time leaves too few bytes in flight.
  constexpr bool PREFETCH = MAXV_ <= 4;
  uint4 raw[MAXV_], nxt[PREFETCH ? MAXV_ : 1];
  int64_t row = (int64_t)blockIdx.x * (NT / 32) + (threadIdx.x >> 5);
  if (PREFETCH && row < N) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * d);
#pragma unroll
    for (int i = 0; i < MAXV_; ++i) {
      const int c = lane + 32 * i;
      if (i < nv && c < dv) raw[i] = __ldg(xr + c);
    }
  }
  for (; row < N; row += warps) {
    if (PREFETCH) {
      if (row + warps < N) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + (row + warps) * d);
#pragma unroll
        for (int i = 0; i < MAXV_; ++i) {
          const int c = lane + 32 * i;
          if (i < nv && c < dv) nxt[i] = __ldg(xr + c);
        }
      }
    } else {
      const uint4* xr = reinterpret_cast<const uint4*>(x + row * d);
#pragma unroll
      for (int i = 0; i < MAXV_; ++i) {
        const int c = lane + 32 * i;
        if (i < nv && c < dv) raw[i] = __ldg(xr + c);
      }
    }
    float sum = 0.f, sq = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV_; ++i) {
      const int c = lane + 32 * i;
      if (i < nv && c < dv) {
        const T* e = reinterpret_cast<const T*>(&raw[i]);
#pragma unroll
        for (int q = 0; q < V; ++q) {
          const float v = DT<T>::to_f(e[q]);
          sum += v;
          sq += v * v;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sum += __shfl_xor_sync(0xffffffffu, sum, o);
      sq += __shfl_xor_sync(0xffffffffu, sq, o);
    }
    float mean = 0.f, rstd;
    if (kind == 0) {
      mean = sum / (float)d;
      float var = 0.f;                        // second pass over the registers: sum (x - mean)^2
#pragma unroll
      for (int i = 0; i < MAXV_; ++i) {
        const int c = lane + 32 * i;
        if (i < nv && c < dv) {
          const T* e = reinterpret_cast<const T*>(&raw[i]);
#pragma unroll
          for (int q = 0; q < V; ++q) {
            const float dlt = DT<T>::to_f(e[q]) - mean;
            var += dlt * dlt;
          }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
      rstd = rsqrtf(var / (float)d + eps);
    } else {
      rstd = rsqrtf(sq / (float)d + eps);
    }
#pragma unroll
    for (int i = 0; i < MAXV_; ++i) {
      const int c = lane + 32 * i;
      if (i < nv && c < dv) {
        const uint4 gv = __ldg(reinterpret_cast<const uint4*>(gamma) + c);
        uint4 bv = make_uint4(0u, 0u, 0u, 0u), lb = make_uint4(0u, 0u, 0u, 0u);
        if (beta) bv = __ldg(reinterpret_cast<const uint4*>(beta) + c);
        if (last_bias) lb = __ldg(reinterpret_cast<const uint4*>(last_bias) + c);
        const T* e = reinterpret_cast<const T*>(&raw[i]);
        const T* g = reinterpret_cast<const T*>(&gv);
        const T* b = reinterpret_cast<const T*>(&bv);
        const T* l = reinterpret_cast<const T*>(&lb);
        T yn[V], yo[V];
#pragma unroll
        for (int q = 0; q < V; ++q) {
          const float v = DT<T>::to_f(e[q]);
          const float nrm = (v - mean) * rstd;
          yn[q] = DT<T>::from_f(kind == 0 ? nrm * DT<T>::to_f(g[q]) + DT<T>::to_f(b[q])
                                          : nrm * (gamma_offset + DT<T>::to_f(g[q])));
          yo[q] = DT<T>::from_f(v + DT<T>::to_f(l[q]));
        }
        *(reinterpret_cast<uint4*>(xn + row * d) + c) = *reinterpret_cast<const uint4*>(yn);
        if (out) *(reinterpret_cast<uint4*>(out + row * d) + c) = *reinterpret_cast<const uint4*>(yo);
      }
    }
    if (PREFETCH) {
#pragma unroll
      for (int i = 0; i < MAXV_; ++i) raw[i] = nxt[i];
    }
  }
}

}  // namespace

int launch_prenorm_init(const void* x, const void* gamma, const void* beta, float eps, int kind,
                        float gamma_offset, const void* last_bias, void* xn, void* out, int64_t N,
                        int d, int dtype, cudaStream_t s) {
  const int V = dtype == D2D_F32 ? 4 : 8;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (d % V != 0 || d / V > 32 * MAXV) return D2D_ERR_UNSUPPORTED;
  if (!al16(x) || !al16(gamma) || !al16(beta) || !al16(last_bias) || !al16(xn) || !al16(out))
    return D2D_ERR_BAD_ARG;
  int64_t grid = ceil_div64(N, NT / 32);
  if (grid > 148 * 16) grid = 148 * 16;
  if (grid < 1) grid = 1;
  const int nv = (d / V + 31) / 32;
#define D2D_PRENORM_CASE(T_, NV_)                                                              \
  prenorm_init_kernel<T_, NV_><<<(unsigned)grid, NT, 0, s>>>(                                   \
      (const T_*)x, (const T_*)gamma, (const T_*)beta, eps, kind, gamma_offset,                 \
      (const T_*)last_bias, (T_*)xn, (T_*)out, N, d)
#define D2D_PRENORM_BY_NV(T_)                                                                  \
  do {                                                                                         \
    if (nv <= 1) D2D_PRENORM_CASE(T_, 1);                                                      \
    else if (nv <= 2) D2D_PRENORM_CASE(T_, 2);                                                 \
    else if (nv <= 3) D2D_PRENORM_CASE(T_, 3);                                                 \
    else if (nv <= 4) D2D_PRENORM_CASE(T_, 4);                                                 \
    else if (nv <= 8) D2D_PRENORM_CASE(T_, 8);                                                 \
    else D2D_PRENORM_CASE(T_, MAXV);                                                           \
  } while (0)
  if (dtype == D2D_F32) D2D_PRENORM_BY_NV(float);
  else D2D_PRENORM_BY_NV(bf16);
#undef D2D_PRENORM_BY_NV
#undef D2D_PRENORM_CASE
  return cudaGetLastError() == cudaSuccess ? D2D_OK : D2D_ERR_LAUNCH;
}

}  // namespace d2d
