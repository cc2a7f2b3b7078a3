// Grouped expert FFN with fused scatter-add, general-shape FFMA kernel.
//
// Serves fp32 (where the upstream kernels forbid TF32,
// architectures/moe/moe_impls.py:153,288, so the products must be true fp32) and
// every shape the tensor-core kernel does not cover (d or H not a multiple of 16,
// H > 128, ...).  One work item = (expert e, 32 rows of its token list):
//   h   = act(T(x[rows] W1[e]) + b1[e])   (* T(x[rows] W_up[e]) for the gated form)
//   out[rows] += T(h W2[e])               vector red.global.add in T
// which fuses architectures/moe/moe_impls.py:93-180 (first layer) and :244-301
// (second layer + atomic add); the [32, H] hidden tile lives in shared memory.
#include "d2d_common.cuh"

namespace d2d {
namespace {

constexpr int NT = 256;
constexpr int TM_MAX = 32;    // rows per work item: 32 or 16
constexpr int KC = 32;        // k-chunk
constexpr int XP = KC + 4;    // padded x row
constexpr int CB = 128;       // output columns per pass (4 per lane)
constexpr int WP = CB + 4;    // padded weight row
constexpr int MAX_E = 256;

// one element's share of a row's norm (ord 1: magnitude, ord 2: square)
__device__ __forceinline__ float norm_term(float v, int ord) { return ord == 1 ? fabsf(v) : v * v; }

// Row sums held as per-thread partials (a row's columns are spread over LC lanes of each of
// the warps of its row group): reduce over the LC lanes, add into the row's shared cell.
template <int RPT, int LR, int LC>
__device__ __forceinline__ void add_row_norms(const float* part, float* rown, int row0, int lc) {
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    float v = part[i];
#pragma unroll
    for (int o = 1; o < LC; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lc == 0) atomicAdd(&rown[row0 + LR * i], v);
  }
}

// TM_ rows per work item: 32, or 16 for small batches (more, lighter work items: with few
// tokens the launch is one work item per SM and its duration is that item's).
template <typename T, bool GLU, int TM_>
__global__ void __launch_bounds__(NT)
experts_simt_kernel(const T* __restrict__ x, const int32_t* __restrict__ token_idx,
                    const int32_t* __restrict__ offsets, const T* __restrict__ w1,
                    const T* __restrict__ b1, const T* __restrict__ w_up,
                    const T* __restrict__ w2, T* __restrict__ out, int64_t N, int d, int E, int H,
                    int act, int* dev_status, T* __restrict__ norms, int norm_layer,
                    int norm_ord) {
  extern __shared__ float sm[];
  constexpr int RG = TM_ / 16, CG = 8 / RG, CW = CB / CG, LC = CW / 4, LR = 32 / LC, RPT = 16 / LR;
  float* xs = sm;                              // [TM_][XP]
  float* ws = xs + TM_ * XP;                   // [KC][WP]
  float* wu = ws + KC * WP;                    // [KC][WP] (gated form only)
  float* hs = wu + (GLU ? KC * WP : 0);        // [TM_][HP]
  const int HP = ((H + 3) & ~3) + 4;
  __shared__ int tstart[MAX_E + 1];
  __shared__ int rows[TM_MAX];
  __shared__ float rown[TM_MAX];               // row sums of the norm by-product
  const int tid = threadIdx.x, lane = tid & 31, ty = tid >> 5;
  // Thread tile of both products: the 8 warps as RG (rows) x CG (columns), lanes LR x LC;
  // thread (i, j) holds row 16*rg + lr + LR*i and column CW*cg + 4*lc + j of the TM_ x 128
  // pass (32 rows: warps 2 x 4, lanes 4 x 8, 4 x 4 outputs; 16 rows: warps 1 x 8, lanes 8 x 4,
  // 2 x 4 outputs).  The lanes of a warp instruction then read LR distinct activation vectors
  // and LC adjacent weight vectors, each set in distinct banks.
  const int rg = ty / CG, cg = ty % CG, lr = lane / LC, lc = lane % LC;
  const int row0 = 16 * rg + lr, col0 = CW * cg + 4 * lc;
  grid_launch_dependents();
  grid_dependency_wait();      // token lists and offsets come from the previous kernel

  if (tid == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      tstart[e] = run;
      const int c = offsets[e + 1] - offsets[e];
      if (c < 0) { report(dev_status, D2D_ERR_INDEX_RANGE); }
      run += c > 0 ? (c + TM_ - 1) / TM_ : 0;
    }
    tstart[E] = run;
  }
  __syncthreads();
  const int total = tstart[E];
  const bool vec_ok = (d % 4 == 0);
  // vector staging of x rows and weight rows: 4-element boundaries everywhere
  const bool vec = (d % 4 == 0) && (H % 4 == 0) &&
                   ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w1) |
                     reinterpret_cast<uintptr_t>(w2) | reinterpret_cast<uintptr_t>(w_up)) % 16 == 0);
  const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);

  for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
    int lo = 0, hi = E;                 // last e with tstart[e] <= tile
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (tstart[mid] <= tile) lo = mid; else hi = mid;
    }
    const int e = lo;
    const int r0 = offsets[e] + (tile - tstart[e]) * TM_;
    const int nrows = min(TM_, offsets[e + 1] - r0);
    __syncthreads();
    if (tid < TM_) {
      int t = tid < nrows ? token_idx[r0 + tid] : -1;
      if (tid < nrows && (t < 0 || t >= N)) { report(dev_status, D2D_ERR_INDEX_RANGE); t = -1; }
      rows[tid] = t;
      rown[tid] = 0.f;
    }
    __syncthreads();
    const T* w1e = w1 + (int64_t)e * d * H;
    const T* wue = GLU ? w_up + (int64_t)e * d * H : nullptr;
    const T* w2e = w2 + (int64_t)e * H * d;

    // ---- first layer: hs = act(x W1 + b1) (* x W_up) ------------------------
    float npart[RPT];                           // this lane's share of its rows' norms
#pragma unroll
    for (int i = 0; i < RPT; ++i) npart[i] = 0.f;
    for (int hc = 0; hc < H; hc += CB) {
      float acc[RPT][4], accu[RPT][4];
#pragma unroll
      for (int i = 0; i < RPT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; accu[i][j] = 0.f; }
      // Vector path: the vectors of k-chunk kc+1 are loaded into registers before the
      // products of chunk kc start, so the load latency hides behind the arithmetic.
      const int xr = tid >> 3, xk = (tid & 7) << 2;          // x tile: row, k offset
      const int wk = tid >> 5, wc = (tid & 31) << 2;         // weight tile: k row (+8 per pass), column
      float4 px = z4, pw[4], pu[4];
      auto prefetch1 = [&](int kc) {
        const int t = xr < TM_ ? rows[xr] : -1;
        px = (t >= 0 && kc + xk < d) ? load4(x + (int64_t)t * d + kc + xk) : z4;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k = wk + 8 * j;
          const bool ok = (kc + k < d) && (hc + wc < H);
          pw[j] = ok ? load4(w1e + (int64_t)(kc + k) * H + hc + wc) : z4;
          if (GLU) pu[j] = ok ? load4(wue + (int64_t)(kc + k) * H + hc + wc) : z4;
        }
      };
      if (vec) prefetch1(0);
      for (int kc = 0; kc < d; kc += KC) {
        __syncthreads();
        if (vec) {
          if (xr < TM_) *reinterpret_cast<float4*>(&xs[xr * XP + xk]) = px;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            *reinterpret_cast<float4*>(&ws[(wk + 8 * j) * WP + wc]) = pw[j];
            if (GLU) *reinterpret_cast<float4*>(&wu[(wk + 8 * j) * WP + wc]) = pu[j];
          }
          if (kc + KC < d) prefetch1(kc + KC);
        } else {
          for (int i = tid; i < TM_ * KC; i += NT) {
            const int r = i / KC, k = i % KC;
            const int t = rows[r];
            xs[r * XP + k] =
                (t >= 0 && kc + k < d) ? DT<T>::to_f(x[(int64_t)t * d + kc + k]) : 0.f;
          }
          for (int i = tid; i < KC * CB; i += NT) {
            const int k = i / CB, c = i % CB;
            const bool ok = (kc + k < d) && (hc + c < H);
            ws[k * WP + c] = ok ? DT<T>::to_f(w1e[(int64_t)(kc + k) * H + hc + c]) : 0.f;
            if (GLU) wu[k * WP + c] = ok ? DT<T>::to_f(wue[(int64_t)(kc + k) * H + hc + c]) : 0.f;
          }
        }
        __syncthreads();
        // Two register sets of operand vectors: the loads of k-group g+1 are issued before
        // the FMAs of group g (8 warps per SM do not hide the shared-memory latency otherwise).
        float4 xa[2][RPT], wv[2][4], uv[2][4];
        auto load_set = [&](int k4, int b) {
#pragma unroll
          for (int i = 0; i < RPT; ++i)
            xa[b][i] = *reinterpret_cast<const float4*>(&xs[(row0 + LR * i) * XP + k4]);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            wv[b][kk] = *reinterpret_cast<const float4*>(&ws[(k4 + kk) * WP + col0]);
            if (GLU) uv[b][kk] = *reinterpret_cast<const float4*>(&wu[(k4 + kk) * WP + col0]);
          }
        };
        auto fma_set = [&](int b) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
              const float xv = kk == 0 ? xa[b][i].x : kk == 1 ? xa[b][i].y
                             : kk == 2 ? xa[b][i].z : xa[b][i].w;
              acc[i][0] = fmaf(xv, wv[b][kk].x, acc[i][0]);
              acc[i][1] = fmaf(xv, wv[b][kk].y, acc[i][1]);
              acc[i][2] = fmaf(xv, wv[b][kk].z, acc[i][2]);
              acc[i][3] = fmaf(xv, wv[b][kk].w, acc[i][3]);
              if (GLU) {
                accu[i][0] = fmaf(xv, uv[b][kk].x, accu[i][0]);
                accu[i][1] = fmaf(xv, uv[b][kk].y, accu[i][1]);
                accu[i][2] = fmaf(xv, uv[b][kk].z, accu[i][2]);
                accu[i][3] = fmaf(xv, uv[b][kk].w, accu[i][3]);
              }
            }
          }
        };
        load_set(0, 0);
#pragma unroll
        for (int k4 = 0; k4 < KC; k4 += 8) {
          load_set(k4 + 4, 1);
          fma_set(0);
          if (k4 + 8 < KC) load_set(k4 + 8, 0);
          fma_set(1);
        }
      }
#pragma unroll
      for (int i = 0; i < RPT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = hc + col0 + j;
          if (c < H) {
            float h = DT<T>::round(acc[i][j]);
            if (b1) h = DT<T>::round(h + DT<T>::to_f(b1[(int64_t)e * H + c]));
            h = DT<T>::round(activate(h, act));
            if (norm_layer == D2D_NORM_OF_INTERMEDIATE) npart[i] += norm_term(h, norm_ord);
            if (GLU) h = DT<T>::round(h * DT<T>::round(accu[i][j]));
            hs[(row0 + LR * i) * HP + c] = h;
          }
        }
    }

    // ---- second layer + scatter-add ----------------------------------------
    for (int dc = 0; dc < d; dc += CB) {
      float acc[RPT][4];
#pragma unroll
      for (int i = 0; i < RPT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
      const int wk = tid >> 5, wc = (tid & 31) << 2;
      float4 pw[4];
      auto prefetch2 = [&](int kc) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k = wk + 8 * j;
          pw[j] = (kc + k < H && dc + wc < d) ? load4(w2e + (int64_t)(kc + k) * d + dc + wc) : z4;
        }
      };
      if (vec) prefetch2(0);
      for (int kc = 0; kc < H; kc += KC) {
        __syncthreads();
        if (vec) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<float4*>(&ws[(wk + 8 * j) * WP + wc]) = pw[j];
          if (kc + KC < H) prefetch2(kc + KC);
        } else {
          for (int i = tid; i < KC * CB; i += NT) {
            const int k = i / CB, c = i % CB;
            ws[k * WP + c] = (kc + k < H && dc + c < d)
                                 ? DT<T>::to_f(w2e[(int64_t)(kc + k) * d + dc + c])
                                 : 0.f;
          }
        }
        __syncthreads();
        const int kn = min(KC, H - kc);
        // four hidden columns per activation vector; two register sets as in the first product
        float4 ha[2][RPT], wv2[2][4];
        auto load2 = [&](int k, int b) {
#pragma unroll
          for (int i = 0; i < RPT; ++i)
            ha[b][i] = *reinterpret_cast<const float4*>(&hs[(row0 + LR * i) * HP + kc + k]);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            wv2[b][kk] = *reinterpret_cast<const float4*>(&ws[(k + kk) * WP + col0]);
        };
        auto fma2 = [&](int b) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
              const float hv = kk == 0 ? ha[b][i].x : kk == 1 ? ha[b][i].y
                             : kk == 2 ? ha[b][i].z : ha[b][i].w;
              acc[i][0] = fmaf(hv, wv2[b][kk].x, acc[i][0]);
              acc[i][1] = fmaf(hv, wv2[b][kk].y, acc[i][1]);
              acc[i][2] = fmaf(hv, wv2[b][kk].z, acc[i][2]);
              acc[i][3] = fmaf(hv, wv2[b][kk].w, acc[i][3]);
            }
          }
        };
        int k = 0;
        if (kn >= 4) load2(0, 0);
        for (; k + 8 <= kn; k += 8) {
          load2(k + 4, 1);
          fma2(0);
          if (k + 12 <= kn) load2(k + 8, 0);
          fma2(1);
        }
        if (k + 4 <= kn) {        // one more whole group, already in set 0
          fma2(0);
          k += 4;
        }
        for (; k < kn; ++k) {
          const float4 wv = *reinterpret_cast<const float4*>(&ws[k * WP + col0]);
#pragma unroll
          for (int i = 0; i < RPT; ++i) {
            const float hv = hs[(row0 + LR * i) * HP + kc + k];
            acc[i][0] = fmaf(hv, wv.x, acc[i][0]);
            acc[i][1] = fmaf(hv, wv.y, acc[i][1]);
            acc[i][2] = fmaf(hv, wv.z, acc[i][2]);
            acc[i][3] = fmaf(hv, wv.w, acc[i][3]);
          }
        }
      }
      const int c0 = dc + col0;
      if (norm_layer == D2D_NORM_OF_OUTPUT) {
#pragma unroll
        for (int i = 0; i < RPT; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (c0 + j < d) npart[i] += norm_term(DT<T>::round(acc[i][j]), norm_ord);
      }
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const int t = rows[row0 + LR * i];
        if (t < 0 || c0 >= d) continue;
        T* o = out + (int64_t)t * d + c0;
        if (vec_ok) {
          red_add_v4(o, DT<T>::round(acc[i][0]), DT<T>::round(acc[i][1]),
                     DT<T>::round(acc[i][2]), DT<T>::round(acc[i][3]));
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (c0 + j < d) red_add_1(o + j, DT<T>::round(acc[i][j]));
        }
      }
    }
    if (norm_layer != 0) {
      add_row_norms<RPT, LR, LC>(npart, rown, row0, lc);
      __syncthreads();
      if (tid < TM_ && rows[tid] >= 0)
        norms[(int64_t)e * N + rows[tid]] =
            DT<T>::from_f(norm_ord == 1 ? rown[tid] : sqrtf(rown[tid]));
    }
  }
}

template <typename T, bool GLU, int TM_>
int launch_tm(const void* x, const int32_t* token_idx, const int32_t* offsets, const void* w1,
              const void* b1, const void* w_up, const void* w2, void* out, int64_t N, int d, int E,
              int H, int act, int* dev_status, cudaStream_t s, NormCapture nc) {
  const int HP = ((H + 3) & ~3) + 4;
  const size_t smem =
      sizeof(float) * ((size_t)TM_ * XP + (size_t)KC * WP * (GLU ? 2 : 1) + (size_t)TM_ * HP);
  if (smem > 200 * 1024) return D2D_ERR_UNSUPPORTED;
  auto k = experts_simt_kernel<T, GLU, TM_>;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return D2D_ERR_LAUNCH;
  const int64_t max_tiles = ceil_div64(N * (int64_t)E, TM_) + E;
  const int grid = (int)(max_tiles < 148 * 4 ? (max_tiles > 0 ? max_tiles : 1) : 148 * 4);
  return launch_pdl(k, dim3((unsigned)grid), dim3(NT), smem, s, (const T*)x, token_idx, offsets,
                    (const T*)w1, (const T*)b1, (const T*)w_up, (const T*)w2, (T*)out, N, d, E, H,
                    act, dev_status, (T*)nc.norms, nc.norms ? nc.layer : 0, nc.ord);
}

// 32-row work items.  (16-row items, instantiable through TM_, were measured on the 1576-token
// fp32 layer: 134 us per layer against 118 us: the loop is bound by shared-memory load
// latency at 8 warps per SM, and the 2 x 4 thread tile has fewer FMAs per load.)
template <typename T, bool GLU>
int launch_t(const void* x, const int32_t* token_idx, const int32_t* offsets, const void* w1,
             const void* b1, const void* w_up, const void* w2, void* out, int64_t N, int d, int E,
             int H, int act, int* dev_status, cudaStream_t s, NormCapture nc) {
  return launch_tm<T, GLU, 32>(x, token_idx, offsets, w1, b1, w_up, w2, out, N, d, E, H, act,
                               dev_status, s, nc);
}

}  // namespace

int launch_experts_simt(const void* x, const int32_t* token_idx, const int32_t* offsets,
                        const void* w1, const void* b1, const void* w_up, const void* w2,
                        void* out, int64_t N, int d, int E, int H, int act, int dtype,
                        int* dev_status, cudaStream_t s, NormCapture nc) {
  if (E > MAX_E) return D2D_ERR_UNSUPPORTED;
  if (dtype == D2D_F32) {
    return w_up ? launch_t<float, true>(x, token_idx, offsets, w1, b1, w_up, w2, out, N, d, E, H,
                                        act, dev_status, s, nc)
                : launch_t<float, false>(x, token_idx, offsets, w1, b1, w_up, w2, out, N, d, E, H,
                                         act, dev_status, s, nc);
  }
  return w_up ? launch_t<bf16, true>(x, token_idx, offsets, w1, b1, w_up, w2, out, N, d, E, H, act,
                                     dev_status, s, nc)
              : launch_t<bf16, false>(x, token_idx, offsets, w1, b1, w_up, w2, out, N, d, E, H,
                                      act, dev_status, s, nc);
}

}  // namespace d2d
