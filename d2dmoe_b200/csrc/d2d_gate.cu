// Router MLP + dynamic-k rule -> bit-packed expert mask (general-shape kernels),
// the rule alone on given scores, the 0/1 routing tensor from the bits, and the
// initial value of the layer output.
//
// Upstream semantics restated by these kernels:
//   scores  = | relu(x Wa^T) Wb^T |        architectures/moe/moefication.py:328-330
//   keep e  iff  s_e >= T(max_e s * mult)  architectures/moe/moefication.py:80-85
// Each Linear output is materialised in the tensor dtype T upstream, so the fp32
// accumulators are rounded to T once after each of the two products, and the
// threshold is rounded to T before the comparison.
#include "d2d_common.cuh"

namespace d2d {

namespace {

constexpr int TM = 32;       // tokens per CTA
constexpr int KC = 32;       // k-chunk staged in shared memory
constexpr int KP = KC + 4;   // padded row (floats): conflict-free float4 reads
constexpr int RC = 128;      // router hidden columns per pass
constexpr int NT = 256;

// max that propagates NaN like torch.max does
__device__ __forceinline__ float nanmax(float a, float b) {
  return (a != a || b != b) ? __int_as_float(0x7fc00000) : fmaxf(a, b);
}

template <typename T>
__device__ __forceinline__ void gate_row(const float* s, int nw, float mult, int lane,
                                         uint32_t* mask_row, int E, T* rt_row = nullptr) {
  // s[j]: this lane's score for expert lane+32j (-inf-like sentinel for e >= E is
  // handled by the caller passing valid flags through E).
  float m = -INFINITY;
  for (int j = 0; j < nw; ++j)
    if (lane + 32 * j < E) m = nanmax(m, s[j]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = nanmax(m, __shfl_xor_sync(0xffffffffu, m, o));
  const float thr = DT<T>::round(__fmul_rn(m, mult));
  for (int j = 0; j < nw; ++j) {
    const bool keep = (lane + 32 * j < E) && (s[j] >= thr);
    const uint32_t w = __ballot_sync(0xffffffffu, keep);
    if (lane == 0) mask_row[j] = w;
    if (rt_row && lane + 32 * j < E) rt_row[lane + 32 * j] = DT<T>::from_f(keep ? 1.f : 0.f);
  }
}

// TM_ tokens per CTA: 32, or 16 when 32-token tiles would leave SMs without a tile.
// GEMM1 thread tile: the 8 warps as RG (rows) x CG (hidden columns), lanes 4 x 8; thread (i, j)
// holds row 16*rg + lr + 4i and column CW*cg + lc + 8j.  The lanes of a warp instruction then
// read 4 distinct x vectors and 8 distinct weight vectors, each set in distinct banks.
template <typename T, int TM_>
__global__ void __launch_bounds__(NT)
router_mask_simt_kernel(const T* __restrict__ x, const T* __restrict__ wa,
                        const T* __restrict__ wb, float mult, uint32_t* __restrict__ mask_bits,
                        T* __restrict__ scores, const T* __restrict__ last_bias, int add_residual,
                        T* __restrict__ out_init, int64_t N, int d, int R, int E,
                        T* __restrict__ rt_out) {
  constexpr int RG = TM_ / 16, CG = 8 / RG, CW = RC / CG, CPT = CW / 8, RPW = TM_ / 8;
  extern __shared__ float sm[];
  float* xs = sm;                      // [TM_][KP]
  float* wsm = xs + TM_ * KP;          // [RC][KP]
  float* hs = wsm + RC * KP;           // [TM_][R]
  const int tid = threadIdx.x, lane = tid & 31, ty = tid >> 5;
  const int rg = ty / CG, cg = ty % CG, lr = lane >> 3, lc = lane & 7;
  const int row0 = 16 * rg + lr, col0 = CW * cg + lc;
  const int64_t t0 = (int64_t)blockIdx.x * TM_;
  grid_launch_dependents();
  grid_dependency_wait();      // x may come from the previous kernel of the stream
  // vector staging needs rows that start on a 4-element boundary
  const bool vec = (d % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(wa)) % 16 == 0);

  for (int rc = 0; rc < R; rc += RC) {
    float acc[4][CPT];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < CPT; ++j) acc[i][j] = 0.f;
    // Vector path: one 4-element vector per thread and pass (row = tid / 8 (+32 per pass),
    // k = 4*(tid%8)).  The vectors of k-chunk kc+1 are loaded into registers before the
    // products of chunk kc start, so the load latency hides behind the arithmetic.
    const int vr = tid >> 3, vk = (tid & 7) << 2;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 px = z, pw[RC / 32];
    auto prefetch = [&](int kc) {
      const int64_t t = t0 + vr;
      px = (vr < TM_ && t < N && kc + vk < d) ? load4(x + t * d + kc + vk) : z;
#pragma unroll
      for (int j = 0; j < RC / 32; ++j) {
        const int c = vr + 32 * j;
        pw[j] = (rc + c < R && kc + vk < d) ? load4(wa + (int64_t)(rc + c) * d + kc + vk) : z;
      }
    };
    if (vec) prefetch(0);
    for (int kc = 0; kc < d; kc += KC) {
      __syncthreads();
      if (vec) {
        if (vr < TM_) *reinterpret_cast<float4*>(&xs[vr * KP + vk]) = px;
#pragma unroll
        for (int j = 0; j < RC / 32; ++j)
          *reinterpret_cast<float4*>(&wsm[(vr + 32 * j) * KP + vk]) = pw[j];
        if (kc + KC < d) prefetch(kc + KC);
      } else {
        for (int i = tid; i < TM_ * KC; i += NT) {
          const int r = i / KC, k = i % KC;
          const int64_t t = t0 + r;
          xs[r * KP + k] = (t < N && kc + k < d) ? DT<T>::to_f(x[t * d + kc + k]) : 0.f;
        }
        for (int i = tid; i < RC * KC; i += NT) {
          const int c = i / KC, k = i % KC;
          wsm[c * KP + k] =
              (rc + c < R && kc + k < d) ? DT<T>::to_f(wa[(int64_t)(rc + c) * d + kc + k]) : 0.f;
        }
      }
      __syncthreads();
      // Two register sets of operand vectors: the loads of k-group g+1 are issued before the
      // FMAs of group g (8 warps per SM do not hide the shared-memory latency otherwise).
      float4 xa[2][4], wv[2][CPT];
      auto load_set = [&](int k4, int b) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          xa[b][i] = *reinterpret_cast<const float4*>(&xs[(row0 + 4 * i) * KP + k4]);
#pragma unroll
        for (int j = 0; j < CPT; ++j)
          wv[b][j] = *reinterpret_cast<const float4*>(&wsm[(col0 + 8 * j) * KP + k4]);
      };
      auto fma_set = [&](int b) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < CPT; ++j) {
            acc[i][j] = fmaf(xa[b][i].x, wv[b][j].x, acc[i][j]);
            acc[i][j] = fmaf(xa[b][i].y, wv[b][j].y, acc[i][j]);
            acc[i][j] = fmaf(xa[b][i].z, wv[b][j].z, acc[i][j]);
            acc[i][j] = fmaf(xa[b][i].w, wv[b][j].w, acc[i][j]);
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
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < CPT; ++j) {
        const int c = rc + col0 + 8 * j;
        if (c < R) hs[(row0 + 4 * i) * R + c] = fmaxf(DT<T>::round(acc[i][j]), 0.f);
      }
  }
  __syncthreads();

  // Wb [E, R] into the (now free) weight staging area as [E][R + 1] floats when it fits: the
  // second product then reads it conflict-free instead of with one strided global load per k
  const int RP = R + 1;
  const bool wb_s = (int64_t)E * RP <= RC * KP;
  if (wb_s) {
    for (int i = tid; i < E * R; i += NT) wsm[(i / R) * RP + (i % R)] = DT<T>::to_f(wb[i]);
    __syncthreads();
  }

  // scores + gate: warp ty owns rows RPW*ty .. RPW*ty + RPW - 1, lane owns experts lane + 32j
  const int nw = (E + 31) / 32;
  float sc[RPW][8];   // [row][word]  (E <= 256)
  for (int j = 0; j < nw; ++j) {
    const int e = lane + 32 * j;
    float a[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) a[i] = 0.f;
    if (e < E) {
      const T* wrow = wb + (int64_t)e * R;
      const float* wsr = wsm + e * RP;
      const float* h0 = hs + (RPW * ty) * R;
      for (int k = 0; k < R; ++k) {
        const float w = wb_s ? wsr[k] : DT<T>::to_f(wrow[k]);
#pragma unroll
        for (int i = 0; i < RPW; ++i) a[i] = fmaf(h0[i * R + k], w, a[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < RPW; ++i) sc[i][j] = fabsf(DT<T>::round(a[i]));
  }
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    const int64_t t = t0 + RPW * ty + i;
    if (t >= N) break;   // warp-uniform
    if (scores)
      for (int j = 0; j < nw; ++j)
        if (lane + 32 * j < E) scores[t * E + lane + 32 * j] = DT<T>::from_f(sc[i][j]);
    gate_row<T>(sc[i], nw, mult, lane, mask_bits + t * nw, E, rt_out ? rt_out + t * E : nullptr);
  }

  if (out_init) {
    const int rows = (int)min((int64_t)TM_, N - t0);
    for (int c = tid; c < d; c += NT) {          // thread = column, rows inside
      const float lb = last_bias ? DT<T>::round(DT<T>::to_f(last_bias[c])) : 0.f;
      for (int r = 0; r < rows; ++r) {
        float v = lb;
        if (add_residual) v = lb + DT<T>::to_f(x[(t0 + r) * d + c]);
        out_init[(t0 + r) * d + c] = DT<T>::from_f(v);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(NT)
mask_from_scores_kernel(const T* __restrict__ scores, float mult, uint32_t* __restrict__ mask_bits,
                        int64_t N, int E) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * NT + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * NT) >> 5;
  const int nw = (E + 31) / 32;
  for (int64_t t = warp; t < N; t += nwarps) {
    float s[8];
    for (int j = 0; j < nw; ++j) {
      const int e = lane + 32 * j;
      s[j] = e < E ? DT<T>::to_f(scores[t * E + e]) : 0.f;
    }
    gate_row<T>(s, nw, mult, lane, mask_bits + t * nw, E);
  }
}

// The other two routing rules of MoeficationMoE.gate on given scores
// (architectures/moe/moefication.py:59-79), one warp per token, lane = expert (+32j):
//   top-k : keep the k largest scores (NaN counts as largest, equal scores: lower index
//           first, as torch.topk does on the host);
//   dynk  : shares = T(s / T(sum s)); experts in descending share order; keep the first,
//           and every further one while the cumulative share before it (fp32 running sum
//           in that order, rounded to T per element, as torch.cumsum does) is < T(tau).
// `before(a, ia, b, ib)`: a precedes b in the descending order used by both rules.
template <typename T> struct Acc { typedef float type; };
template <> struct Acc<float> { typedef double type; };

__device__ __forceinline__ bool before(float a, int ia, float b, int ib) {
  const bool an = a != a, bn = b != b;
  if (an || bn) return an && (!bn || ia < ib);
  return a > b || (a == b && ia < ib);
}

template <typename T>
__global__ void __launch_bounds__(NT)
gate_rule_kernel(const T* __restrict__ scores, int rule, int k, float tau,
                 uint32_t* __restrict__ mask_bits, int64_t N, int E) {
  __shared__ float sorted_s[NT / 32][256];
  const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
  const int64_t warp = ((int64_t)blockIdx.x * NT + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * NT) >> 5;
  const int nw = (E + 31) / 32;
  const float tau_t = DT<T>::round(tau);
  float* srt = sorted_s[wi];
  for (int64_t t = warp; t < N; t += nwarps) {
    float s[8];
    int rank[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane + 32 * j;
      s[j] = (j < nw && e < E) ? DT<T>::to_f(scores[t * E + e]) : 0.f;
      rank[j] = 0;
    }
    if (rule == D2D_RULE_DYNK) {
      float tot = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < nw && lane + 32 * j < E) tot += s[j];
      for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
      tot = DT<T>::round(tot);
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j] = DT<T>::round(s[j] / tot);
    }
    // rank of each of my experts = number of experts that precede it
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      if (jj >= nw) break;
      for (int l = 0; l < 32; ++l) {
        const int eo = l + 32 * jj;
        if (eo >= E) break;                    // warp-uniform
        const float v = __shfl_sync(0xffffffffu, s[jj], l);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < nw && before(v, eo, s[j], lane + 32 * j)) ++rank[j];
      }
    }
    bool keep[8];
    if (rule == D2D_RULE_TOPK) {
#pragma unroll
      for (int j = 0; j < 8; ++j) keep[j] = rank[j] < k;
    } else {
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < nw && lane + 32 * j < E) srt[rank[j]] = s[j];
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 8; ++j) keep[j] = rank[j] == 0;
      // running sum in the accumulation type torch.cumsum uses on the host: double for
      // fp32 tensors, float for bf16
      typename Acc<T>::type acc = 0;
      for (int r = 0; r + 1 < E; ++r) {
        acc += srt[r];
        const bool more = DT<T>::round((float)acc) < tau_t;   // expert of rank r+1 still needed
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (rank[j] == r + 1) keep[j] = more;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j >= nw) break;
      const uint32_t word = __ballot_sync(0xffffffffu, keep[j] && lane + 32 * j < E);
      if (lane == 0) mask_bits[t * nw + j] = word;
    }
  }
}

// The rule on given scores, fused with what the layer needs next: the compaction's counts
// table (per 128-token tile) and the output's initial value.  One CTA = one 128-token
// tile; warp w handles tokens 16w..16w+15 (lane = expert), then all threads write the
// tile's initial output rows with 16-byte stores.  Needs d % (16/sizeof(T)) == 0.
template <typename T>
__global__ void __launch_bounds__(NT)
gate_scores_fused_kernel(const T* __restrict__ scores, float mult,
                         uint32_t* __restrict__ mask_bits, T* __restrict__ rt,
                         uint8_t* __restrict__ tile_counts, int EP,
                         const T* __restrict__ x, const T* __restrict__ last_bias,
                         int add_residual, T* __restrict__ out, int64_t N, int d, int E) {
  __shared__ int cnt[256];
  constexpr int V = 16 / sizeof(T);
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int nw = (E + 31) / 32;
  const int64_t t0 = (int64_t)blockIdx.x * 128;
  for (int e = tid; e < E; e += NT) cnt[e] = 0;
  // the tile's initial output rows first: these stores depend on nothing the rule computes
  // and drain while it runs.  Warp w writes rows w, w+8, ...; a lane keeps its 16-byte
  // column pieces of last_bias in registers.
  if (out) {
    const int dv = d / V;
    const int rows = (int)min((int64_t)128, N - t0);
    for (int cv = lane; cv < dv; cv += 32) {
      uint4 bz = make_uint4(0u, 0u, 0u, 0u);
      if (last_bias) bz = __ldg(reinterpret_cast<const uint4*>(last_bias) + cv);
#pragma unroll 4
      for (int r = w; r < rows; r += NT / 32) {
        uint4 o = bz;
        if (add_residual) {
          const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + (t0 + r) * d) + cv);
          const T* a = reinterpret_cast<const T*>(&bz);
          const T* b = reinterpret_cast<const T*>(&xv);
          T rr[V];
#pragma unroll
          for (int q = 0; q < V; ++q)
            rr[q] = DT<T>::from_f(DT<T>::to_f(a[q]) + DT<T>::to_f(b[q]));
          o = *reinterpret_cast<const uint4*>(rr);
        }
        *(reinterpret_cast<uint4*>(out + (t0 + r) * d) + cv) = o;
      }
    }
  }
  __syncthreads();
  int mine[8] = {0, 0, 0, 0, 0, 0, 0, 0};       // kept-count of expert lane+32j over my tokens
  // warp w applies the rule to tokens 16w..16w+15 (lane = expert); the scores of four tokens
  // are loaded before the first of them is reduced, so the loads overlap
  for (int i0 = 0; i0 < 16; i0 += 4) {
    float s[4][8];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t t = t0 + w * 16 + i0 + u;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int e = lane + 32 * j;
        s[u][j] = (j < nw && t < N && e < E) ? DT<T>::to_f(scores[t * E + e]) : 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t t = t0 + w * 16 + i0 + u;
      if (t >= N) break;                           // warp-uniform
      float m = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < nw && lane + 32 * j < E) m = nanmax(m, s[u][j]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = nanmax(m, __shfl_xor_sync(0xffffffffu, m, o));
      const float thr = DT<T>::round(__fmul_rn(m, mult));
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (j >= nw) break;
        const bool keep = (lane + 32 * j < E) && (s[u][j] >= thr);
        const uint32_t word = __ballot_sync(0xffffffffu, keep);
        if (lane == 0) mask_bits[t * nw + j] = word;
        if (rt && lane + 32 * j < E) rt[t * E + lane + 32 * j] = DT<T>::from_f(keep ? 1.0f : 0.0f);
        mine[j] += keep ? 1 : 0;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j)
    if (j < nw && lane + 32 * j < E && mine[j]) atomicAdd(&cnt[lane + 32 * j], mine[j]);
  __syncthreads();
  for (int e = tid; e < EP; e += NT)
    tile_counts[(int64_t)blockIdx.x * EP + e] = (uint8_t)(e < E ? cnt[e] : 0);
}

// The same kernel for rows of at most 8 sixteen-byte vectors (E <= 64 in bf16, E <= 32 in
// fp32, E * sizeof(T) a multiple of 16): one LANE per token.  A lane loads its token's
// whole score row with vector loads and finds the row maximum, the threshold and the mask
// word(s) in its own registers, with no cross-lane traffic, so a warp settles 32 tokens in
// the time the warp-per-token form needs for one; warps 0-3 take the tile's 128 tokens.
// The per-expert counts of the tile come from one ballot per expert and warp.
template <typename T, int NV>
__global__ void __launch_bounds__(NT)
gate_scores_fused_rows_kernel(const T* __restrict__ scores, float mult,
                              uint32_t* __restrict__ mask_bits, T* __restrict__ rt,
                              uint8_t* __restrict__ tile_counts, int EP,
                              const T* __restrict__ x, const T* __restrict__ last_bias,
                              int add_residual, T* __restrict__ out, int64_t N, int d, int E) {
  __shared__ int cnt[64];
  constexpr int V = 16 / sizeof(T);
  constexpr int EMAX = NV * V;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int nw = (E + 31) / 32;
  const int64_t t0 = (int64_t)blockIdx.x * 128;
  if (tid < 64) cnt[tid] = 0;
  // this lane's score row first: the loads fly while the initial output rows are issued
  const int64_t t = t0 + w * 32 + lane;
  uint4 raw[NV];
  if (w < 4) {
#pragma unroll
    for (int v = 0; v < NV; ++v)
      raw[v] = t < N ? __ldg(reinterpret_cast<const uint4*>(scores + t * E) + v)
                     : make_uint4(0u, 0u, 0u, 0u);
  }
  if (out) {
    const int dv = d / V;
    const int rows = (int)min((int64_t)128, N - t0);
    for (int cv = lane; cv < dv; cv += 32) {
      uint4 bz = make_uint4(0u, 0u, 0u, 0u);
      if (last_bias) bz = __ldg(reinterpret_cast<const uint4*>(last_bias) + cv);
#pragma unroll 4
      for (int r = w; r < rows; r += NT / 32) {
        uint4 o = bz;
        if (add_residual) {
          const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + (t0 + r) * d) + cv);
          const T* a = reinterpret_cast<const T*>(&bz);
          const T* b = reinterpret_cast<const T*>(&xv);
          T rr[V];
#pragma unroll
          for (int q = 0; q < V; ++q)
            rr[q] = DT<T>::from_f(DT<T>::to_f(a[q]) + DT<T>::to_f(b[q]));
          o = *reinterpret_cast<const uint4*>(rr);
        }
        *(reinterpret_cast<uint4*>(out + (t0 + r) * d) + cv) = o;
      }
    }
  }
  __syncthreads();
  if (w < 4) {
    const T* sv = reinterpret_cast<const T*>(raw);
    float m = -INFINITY;
#pragma unroll
    for (int e = 0; e < EMAX; ++e)
      if (e < E) m = nanmax(m, DT<T>::to_f(sv[e]));
    const float thr = DT<T>::round(__fmul_rn(m, mult));
    uint32_t word[2] = {0u, 0u};
    uint4 one[NV];
    T* ov = reinterpret_cast<T*>(one);
#pragma unroll
    for (int e = 0; e < EMAX; ++e) {
      const bool keep = e < E && DT<T>::to_f(sv[e]) >= thr;
      if (keep) word[e >> 5] |= 1u << (e & 31);
      ov[e] = DT<T>::from_f(keep ? 1.0f : 0.0f);
    }
    if (t < N) {
      for (int j = 0; j < nw; ++j) mask_bits[t * nw + j] = word[j];
      if (rt) {
#pragma unroll
        for (int v = 0; v < NV; ++v) *(reinterpret_cast<uint4*>(rt + t * E) + v) = one[v];
      }
    }
    for (int e = 0; e < E; ++e) {
      const int c = __popc(__ballot_sync(0xffffffffu, t < N && ((word[e >> 5] >> (e & 31)) & 1u)));
      if (lane == 0 && c) atomicAdd(&cnt[e], c);
    }
  }
  __syncthreads();
  for (int e = tid; e < EP; e += NT)
    tile_counts[(int64_t)blockIdx.x * EP + e] = (uint8_t)(e < E ? cnt[e] : 0);
}

template <typename T>
__global__ void __launch_bounds__(NT)
init_out_kernel(const T* __restrict__ x, const T* __restrict__ last_bias, int add_residual,
                T* __restrict__ out, int64_t total, int d) {
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * NT) {
    const int c = (int)(i % d);
    float v = last_bias ? DT<T>::to_f(last_bias[c]) : 0.f;
    if (add_residual) v = DT<T>::round(v) + DT<T>::to_f(x[i]);
    out[i] = DT<T>::from_f(v);
  }
}

// 16 bytes per thread: V = 16 / sizeof(T) columns of one row (d % V == 0, 16-byte aligned)
template <typename T>
__global__ void __launch_bounds__(NT)
init_out_vec_kernel(const T* __restrict__ x, const T* __restrict__ last_bias, int add_residual,
                    T* __restrict__ out, int64_t total_vec, int dv) {
  constexpr int V = 16 / sizeof(T);
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < total_vec;
       i += (int64_t)gridDim.x * NT) {
    const int cv = (int)(i % dv);
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if (last_bias) o = __ldg(reinterpret_cast<const uint4*>(last_bias) + cv);
    if (add_residual) {
      const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x) + i);
      const T* a = reinterpret_cast<const T*>(&o);
      const T* b = reinterpret_cast<const T*>(&xv);
      T r[V];
#pragma unroll
      for (int q = 0; q < V; ++q) r[q] = DT<T>::from_f(DT<T>::to_f(a[q]) + DT<T>::to_f(b[q]));
      o = *reinterpret_cast<const uint4*>(r);
    }
    *(reinterpret_cast<uint4*>(out) + i) = o;
  }
}

template <typename T>
__global__ void __launch_bounds__(NT)
expand_mask_kernel(const uint32_t* __restrict__ mask_bits, T* __restrict__ rt, int64_t total, int E) {
  const int nw = (E + 31) / 32;
  for (int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * NT) {
    const int64_t t = i / E;
    const int e = (int)(i % E);
    const uint32_t w = mask_bits[t * nw + (e >> 5)];
    rt[i] = DT<T>::from_f(((w >> (e & 31)) & 1u) ? 1.0f : 0.0f);
  }
}

template <typename T>
__global__ void __launch_bounds__(NT)
pack_mask_kernel(const T* __restrict__ rt, uint32_t* __restrict__ mask_bits, int64_t N, int E) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * NT + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * NT) >> 5;
  const int nw = (E + 31) / 32;
  for (int64_t t = warp; t < N; t += nwarps)
    for (int j = 0; j < nw; ++j) {
      const int e = lane + 32 * j;
      const bool keep = e < E && DT<T>::to_f(rt[t * E + e]) > 0.0f;
      const uint32_t w = __ballot_sync(0xffffffffu, keep);
      if (lane == 0) mask_bits[t * nw + j] = w;
    }
}

inline int grid_for(int64_t work, int per_block, int cap) {
  int64_t g = ceil_div64(work, per_block);
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return (int)g;
}

template <typename T, int TM_>
int launch_router_simt_t(const void* x, const void* wa, const void* wb, float mult,
                         uint32_t* mask_bits, void* scores, const void* last_bias,
                         int add_residual, void* out_init, int64_t N, int d, int R, int E,
                         cudaStream_t s, void* rt_out) {
  const size_t smem = sizeof(float) * ((size_t)TM_ * KP + (size_t)RC * KP + (size_t)TM_ * R);
  const int64_t grid = ceil_div64(N, TM_);
  if (grid > 0x7fffffffLL) return D2D_ERR_UNSUPPORTED;
  auto k = router_mask_simt_kernel<T, TM_>;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess)
    return D2D_ERR_LAUNCH;
  return launch_pdl(k, dim3((unsigned)grid), dim3(NT), smem, s, (const T*)x, (const T*)wa,
                    (const T*)wb, mult, mask_bits, (T*)scores, (const T*)last_bias, add_residual,
                    (T*)out_init, N, d, R, E, (T*)rt_out);
}

}  // namespace

int launch_router_mask_simt(const void* x, const void* wa, const void* wb, float mult,
                            uint32_t* mask_bits, void* scores, const void* last_bias,
                            int add_residual, void* out_init, int64_t N, int d, int R, int E,
                            int dtype, int* dev_status, cudaStream_t s, void* rt_out) {
  (void)dev_status;
  if (E > 256 || R > 1024) return D2D_ERR_UNSUPPORTED;
  // 16-token tiles while 32-token tiles would not give every SM of a B200 a tile
  const bool small = ceil_div64(N, 32) < 148;
#define D2D_ROUTER_SIMT(T_, TM_)                                                                \
  launch_router_simt_t<T_, TM_>(x, wa, wb, mult, mask_bits, scores, last_bias, add_residual,   \
                                out_init, N, d, R, E, s, rt_out)
  if (dtype == D2D_F32) return small ? D2D_ROUTER_SIMT(float, 16) : D2D_ROUTER_SIMT(float, 32);
  return small ? D2D_ROUTER_SIMT(bf16, 16) : D2D_ROUTER_SIMT(bf16, 32);
#undef D2D_ROUTER_SIMT
}

int launch_mask_from_scores(const void* scores, float mult, uint32_t* mask_bits, int64_t N, int E,
                            int dtype, int* dev_status, cudaStream_t s) {
  (void)dev_status;
  if (E > 256) return D2D_ERR_UNSUPPORTED;
  const int grid = grid_for(N, NT / 32, 148 * 8);
  if (dtype == D2D_F32)
    mask_from_scores_kernel<float><<<grid, NT, 0, s>>>((const float*)scores, mult, mask_bits, N, E);
  else
    mask_from_scores_kernel<bf16><<<grid, NT, 0, s>>>((const bf16*)scores, mult, mask_bits, N, E);
  return cudaGetLastError() == cudaSuccess ? D2D_OK : D2D_ERR_LAUNCH;
}

int launch_gate_rule(const void* scores, int rule, int k, float tau, uint32_t* mask_bits,
                     int64_t N, int E, int dtype, cudaStream_t s) {
  if (E > 256) return D2D_ERR_UNSUPPORTED;
  const int grid = grid_for(N, NT / 32, 148 * 8);
  if (dtype == D2D_F32)
    gate_rule_kernel<float><<<grid, NT, 0, s>>>((const float*)scores, rule, k, tau, mask_bits, N, E);
  else
    gate_rule_kernel<bf16><<<grid, NT, 0, s>>>((const bf16*)scores, rule, k, tau, mask_bits, N, E);
  return cudaGetLastError() == cudaSuccess ? D2D_OK : D2D_ERR_LAUNCH;
}

// returns D2D_ERR_UNSUPPORTED when the shape does not allow the fused form (caller then uses
// the separate kernels)
int launch_gate_scores_fused(const void* scores, float mult, uint32_t* mask_bits, void* rt,
                             int32_t* tile_counts, const void* x, const void* last_bias,
                             int add_residual, void* out, int64_t N, int d, int E, int dtype,
                             cudaStream_t s) {
  const int V = dtype == D2D_F32 ? 4 : 8;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (E > 256 || d % V != 0 || !al16(out) || !al16(x) || !al16(last_bias))
    return D2D_ERR_UNSUPPORTED;
  const int64_t grid = ceil_div64(N, 128);
  if (grid > 0x7fffffffLL) return D2D_ERR_UNSUPPORTED;
  // score rows of whole 16-byte vectors, at most 8 of them: one lane per token
  const int row_bytes = E * (dtype == D2D_F32 ? 4 : 2);
  const bool rows_form = row_bytes % 16 == 0 && row_bytes <= 128 && al16(scores) &&
                         (rt == nullptr || al16(rt));
#define D2D_ROWS_CASE(T, NVV)                                                                 \
  case NVV:                                                                                   \
    gate_scores_fused_rows_kernel<T, NVV><<<(unsigned)grid, NT, 0, s>>>(                      \
        (const T*)scores, mult, mask_bits, (T*)rt, reinterpret_cast<uint8_t*>(tile_counts),   \
        compact_row_cells(E), (const T*)x, (const T*)last_bias, add_residual, (T*)out, N, d,  \
        E);                                                                                   \
    break;
  if (rows_form) {
    if (dtype == D2D_F32) {
      switch (row_bytes / 16) {
        D2D_ROWS_CASE(float, 1) D2D_ROWS_CASE(float, 2) D2D_ROWS_CASE(float, 3)
        D2D_ROWS_CASE(float, 4) D2D_ROWS_CASE(float, 5) D2D_ROWS_CASE(float, 6)
        D2D_ROWS_CASE(float, 7) D2D_ROWS_CASE(float, 8)
      }
    } else {
      switch (row_bytes / 16) {
        D2D_ROWS_CASE(bf16, 1) D2D_ROWS_CASE(bf16, 2) D2D_ROWS_CASE(bf16, 3)
        D2D_ROWS_CASE(bf16, 4) D2D_ROWS_CASE(bf16, 5) D2D_ROWS_CASE(bf16, 6)
        D2D_ROWS_CASE(bf16, 7) D2D_ROWS_CASE(bf16, 8)
      }
    }
    return cudaGetLastError() == cudaSuccess ? D2D_OK : D2D_ERR_LAUNCH;
  }
#undef D2D_ROWS_CASE
  if (dtype == D2D_F32)
    gate_scores_fused_kernel<float><<<(unsigned)grid, NT, 0, s>>>(
        (const float*)scores, mult, mask_bits, (float*)rt, reinterpret_cast<uint8_t*>(tile_counts),
        compact_row_cells(E), (const float*)x,
        (const float*)last_bias, add_residual, (float*)out, N, d, E);
  else
    gate_scores_fused_kernel<bf16><<<(unsigned)grid, NT, 0, s>>>(
        (const bf16*)scores, mult, mask_bits, (bf16*)rt, reinterpret_cast<uint8_t*>(tile_counts),
        compact_row_cells(E), (const bf16*)x,
        (const bf16*)last_bias, add_residual, (bf16*)out, N, d, E);
  return cudaGetLastError() == cudaSuccess ? D2D_OK : D2D_ERR_LAUNCH;
}

int launch_init_out(const void* x, const void* last_bias, int add_residual, void* out, int64_t N,
                    int d, int dtype, cudaStream_t s) {
  const int64_t total = N * d;
  const int V = dtype == D2D_F32 ? 4 : 8;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (d % V == 0 && al16(out) && al16(x) && al16(last_bias)) {
    const int grid = grid_for(total / V, NT * 4, 148 * 16);
    if (dtype == D2D_F32)
      init_out_vec_kernel<float><<<grid, NT, 0, s>>>((const float*)x, (const float*)last_bias,
                                                     add_residual, (float*)out, total / V, d / V);
    else
      init_out_vec_kernel<bf16><<<grid, NT, 0, s>>>((const bf16*)x, (const bf16*)last_bias,
                                                    add_residual, (bf16*)out, total / V, d / V);
    return cudaGetLastError() == cudaSuccess ? D2D_OK : D2D_ERR_LAUNCH;
  }
  const int grid = grid_for(total, NT * 8, 148 * 8);
  if (dtype == D2D_F32)
    init_out_kernel<float><<<grid, NT, 0, s>>>((const float*)x, (const float*)last_bias,
                                               add_residual, (float*)out, total, d);
  else
    init_out_kernel<bf16><<<grid, NT, 0, s>>>((const bf16*)x, (const bf16*)last_bias,
                                              add_residual, (bf16*)out, total, d);
  return cudaGetLastError() == cudaSuccess ? D2D_OK : D2D_ERR_LAUNCH;
}

int launch_pack_mask(const void* rt, uint32_t* mask_bits, int64_t N, int E, int dtype,
                     cudaStream_t s) {
  const int grid = grid_for(N, NT / 32, 148 * 8);
  if (dtype == D2D_F32)
    pack_mask_kernel<float><<<grid, NT, 0, s>>>((const float*)rt, mask_bits, N, E);
  else
    pack_mask_kernel<bf16><<<grid, NT, 0, s>>>((const bf16*)rt, mask_bits, N, E);
  return cudaGetLastError() == cudaSuccess ? D2D_OK : D2D_ERR_LAUNCH;
}

int launch_expand_mask(const uint32_t* mask_bits, void* rt, int64_t N, int E, int dtype,
                       cudaStream_t s) {
  const int64_t total = N * E;
  const int grid = grid_for(total, NT * 4, 148 * 8);
  if (dtype == D2D_F32)
    expand_mask_kernel<float><<<grid, NT, 0, s>>>(mask_bits, (float*)rt, total, E);
  else
    expand_mask_kernel<bf16><<<grid, NT, 0, s>>>(mask_bits, (bf16*)rt, total, E);
  return cudaGetLastError() == cudaSuccess ? D2D_OK : D2D_ERR_LAUNCH;
}

}  // namespace d2d
