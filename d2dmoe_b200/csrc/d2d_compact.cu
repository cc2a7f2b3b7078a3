// Bit mask -> per-expert token lists + offsets (warp-ballot / prefix-sum compaction).
//
// Replaces the upstream index preparation (architectures/moe/moe_layers.py:241-249:
// int32 cast of the routing tensor, argsort along the token dimension, column sums).
// The sort only serves to bring each expert's tokens to the front of its column;
// a compaction gives the same set per expert, here in ascending token order.
//
// Two launches:
//   count   : counts[tile][e] = tokens of the 128-token tile that keep expert e, one BYTE
//             per cell (a tile holds at most 128 tokens), rows padded to EP cells
//             (skipped when the router kernel already wrote the table)
//   scatter : one CTA per 256 tokens sweeps the byte table with 16-byte loads (sum over all
//             tiles = the expert totals, sum over earlier tiles = its own base), scans the
//             totals over the experts and writes its token indices.
// Every CTA reads the whole table, but at one byte per cell that is 12 KB for a ViT-B/16
// layer (394 tiles x 32) and 128 KB for 131072 tokens x 128 experts, out of L2.
// Integer work, bit-exact by construction; HBM traffic is the mask (read twice)
// plus 4 bytes per kept token-expert pair.
#include "d2d_common.cuh"

namespace d2d {
namespace {

constexpr int NT = 256;
constexpr int NTS = 256;                 // scatter CTA: one warp per row of 32 tokens
constexpr int ROWS = 8;                  // rows of 32 tokens per scatter CTA (one per warp)
constexpr int CHUNK = ROWS * 32;
constexpr int CTILE = 128;               // granularity of the counts table
constexpr int TILES_PER_CHUNK = CHUNK / CTILE;
constexpr int MAX_E = 256;

// one warp = one 128-token tile; lane b ends up with the count of expert 32j+b
__global__ void __launch_bounds__(NT)
compact_count_kernel(const uint32_t* __restrict__ mask_bits, uint8_t* __restrict__ counts,
                     int64_t N, int E, int EP) {
  const int lane = threadIdx.x & 31;
  const int64_t tile = (int64_t)blockIdx.x * (NT / 32) + (threadIdx.x >> 5);
  if (tile * CTILE >= N) return;
  const int nw = (E + 31) / 32;
  for (int j = 0; j * 32 < EP; ++j) {
    uint32_t w[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int64_t t = tile * CTILE + r * 32 + lane;
      w[r] = (t < N && j < nw) ? mask_bits[t * nw + j] : 0u;
    }
    int mine = 0;
    const int nb = max(0, min(32, E - 32 * j));
    for (int b = 0; b < nb; ++b) {
      int cb = 0;
#pragma unroll
      for (int r = 0; r < 4; ++r) cb += __popc(__ballot_sync(0xffffffffu, (w[r] >> b) & 1u));
      if (lane == b) mine = cb;
    }
    if (32 * j + lane < EP) counts[tile * EP + 32 * j + lane] = (uint8_t)mine;   // pads are 0
  }
}

__global__ void __launch_bounds__(NTS)
compact_scatter_kernel(const uint32_t* __restrict__ mask_bits, const uint8_t* __restrict__ counts,
                       int32_t* __restrict__ token_idx, int32_t* __restrict__ offsets, int64_t N,
                       int E, int EP, int ntiles, int* dev_status) {
  extern __shared__ int sm[];
  int* cnt = sm;                 // [ROWS][E] -> becomes each row's write base
  int* tot = cnt + ROWS * E;     // [EP]  total per expert, then exclusive offsets
  int* pre = tot + EP;           // [EP]  tokens of expert e in earlier chunks
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int nw = (E + 31) / 32;
  const int chunk = blockIdx.x;
  const int64_t t = (int64_t)chunk * CHUNK + w * 32 + lane;

  grid_launch_dependents();
  for (int i = tid; i < ROWS * E; i += NTS) cnt[i] = 0;
  for (int e = tid; e < 2 * EP; e += NTS) tot[e] = 0;      // tot and pre are adjacent
  __syncthreads();
  grid_dependency_wait();      // mask and counts table come from the previous kernel
  // this thread's mask words (warps 0..ROWS-1: one row of 32 tokens each); the loads are in
  // flight during the table sweep and the words stay in registers for both passes
  uint32_t word[MAX_E / 32];
#pragma unroll
  for (int j = 0; j < MAX_E / 32; ++j)
    word[j] = (w < ROWS && j < nw && t < N) ? mask_bits[t * nw + j] : 0u;
  // sweep of the byte table: thread (tsub, g) adds up the 16 cells of group g over the tiles
  // tsub, tsub + stride, ...; sums over all tiles and over the tiles before this chunk
  {
    const int G = EP >> 4;                      // 16-cell groups per table row (power of two)
    const int g = tid & (G - 1), tsub = tid / G, stride = NTS / G;
    const int first_tile = chunk * TILES_PER_CHUNK;
    int a[16], b[16];
#pragma unroll
    for (int q = 0; q < 16; ++q) a[q] = b[q] = 0;
    for (int t0 = tsub; t0 < ntiles; t0 += 4 * stride) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {      // four independent loads in flight
        const int tt = t0 + u * stride;
        v[u] = tt < ntiles ? __ldg(reinterpret_cast<const uint4*>(counts + (int64_t)tt * EP) + g)
                           : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t ww[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
        const bool before = t0 + u * stride < first_tile;
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          const int c = (ww[q >> 2] >> (8 * (q & 3))) & 0xff;
          a[q] += c;
          if (before) b[q] += c;
        }
      }
    }
    // lanes that hold the same group (lane mod G equal) are added up by shuffles, then one
    // lane per group and warp adds into shared memory
    for (int o = 16; o >= G; o >>= 1) {
#pragma unroll
      for (int q = 0; q < 16; ++q) {
        a[q] += __shfl_xor_sync(0xffffffffu, a[q], o);
        b[q] += __shfl_xor_sync(0xffffffffu, b[q], o);
      }
    }
    if (lane < G && lane < 32) {
#pragma unroll
      for (int q = 0; q < 16; ++q) {
        if (a[q]) atomicAdd(&tot[16 * g + q], a[q]);
        if (b[q]) atomicAdd(&pre[16 * g + q], b[q]);
      }
    }
  }
  // per-row popcounts of this chunk
#pragma unroll
  for (int j = 0; j < MAX_E / 32; ++j) {
    if (j >= nw || w >= ROWS) break;
    if (__ballot_sync(0xffffffffu, word[j] != 0u) == 0u) continue;
    const int nb = min(32, E - 32 * j);
    int mine = 0;
    for (int b = 0; b < nb; ++b) {
      const int cb = __popc(__ballot_sync(0xffffffffu, (word[j] >> b) & 1u));
      if (lane == b) mine = cb;
    }
    if (lane < nb) cnt[w * E + 32 * j + lane] = mine;
  }
  __syncthreads();
  // exclusive scan of the expert totals (E <= 256: one warp, 8 values per lane)
  if (w == 0) {
    int v[8], s = 0;
    for (int k = 0; k < 8; ++k) {
      const int e = lane * 8 + k;
      v[k] = e < E ? tot[e] : 0;
      s += v[k];
    }
    int incl = s;
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    int run = incl - s;
    for (int k = 0; k < 8; ++k) {
      const int e = lane * 8 + k;
      if (e < E) tot[e] = run;
      run += v[k];
    }
    if (lane == 31) {
      if (chunk == 0) offsets[E] = incl;
      if ((int64_t)incl > N * (int64_t)E) report(dev_status, D2D_ERR_INDEX_RANGE);
    }
  }
  __syncthreads();
  for (int e = tid; e < E; e += NTS) {
    if (chunk == 0) offsets[e] = tot[e];
    int run = tot[e] + pre[e];
    for (int row = 0; row < ROWS; ++row) {
      const int c = cnt[row * E + e];
      cnt[row * E + e] = run;
      run += c;
    }
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < MAX_E / 32; ++j) {
    if (j >= nw || w >= ROWS) break;
    if (__ballot_sync(0xffffffffu, word[j] != 0u) == 0u) continue;
    const int nb = min(32, E - 32 * j);
    for (int b = 0; b < nb; ++b) {
      const uint32_t bit = (word[j] >> b) & 1u;
      const uint32_t v = __ballot_sync(0xffffffffu, bit);
      if (bit) {
        const int rank = __popc(v & ((1u << lane) - 1u));
        token_idx[cnt[w * E + 32 * j + b] + rank] = (int32_t)t;
      }
    }
  }
}

}  // namespace

// cells per row of the byte table: the next power of two >= E, at least 16 (rows are read
// in 16-byte groups; a power of two lets one warp's lanes split into equal groups)
int compact_row_cells(int E) {
  int ep = 16;
  while (ep < E) ep <<= 1;
  return ep;
}

// the byte table needs ntiles * EP bytes; this (four bytes per tile and expert) is what
// d2d_workspace_bytes has always reported and covers it for every E
size_t compact_workspace_bytes(int64_t n_max, int E) {
  const int64_t ntiles = ceil_div64(n_max > 0 ? n_max : 1, CTILE);
  return (size_t)(ntiles + 1) * (size_t)E * sizeof(int32_t);
}

int launch_compact(const uint32_t* mask_bits, int32_t* token_idx, int32_t* offsets, int64_t N,
                   int E, int32_t* counts_ws, int* dev_status, cudaStream_t s,
                   bool counts_ready) {
  if (E > MAX_E || E < 1) return D2D_ERR_UNSUPPORTED;
  if (N * (int64_t)E > 0x7fffffffLL) return D2D_ERR_UNSUPPORTED;   // int32 offsets
  if (N == 0) {
    // no tokens: every list is empty; no kernel reads the (unwritten) counts table
    return cudaMemsetAsync(offsets, 0, sizeof(int32_t) * ((size_t)E + 1), s) == cudaSuccess
               ? D2D_OK
               : D2D_ERR_LAUNCH;
  }
  const int EP = compact_row_cells(E);
  const int64_t ntiles = ceil_div64(N, CTILE);
  const int64_t nchunks = ceil_div64(N, CHUNK);
  uint8_t* counts = reinterpret_cast<uint8_t*>(counts_ws);
  if (!counts_ready) {
    compact_count_kernel<<<(unsigned)ceil_div64(ntiles, NT / 32), NT, 0, s>>>(mask_bits, counts, N,
                                                                             E, EP);
    if (cudaGetLastError() != cudaSuccess) return D2D_ERR_LAUNCH;
  }
  const size_t smem = sizeof(int) * ((size_t)ROWS * E + 2 * (size_t)EP);
  return launch_pdl(compact_scatter_kernel, dim3((unsigned)nchunks), dim3(NTS), smem, s, mask_bits,
                    (const uint8_t*)counts, token_idx, offsets, N, E, EP, (int)ntiles, dev_status);
}

}  // namespace d2d

// ---------------------------------------------------------------------------
// Compaction for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to hand over a workspace: a plugin slot
// that passes only the operator's inputs and outputs, a runtime whose memory pool
// is frozen after start-up, or a latency-critical loop that must never enter the
// driver's allocator.  For them the counts
// table lives in the library itself, in a fixed device array that every GPU
// loading the library holds until the process exits.
//
// Limit: D2D_NOALLOC_MAX_CELLS table cells = ceil(N/128) * E (1 MiB); e.g. 262144
// tokens x 128 experts, or 1M tokens x 32 experts.  Larger requests are refused with
// D2D_ERR_SCRATCH_LIMIT before anything is launched.
//
// The table is shared by every call in the process and keeps the previous call's
// contents.  Nothing in it needs clearing: for N > 0 the count kernel writes every cell
// (padding included) of each of the ceil(N/128) tile rows and the scatter kernel reads
// nothing else; for N = 0 no kernel touches the table (the offsets are simply set to zero).
// Two calls that run concurrently on one GPU (different streams) would overwrite
// each other's counts: keep such calls on one stream or order them with events.
// ---------------------------------------------------------------------------
#define D2D_NOALLOC_MAX_CELLS (2048 * 128)

static __device__ __align__(256) int32_t g_noalloc_counts[D2D_NOALLOC_MAX_CELLS];

namespace {

constexpr int kMaxDevices = 64;
int32_t* g_noalloc_ptr[kMaxDevices] = {nullptr};   // per device: address of the array there

// Device address of g_noalloc_counts on the current device.  In host code the
// array's name is only a handle for the runtime, not an address a kernel may use;
// the address comes from cudaGetSymbolAddress, asked once per device while that
// device is current.
int noalloc_scratch(int32_t** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return D2D_ERR_NO_DEVICE;
  int32_t* p = __atomic_load_n(&g_noalloc_ptr[dev], __ATOMIC_ACQUIRE);
  if (!p) {
    void* sym = nullptr;
    if (cudaGetSymbolAddress(&sym, g_noalloc_counts) != cudaSuccess || !sym) {
      cudaGetLastError();
      return D2D_ERR_NO_DEVICE;
    }
    p = static_cast<int32_t*>(sym);
    __atomic_store_n(&g_noalloc_ptr[dev], p, __ATOMIC_RELEASE);
  }
  *out = p;
  return D2D_OK;
}

}  // namespace

extern "C" int d2d_compact_noalloc(const uint32_t* mask_bits, int32_t* token_idx, int32_t* offsets,
                                   int64_t N, int E, int* dev_status, d2d_stream_t stream) {
  if (!mask_bits || !token_idx || !offsets || N < 0 || E < 1) return D2D_ERR_BAD_ARG;
  const int64_t ntiles = d2d::ceil_div64(N > 0 ? N : 1, d2d::CTILE);
  // documented limit, and the table's actual bytes (rows are padded to at least 16 cells)
  if (ntiles * (int64_t)E > D2D_NOALLOC_MAX_CELLS ||
      ntiles * (int64_t)d2d::compact_row_cells(E > 0 && E <= 256 ? E : 256) >
          (int64_t)sizeof(int32_t) * D2D_NOALLOC_MAX_CELLS)
    return D2D_ERR_SCRATCH_LIMIT;
  int32_t* counts = nullptr;
  const int rc = noalloc_scratch(&counts);   // first call on a device looks the address up
  if (rc != D2D_OK) return rc;
  return d2d::launch_compact(mask_bits, token_idx, offsets, N, E, counts, dev_status,
                             (cudaStream_t)stream, false);
}
