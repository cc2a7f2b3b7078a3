// bf16 tensor-core path (tcgen05 + TMEM) of the two MLP-shaped stages of the layer:
//
//   experts : per (expert e, 128 rows of its token list)
//               h   = act(bf16(x[rows] W1[e]) + b1[e]) (* bf16(x[rows] W_up[e]))
//               out[rows] += bf16(h W2[e])               red.global.add bf16x2
//             fusing architectures/moe/moe_impls.py:93-180 (gathered first layer) and
//             :244-301 (second layer + atomic add); h never leaves the SM.
//   router  : per 128 consecutive tokens
//               s = |bf16(relu(bf16(x Wa^T)) Wb^T)|, keep e iff s_e >= bf16(max s * mult)
//             (architectures/moe/moefication.py:328-330 and :80-85), written as mask
//             bits (and, on request, as the 0/1 routing tensor); the same CTA writes the
//             layer output's initial value and the compaction's counts table.
//
// Both are one persistent kernel (one CTA per SM: 480 threads in the router form, 608 in
// the experts form; tile = 128 rows): GEMM1 (K = d) into a double-buffered TMEM accumulator,
// an epilogue that turns it into the bf16 A operand of GEMM2 in shared memory, GEMM2
// (K = hidden width) per 128-column chunk into a second double-buffered TMEM accumulator,
// and a second epilogue.
//
// Warp roles:
//   experts form
//     warps 0-3   epilogue 1: accumulator 1 -> + b1, activation (x up-projection) -> hidden tile
//     warps 4-7   accumulator 2 -> bf16 -> two alternating 4 KB staging blocks per warp
//     warps 15-18 read the blocks back row-contiguous and add them to out[token] with
//                 red.global.add.noftz.v4.bf16x2 (4 cache lines per instruction)
//     warps 11-14 gather the tile's token rows of x with 16-byte cp.async into ring A in the
//                 128-byte-swizzled K-major layout the MMA descriptors expect; stage barriers
//                 are signalled by cp.async.mbarrier.arrive.  (Selectable instead: warp 11
//                 gathers them with TMA tile::gather4 copies, four rows per copy.)
//   router form
//     warps 0-7   two epilogue groups of four: epilogue 1 (ReLU hidden tile), then group 0:
//                 |.|, row max, threshold, mask word, the row of the 0/1 routing tensor,
//                 per-tile expert counts for the compaction; warp 7 issues the output's
//                 initial rows as TMA row stores
//     warp 11     one lane issues one tiled TMA box (128 rows x 64 columns of x) per stage
//   both
//     warp  8     TMEM allocation; one thread issues the GEMM1 stream (tcgen05.mma / commit)
//     warp  9     one thread issues the GEMM2 stream on its own weight ring
//     warp 10     one thread streams packed weight tiles with cp.async.bulk (TMA, 1-D) into
//                 the two weight rings, whichever has a free stage
// Weights are packed once (d2d_prepack_*) into exactly the shared-memory images the
// MMA reads, so a weight tile is one contiguous bulk copy.  No multicast loads.
//
// Every wait is bounded: when one runs out the kernel records D2D_ERR_TIMEOUT in the
// status word, all roles leave their loops, TMEM is freed and the kernel returns.
#include <atomic>
#include <mutex>

#include "d2d_tmap.cuh"
#include "d2d_umma_api.cuh"
#include "d2d_umma_ptx.cuh"

namespace d2d {
using namespace umma;
namespace {

constexpr int NA_MAX = 6;            // ring A stages (upper bound)
constexpr int NB_MAX = 6;            // ring B stages (upper bound)
constexpr int SLOTS_TOTAL = 14;      // ring A + ring B + hidden tile + staging (224 KB)
constexpr int NTHREADS = 480;            // router form
constexpr int NTHREADS_EXPERTS = 608;    // + four warps that write the output rows
constexpr int WARP_MMA1 = 8, WARP_MMA2 = 9, WARP_BULK = 10, WARP_PROD0 = 11, WARP_WR0 = 15;
constexpr int MAX_E = 128;
constexpr int MODE_EXPERTS = 0, MODE_ROUTER = 1;

struct Geo {
  int kc1;       // d / 64
  int nsub;      // weight subtiles per k-chunk of GEMM1 (gate/up, or two halves of a wide router)
  int nsubw;     // columns per subtile (<= 128, multiple of 16)
  int K2;        // GEMM2 reduction = hidden width held in shared memory
  int kc2;       // ceil(K2 / 64)
  int nd;        // GEMM2 output columns per chunk (<= 128, multiple of 16)
  int nc;        // number of chunks
  int nb;        // ring B1 stages (W1 tiles, consumed by the GEMM1 warp)
  int nb2;       // ring B2 stages (W2 pieces, consumed by the GEMM2 warp)
  int na;        // ring A stages
  int stg;       // 16 KB slots of epilogue staging (experts: 2 = 32 rows x 128 B per warp)
  long long w1_bytes, bias_off, stride;   // packed layout per expert
};

struct Params {
  const bf16* x;
  long long N;
  int d;
  const uint8_t* packed;
  Geo g;
  // experts
  const int32_t* token_idx;
  const int32_t* offsets;
  int E;
  bf16* out;
  int act, glu;
  // router
  float mult;
  uint32_t* mask_bits;
  bf16* scores;
  bf16* rt_out;             // optional: 0/1 routing tensor [N, E]
  const bf16* last_bias;
  int add_residual;
  bf16* out_init;
  uint8_t* tile_counts;     // [tiles][EP] bytes: per-expert kept-token counts of each 128-token tile
  int EP;                   // cells per table row (compact_row_cells(E))
  int* dev_status;
  uint32_t wait_limit;      // polls per bounded wait
  int withhold;             // test hook: CTA 0 never loads its first weight tile
  int tma_gather;           // experts: rows by TMA tile::gather4 instead of cp.async
  bf16* norms;              // experts, optional: [E, N] norms of each computed pair's activations
  int norm_layer, norm_ord; // D2D_NORM_OF_INTERMEDIATE / D2D_NORM_OF_OUTPUT (0: none); 1 or 2
};

Geo experts_geo(int d, int H, bool glu) {
  Geo g;
  g.kc1 = d / 64;
  g.nsub = glu ? 2 : 1;
  g.nsubw = H;
  g.K2 = H;
  g.kc2 = (H + 63) / 64;
  g.nd = (d % 128 == 0) ? 128 : 64;
  g.nc = d / g.nd;
  g.stg = 2;                       // 8 epilogue warps x 4 KB
  g.na = 4;
  g.nb = glu ? 4 : 3;
  g.nb2 = min(NB_MAX, SLOTS_TOTAL - g.na - g.nb - g.kc2 - g.stg);
  g.w1_bytes = (long long)g.kc1 * g.nsub * g.nsubw * 128;
  g.bias_off = g.w1_bytes + (long long)g.nc * g.kc2 * g.nd * 128;
  g.stride = (g.bias_off + 512 + 1023) / 1024 * 1024;
  return g;
}

Geo router_geo(int d, int R, int E) {
  Geo g;
  g.kc1 = d / 64;
  g.nsub = R > 128 ? 2 : 1;
  g.nsubw = R / g.nsub;
  g.K2 = R;
  g.kc2 = (R + 63) / 64;
  g.nd = (E + 15) / 16 * 16;
  g.nc = 1;
  g.stg = 1;                       // one slot holds the last_bias row for the TMA row stores
  g.na = g.kc2 > 2 ? 4 : 5;
  g.nb = 4;
  g.nb2 = min(NB_MAX, SLOTS_TOTAL - g.na - g.nb - g.kc2 - g.stg);
  g.w1_bytes = (long long)g.kc1 * g.nsub * g.nsubw * 128;
  g.bias_off = g.w1_bytes + (long long)g.nc * g.kc2 * g.nd * 128;
  g.stride = (g.bias_off + 512 + 1023) / 1024 * 1024;
  return g;
}

// ---------------------------------------------------------------------------
// shared-memory bookkeeping
// ---------------------------------------------------------------------------
struct Ctl {
  unsigned long long fullA[NA_MAX], emptyA[NA_MAX], fullB[NB_MAX], emptyB[NB_MAX];
  unsigned long long fullB2[NB_MAX], emptyB2[NB_MAX];
  unsigned long long acc1_full[2], acc1_empty[2], hs_full, hs_empty, acc2_full[2], acc2_empty[2];
  unsigned long long sfull[2][4], sempty[2][4];   // staging unit of (epilogue group, row quarter)
  uint32_t tmem_base;
  int abort_flag;
  int wait_limit;                  // must follow abort_flag (mbar_wait reads abort_flag[1])
  int total_tiles;
  alignas(16) float bias_s[128];   // (read as float4) b1 of the current tile's expert
  int total_full;                  // experts: number of full 128-row tiles (they come first)
  int dense_tpe;                   // experts: > 0 = every expert lists all N tokens: tiles per expert
  uint8_t pidx[MAX_E];             // experts: expert of the k-th partial (tail) tile
  union {
    int tstart[MAX_E + 1];  // experts: first FULL tile of each expert
    int tile_cnt[MAX_E];    // router: per-expert counts of the current tile
  };
};

struct Tile {
  int e, r0, nrows;
};

template <int MODE>
__device__ __forceinline__ Tile tile_info(const Params& p, const Ctl* c, int tile) {
  Tile t;
  if (MODE == MODE_ROUTER) {
    t.e = 0;
    t.r0 = tile * TILE_M;
    t.nrows = (int)min((long long)TILE_M, p.N - (long long)t.r0);
  } else {
    // Every expert runs on every token (mode 'all' upstream: router training, label capture):
    // token-tile-major order, the E tiles of one 128-token window next to each other, so that
    // the window's rows of x and out are read from and added to in L2 instead of being
    // streamed through DRAM once per expert.
    if (c->dense_tpe > 0) {
      const int j = tile / p.E;
      t.e = tile - j * p.E;
      t.r0 = p.offsets[t.e] + j * TILE_M;
      t.nrows = (int)min((long long)TILE_M, p.N - (long long)j * TILE_M);
      return t;
    }
    // Tile order: every full 128-row tile (expert-major), then the experts' partial tail
    // tiles.  With the static round-robin over CTAs the last, incomplete round of a launch
    // is then made of the cheap partial tiles.
    if (tile < c->total_full) {
      int lo = 0, hi = p.E;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (c->tstart[mid] <= tile) lo = mid; else hi = mid;
      }
      t.e = lo;
      t.r0 = p.offsets[lo] + (tile - c->tstart[lo]) * TILE_M;
      t.nrows = TILE_M;
    } else {
      t.e = c->pidx[tile - c->total_full];
      const int n = p.offsets[t.e + 1] - p.offsets[t.e];
      t.r0 = p.offsets[t.e] + (n / TILE_M) * TILE_M;
      t.nrows = n % TILE_M;
    }
  }
  return t;
}

// With one weight subtile per k-chunk (nsub == 1) the first accumulator is double
// buffered and GEMM1 of the next tile is issued before GEMM2 of the current one, so the
// tensor pipe works while the epilogue warps turn acc1 into the hidden tile.
__device__ __forceinline__ bool lookahead(const Geo& g) { return g.nsub == 1; }

// ---------------------------------------------------------------------------
// roles
// ---------------------------------------------------------------------------
// Ring A producer of the expert form, default path (four warps): the rows of the tile's
// token list by 16-byte cp.async (4 rows x 128 bytes per warp instruction, software
// swizzle); the stage barrier is signalled by cp.async.mbarrier.arrive.  Measured against
// the TMA gather below on the ViT-B/16 layer: 61 vs 101 us per launch, so this is the path
// that runs.
__device__ void role_producer_cpasync(const Params& p, Ctl* c, uint32_t ringA, int pt) {
  constexpr int MODE = MODE_EXPERTS;
  const int lane = pt & 31, pw = pt >> 5;
  const int j = lane & 7;
  uint32_t dstoff[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = pw * 32 + i * 4 + (lane >> 3);
    dstoff[i] = (row >> 3) * 1024 + (row & 7) * 128 + ((j ^ (row & 7)) << 4);
  }
  volatile int* af = &c->abort_flag;
  uint32_t s = 0, ph = 0;
  for (int tile = blockIdx.x; tile < c->total_tiles; tile += gridDim.x) {
    const Tile t = tile_info<MODE>(p, c, tile);
    const bf16* src[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int row = pw * 32 + i * 4 + (lane >> 3);
      row = min(row, t.nrows - 1);      // rows past the tail repeat the last row; masked later
      long long tok = p.token_idx[t.r0 + row];
      if (tok < 0 || tok >= p.N) {
        report(p.dev_status, D2D_ERR_INDEX_RANGE);
        tok = 0;
      }
      src[i] = p.x + tok * p.d + j * 8;
    }
    for (int kc = 0; kc < p.g.kc1; ++kc) {
      if (!mbar_wait_fast(smem_u32(&c->emptyA[s]), ph ^ 1, af, p.dev_status)) return;
      const uint32_t base = ringA + s * SLOT;
#pragma unroll
      for (int i = 0; i < 8; ++i) cp_async16(base + dstoff[i], src[i] + kc * 64);
      cp_async_arrive_noinc(smem_u32(&c->fullA[s]));
      if (++s == (uint32_t)p.g.na) {
        s = 0;
        ph ^= 1;
      }
    }
  }
}

// Ring A producer by TMA (one warp): the tile's rows of x into the 128-byte-swizzled K-major
// stage the MMA descriptor describes, 64 columns (128 bytes per row) per stage.
//   router:  rows are consecutive: one lane issues one 128-row box per stage; rows past the
//            last token arrive as zeros.
//   experts: (selectable, slower than the cp.async gather: the TMA unit spends a request per
//            128-byte row) lane l gathers rows 4l..4l+3 of the tile with one tile::gather4
//            copy (four token indices -> four consecutive 128-byte rows, 512 bytes per lane).
// Lane 0 posts the stage's 16 KB on its barrier; the copies complete on it.
template <int MODE>
__device__ void role_producer(const Params& p, Ctl* c, const CUtensorMap* tmx, uint32_t ringA,
                              int lane) {
  volatile int* af = &c->abort_flag;
  uint32_t s = 0, ph = 0;
  for (int tile = blockIdx.x; tile < c->total_tiles; tile += gridDim.x) {
    const Tile t = tile_info<MODE>(p, c, tile);
    int tok[4] = {0, 0, 0, 0};
    if (MODE == MODE_EXPERTS) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = min(4 * lane + i, t.nrows - 1);   // rows past the tail repeat the last row
        tok[i] = p.token_idx[t.r0 + row];
        if (tok[i] < 0 || tok[i] >= p.N) {
          report(p.dev_status, D2D_ERR_INDEX_RANGE);
          tok[i] = 0;
        }
      }
    }
    for (int kc = 0; kc < p.g.kc1; ++kc) {
      if (!mbar_wait_fast(smem_u32(&c->emptyA[s]), ph ^ 1, af, p.dev_status)) return;
      const uint32_t bar = smem_u32(&c->fullA[s]);
      if (lane == 0) mbar_arrive_expect_tx(bar, SLOT);
      if (MODE == MODE_EXPERTS) {
        tma_gather4(ringA + s * SLOT + lane * 512, tmx, kc * 64, tok[0], tok[1], tok[2], tok[3],
                    bar);
      } else if (lane == 0) {
        tma_load_2d(ringA + s * SLOT, tmx, kc * 64, t.r0, bar);
      }
      if (++s == (uint32_t)p.g.na) {
        s = 0;
        ph ^= 1;
      }
    }
  }
}

// The three issuing roles below (weight loads, GEMM1, GEMM2) each run in ONE thread of
// their warp for the whole launch: their loops are chains of dependent instructions, so
// warp votes, elections and re-convergence per k-chunk only lengthen the chain.

// Weight tiles for both rings.  The two streams (W1 tiles for the GEMM1 thread, W2 pieces
// for the GEMM2 thread) advance independently: whichever ring has a free stage gets its
// next tile, so neither GEMM waits for the other's weights.
template <int MODE>
__device__ void role_bulk(const Params& p, Ctl* c, uint32_t ringB, uint32_t ringB2) {
  volatile int* af = &c->abort_flag;
  const Geo& g = p.g;
  const uint32_t b1 = g.nsubw * 128, b2 = g.nd * 128;
  const int n1 = g.kc1 * g.nsub, n2 = g.nc * g.kc2;
  const int step = gridDim.x, total = c->total_tiles;
  const uint32_t fullB = smem_u32(c->fullB), emptyB = smem_u32(c->emptyB);
  const uint32_t fullB2 = smem_u32(c->fullB2), emptyB2 = smem_u32(c->emptyB2);
  RingPos r1 = {0, 0}, r2 = {0, 0};
  int t1 = blockIdx.x, t2 = blockIdx.x, j1 = 0, j2 = 0;
  const uint8_t *pe1 = nullptr, *pe2 = nullptr;
  if (t1 < total) pe1 = pe2 = p.packed + (long long)tile_info<MODE>(p, c, t1).e * g.stride;
  uint32_t idle = 0;
  bool withheld = (p.withhold & 1) != 0 && blockIdx.x == 0;
  while (t1 < total || t2 < total) {
    bool progress = false;
    if (t1 < total && mbar_test_wait(emptyB + 8 * r1.s, r1.ph ^ 1)) {
      const uint32_t bar = fullB + 8 * r1.s;
      if (withheld) {
        withheld = false;      // test hook: this stage never fills, its consumer's wait runs out
      } else {
        mbar_arrive_expect_tx(bar, b1);
        bulk_g2s(ringB + r1.s * SLOT, pe1 + (long long)j1 * b1, b1, bar);
      }
      r1.next(g.nb);
      if (++j1 == n1) {
        j1 = 0;
        t1 += step;
        if (t1 < total) pe1 = p.packed + (long long)tile_info<MODE>(p, c, t1).e * g.stride;
      }
      progress = true;
    }
    if (t2 < total && mbar_test_wait(emptyB2 + 8 * r2.s, r2.ph ^ 1)) {
      const uint32_t bar = fullB2 + 8 * r2.s;
      mbar_arrive_expect_tx(bar, b2);
      bulk_g2s(ringB2 + r2.s * SLOT, pe2 + g.w1_bytes + (long long)j2 * b2, b2, bar);
      r2.next(g.nb2);
      if (++j2 == n2) {
        j2 = 0;
        t2 += step;
        if (t2 < total) pe2 = p.packed + (long long)tile_info<MODE>(p, c, t2).e * g.stride;
      }
      progress = true;
    }
    if (progress) {
      idle = 0;
    } else {
      if (++idle > 64) __nanosleep(idle > 4096 ? 256 : 32);
      if ((idle & 63) == 0 && *af != 0) return;
      if (idle >= p.wait_limit) {
        *af = 1;
        report(p.dev_status, D2D_ERR_TIMEOUT);
        return;
      }
    }
  }
}

// GEMM1 stream: acc1[buffer][sub] = A(rows, d) * W1sub(d, nsubw), one tile after another.
// Only the low word of a shared-memory descriptor changes with the stage and the k-step
// (16-byte units: one slot = 1024, one k-step of 16 elements = 2).
template <int MODE>
__device__ void role_mma1(const Params& p, Ctl* c, uint32_t ringA, uint32_t ringB,
                          uint32_t tmem) {
  volatile int* af = &c->abort_flag;
  const Geo& g = p.g;
  const uint32_t idesc1 = instr_desc(TILE_M, g.nsubw);
  const uint64_t dA = smem_desc(ringA), dB = smem_desc(ringB);
  const uint32_t hi = (uint32_t)(dA >> 32), alo0 = (uint32_t)dA, blo0 = (uint32_t)dB;
  const uint32_t fullA = smem_u32(c->fullA), emptyA = smem_u32(c->emptyA);
  const uint32_t fullB = smem_u32(c->fullB), emptyB = smem_u32(c->emptyB);
  const bool la = lookahead(g), two = g.nsub == 2;
  const uint32_t na = g.na, nb = g.nb;
  const int kc1 = g.kc1, total = c->total_tiles;
  uint32_t sa = 0, pha = 0, sb = 0, phb = 0, i = 0;
  for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++i) {
    const uint32_t b = la ? (i & 1) : 0;
    const uint32_t use = la ? (i >> 1) : i;              // how often this buffer was used
    const uint32_t acc = tmem + (la ? b * 128 : 0);
    // the epilogue warps must have read the previous contents of this buffer
    if (!mbar_wait_fast(smem_u32(&c->acc1_empty[b]), (use & 1) ^ 1, af, p.dev_status)) return;
    tc_fence_after();
    for (int kc = 0; kc < kc1; ++kc) {
      const uint32_t alo = alo0 + sa * (SLOT >> 4), blo = blo0 + sb * (SLOT >> 4);
      if (!mbar_wait_fast(fullA + 8 * sa, pha, af, p.dev_status)) return;
      if (!mbar_wait_fast(fullB + 8 * sb, phb, af, p.dev_status)) return;
      tc_fence_after();
#pragma unroll
      for (uint32_t k = 0; k < 4; ++k)
        umma_bf16(acc, ((uint64_t)hi << 32) | (alo + 2 * k), ((uint64_t)hi << 32) | (blo + 2 * k),
                  idesc1, (kc | k) != 0);
      umma_commit(emptyB + 8 * sb);
      if (++sb == nb) {
        sb = 0;
        phb ^= 1;
      }
      if (two) {
        const uint32_t blo1 = blo0 + sb * (SLOT >> 4);
        if (!mbar_wait_fast(fullB + 8 * sb, phb, af, p.dev_status)) return;
        tc_fence_after();
#pragma unroll
        for (uint32_t k = 0; k < 4; ++k)
          umma_bf16(acc + 128, ((uint64_t)hi << 32) | (alo + 2 * k),
                    ((uint64_t)hi << 32) | (blo1 + 2 * k), idesc1, (kc | k) != 0);
        umma_commit(emptyB + 8 * sb);
        if (++sb == nb) {
          sb = 0;
          phb ^= 1;
        }
      }
      umma_commit(emptyA + 8 * sa);
      if (++sa == na) {
        sa = 0;
        pha ^= 1;
      }
    }
    umma_commit(smem_u32(&c->acc1_full[b]));
  }
}

// GEMM2 stream: acc2[chunk & 1] = Hs(rows, K2) * W2chunk(K2, nd) for every chunk of a tile.
template <int MODE>
__device__ void role_mma2(const Params& p, Ctl* c, uint32_t ringB2, uint32_t hs,
                          uint32_t tmem) {
  volatile int* af = &c->abort_flag;
  const Geo& g = p.g;
  const uint32_t idesc2 = instr_desc(TILE_M, g.nd);
  const uint64_t dB = smem_desc(ringB2), dH = smem_desc(hs);
  const uint32_t hi = (uint32_t)(dB >> 32), blo0 = (uint32_t)dB, hlo0 = (uint32_t)dH;
  const uint32_t fullB2 = smem_u32(c->fullB2), emptyB2 = smem_u32(c->emptyB2);
  const uint32_t nb2 = g.nb2;
  const int nc = g.nc, kc2 = g.kc2, total = c->total_tiles;
  uint32_t s = 0, ph = 0, accbits = 0, i = 0;
  for (int tile = blockIdx.x; tile < total; tile += gridDim.x, ++i) {
    if (!mbar_wait_fast(smem_u32(&c->hs_full), i & 1, af, p.dev_status)) return;
    tc_fence_after();
    for (int nci = 0; nci < nc; ++nci) {
      const uint32_t buf = nci & 1;
      const uint32_t acc = tmem + 256 + buf * 128;
      for (int k2 = 0; k2 < kc2; ++k2) {
        const uint32_t blo = blo0 + s * (SLOT >> 4), hlo = hlo0 + k2 * (SLOT >> 4);
        if (!mbar_wait_fast(fullB2 + 8 * s, ph, af, p.dev_status)) return;
        if (k2 == 0) {
          if (!mbar_wait_fast(smem_u32(&c->acc2_empty[buf]), ((accbits >> buf) & 1) ^ 1, af,
                              p.dev_status))
            return;
          accbits ^= 1u << buf;
        }
        tc_fence_after();
        const int ksteps = min(4, (g.K2 - k2 * 64) >> 4);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (k < ksteps)
            umma_bf16(acc, ((uint64_t)hi << 32) | (hlo + 2 * k), ((uint64_t)hi << 32) | (blo + 2 * k),
                      idesc2, (k2 | k) != 0);
        umma_commit(emptyB2 + 8 * s);
        if (++s == nb2) {
          s = 0;
          ph ^= 1;
        }
      }
      umma_commit(smem_u32(&c->acc2_full[buf]));
    }
    umma_commit(smem_u32(&c->hs_empty));
  }
}

// Router form, 16 hidden columns of epilogue 1: relu(T(x Wa^T)) as 8 packed bf16 pairs
__device__ __forceinline__ void ep1_router_pairs(const uint32_t* v, uint32_t* w) {
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    __nv_bfloat162 h =
        __floats2bfloat162_rn(__uint_as_float(v[2 * q]), __uint_as_float(v[2 * q + 1]));
    h = __hmax2(h, __float2bfloat162_rn(0.f));
    w[q] = *reinterpret_cast<uint32_t*>(&h);
  }
}

// Router form, epilogue warps: 8 warps in two groups.  Warp w reads TMEM lanes
// 32*(w%4)..+31 (= tile rows); group w/4 takes every other 16-column block of epilogue 1;
// group 0 then turns the scores into mask words and counts.
__device__ void role_epilogue_router(const Params& p, Ctl* c, uint32_t hs, uint32_t stg,
                                     uint32_t tmem, int et) {
  constexpr int MODE = MODE_ROUTER;
  volatile int* af = &c->abort_flag;
  const Geo& g = p.g;
  const int lane = et & 31, w8 = et >> 5, grp = w8 >> 2;
  const int r = et & 127;                                   // tile row = TMEM lane
  const uint32_t lane_base = (uint32_t)(r & ~31) << 16;
  const uint32_t hs_row = hs + (r >> 3) * 1024 + (r & 7) * 128;
  const bool la = lookahead(g);
  uint32_t i = 0, ph_mine = 0;
  // Without residual: every token's initial output is the same row (last_bias or
  // zeros).  Keep that row in shared memory and let the TMA engine write it once per
  // token, instead of spending the epilogue warps' store bandwidth on it.
  const bool tma_init = p.out_init && !p.add_residual && p.d * 2 <= SLOT;
  if (tma_init) {
    for (int c8 = et; c8 < (p.d >> 3); c8 += 256) {
      uint4 bz = make_uint4(0u, 0u, 0u, 0u);
      if (p.last_bias) bz = __ldg(reinterpret_cast<const uint4*>(p.last_bias) + c8);
      st_shared_v4(stg + c8 * 16, bz.x, bz.y, bz.z, bz.w);
    }
    fence_proxy_async();
    asm volatile("bar.sync 4, 256;" ::: "memory");
  }
  for (int tile = blockIdx.x; tile < c->total_tiles; tile += gridDim.x, ++i) {
    const Tile t = tile_info<MODE>(p, c, tile);
    if (tma_init) {
      if (w8 == 7) {
        for (int row = lane; row < t.nrows; row += 32)
          bulk_s2g(p.out_init + ((long long)t.r0 + row) * p.d, stg, (uint32_t)p.d * 2);
        bulk_commit();
      }
    } else if (p.out_init) {
      // initial value of the layer output for this tile's tokens: last_bias (+ x).
      // Lane = one 16-byte column piece (kept in a register), rows of this warp inside.
      const int v8 = p.d >> 3;
      for (int c8 = lane; c8 < v8; c8 += 32) {
        uint4 bz = make_uint4(0u, 0u, 0u, 0u);
        if (p.last_bias) bz = __ldg(reinterpret_cast<const uint4*>(p.last_bias) + c8);
#pragma unroll 4
        for (int row = w8; row < t.nrows; row += 8) {
          const long long rowoff = ((long long)t.r0 + row) * p.d;
          uint4 o = bz;
          if (p.add_residual) {
            const uint4 xv = *(reinterpret_cast<const uint4*>(p.x + rowoff) + c8);
            const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&bz);
            const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&xv);
            uint32_t ww[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 fa = __bfloat1622float2(a[q]), fb = __bfloat1622float2(b[q]);
              ww[q] = pack_bf16x2(fa.x + fb.x, fa.y + fb.y);
            }
            o = make_uint4(ww[0], ww[1], ww[2], ww[3]);
          }
          *(reinterpret_cast<uint4*>(p.out_init + rowoff) + c8) = o;
        }
      }
    }
    // ---- epilogue 1: acc1 -> bf16 hidden tile in shared memory ------------------
    const uint32_t b1 = la ? (i & 1) : 0;
    const uint32_t acc1 = tmem + lane_base + (la ? b1 * 128 : 0);
    if (!mbar_wait_fast(smem_u32(&c->acc1_full[b1]), la ? ((i >> 1) & 1) : (i & 1), af,
                        p.dev_status))
      return;
    if (!mbar_wait_fast(smem_u32(&c->hs_empty), (i & 1) ^ 1, af, p.dev_status)) return;
    tc_fence_after();
    const int nblk = g.nsubw >> 4;
    for (int bi = grp; bi < g.nsub * nblk; bi += 2) {
      const int sub = bi / nblk, c0 = (bi - sub * nblk) << 4;
      uint32_t v[16], w[8];
      tmem_ld16(acc1 + sub * 128 + c0, v);
      tmem_wait_ld();
      ep1_router_pairs(v, w);
      const int hc = sub * g.nsubw + c0;          // hidden column of v[0]
      const uint32_t base = hs_row + (hc >> 6) * SLOT;
      const int j0 = (hc & 63) >> 3;
      st_shared_v4(base + (((j0) ^ (r & 7)) << 4), w[0], w[1], w[2], w[3]);
      st_shared_v4(base + (((j0 + 1) ^ (r & 7)) << 4), w[4], w[5], w[6], w[7]);
    }
    tc_fence_before();
    mbar_arrive(smem_u32(&c->acc1_empty[b1]));     // acc1 buffer read completely
    fence_proxy_async();     // ordinary shared stores -> visible to the MMA's async reads
    mbar_arrive(smem_u32(&c->hs_full));
    // ---- scores -> mask words, counts ---------------------------------------------
    if (grp == 0) {
      if (!mbar_wait_fast(smem_u32(&c->acc2_full[0]), ph_mine, af, p.dev_status)) return;
      ph_mine ^= 1;
      tc_fence_after();
      const int E = p.E;
      const long long trow = (long long)t.r0 + r;
      float m = -INFINITY;
      for (int c0 = 0; c0 < g.nd; c0 += 16) {
        uint32_t v[16];
        tmem_ld16(tmem + lane_base + 256 + c0, v);
        tmem_wait_ld();
#pragma unroll
        for (int q = 0; q < 16; ++q)
          if (c0 + q < E) m = nanmax(m, fabsf(bfr(__uint_as_float(v[q]))));
      }
      const float thr = bfr(__fmul_rn(m, p.mult));
      const int nw = (E + 31) >> 5;
      uint32_t word = 0, mw[4] = {0u, 0u, 0u, 0u};
      for (int c0 = 0; c0 < g.nd; c0 += 16) {
        uint32_t v[16], blk = 0;
        tmem_ld16(tmem + lane_base + 256 + c0, v);
        tmem_wait_ld();
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          const float sc = fabsf(bfr(__uint_as_float(v[q])));
          if (c0 + q < E) {
            if (sc >= thr) {
              word |= 1u << ((c0 + q) & 31);
              blk |= 1u << q;
            }
            if (p.scores && r < t.nrows) p.scores[trow * E + c0 + q] = __float2bfloat16_rn(sc);
          }
        }
        if (p.rt_out && r < t.nrows && c0 < E) {
          // this row's 0/1 routing entries of the block (bf16 1.0 = 0x3F80)
          bf16* dst = p.rt_out + trow * E + c0;
          if ((E & 7) == 0) {
            uint32_t w8[8];
#pragma unroll
            for (int q = 0; q < 8; ++q)
              w8[q] = ((blk >> (2 * q)) & 1u ? 0x3F80u : 0u) |
                      ((blk >> (2 * q + 1)) & 1u ? 0x3F800000u : 0u);
            *reinterpret_cast<uint4*>(dst) = make_uint4(w8[0], w8[1], w8[2], w8[3]);
            if (c0 + 16 <= E) *reinterpret_cast<uint4*>(dst + 8) = make_uint4(w8[4], w8[5], w8[6], w8[7]);
          } else {
            for (int q = 0; q < 16 && c0 + q < E; ++q)
              dst[q] = __float2bfloat16_rn((blk >> q) & 1u ? 1.0f : 0.0f);
          }
        }
        if (((c0 + 16) & 31) == 0 || c0 + 16 >= g.nd) {
          const int jw = c0 >> 5;
          if (r < t.nrows && jw < nw) {
            p.mask_bits[trow * nw + jw] = word;
            mw[jw & 3] = word;
          }
          word = 0;
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(&c->acc2_empty[0]));
      if (p.tile_counts) {
        // per-expert counts of this tile for the compaction: ballots per warp, summed
        // over the group's four warps in shared memory
        if (r < E) c->tile_cnt[r] = 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        for (int jw = 0; jw < nw; ++jw) {
          const int nb = min(32, E - 32 * jw);
          int mine = 0;
          for (int b = 0; b < nb; ++b) {
            const int cb = __popc(__ballot_sync(0xffffffffu, (mw[jw] >> b) & 1u));
            if (lane == b) mine = cb;
          }
          if (lane < nb && mine) atomicAdd(&c->tile_cnt[32 * jw + lane], mine);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (r < p.EP) p.tile_counts[(long long)tile * p.EP + r] = (uint8_t)(r < E ? c->tile_cnt[r] : 0);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// experts form: epilogue roles
// ---------------------------------------------------------------------------
// 16 hidden columns as 8 packed bf16 pairs, with the upstream rounding points
// (T(x W1), + b1, activation, x T(x W_up)) done in packed bf16 arithmetic: one
// float->bf16x2 conversion per pair instead of one conversion per rounding point.
// nord != 0: nacc also collects the row's norm terms of the activation (before the gating
// product), 1 = magnitudes, 2 = squares.
template <int ACT>
__device__ __forceinline__ void ep1_pairs(const uint32_t* v, const uint32_t* u, const uint32_t* bp,
                                          bool glu, uint32_t* w, float& nacc, int nord) {
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    __nv_bfloat162 h =
        __floats2bfloat162_rn(__uint_as_float(v[2 * q]), __uint_as_float(v[2 * q + 1]));
    h = __hadd2_rn(h, *reinterpret_cast<const __nv_bfloat162*>(&bp[q]));
    if (ACT == D2D_RELU) {
      h = __hmax2(h, __float2bfloat162_rn(0.f));
    } else {
      const float2 f = __bfloat1622float2(h);
      h = __floats2bfloat162_rn(activate(f.x, ACT), activate(f.y, ACT));
    }
    if (nord != 0) {
      const float2 f = __bfloat1622float2(h);
      nacc += nord == 1 ? fabsf(f.x) + fabsf(f.y) : fmaf(f.x, f.x, f.y * f.y);
    }
    if (glu) {
      const __nv_bfloat162 uu =
          __floats2bfloat162_rn(__uint_as_float(u[2 * q]), __uint_as_float(u[2 * q + 1]));
      h = __hmul2_rn(h, uu);
    }
    w[q] = *reinterpret_cast<uint32_t*>(&h);
  }
}

// Warps 0-3: accumulator 1 -> bias, activation (x up-projection) -> bf16 hidden tile in
// shared memory, one tile after another.  Thread = tile row = TMEM lane.
__device__ void role_ep1_experts(const Params& p, Ctl* c, uint32_t hs, uint32_t tmem, int et) {
  volatile int* af = &c->abort_flag;
  const Geo& g = p.g;
  const int r = et;
  const uint32_t lane_base = (uint32_t)(r & ~31) << 16;
  const uint32_t hs_row = hs + (r >> 3) * 1024 + (r & 7) * 128;
  const bool la = lookahead(g);
  uint32_t* bias_p = reinterpret_cast<uint32_t*>(c->bias_s);   // [2][64] packed pairs
  const int npair = g.nsubw >> 1;
  uint32_t i = 0;
  for (int tile = blockIdx.x; tile < c->total_tiles; tile += gridDim.x, ++i) {
    const Tile t = tile_info<MODE_EXPERTS>(p, c, tile);
    // this expert's bias as bf16 pairs; two copies alternate so that a warp already on the
    // next tile never overwrites pairs another warp still reads
    uint32_t* bp = bias_p + (i & 1) * 64;
    if (et < npair) {
      const float2 b = __ldg(reinterpret_cast<const float2*>(p.packed + (long long)t.e * g.stride +
                                                             g.bias_off) + et);
      bp[et] = pack_bf16x2(b.x, b.y);
    }
    asm volatile("bar.sync 2, 128;" ::: "memory");
    // labels by-product (intermediate layer): this thread's row, its token loaded up front
    const int nord = p.norm_layer == D2D_NORM_OF_INTERMEDIATE ? p.norm_ord : 0;
    float nacc = 0.f;
    int ntok = -1;
    if (nord != 0 && r < t.nrows) ntok = p.token_idx[t.r0 + r];
    const uint32_t b1 = la ? (i & 1) : 0;
    const uint32_t acc1 = tmem + lane_base + (la ? b1 * 128 : 0);
    if (!mbar_wait_fast(smem_u32(&c->acc1_full[b1]), la ? ((i >> 1) & 1) : (i & 1), af,
                        p.dev_status))
      return;
    if (!mbar_wait_fast(smem_u32(&c->hs_empty), (i & 1) ^ 1, af, p.dev_status)) return;
    tc_fence_after();
    for (int c0 = 0; c0 < g.nsubw; c0 += 16) {
      uint32_t v[16], u[16], w[8], bb[8];
      tmem_ld16(acc1 + c0, v);
      if (p.glu) tmem_ld16(acc1 + 128 + c0, u);
      const uint4 q0 = *reinterpret_cast<const uint4*>(bp + (c0 >> 1));
      const uint4 q1 = *reinterpret_cast<const uint4*>(bp + (c0 >> 1) + 4);
      bb[0] = q0.x; bb[1] = q0.y; bb[2] = q0.z; bb[3] = q0.w;
      bb[4] = q1.x; bb[5] = q1.y; bb[6] = q1.z; bb[7] = q1.w;
      tmem_wait_ld();
      switch (p.act) {      // uniform branch around the element loop
        case D2D_RELU: ep1_pairs<D2D_RELU>(v, u, bb, p.glu != 0, w, nacc, nord); break;
        case D2D_GELU: ep1_pairs<D2D_GELU>(v, u, bb, p.glu != 0, w, nacc, nord); break;
        case D2D_TANH: ep1_pairs<D2D_TANH>(v, u, bb, p.glu != 0, w, nacc, nord); break;
        case D2D_LEAKY_RELU: ep1_pairs<D2D_LEAKY_RELU>(v, u, bb, p.glu != 0, w, nacc, nord); break;
        default: ep1_pairs<D2D_GELU_TANH>(v, u, bb, p.glu != 0, w, nacc, nord); break;
      }
      const uint32_t base = hs_row + (c0 >> 6) * SLOT;
      const int j0 = (c0 & 63) >> 3;
      st_shared_v4(base + (((j0) ^ (r & 7)) << 4), w[0], w[1], w[2], w[3]);
      st_shared_v4(base + (((j0 + 1) ^ (r & 7)) << 4), w[4], w[5], w[6], w[7]);
    }
    tc_fence_before();
    mbar_arrive(smem_u32(&c->acc1_empty[b1]));     // acc1 buffer read completely
    fence_proxy_async();     // ordinary shared stores -> visible to the MMA's async reads
    mbar_arrive(smem_u32(&c->hs_full));
    if (ntok >= 0 && ntok < p.N)
      p.norms[(long long)t.e * p.N + ntok] = __float2bfloat16_rn(nord == 1 ? nacc : sqrtf(nacc));
  }
}

// Warps 4-7: accumulator 2 -> bf16 -> staging blocks.  Warp q owns two 32-row x 128-byte
// blocks and fills them alternately; writer warp q adds them to the output rows.  This
// role never touches global memory, so the accumulators are handed back to the GEMM2
// warp as fast as the write path drains.
__device__ void role_ep2_experts(const Params& p, Ctl* c, uint32_t stg, uint32_t tmem, int et) {
  volatile int* af = &c->abort_flag;
  const Geo& g = p.g;
  const int lane = et & 31, q = et >> 5;
  const uint32_t lane_base = (uint32_t)(et & ~31) << 16;
  const int halves = g.nd >> 6;
  uint32_t phbits = 0, n = 0;
  const int nord = p.norm_layer == D2D_NORM_OF_OUTPUT ? p.norm_ord : 0;
  for (int tile = blockIdx.x; tile < c->total_tiles; tile += gridDim.x) {
    // labels by-product (output layer): thread = tile row; norm terms of the bf16 outputs
    float nacc = 0.f;
    int ntok = -1, ne = 0;
    if (nord != 0) {
      const Tile t = tile_info<MODE_EXPERTS>(p, c, tile);
      ne = t.e;
      if (et < t.nrows) ntok = p.token_idx[t.r0 + et];
    }
    for (int nci = 0; nci < g.nc; ++nci) {
      const uint32_t buf = nci & 1;
      if (!mbar_wait_fast(smem_u32(&c->acc2_full[buf]), (phbits >> buf) & 1, af, p.dev_status))
        return;
      phbits ^= 1u << buf;
      tc_fence_after();
      for (int hf = 0; hf < halves; ++hf, ++n) {
        uint32_t v[64];
        tmem_ld32(tmem + lane_base + 256 + buf * 128 + hf * 64, v);
        tmem_ld32(tmem + lane_base + 256 + buf * 128 + hf * 64 + 32, v + 32);
        tmem_wait_ld();
        if (hf == halves - 1) {     // accumulator buffer read completely: hand it back
          tc_fence_before();
          mbar_arrive(smem_u32(&c->acc2_empty[buf]));
        }
        const uint32_t blk = n & 1;
        if (!mbar_wait_fast(smem_u32(&c->sempty[blk][q]), ((n >> 1) & 1) ^ 1, af, p.dev_status))
          return;
        const uint32_t dst = stg + (blk * 4 + q) * 4096 + lane * 128;
        // piece XOR row: conflict-free 16-byte stores
#pragma unroll
        for (int pc = 0; pc < 8; ++pc) {
          uint32_t ww[4];
#pragma unroll
          for (int k = 0; k < 4; ++k)
            ww[k] = pack_bf16x2(__uint_as_float(v[8 * pc + 2 * k]),
                                __uint_as_float(v[8 * pc + 2 * k + 1]));
          st_shared_v4(dst + ((pc ^ (lane & 7)) << 4), ww[0], ww[1], ww[2], ww[3]);
          if (nord != 0) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float lo = __uint_as_float(ww[k] << 16), hi = __uint_as_float(ww[k] & 0xffff0000u);
              nacc += nord == 1 ? fabsf(lo) + fabsf(hi) : fmaf(lo, lo, hi * hi);
            }
          }
        }
        mbar_arrive(smem_u32(&c->sfull[blk][q]));
      }
    }
    if (ntok >= 0 && ntok < p.N)
      p.norms[(long long)ne * p.N + ntok] = __float2bfloat16_rn(nord == 1 ? nacc : sqrtf(nacc));
  }
}

// Writer warps: warp q adds the staged bf16 blocks of row quarter q to the output rows.
// The global write path takes about 24 bytes per clock and SM for vector reds whichever
// warps issue them, so it gets warps of its own.  A lane reads its rows back
// row-contiguous (8 lanes cover one row's 128 bytes), so one red instruction touches 4
// cache lines instead of 32.
__device__ void role_writer(const Params& p, Ctl* c, uint32_t stg, int wt) {
  volatile int* af = &c->abort_flag;
  const Geo& g = p.g;
  const int lane = wt & 31, q = wt >> 5;
  const int rl = lane >> 3, pl = lane & 7;
  const int halves = g.nd >> 6;
  uint32_t n = 0;
  int tile = blockIdx.x;
  const int total = c->total_tiles, step = gridDim.x;
  Tile t = {0, 0, 0};
  long long tok = -1;
  if (tile < total) {
    t = tile_info<MODE_EXPERTS>(p, c, tile);
    const int r = q * 32 + lane;
    if (r < t.nrows) tok = p.token_idx[t.r0 + r];
  }
  for (; tile < total; tile += step) {
    if (tok < 0 || tok >= p.N) tok = -1;      // out-of-range indices are reported by the producer
    bf16* orow[8];
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const long long tk = __shfl_sync(0xffffffffu, tok, it * 4 + rl);
      orow[it] = tk < 0 ? nullptr : p.out + tk * p.d + pl * 8;
    }
    // rows of the next tile: the load is in flight while this tile's blocks are written
    tok = -1;
    if (tile + step < total) {
      t = tile_info<MODE_EXPERTS>(p, c, tile + step);
      const int r = q * 32 + lane;
      if (r < t.nrows) tok = p.token_idx[t.r0 + r];
    }
    for (int nci = 0; nci < g.nc; ++nci) {
      for (int hf = 0; hf < halves; ++hf, ++n) {
        const uint32_t blk = n & 1;
        const uint32_t src = stg + (blk * 4 + q) * 4096;
        if (!mbar_wait_fast(smem_u32(&c->sfull[blk][q]), (n >> 1) & 1, af, p.dev_status)) return;
        uint4 val[8];
#pragma unroll
        for (int it = 0; it < 8; ++it) {      // all shared loads first, then all reds
          const int rr = it * 4 + rl;
          val[it] = ld_shared_v4(src + rr * 128 + ((pl ^ (rr & 7)) << 4));
        }
        mbar_arrive(smem_u32(&c->sempty[blk][q]));   // block may be overwritten
        const int col = nci * g.nd + hf * 64;
#pragma unroll
        for (int it = 0; it < 8; ++it)
          if (orow[it])
            red_add_bf16x8(orow[it] + col, val[it].x, val[it].y, val[it].z, val[it].w);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(MODE == MODE_EXPERTS ? NTHREADS_EXPERTS : NTHREADS, 1)
mlp_tiles_kernel(const Params p, const __grid_constant__ CUtensorMap tmx) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - raw);
  const uint32_t ringA = base;
  const uint32_t ringB = ringA + p.g.na * SLOT;
  const uint32_t ringB2 = ringB + p.g.nb * SLOT;
  const uint32_t hs = ringB2 + p.g.nb2 * SLOT;
  const uint32_t stg = hs + p.g.kc2 * SLOT;
  Ctl* c = reinterpret_cast<Ctl*>(
      aligned + (size_t)(p.g.na + p.g.nb + p.g.nb2 + p.g.kc2 + p.g.stg) * SLOT);
  const int tid = threadIdx.x, warp = tid >> 5;
  // Programmatic dependent launch: the next kernel of the stream may be scheduled as soon as
  // every CTA of this one has passed this point (its CTAs still wait for this grid to
  // finish before they read anything); this CTA in turn initialises its barriers while the
  // previous kernel drains and reads global memory only after the wait below.
  grid_launch_dependents();

  if (tid == 0) {
    for (int i = 0; i < NA_MAX; ++i) {
      mbar_init(smem_u32(&c->fullA[i]), (MODE == MODE_EXPERTS && !p.tma_gather) ? 128 : 1);
      mbar_init(smem_u32(&c->emptyA[i]), 1);
    }
    for (int i = 0; i < NB_MAX; ++i) {
      mbar_init(smem_u32(&c->fullB[i]), 1);
      mbar_init(smem_u32(&c->emptyB[i]), 1);
      mbar_init(smem_u32(&c->fullB2[i]), 1);
      mbar_init(smem_u32(&c->emptyB2[i]), 1);
    }
    // experts form: warps 0-3 write the hidden tile, warps 4-7 read accumulator 2
    constexpr uint32_t EP1_THREADS = MODE == MODE_EXPERTS ? 128 : 256;
    mbar_init(smem_u32(&c->hs_full), EP1_THREADS);
    mbar_init(smem_u32(&c->hs_empty), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&c->acc1_full[i]), 1);
      mbar_init(smem_u32(&c->acc1_empty[i]), EP1_THREADS);
      mbar_init(smem_u32(&c->acc2_full[i]), 1);
      mbar_init(smem_u32(&c->acc2_empty[i]), 128);
      for (int q = 0; q < 4; ++q) {
        mbar_init(smem_u32(&c->sfull[i][q]), 32);
        mbar_init(smem_u32(&c->sempty[i][q]), 32);
      }
    }
    c->abort_flag = 0;
    c->wait_limit = (int)p.wait_limit;
    if (MODE == MODE_ROUTER) c->total_tiles = (int)((p.N + TILE_M - 1) / TILE_M);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  grid_dependency_wait();
  if (MODE == MODE_EXPERTS && warp == 1) {
    // tile tables: all offsets loaded in parallel (lane l owns experts 4l..4l+3), exclusive
    // scans across the warp of the full-tile counts and of the "has a partial tile" flags
    const int lane = tid & 31;
    int off[5], nt[4], pt[4], sum = 0, psum = 0;
    bool all_n = true;               // every expert of this lane lists exactly N tokens
#pragma unroll
    for (int q = 0; q < 5; ++q) {
      const int e = 4 * lane + q;
      off[q] = e <= p.E ? p.offsets[e] : 0;
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int e = 4 * lane + q;
      const int n = e < p.E ? off[q + 1] - off[q] : 0;
      if (e < p.E && n != p.N) all_n = false;
      if (e < p.E && (n < 0 || off[q + 1] > p.N * (long long)p.E))
        report(p.dev_status, D2D_ERR_INDEX_RANGE);
      nt[q] = n > 0 ? n / TILE_M : 0;
      pt[q] = (n > 0 && n % TILE_M != 0) ? 1 : 0;
      sum += nt[q];
      psum += pt[q];
    }
    int incl = sum, pincl = psum;
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      const int w = __shfl_up_sync(0xffffffffu, pincl, o);
      if (lane >= o) {
        incl += v;
        pincl += w;
      }
    }
    int run = incl - sum, prun = pincl - psum;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int e = 4 * lane + q;
      if (e <= p.E) c->tstart[e] = run;
      if (pt[q]) c->pidx[prun] = (uint8_t)e;
      run += nt[q];
      prun += pt[q];
    }
    const bool dense = __all_sync(0xffffffffu, all_n) && p.N > 0 && p.E > 1;
    if (lane == 31) {
      c->total_full = incl;
      c->total_tiles = incl + pincl;
      c->dense_tpe = dense ? (int)((p.N + TILE_M - 1) / TILE_M) : 0;    // same tile count either way
    }
  }
  if (warp == WARP_MMA1) tmem_alloc(smem_u32(&c->tmem_base), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = c->tmem_base;

  if (MODE == MODE_EXPERTS && warp < 4) {
    role_ep1_experts(p, c, hs, tmem, tid);
  } else if (MODE == MODE_EXPERTS && warp < 8) {
    role_ep2_experts(p, c, stg, tmem, tid - 128);
  } else if (warp < 8) {
    role_epilogue_router(p, c, hs, stg, tmem, tid);
    bulk_wait_all();       // TMA row stores read shared memory: finish before the CTA ends
  } else if (warp == WARP_MMA1) {
    if (elect_one()) role_mma1<MODE>(p, c, ringA, ringB, tmem);
    __syncwarp();
  } else if (warp == WARP_MMA2) {
    if (elect_one()) role_mma2<MODE>(p, c, ringB2, hs, tmem);
    __syncwarp();
  } else if (warp == WARP_BULK) {
    if (elect_one()) role_bulk<MODE>(p, c, ringB, ringB2);
    __syncwarp();
  } else if (warp < WARP_WR0) {
    if (MODE == MODE_EXPERTS && !p.tma_gather) {
      role_producer_cpasync(p, c, ringA, tid - WARP_PROD0 * 32);
      cp_async_wait_all();
    } else if (warp == WARP_PROD0) {
      role_producer<MODE>(p, c, &tmx, ringA, tid & 31);
    }
  } else if (MODE == MODE_EXPERTS) {
    role_writer(p, c, stg, tid - WARP_WR0 * 32);
  }

  // A launch that gave up may still have copies and MMAs in flight that use this CTA's
  // shared and tensor memory: give them time to land before both are released.
  if (*reinterpret_cast<volatile int*>(&c->abort_flag) != 0)
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------------
// weight packing
// ---------------------------------------------------------------------------
__global__ void prepack_experts_kernel(const bf16* __restrict__ w1, const bf16* __restrict__ b1,
                                       const bf16* __restrict__ w_up, const bf16* __restrict__ w2,
                                       uint8_t* __restrict__ packed, Geo g, int d, int E, int H) {
  const int e = blockIdx.y;
  uint8_t* pe = packed + (long long)e * g.stride;
  const long long n1 = (long long)g.kc1 * g.nsub * g.nsubw * 64;
  const long long n2 = (long long)g.nc * g.kc2 * g.nd * 64;
  const bf16 zero = __float2bfloat16_rn(0.f);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n1 + n2 + g.nsubw;
       i += (long long)gridDim.x * blockDim.x) {
    if (i < n1) {
      const int k = (int)(i % 64);
      const int n = (int)((i / 64) % g.nsubw);
      const int sub = (int)((i / (64LL * g.nsubw)) % g.nsub);
      const int kc = (int)(i / (64LL * g.nsubw * g.nsub));
      const bf16* src = sub == 0 ? w1 : w_up;
      const bf16 v = src[((long long)e * d + kc * 64 + k) * H + n];
      *reinterpret_cast<bf16*>(pe + (long long)(kc * g.nsub + sub) * g.nsubw * 128 + swz(n, k)) = v;
    } else if (i < n1 + n2) {
      const long long q = i - n1;
      const int k = (int)(q % 64);
      const int n = (int)((q / 64) % g.nd);
      const int k2 = (int)((q / (64LL * g.nd)) % g.kc2);
      const int nci = (int)(q / (64LL * g.nd * g.kc2));
      const int kk = k2 * 64 + k;
      const bf16 v = kk < H ? w2[((long long)e * H + kk) * d + nci * g.nd + n] : zero;
      *reinterpret_cast<bf16*>(pe + g.w1_bytes + (long long)(nci * g.kc2 + k2) * g.nd * 128 +
                               swz(n, k)) = v;
    } else {
      const int h = (int)(i - n1 - n2);
      reinterpret_cast<float*>(pe + g.bias_off)[h] =
          b1 ? __bfloat162float(b1[(long long)e * H + h]) : 0.f;
    }
  }
}

__global__ void prepack_router_kernel(const bf16* __restrict__ wa, const bf16* __restrict__ wb,
                                      uint8_t* __restrict__ packed, Geo g, int d, int R, int E) {
  const long long n1 = (long long)g.kc1 * g.nsub * g.nsubw * 64;
  const long long n2 = (long long)g.kc2 * g.nd * 64;
  const bf16 zero = __float2bfloat16_rn(0.f);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n1 + n2;
       i += (long long)gridDim.x * blockDim.x) {
    if (i < n1) {
      const int k = (int)(i % 64);
      const int n = (int)((i / 64) % g.nsubw);
      const int sub = (int)((i / (64LL * g.nsubw)) % g.nsub);
      const int kc = (int)(i / (64LL * g.nsubw * g.nsub));
      const bf16 v = wa[(long long)(sub * g.nsubw + n) * d + kc * 64 + k];
      *reinterpret_cast<bf16*>(packed + (long long)(kc * g.nsub + sub) * g.nsubw * 128 +
                               swz(n, k)) = v;
    } else {
      const long long q = i - n1;
      const int k = (int)(q % 64);
      const int n = (int)((q / 64) % g.nd);
      const int k2 = (int)(q / (64LL * g.nd));
      const int kk = k2 * 64 + k;
      const bf16 v = (n < E && kk < R) ? wb[(long long)n * R + kk] : zero;
      *reinterpret_cast<bf16*>(packed + g.w1_bytes + (long long)k2 * g.nd * 128 + swz(n, k)) = v;
    }
  }
}

// Facts of one device, looked up with that device current.  The shared-memory opt-in of
// a kernel (cudaFuncSetAttribute) holds for the current device only, as does the SM count,
// so both are cached per device index; the lock makes first use from several host threads
// safe.
constexpr int MAX_DEVICES = 64;
struct DeviceFacts {
  int sms = 0;
  size_t smem_optin[2] = {0, 0};      // per MODE: largest dynamic shared memory opted in
};
DeviceFacts g_dev[MAX_DEVICES];
std::mutex g_dev_lock;

// test hooks (d2d_debug_configure): process-wide, read at launch
std::atomic<uint32_t> g_wait_limit{WAIT_LIMIT};
std::atomic<int> g_withhold{0};
// expert rows: 0/1 = 16-byte cp.async gather (default), 2 = TMA tile::gather4
std::atomic<int> g_experts_kernel{0};

static_assert(1024 + (size_t)SLOTS_TOTAL * SLOT + sizeof(Ctl) + 64 <= 232448,
              "shared-memory plan exceeds the 227 KB a CTA may use");

size_t smem_bytes(const Geo& g) {
  return 1024 + (size_t)(g.na + g.nb + g.nb2 + g.kc2 + g.stg) * SLOT + sizeof(Ctl) + 64;
}

template <int MODE>
int launch(Params& p, long long max_tiles, cudaStream_t s) {
  const size_t smem = smem_bytes(p.g);
  auto k = mlp_tiles_kernel<MODE>;
  int dev = -1, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    cudaGetLastError();
    return D2D_ERR_NO_DEVICE;
  }
  {
    std::lock_guard<std::mutex> hold(g_dev_lock);
    DeviceFacts& f = g_dev[dev];
    if (f.sms == 0 &&
        (cudaDeviceGetAttribute(&f.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
         f.sms <= 0)) {
      cudaGetLastError();
      f.sms = 0;
      return D2D_ERR_NO_DEVICE;
    }
    if (f.smem_optin[MODE] < smem) {
      if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
          cudaSuccess) {
        cudaGetLastError();
        return D2D_ERR_LAUNCH;
      }
      f.smem_optin[MODE] = smem;
    }
    sms = f.sms;
  }
  p.wait_limit = g_wait_limit.load();
  p.withhold = g_withhold.load();
  // x as a tensor map: boxes of 64 columns x 1 row (gathered by fours) for the expert lists,
  // 64 columns x 128 consecutive rows for the router
  alignas(64) CUtensorMap tmx;
  const int rc = encode_tmap_2d_b16(&tmx, p.x, (uint64_t)p.d, (uint64_t)p.N, (uint64_t)p.d * 2, 64,
                                    MODE == MODE_EXPERTS ? 1 : TILE_M, true);
  if (rc != D2D_OK) return rc == D2D_ERR_BAD_ARG ? D2D_ERR_LAUNCH : rc;
  long long grid = max_tiles < sms ? max_tiles : sms;
  if (grid < 1) grid = 1;
  return launch_pdl(k, dim3((unsigned)grid), dim3(MODE == MODE_EXPERTS ? NTHREADS_EXPERTS : NTHREADS),
                    smem, s, p, tmx);
}

}  // namespace

// ---------------------------------------------------------------------------
// host interface
// ---------------------------------------------------------------------------
bool umma_experts_supported(int d, int E, int H, bool glu, int dtype) {
  (void)glu;
  return dtype == D2D_BF16 && d >= 64 && d % 64 == 0 && (d % 128 == 0 || d == 64) && H >= 16 &&
         H <= 128 && H % 16 == 0 && E >= 1 && E <= MAX_E;
}

size_t umma_experts_packed_bytes(int d, int E, int H, bool glu) {
  return (size_t)experts_geo(d, H, glu).stride * (size_t)E;
}

int launch_prepack_experts(const void* w1, const void* b1, const void* w_up, const void* w2,
                           void* packed, int d, int E, int H, cudaStream_t s) {
  const Geo g = experts_geo(d, H, w_up != nullptr);
  dim3 grid(64, E);
  prepack_experts_kernel<<<grid, 256, 0, s>>>((const bf16*)w1, (const bf16*)b1, (const bf16*)w_up,
                                              (const bf16*)w2, (uint8_t*)packed, g, d, E, H);
  return cudaGetLastError() == cudaSuccess ? D2D_OK : D2D_ERR_LAUNCH;
}

int launch_experts_umma(const void* x, const int32_t* token_idx, const int32_t* offsets,
                        const void* packed, void* out, int64_t N, int d, int E, int H, bool glu,
                        int act, int* dev_status, cudaStream_t s, NormCapture nc) {
  Params p = {};
  p.x = (const bf16*)x;
  p.N = N;
  p.d = d;
  p.packed = (const uint8_t*)packed;
  p.g = experts_geo(d, H, glu);
  p.token_idx = token_idx;
  p.offsets = offsets;
  p.E = E;
  p.out = (bf16*)out;
  p.act = act;
  p.glu = glu ? 1 : 0;
  p.dev_status = dev_status;
  p.tma_gather = g_experts_kernel.load() == 2 ? 1 : 0;
  p.norms = (bf16*)nc.norms;
  p.norm_layer = nc.norms ? nc.layer : 0;
  p.norm_ord = nc.ord;
  const long long max_tiles = (N * (long long)E + TILE_M - 1) / TILE_M + E;
  return launch<MODE_EXPERTS>(p, max_tiles, s);
}

void umma_debug_select_experts_kernel(int which) {
  g_experts_kernel.store(which == 2 ? 2 : 0);
}

void umma_debug_configure(int wait_limit_log2, int withhold_weight_tile) {
  g_wait_limit.store(wait_limit_log2 >= 4 && wait_limit_log2 <= 22 ? 1u << wait_limit_log2
                                                                    : WAIT_LIMIT);
  g_withhold.store(withhold_weight_tile ? 1 : 0);
}

bool umma_router_supported(int d, int R, int E, int dtype) {
  return dtype == D2D_BF16 && d >= 64 && d % 64 == 0 && R >= 16 && R % 16 == 0 &&
         (R <= 128 || R == 256) && E >= 1 && E <= MAX_E;
}

size_t umma_router_packed_bytes(int d, int R, int E) { return (size_t)router_geo(d, R, E).stride; }

int launch_prepack_router(const void* wa, const void* wb, void* packed, int d, int R, int E,
                          cudaStream_t s) {
  const Geo g = router_geo(d, R, E);
  prepack_router_kernel<<<64, 256, 0, s>>>((const bf16*)wa, (const bf16*)wb, (uint8_t*)packed, g, d,
                                           R, E);
  return cudaGetLastError() == cudaSuccess ? D2D_OK : D2D_ERR_LAUNCH;
}

int launch_router_mask_umma(const void* x, const void* packed, float mult, uint32_t* mask_bits,
                            void* scores, void* rt_out, const void* last_bias, int add_residual,
                            void* out_init, int32_t* tile_counts, int64_t N, int d, int R, int E,
                            int* dev_status, cudaStream_t s) {
  Params p = {};
  p.x = (const bf16*)x;
  p.N = N;
  p.d = d;
  p.packed = (const uint8_t*)packed;
  p.g = router_geo(d, R, E);
  p.E = E;
  p.mult = mult;
  p.mask_bits = mask_bits;
  p.scores = (bf16*)scores;
  p.rt_out = (bf16*)rt_out;
  p.last_bias = (const bf16*)last_bias;
  p.add_residual = add_residual;
  p.out_init = (bf16*)out_init;
  p.tile_counts = reinterpret_cast<uint8_t*>(tile_counts);
  p.EP = compact_row_cells(E);
  p.dev_status = dev_status;
  return launch<MODE_ROUTER>(p, (N + TILE_M - 1) / TILE_M, s);
}

}  // namespace d2d
