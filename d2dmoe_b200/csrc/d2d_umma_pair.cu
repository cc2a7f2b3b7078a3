// Expert FFN on CTA pairs: tcgen05.mma.cta_group::2 over 256 rows of one expert's token list.
//
//   per (expert e, 256 entries of its token list), CTA r of the pair owning 128 of the rows:
//     h   = act(bf16(x[rows] W1[e]) + b1[e]) (* bf16(x[rows] W_up[e]))
//     out[rows] += bf16(h W2[e])                         red.global.add bf16x2
//   fusing architectures/moe/moe_impls.py:93-180 (gathered first layer) and :244-301
//   (second layer + atomic add); h never leaves the SM.
//
// Why pairs: with one CTA per tile every 128 rows pull a full copy of the expert's weights
// (W1 and W2 tiles) through the SM's memory interface, which bounds the tile period.  Two
// CTAs on neighbouring SMs form a cluster; each gathers its own 128 rows and loads only
// HALF of every weight tile (its half of the tile's N dimension), and one MMA instruction
// of the leader CTA multiplies both CTAs' row tiles with the two halves: half the weight
// bytes per row, and the weight rings take half the shared memory.
//
// Roles per CTA (608 threads), same as the single-CTA kernel of d2d_umma.cu:
//   warps 0-3   epilogue 1: accumulator 1 -> bias/activation(/x up) -> bf16 hidden tile
//   warps 4-7   epilogue 2: accumulator 2 -> bf16 -> staging blocks
//   warp  8     TMEM allocation (pair-wide); leader: GEMM1 issue thread; peer: relay thread
//   warp  9     leader: GEMM2 issue thread; peer: relay thread
//   warp 10     weight half-tiles by cp.async.bulk into this CTA's rings
//   warps 11-14 gather this CTA's token rows (16-byte cp.async, software swizzle)
//   warps 15-18 add the staged blocks to out[token] (red.global.add.noftz.v4.bf16x2)
// The leader's issue threads wait on "full" barriers of the LEADER that count the leader's
// own producers plus one arrival of the peer's relay thread (which forwards the peer's
// local "full" events); MMA completion is signalled to the barriers of both CTAs with
// tcgen05.commit ... multicast::cluster; the epilogue warps of both CTAs hand accumulators
// and the hidden tile back by arriving on the leader's barriers.  No multicast LOADS.
//
// Every wait is bounded: when one runs out the kernel records D2D_ERR_TIMEOUT in the
// status word, all roles leave their loops, both CTAs meet at the cluster barrier, TMEM
// is freed and the kernel returns.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "d2d_umma_api.cuh"
#include "d2d_umma_ptx.cuh"

namespace d2d {
using namespace umma;
namespace {

constexpr int HSLOT = SLOT / 2;      // 8 KB: stage stride of the weight half-tile rings
constexpr int NA_MAX = 6, NB_MAX = 8;
constexpr int NTHREADS = 608;
constexpr int WARP_MMA1 = 8, WARP_MMA2 = 9, WARP_BULK = 10, WARP_PROD0 = 11, WARP_WR0 = 15;
constexpr int MAX_E = 128;
constexpr int PAIR_M = 2 * TILE_M;   // rows of a pair tile

struct Geo {
  int kc1;       // d / 64
  int nsub;      // weight subtiles per k-chunk of GEMM1 (1, or 2 = gate and up)
  int nsubw;     // columns per subtile = H
  int K2;        // GEMM2 reduction = H
  int kc2;       // ceil(H / 64)
  int nd;        // GEMM2 output columns per chunk
  int nc;        // number of chunks
  int na, nb, nb2;                        // ring depths
  long long w1_bytes, bias_off, stride;   // packed layout per expert (d2d_prepack_experts)
};

struct Params {
  const bf16* x;
  long long N;
  int d;
  const uint8_t* packed;
  Geo g;
  const int32_t* token_idx;
  const int32_t* offsets;
  int E;
  bf16* out;
  int act, glu;
  int* dev_status;
  uint32_t wait_limit;
  int withhold;
};

// Must describe the same packed layout as experts_geo of d2d_umma.cu.
Geo pair_geo(int d, int H, bool glu) {
  Geo g;
  g.kc1 = d / 64;
  g.nsub = glu ? 2 : 1;
  g.nsubw = H;
  g.K2 = H;
  g.kc2 = (H + 63) / 64;
  g.nd = (d % 128 == 0) ? 128 : 64;
  g.nc = d / g.nd;
  // 14 slots of 16 KB: hidden tile kc2, staging 2, the rest for the three rings
  const int free16 = 14 - g.kc2 - 2;                 // 10 or 11
  g.na = free16 >= 11 ? 6 : 5;
  const int half_slots = 2 * (free16 - g.na);        // 8 KB stages left for the weight rings
  g.nb = glu ? 6 : half_slots / 2;
  g.nb2 = half_slots - g.nb;
  if (g.nb2 > NB_MAX) g.nb2 = NB_MAX;
  g.w1_bytes = (long long)g.kc1 * g.nsub * g.nsubw * 128;
  g.bias_off = g.w1_bytes + (long long)g.nc * g.kc2 * g.nd * 128;
  g.stride = (g.bias_off + 512 + 1023) / 1024 * 1024;
  return g;
}

// ---------------------------------------------------------------------------
// PTX wrappers of the pair (cta_group::2 / cluster) forms
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// arrive on the barrier at the same shared-memory offset in CTA `cta` of the cluster
__device__ __forceinline__ void mbar_arrive_remote(uint32_t local_bar, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_bar), "r"(cta));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(r) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
// D[tmem of both CTAs] (+)= A[smem of each CTA, 128 rows] * B[halves in both CTAs' smem]
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the barrier at this shared-memory offset in BOTH CTAs of the pair receives one arrival
// once every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma2_commit(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(bar),
      "h"(mask)
      : "memory");
}

// ---------------------------------------------------------------------------
// shared-memory bookkeeping
// ---------------------------------------------------------------------------
struct Ctl {
  unsigned long long fullA[NA_MAX], emptyA[NA_MAX], fullB[NB_MAX], emptyB[NB_MAX];
  unsigned long long fullB2[NB_MAX], emptyB2[NB_MAX];
  unsigned long long acc1_full[2], acc1_empty[2], hs_full, hs_empty, acc2_full[2], acc2_empty[2];
  unsigned long long sfull[2][4], sempty[2][4];   // staging unit of (block, row quarter)
  uint32_t tmem_base;
  int abort_flag;
  int wait_limit;                  // must follow abort_flag (mbar_wait reads abort_flag[1])
  int total_tiles;
  alignas(16) float bias_s[128];   // two copies of the current expert's b1 as bf16 pairs
  int total_full;                  // number of full 256-row tiles (they come first)
  uint8_t pidx[MAX_E];             // expert of the k-th partial (tail) tile
  int tstart[MAX_E + 1];           // first full tile of each expert
};

struct Tile {
  int e;        // expert
  int r0;       // first entry of this CTA's rows in token_idx
  int nrows;    // this CTA's rows (0..128)
};

// Pair-tile order: every full 256-row tile (expert-major), then the experts' partial tail
// tiles.  A tail of n rows is split evenly: the leader takes ceil(n/2), the peer the rest.
__device__ __forceinline__ Tile tile_info(const Params& p, const Ctl* c, int tile, uint32_t rank) {
  Tile t;
  int r0, n;
  if (tile < c->total_full) {
    int lo = 0, hi = p.E;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (c->tstart[mid] <= tile) lo = mid; else hi = mid;
    }
    t.e = lo;
    r0 = p.offsets[lo] + (tile - c->tstart[lo]) * PAIR_M;
    n = PAIR_M;
  } else {
    t.e = c->pidx[tile - c->total_full];
    const int cnt = p.offsets[t.e + 1] - p.offsets[t.e];
    r0 = p.offsets[t.e] + (cnt / PAIR_M) * PAIR_M;
    n = cnt % PAIR_M;
  }
  const int half = (n + 1) >> 1;
  t.r0 = r0 + (rank ? half : 0);
  t.nrows = rank ? n - half : half;
  return t;
}

// ---------------------------------------------------------------------------
// roles
// ---------------------------------------------------------------------------
__device__ void role_producer(const Params& p, Ctl* c, uint32_t ringA, int pt, uint32_t rank) {
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
  for (int tile = blockIdx.x >> 1; tile < c->total_tiles; tile += gridDim.x >> 1) {
    const Tile t = tile_info(p, c, tile, rank);
    const bf16* src[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int row = pw * 32 + i * 4 + (lane >> 3);
      row = max(0, min(row, t.nrows - 1));      // rows past the tail repeat the last row
      long long tok = 0;
      if (t.nrows > 0) {
        tok = p.token_idx[t.r0 + row];
        if (tok < 0 || tok >= p.N) {
          report(p.dev_status, D2D_ERR_INDEX_RANGE);
          tok = 0;
        }
      }
      src[i] = p.x + tok * p.d + j * 8;
    }
    for (int kc = 0; kc < p.g.kc1; ++kc) {
      if (!mbar_wait_fast(smem_u32(&c->emptyA[s]), ph ^ 1, af, p.dev_status)) return;
      const uint32_t base = ringA + s * SLOT;
      if (t.nrows > 0 && !(p.withhold & 4)) {   // a CTA without rows in a tail tile leaves the stage as it is
#pragma unroll
        for (int i = 0; i < 8; ++i) cp_async16(base + dstoff[i], src[i] + kc * 64);
      }
      cp_async_arrive_noinc(smem_u32(&c->fullA[s]));
      if (++s == (uint32_t)p.g.na) {
        s = 0;
        ph ^= 1;
      }
    }
  }
}

// Weight half-tiles for both rings of this CTA: rows [rank * n/2, (rank+1) * n/2) of every
// packed tile (n = tile rows = MMA N), i.e. one contiguous half of the tile image.
__device__ void role_bulk(const Params& p, Ctl* c, uint32_t ringB, uint32_t ringB2,
                          uint32_t rank) {
  volatile int* af = &c->abort_flag;
  const Geo& g = p.g;
  const uint32_t b1 = g.nsubw * 128, b2 = g.nd * 128;          // full tile bytes
  const uint32_t h1 = b1 >> 1, h2 = b2 >> 1;                   // this CTA's half
  const int n1 = g.kc1 * g.nsub, n2 = g.nc * g.kc2;
  const int step = gridDim.x >> 1, total = c->total_tiles;
  const uint32_t fullB = smem_u32(c->fullB), emptyB = smem_u32(c->emptyB);
  const uint32_t fullB2 = smem_u32(c->fullB2), emptyB2 = smem_u32(c->emptyB2);
  RingPos r1 = {0, 0}, r2 = {0, 0};
  int t1 = blockIdx.x >> 1, t2 = blockIdx.x >> 1, j1 = 0, j2 = 0;
  const uint8_t *pe1 = nullptr, *pe2 = nullptr;
  if (t1 < total) pe1 = pe2 = p.packed + (long long)tile_info(p, c, t1, rank).e * g.stride;
  uint32_t idle = 0;
  bool withheld = (p.withhold & 1) != 0 && blockIdx.x == 0;
  while (t1 < total || t2 < total) {
    bool progress = false;
    if (t1 < total && mbar_test_wait(emptyB + 8 * r1.s, r1.ph ^ 1)) {
      const uint32_t bar = fullB + 8 * r1.s;
      if (withheld) {
        withheld = false;      // test hook: this stage never fills, its consumer's wait runs out
      } else {
        if (p.withhold & 8) {
          mbar_arrive(bar);
        } else {
          mbar_arrive_expect_tx(bar, h1);
          bulk_g2s(ringB + r1.s * HSLOT, pe1 + (long long)j1 * b1 + rank * h1, h1, bar);
        }
      }
      r1.next(g.nb);
      if (++j1 == n1) {
        j1 = 0;
        t1 += step;
        if (t1 < total) pe1 = p.packed + (long long)tile_info(p, c, t1, rank).e * g.stride;
      }
      progress = true;
    }
    if (t2 < total && mbar_test_wait(emptyB2 + 8 * r2.s, r2.ph ^ 1)) {
      const uint32_t bar = fullB2 + 8 * r2.s;
      if (p.withhold & 8) {
        mbar_arrive(bar);
      } else {
        mbar_arrive_expect_tx(bar, h2);
        bulk_g2s(ringB2 + r2.s * HSLOT, pe2 + g.w1_bytes + (long long)j2 * b2 + rank * h2, h2, bar);
      }
      r2.next(g.nb2);
      if (++j2 == n2) {
        j2 = 0;
        t2 += step;
        if (t2 < total) pe2 = p.packed + (long long)tile_info(p, c, t2, rank).e * g.stride;
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

// GEMM1 stream.  Leader: acc1[buffer][sub] = A(256 rows, d) * W1sub(d, H), one pair tile
// after another; a stage is used once the leader's barrier has the leader's own arrivals
// and the peer's relay.  Peer: forwards "this CTA's stage is full" to the leader's barriers.
__device__ void role_mma1(const Params& p, Ctl* c, uint32_t ringA, uint32_t ringB, uint32_t tmem,
                          uint32_t rank) {
  volatile int* af = &c->abort_flag;
  const Geo& g = p.g;
  const uint32_t idesc1 = instr_desc(PAIR_M, g.nsubw);
  const uint64_t dA = smem_desc(ringA), dB = smem_desc(ringB);
  const uint32_t hi = (uint32_t)(dA >> 32), alo0 = (uint32_t)dA, blo0 = (uint32_t)dB;
  const uint32_t fullA = smem_u32(c->fullA), emptyA = smem_u32(c->emptyA);
  const uint32_t fullB = smem_u32(c->fullB), emptyB = smem_u32(c->emptyB);
  const bool la = g.nsub == 1, two = g.nsub == 2;
  const uint32_t na = g.na, nb = g.nb;
  const int kc1 = g.kc1, total = c->total_tiles;
  uint32_t sa = 0, pha = 0, sb = 0, phb = 0, i = 0;
  if (rank != 0) {
    for (int tile = blockIdx.x >> 1; tile < total; tile += gridDim.x >> 1) {
      for (int kc = 0; kc < kc1; ++kc) {
        for (int sub = 0; sub < g.nsub; ++sub) {
          if (!mbar_wait_fast(fullB + 8 * sb, phb, af, p.dev_status)) return;
          mbar_arrive_remote(fullB + 8 * sb, 0);
          if (++sb == nb) {
            sb = 0;
            phb ^= 1;
          }
        }
        if (!mbar_wait_fast(fullA + 8 * sa, pha, af, p.dev_status)) return;
        fence_proxy_async();      // gathered rows (cp.async) before the leader's MMA reads them
        mbar_arrive_remote(fullA + 8 * sa, 0);
        if (++sa == na) {
          sa = 0;
          pha ^= 1;
        }
      }
    }
    return;
  }
  for (int tile = blockIdx.x >> 1; tile < total; tile += gridDim.x >> 1, ++i) {
    const uint32_t b = la ? (i & 1) : 0;
    const uint32_t use = la ? (i >> 1) : i;              // how often this buffer was used
    const uint32_t acc = tmem + (la ? b * 128 : 0);
    // the epilogue warps of both CTAs must have read the previous contents of this buffer
    if (!mbar_wait_fast(smem_u32(&c->acc1_empty[b]), (use & 1) ^ 1, af, p.dev_status)) return;
    tc_fence_after();
    for (int kc = 0; kc < kc1; ++kc) {
      const uint32_t alo = alo0 + sa * (SLOT >> 4), blo = blo0 + sb * (HSLOT >> 4);
      if (!mbar_wait_fast(fullA + 8 * sa, pha, af, p.dev_status)) return;
      if (!mbar_wait_fast(fullB + 8 * sb, phb, af, p.dev_status)) return;
      tc_fence_after();
      if (!(p.withhold & 16))
#pragma unroll
      for (uint32_t k = 0; k < 4; ++k)
        umma2_bf16(acc, ((uint64_t)hi << 32) | (alo + 2 * k), ((uint64_t)hi << 32) | (blo + 2 * k),
                   idesc1, (kc | k) != 0);
      umma2_commit(emptyB + 8 * sb);
      if (++sb == nb) {
        sb = 0;
        phb ^= 1;
      }
      if (two) {
        const uint32_t blo1 = blo0 + sb * (HSLOT >> 4);
        if (!mbar_wait_fast(fullB + 8 * sb, phb, af, p.dev_status)) return;
        tc_fence_after();
#pragma unroll
        for (uint32_t k = 0; k < 4; ++k)
          umma2_bf16(acc + 128, ((uint64_t)hi << 32) | (alo + 2 * k),
                     ((uint64_t)hi << 32) | (blo1 + 2 * k), idesc1, (kc | k) != 0);
        umma2_commit(emptyB + 8 * sb);
        if (++sb == nb) {
          sb = 0;
          phb ^= 1;
        }
      }
      umma2_commit(emptyA + 8 * sa);
      if (++sa == na) {
        sa = 0;
        pha ^= 1;
      }
    }
    umma2_commit(smem_u32(&c->acc1_full[b]));
  }
}

// GEMM2 stream.  Leader: acc2[chunk & 1] = Hs(256 rows, H) * W2chunk(H, nd) for every chunk
// of a pair tile.  Peer: forwards its W2 stages' "full" events.
__device__ void role_mma2(const Params& p, Ctl* c, uint32_t ringB2, uint32_t hs, uint32_t tmem,
                          uint32_t rank) {
  volatile int* af = &c->abort_flag;
  const Geo& g = p.g;
  const uint32_t idesc2 = instr_desc(PAIR_M, g.nd);
  const uint64_t dB = smem_desc(ringB2), dH = smem_desc(hs);
  const uint32_t hi = (uint32_t)(dB >> 32), blo0 = (uint32_t)dB, hlo0 = (uint32_t)dH;
  const uint32_t fullB2 = smem_u32(c->fullB2), emptyB2 = smem_u32(c->emptyB2);
  const uint32_t nb2 = g.nb2;
  const int nc = g.nc, kc2 = g.kc2, total = c->total_tiles;
  uint32_t s = 0, ph = 0, accbits = 0, i = 0;
  if (rank != 0) {
    for (int tile = blockIdx.x >> 1; tile < total; tile += gridDim.x >> 1, ++i) {
      for (int q = 0; q < nc * kc2; ++q) {
        if (!mbar_wait_fast(fullB2 + 8 * s, ph, af, p.dev_status)) return;
        mbar_arrive_remote(fullB2 + 8 * s, 0);
        if (++s == nb2) {
          s = 0;
          ph ^= 1;
        }
      }
    }
    // the leader's last multicast arrival for this CTA (hidden tile released) has landed
    if (i > 0) mbar_wait_fast(smem_u32(&c->hs_empty), (i - 1) & 1, af, p.dev_status);
    return;
  }
  for (int tile = blockIdx.x >> 1; tile < total; tile += gridDim.x >> 1, ++i) {
    if (!mbar_wait_fast(smem_u32(&c->hs_full), i & 1, af, p.dev_status)) return;
    tc_fence_after();
    for (int nci = 0; nci < nc; ++nci) {
      const uint32_t buf = nci & 1;
      const uint32_t acc = tmem + 256 + buf * 128;
      for (int k2 = 0; k2 < kc2; ++k2) {
        const uint32_t blo = blo0 + s * (HSLOT >> 4), hlo = hlo0 + k2 * (SLOT >> 4);
        if (!mbar_wait_fast(fullB2 + 8 * s, ph, af, p.dev_status)) return;
        if (k2 == 0) {
          if (!mbar_wait_fast(smem_u32(&c->acc2_empty[buf]), ((accbits >> buf) & 1) ^ 1, af,
                              p.dev_status))
            return;
          accbits ^= 1u << buf;
        }
        tc_fence_after();
        const int ksteps = min(4, (g.K2 - k2 * 64) >> 4);
        if (!(p.withhold & 16))
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (k < ksteps)
            umma2_bf16(acc, ((uint64_t)hi << 32) | (hlo + 2 * k), ((uint64_t)hi << 32) | (blo + 2 * k),
                       idesc2, (k2 | k) != 0);
        umma2_commit(emptyB2 + 8 * s);
        if (++s == nb2) {
          s = 0;
          ph ^= 1;
        }
      }
      umma2_commit(smem_u32(&c->acc2_full[buf]));
    }
    umma2_commit(smem_u32(&c->hs_empty));
  }
  // every MMA of this launch has completed once the last hidden tile is released
  if (i > 0) mbar_wait_fast(smem_u32(&c->hs_empty), (i - 1) & 1, af, p.dev_status);
}

// 16 hidden columns as 8 packed bf16 pairs, with the upstream rounding points
// (T(x W1), + b1, activation, x T(x W_up)) done in packed bf16 arithmetic.
template <int ACT>
__device__ __forceinline__ void ep1_pairs(const uint32_t* v, const uint32_t* u, const uint32_t* bp,
                                          bool glu, uint32_t* w) {
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
    if (glu) {
      const __nv_bfloat162 uu =
          __floats2bfloat162_rn(__uint_as_float(u[2 * q]), __uint_as_float(u[2 * q + 1]));
      h = __hmul2_rn(h, uu);
    }
    w[q] = *reinterpret_cast<uint32_t*>(&h);
  }
}

// Warps 0-3: accumulator 1 -> bias, activation (x up-projection) -> bf16 hidden tile in this
// CTA's shared memory.  Thread = tile row = TMEM lane.  One lane per warp then tells the
// leader that the accumulator may be overwritten and that the hidden tile is ready.
__device__ void role_ep1(const Params& p, Ctl* c, uint32_t hs, uint32_t tmem, int et,
                         uint32_t rank) {
  volatile int* af = &c->abort_flag;
  const Geo& g = p.g;
  const int r = et, lane = et & 31;
  const uint32_t lane_base = (uint32_t)(r & ~31) << 16;
  const uint32_t hs_row = hs + (r >> 3) * 1024 + (r & 7) * 128;
  const bool la = g.nsub == 1;
  uint32_t* bias_p = reinterpret_cast<uint32_t*>(c->bias_s);   // [2][64] packed pairs
  const int npair = g.nsubw >> 1;
  uint32_t i = 0;
  for (int tile = blockIdx.x >> 1; tile < c->total_tiles; tile += gridDim.x >> 1, ++i) {
    const Tile t = tile_info(p, c, tile, rank);
    uint32_t* bp = bias_p + (i & 1) * 64;
    if (et < npair) {
      const float2 b = __ldg(reinterpret_cast<const float2*>(p.packed + (long long)t.e * g.stride +
                                                             g.bias_off) + et);
      bp[et] = pack_bf16x2(b.x, b.y);
    }
    asm volatile("bar.sync 2, 128;" ::: "memory");
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
        case D2D_RELU: ep1_pairs<D2D_RELU>(v, u, bb, p.glu != 0, w); break;
        case D2D_GELU: ep1_pairs<D2D_GELU>(v, u, bb, p.glu != 0, w); break;
        case D2D_TANH: ep1_pairs<D2D_TANH>(v, u, bb, p.glu != 0, w); break;
        case D2D_LEAKY_RELU: ep1_pairs<D2D_LEAKY_RELU>(v, u, bb, p.glu != 0, w); break;
        default: ep1_pairs<D2D_GELU_TANH>(v, u, bb, p.glu != 0, w); break;
      }
      const uint32_t base = hs_row + (c0 >> 6) * SLOT;
      const int j0 = (c0 & 63) >> 3;
      st_shared_v4(base + (((j0) ^ (r & 7)) << 4), w[0], w[1], w[2], w[3]);
      st_shared_v4(base + (((j0 + 1) ^ (r & 7)) << 4), w[4], w[5], w[6], w[7]);
    }
    tc_fence_before();
    fence_proxy_async();     // ordinary shared stores -> visible to the MMA's async reads
    __syncwarp();
    if (lane == 0) {
      mbar_arrive_remote(smem_u32(&c->acc1_empty[b1]), 0);     // acc1 buffer read completely
      mbar_arrive_remote(smem_u32(&c->hs_full), 0);
    }
  }
}

// Warps 4-7: accumulator 2 -> bf16 -> staging blocks of this CTA.
__device__ void role_ep2(const Params& p, Ctl* c, uint32_t stg, uint32_t tmem, int et) {
  volatile int* af = &c->abort_flag;
  const Geo& g = p.g;
  const int lane = et & 31, q = et >> 5;
  const uint32_t lane_base = (uint32_t)(et & ~31) << 16;
  const int halves = g.nd >> 6;
  uint32_t phbits = 0, n = 0;
  for (int tile = blockIdx.x >> 1; tile < c->total_tiles; tile += gridDim.x >> 1) {
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
          __syncwarp();
          if (lane == 0) mbar_arrive_remote(smem_u32(&c->acc2_empty[buf]), 0);
        }
        const uint32_t blk = n & 1;
        if (!mbar_wait_fast(smem_u32(&c->sempty[blk][q]), ((n >> 1) & 1) ^ 1, af, p.dev_status))
          return;
        const uint32_t dst = stg + (blk * 4 + q) * 4096 + lane * 128;
#pragma unroll
        for (int pc = 0; pc < 8; ++pc) {      // piece XOR row: conflict-free 16-byte stores
          uint32_t ww[4];
#pragma unroll
          for (int k = 0; k < 4; ++k)
            ww[k] = pack_bf16x2(__uint_as_float(v[8 * pc + 2 * k]),
                                __uint_as_float(v[8 * pc + 2 * k + 1]));
          st_shared_v4(dst + ((pc ^ (lane & 7)) << 4), ww[0], ww[1], ww[2], ww[3]);
        }
        mbar_arrive(smem_u32(&c->sfull[blk][q]));
      }
    }
  }
}

// Writer warps: warp q adds the staged bf16 blocks of row quarter q to the output rows,
// read back row-contiguous so that one red instruction touches 4 cache lines.
__device__ void role_writer(const Params& p, Ctl* c, uint32_t stg, int wt, uint32_t rank) {
  volatile int* af = &c->abort_flag;
  const Geo& g = p.g;
  const int lane = wt & 31, q = wt >> 5;
  const int rl = lane >> 3, pl = lane & 7;
  const int halves = g.nd >> 6;
  uint32_t n = 0;
  int tile = blockIdx.x >> 1;
  const int total = c->total_tiles, step = gridDim.x >> 1;
  Tile t = {0, 0, 0};
  long long tok = -1;
  if (tile < total) {
    t = tile_info(p, c, tile, rank);
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
    tok = -1;      // rows of the next tile: the load is in flight while this tile is written
    if (tile + step < total) {
      t = tile_info(p, c, tile + step, rank);
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
          if (orow[it] && !(p.withhold & 2))
            red_add_bf16x8(orow[it] + col, val[it].x, val[it].y, val[it].z, val[it].w);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(NTHREADS, 1) experts_pair_kernel(const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - raw);
  const Geo& g = p.g;
  const uint32_t ringA = base;
  const uint32_t ringB = ringA + g.na * SLOT;
  const uint32_t ringB2 = ringB + g.nb * HSLOT;
  const uint32_t hs = ringB2 + g.nb2 * HSLOT;          // (na*2 + nb + nb2) * 8 KB: 1 KB aligned
  const uint32_t stg = hs + g.kc2 * SLOT;
  Ctl* c = reinterpret_cast<Ctl*>(aligned + (size_t)(g.na + g.kc2 + 2) * SLOT +
                                  (size_t)(g.nb + g.nb2) * HSLOT);
  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t rank = cluster_ctarank();
  grid_launch_dependents();

  if (tid == 0) {
    // barriers of the leader that also count the peer: +1 relay arrival on the "full"
    // barriers; the epilogue hand-backs get one arrival per warp from both CTAs
    const uint32_t extra = rank == 0 ? 1 : 0;
    for (int i = 0; i < NA_MAX; ++i) {
      mbar_init(smem_u32(&c->fullA[i]), 128 + extra);
      mbar_init(smem_u32(&c->emptyA[i]), 1);
    }
    for (int i = 0; i < NB_MAX; ++i) {
      mbar_init(smem_u32(&c->fullB[i]), 1 + extra);
      mbar_init(smem_u32(&c->emptyB[i]), 1);
      mbar_init(smem_u32(&c->fullB2[i]), 1 + extra);
      mbar_init(smem_u32(&c->emptyB2[i]), 1);
    }
    mbar_init(smem_u32(&c->hs_full), 8);
    mbar_init(smem_u32(&c->hs_empty), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&c->acc1_full[i]), 1);
      mbar_init(smem_u32(&c->acc1_empty[i]), 8);
      mbar_init(smem_u32(&c->acc2_full[i]), 1);
      mbar_init(smem_u32(&c->acc2_empty[i]), 8);
      for (int q = 0; q < 4; ++q) {
        mbar_init(smem_u32(&c->sfull[i][q]), 32);
        mbar_init(smem_u32(&c->sempty[i][q]), 32);
      }
    }
    c->abort_flag = 0;
    c->wait_limit = (int)p.wait_limit;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  grid_dependency_wait();
  if (warp == 1) {
    // pair-tile tables: all offsets loaded in parallel (lane l owns experts 4l..4l+3),
    // exclusive scans across the warp of the full-tile counts and of the tail flags
    const int lane = tid & 31;
    int off[5], nt[4], pt[4], sum = 0, psum = 0;
#pragma unroll
    for (int q = 0; q < 5; ++q) {
      const int e = 4 * lane + q;
      off[q] = e <= p.E ? p.offsets[e] : 0;
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int e = 4 * lane + q;
      const int n = e < p.E ? off[q + 1] - off[q] : 0;
      if (e < p.E && (n < 0 || off[q + 1] > p.N * (long long)p.E))
        report(p.dev_status, D2D_ERR_INDEX_RANGE);
      nt[q] = n > 0 ? n / PAIR_M : 0;
      pt[q] = (n > 0 && n % PAIR_M != 0) ? 1 : 0;
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
    if (lane == 31) {
      c->total_full = incl;
      c->total_tiles = incl + pincl;
    }
  }
  if (warp == WARP_MMA1) tmem_alloc2(smem_u32(&c->tmem_base), 512);
  tc_fence_before();
  __syncthreads();
  // both CTAs' barriers are initialised before any remote arrival or multicast commit
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem = c->tmem_base;

  if (warp < 4) {
    role_ep1(p, c, hs, tmem, tid, rank);
  } else if (warp < 8) {
    role_ep2(p, c, stg, tmem, tid - 128);
  } else if (warp == WARP_MMA1) {
    if (elect_one()) role_mma1(p, c, ringA, ringB, tmem, rank);
    __syncwarp();
  } else if (warp == WARP_MMA2) {
    if (elect_one()) role_mma2(p, c, ringB2, hs, tmem, rank);
    __syncwarp();
  } else if (warp == WARP_BULK) {
    if (elect_one()) role_bulk(p, c, ringB, ringB2, rank);
    __syncwarp();
  } else if (warp < WARP_WR0) {
    role_producer(p, c, ringA, tid - WARP_PROD0 * 32, rank);
    cp_async_wait_all();
  } else {
    role_writer(p, c, stg, tid - WARP_WR0 * 32, rank);
  }

  // A launch that gave up may still have copies and MMAs in flight that use the shared and
  // tensor memory of both CTAs: give them time to land before either is released.
  if (*reinterpret_cast<volatile int*>(&c->abort_flag) != 0)
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  tc_fence_before();
  __syncthreads();
  // neither CTA leaves (or frees tensor memory) while its partner may still arrive on its
  // barriers or have MMAs reading its shared memory
  cluster_sync_all();
  if (warp == WARP_MMA1) {
    tc_fence_after();
    tmem_dealloc2(tmem, 512);
  }
}

// ---------------------------------------------------------------------------
// launch
// ---------------------------------------------------------------------------
constexpr int MAX_DEVICES = 64;
struct DeviceFacts {
  int pairs = -1;            // CTA pairs that can be resident at once (0 = cannot launch)
  size_t smem_optin = 0;
};
DeviceFacts g_dev[MAX_DEVICES];
std::mutex g_dev_lock;

size_t smem_bytes(const Geo& g) {
  return 1024 + (size_t)(g.na + g.kc2 + 2) * SLOT + (size_t)(g.nb + g.nb2) * HSLOT + sizeof(Ctl) +
         64;
}

static_assert(1024 + (size_t)14 * SLOT + sizeof(Ctl) + 64 <= 232448,
              "shared-memory plan exceeds the 227 KB a CTA may use");

}  // namespace

bool pair_experts_supported(int d, int E, int H, bool glu, int dtype) {
  return umma_experts_supported(d, E, H, glu, dtype);
}

int launch_experts_pair(const void* x, const int32_t* token_idx, const int32_t* offsets,
                        const void* packed, void* out, int64_t N, int d, int E, int H, bool glu,
                        int act, int* dev_status, uint32_t wait_limit, int withhold,
                        cudaStream_t s) {
  Params p = {};
  p.x = (const bf16*)x;
  p.N = N;
  p.d = d;
  p.packed = (const uint8_t*)packed;
  p.g = pair_geo(d, H, glu);
  p.token_idx = token_idx;
  p.offsets = offsets;
  p.E = E;
  p.out = (bf16*)out;
  p.act = act;
  p.glu = glu ? 1 : 0;
  p.dev_status = dev_status;
  p.wait_limit = wait_limit;
  p.withhold = withhold;
  const size_t smem = smem_bytes(p.g);
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    cudaGetLastError();
    return D2D_ERR_NO_DEVICE;
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.blockDim = dim3(NTHREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cfg.attrs = attr;
  int pairs = 0;
  {
    std::lock_guard<std::mutex> hold(g_dev_lock);
    DeviceFacts& f = g_dev[dev];
    if (f.smem_optin < smem) {
      if (cudaFuncSetAttribute(experts_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return D2D_ERR_LAUNCH;
      }
      f.smem_optin = smem;
      f.pairs = -1;
    }
    if (f.pairs < 0) {
      int sms = 0, n = 0;
      if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        sms = 0;
      cfg.gridDim = dim3((unsigned)(sms > 1 ? sms & ~1 : 2));
      cfg.numAttrs = 1;      // the occupancy query looks at the cluster shape only
      if (cudaOccupancyMaxActiveClusters(&n, experts_pair_kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
      }
      f.pairs = n < sms / 2 ? n : sms / 2;
    }
    pairs = f.pairs;
  }
  if (pairs < 1) return D2D_ERR_UNSUPPORTED;
  if (getenv("D2D_DEBUG")) fprintf(stderr, "pair kernel: %d resident pairs, smem %zu\n", pairs, smem);
  const long long max_tiles = (N * (long long)E + PAIR_M - 1) / PAIR_M + E;
  long long np = max_tiles < pairs ? max_tiles : pairs;
  if (np < 1) np = 1;
  cfg.gridDim = dim3((unsigned)(2 * np));
  cfg.numAttrs = 2;
  if (cudaLaunchKernelEx(&cfg, experts_pair_kernel, p) == cudaSuccess) return D2D_OK;
  cudaGetLastError();
  return D2D_ERR_LAUNCH;
}

}  // namespace d2d
