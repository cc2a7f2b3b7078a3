/*
 * C restatement of the integer stages of the D2DMoE MoE-FFN layer.  TEST INFRASTRUCTURE ONLY:
 * it checks the CUDA path (tests, smoke); nothing in the product links or calls it.
 *
 *   d2d_oracle_mask_*   the 'dynk_max' rule of MoeficationMoE.gate
 *                       (architectures/moe/moefication.py:80-85): keep expert e iff
 *                       s_e >= T(max_e(s) * mult), mult = (float)(1.0 - tau); the row max
 *                       propagates NaN like torch.max, the threshold is rounded to the
 *                       score dtype T before the comparison.
 *   d2d_oracle_rule_*   the 'topk' and cumulative 'dynk' rules of the same gate
 *                       (architectures/moe/moefication.py:59-79) on given scores.
 *   d2d_oracle_compact  per-expert token lists and offsets: the set the upstream index
 *                       preparation selects (architectures/moe/moe_layers.py:241-249: first
 *                       bincount[e] rows of a descending argsort of column e), listed in
 *                       ascending token order.
 *
 * Pinned by tests/test_oracle_golden.py against routing tensors produced by the upstream
 * modules (tests/golden).  Build: gcc -O2 -shared -fPIC oracle/d2d_oracle.c -o oracle/_build/libd2d_oracle.so
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static float bf16_to_f(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* round-to-nearest-even fp32 -> bf16 -> fp32, NaN kept */
static float round_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return f;
  u += 0x7fffu + ((u >> 16) & 1u);
  u &= 0xffff0000u;
  memcpy(&f, &u, 4);
  return f;
}

static void mask_row(const float* s, int E, float mult, int is_bf16, uint32_t* words) {
  int nw = (E + 31) / 32;
  float m = -INFINITY;
  int nan = 0;
  for (int e = 0; e < E; ++e) {
    if (s[e] != s[e]) nan = 1;
    if (s[e] > m) m = s[e];
  }
  if (nan) m = NAN;
  volatile float prod = m * mult; /* one fp32 multiply, no contraction */
  float thr = is_bf16 ? round_bf16(prod) : prod;
  for (int j = 0; j < nw; ++j) words[j] = 0;
  for (int e = 0; e < E; ++e)
    if (s[e] >= thr) words[e >> 5] |= 1u << (e & 31);
}

void d2d_oracle_mask_f32(const float* scores, float mult, uint32_t* bits, long N, int E) {
  int nw = (E + 31) / 32;
  for (long t = 0; t < N; ++t) mask_row(scores + t * E, E, mult, 0, bits + t * nw);
}

void d2d_oracle_mask_bf16(const uint16_t* scores, float mult, uint32_t* bits, long N, int E) {
  int nw = (E + 31) / 32;
  float row[256];
  for (long t = 0; t < N; ++t) {
    for (int e = 0; e < E; ++e) row[e] = bf16_to_f(scores[t * E + e]);
    mask_row(row, E, mult, 1, bits + t * nw);
  }
}

/* descending order used by both rules below: NaN first, equal values by ascending index
 * (what torch.topk / torch.sort return on the host for the fixtures' inputs; which member of a
 * group of equal values comes first is not defined upstream) */
static int before(float a, int ia, float b, int ib) {
  int an = a != a, bn = b != b;
  if (an || bn) return an && (!bn || ia < ib);
  return a > b || (a == b && ia < ib);
}

/* rule 1 = 'topk' (architectures/moe/moefication.py:59-63): keep the k largest scores.
 * rule 2 = 'dynk' (architectures/moe/moefication.py:64-79): shares = T(s / T(sum s)); experts in
 * descending share order; keep the first and every further one while the cumulative share
 * before it, accumulated in torch.cumsum's host accumulation type (double for fp32, float for
 * bf16) and rounded to T per element, is < T(tau). */
static void rule_row(const float* s_in, int E, int rule, int k, float tau, int is_bf16,
                     uint32_t* words) {
  float s[256];
  int rank[256];
  int nw = (E + 31) / 32;
  for (int e = 0; e < E; ++e) s[e] = s_in[e];
  if (rule == 2) {
    float tot = 0.f;
    for (int e = 0; e < E; ++e) tot += s[e];
    if (is_bf16) tot = round_bf16(tot);
    for (int e = 0; e < E; ++e) {
      volatile float q = s[e] / tot;
      s[e] = is_bf16 ? round_bf16(q) : q;
    }
  }
  for (int i = 0; i < E; ++i) {
    int r = 0;
    for (int j = 0; j < E; ++j)
      if (j != i && before(s[j], j, s[i], i)) ++r;
    rank[i] = r;
  }
  for (int j = 0; j < nw; ++j) words[j] = 0;
  if (rule == 1) {
    for (int e = 0; e < E; ++e)
      if (rank[e] < k) words[e >> 5] |= 1u << (e & 31);
    return;
  }
  float sorted[256];
  int more[256]; /* more[r]: the expert of rank r is kept */
  for (int e = 0; e < E; ++e) sorted[rank[e]] = s[e];
  float tau_t = is_bf16 ? round_bf16(tau) : tau;
  double accd = 0.0;
  float accf = 0.f;
  more[0] = 1;
  for (int r = 0; r + 1 < E; ++r) {
    float c;
    if (is_bf16) {
      accf += sorted[r];
      c = round_bf16(accf);
    } else {
      accd += (double)sorted[r];
      c = (float)accd;
    }
    more[r + 1] = c < tau_t;
  }
  for (int e = 0; e < E; ++e)
    if (more[rank[e]]) words[e >> 5] |= 1u << (e & 31);
}

void d2d_oracle_rule_f32(const float* scores, int rule, int k, float tau, uint32_t* bits, long N,
                         int E) {
  int nw = (E + 31) / 32;
  for (long t = 0; t < N; ++t) rule_row(scores + t * E, E, rule, k, tau, 0, bits + t * nw);
}

void d2d_oracle_rule_bf16(const uint16_t* scores, int rule, int k, float tau, uint32_t* bits,
                          long N, int E) {
  int nw = (E + 31) / 32;
  float row[256];
  for (long t = 0; t < N; ++t) {
    for (int e = 0; e < E; ++e) row[e] = bf16_to_f(scores[t * E + e]);
    rule_row(row, E, rule, k, tau, 1, bits + t * nw);
  }
}

/* offsets[E+1], token_idx[sum of counts]; returns the total */
long d2d_oracle_compact(const uint32_t* bits, long N, int E, int32_t* offsets, int32_t* token_idx) {
  int nw = (E + 31) / 32;
  long pos = 0;
  for (int e = 0; e < E; ++e) {
    offsets[e] = (int32_t)pos;
    for (long t = 0; t < N; ++t)
      if ((bits[t * nw + (e >> 5)] >> (e & 31)) & 1u) token_idx[pos++] = (int32_t)t;
  }
  offsets[E] = (int32_t)pos;
  return pos;
}
