/*
 * C restatement of the integer stages of the D2DMoE MoE-FFN layer.  TEST INFRASTRUCTURE ONLY:
 * it checks the CUDA path (tests, smoke); nothing in the product links or calls it.
 *
 *   d2d_oracle_mask_*   the 'dynk_max' rule of MoeficationMoE.gate
 *                       (architectures/moe/moefication.py:80-85): keep expert e iff
 *                       s_e >= T(max_e(s) * mult), mult = (float)(1.0 - tau); the row max
 *                       propagates NaN like torch.max, the threshold is rounded to the
 *                       score dtype T before the comparison.
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
