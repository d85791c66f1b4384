/*
 * Plain-C restatement of the reference's CPU path for the GLQ compressed-weight matmul.
 * TEST INFRASTRUCTURE ONLY: the checker for the CUDA kernels and the timed CPU baseline of the
 * benchmark.  Nothing on the product path links or calls this file.
 *
 * Parity status: PINNED — tests/test_oracle_c.py checks every function here bit-for-bit against
 * the numpy oracle (oracle/glq_oracle.py), which is itself pinned to outputs of the reference
 * stored in tests/golden/.
 *
 * Citations are paths inside the cnygaard/glq project.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- fp16 <-> fp32 (IEEE binary16, round to nearest even) -------------------------------- */
static float h2f(uint16_t h) {
  uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 0x1F, m = h & 0x3FF, u;
  if (e == 0) {
    if (m == 0) u = s;
    else {
      int sh = 0;
      while (!(m & 0x400)) { m <<= 1; ++sh; }
      u = s | ((uint32_t)(127 - 15 - sh + 1) << 23) | ((m & 0x3FF) << 13);
    }
  } else if (e == 31) u = s | 0x7F800000u | (m << 13);
  else u = s | ((e + 112) << 23) | (m << 13);
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static uint16_t f2h(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint32_t s = (u >> 16) & 0x8000u;
  int32_t e = (int32_t)((u >> 23) & 0xFF) - 127 + 15;
  uint32_t m = u & 0x7FFFFFu;
  if (((u >> 23) & 0xFF) == 0xFF) return (uint16_t)(s | 0x7C00u | (m ? 0x200u : 0));
  if (e >= 31) return (uint16_t)(s | 0x7C00u);
  if (e <= 0) {
    if (e < -10) return (uint16_t)s;
    m |= 0x800000u;
    int sh = 14 - e;
    uint32_t r = m >> sh, rem = m & ((1u << sh) - 1), half = 1u << (sh - 1);
    if (rem > half || (rem == half && (r & 1))) ++r;
    return (uint16_t)(s | r);
  }
  uint32_t r = (uint32_t)(e << 10) | (m >> 13), rem = m & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) ++r;
  return (uint16_t)(s | r);
}

/* ---- 3INST decode: glq/trellis.py:122-134 -------------------------------------------------- */
uint16_t glqo_decode_3inst(uint32_t state) {
  uint32_t h = (state & 0xFFFFu) * 89226354u + 64248484u;
  uint32_t r = (h & 0x8FFF8FFFu) ^ 0x3B603B60u;
  /* both halves are read as fp16 and added in fp16: the exact sum of two fp16 values fits a float,
     so rounding that float to fp16 once is the fp16 addition */
  return f2h(h2f((uint16_t)(r >> 16)) + h2f((uint16_t)(r & 0xFFFFu)));
}

/* ---- trellis kernel layout -> dense fp16 (m, n): glq/trellis.py:629-643 with :580-602, :486-523
 * group (rp, cp) of 2x2 tiles = 128*K bytes indexed (lane, ni, mi, byte); a lane's K bytes are a
 * little-endian chunk of 8K bits; a tile's stream is its 32 chunks MSB-first, cyclic; weight
 * p = 8*lane + j has state = stream bits [pK, pK+16); (lane, j) -> row 8a+g, col 8c+2t+e. */
void glqo_trellis_decode(const uint8_t* packed, int m, int n, int K, uint16_t* out /* (m, n) fp16 bits */) {
  const int RP = m / 32, CP = n / 32;
#pragma omp parallel for collapse(2) schedule(static)
  for (int rp = 0; rp < RP; ++rp) {
    for (int cp = 0; cp < CP; ++cp) {
      const uint8_t* g = packed + ((size_t)rp * CP + cp) * 128 * K;
      for (int ni = 0; ni < 2; ++ni)
        for (int mi = 0; mi < 2; ++mi) {
          uint8_t bits[256 * 4 + 16];
          for (int lane = 0; lane < 32; ++lane) {
            uint32_t chunk = 0;
            for (int b = 0; b < K; ++b) chunk |= (uint32_t)g[((lane * 2 + ni) * 2 + mi) * K + b] << (8 * b);
            for (int b = 0; b < 8 * K; ++b) bits[lane * 8 * K + b] = (chunk >> (8 * K - 1 - b)) & 1;
          }
          for (int b = 0; b < 16; ++b) bits[256 * K + b] = bits[b];
          for (int lane = 0; lane < 32; ++lane)
            for (int j = 0; j < 8; ++j) {
              const int p = lane * 8 + j;
              uint32_t st = 0;
              for (int b = 0; b < 16; ++b) st = (st << 1) | bits[p * K + b];
              const int gq = lane >> 2, t = lane & 3, c = (j >> 2) & 1, a = (j >> 1) & 1, e = j & 1;
              const int row = rp * 32 + mi * 16 + 8 * a + gq, col = cp * 32 + ni * 16 + 8 * c + 2 * t + e;
              out[(size_t)row * n + col] = glqo_decode_3inst(st);
            }
        }
    }
  }
}

/* W = dec1 + dec2 * s2 in fp32 (multiply then add): glq/trellis.py:923-933 */
void glqo_trellis_decode_f32(const uint8_t* p1, int K1, const uint8_t* p2, int K2, float s2, int m, int n,
                             float* out) {
  uint16_t* t = (uint16_t*)malloc((size_t)m * n * 2);
  glqo_trellis_decode(p1, m, n, K1, t);
#pragma omp parallel for schedule(static)
  for (long i = 0; i < (long)m * n; ++i) out[i] = h2f(t[i]);
  if (p2) {
    glqo_trellis_decode(p2, m, n, K2, t);
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)m * n; ++i) {
      volatile float prod = h2f(t[i]) * s2;     /* keep the product rounded: no fused multiply-add */
      out[i] = out[i] + prod;
    }
  }
  free(t);
}

/* ---- E8 shell: glq/codebook.py:280-282, N-stage sum glq/quantized_linear.py:1177-1194 ------- */
void glqo_e8_decode(const uint16_t* const* q, const uint32_t* const* table, const int* entries,
                    const float* scale, int n_stages, int m, int n, float* out) {
  const long total = (long)m * (n / 8);
#pragma omp parallel for schedule(static)
  for (long i = 0; i < total; ++i) {
    float v[8];
    uint32_t e = table[0][q[0][i] % (uint32_t)entries[0]];
    for (int k = 0; k < 8; ++k) v[k] = (float)((e >> (4 * k)) & 0xF) * 0.5f - 3.0f;
    for (int s = 1; s < n_stages; ++s) {
      e = table[s][q[s][i] % (uint32_t)entries[s]];
      for (int k = 0; k < 8; ++k) {
        volatile float prod = ((float)((e >> (4 * k)) & 0xF) * 0.5f - 3.0f) * scale[s];
        v[k] = v[k] + prod;
      }
    }
    memcpy(out + i * 8, v, sizeof v);
  }
}

/* ---- Walsh-Hadamard: glq/hadamard.py:10-28 (ascending distance, a+b / a-b, one 1/sqrt(n)) --- */
void glqo_fht(float* x, int n) {
  for (int h = 1; h < n; h <<= 1)
    for (int i = 0; i < n; i += 2 * h)
      for (int j = i; j < i + h; ++j) {
        float a = x[j], b = x[j + h];
        x[j] = a + b;
        x[j + h] = a - b;
      }
  const float d = sqrtf((float)n);
  for (int i = 0; i < n; ++i) x[i] = x[i] / d;
}

void glqo_block_fht(float* x, const int* blocks, int n_blocks) {
  int off = 0;
  for (int b = 0; b < n_blocks; ++b) { glqo_fht(x + off, blocks[b]); off += blocks[b]; }
}

/* ---- layer: y = [SU * H_m(wscale * W (H_n(SV * pad(x))))][:out]
 * glq/quantized_linear.py:1149-1154, 1176-1195, 1225-1231 (E8) and :986-1010 (trellis) ---------- */
void glqo_linear_forward(const float* x, int B, int in_f, const float* W, int m, int n, const uint16_t* su,
                         const uint16_t* sv, float wscale, const int* blocks_n, int nbn, const int* blocks_m,
                         int nbm, int out_f, float* y /* (B, out_f) */) {
  float* xr = (float*)calloc((size_t)B * n, sizeof(float));
  float* yr = (float*)malloc((size_t)B * m * sizeof(float));
  for (int b = 0; b < B; ++b) {
    for (int i = 0; i < in_f; ++i) xr[(size_t)b * n + i] = x[(size_t)b * in_f + i] * h2f(sv[i]);
    glqo_block_fht(xr + (size_t)b * n, blocks_n, nbn);
  }
#pragma omp parallel for schedule(static)
  for (int r = 0; r < m; ++r)
    for (int b = 0; b < B; ++b) {
      double acc = 0.0;
      const float* w = W + (size_t)r * n;
      const float* xv = xr + (size_t)b * n;
      for (int i = 0; i < n; ++i) acc += (double)w[i] * xv[i];
      yr[(size_t)b * m + r] = (float)acc * wscale;
    }
  for (int b = 0; b < B; ++b) {
    glqo_block_fht(yr + (size_t)b * m, blocks_m, nbm);
    for (int r = 0; r < out_f; ++r) y[(size_t)b * out_f + r] = yr[(size_t)b * m + r] * h2f(su[r]);
  }
  free(xr);
  free(yr);
}

/* One whole trellis linear from packed storage (decode every call, as the reference's CPU path
 * does, glq/quantized_linear.py:986-1010): the unit the CPU baseline times. */
void glqo_trellis_linear(const float* x, int B, const uint8_t* p1, int K1, const uint8_t* p2, int K2, float s2,
                         int m, int n, const uint16_t* su, const uint16_t* sv, float wscale, const int* blocks_n,
                         int nbn, const int* blocks_m, int nbm, float* y) {
  float* W = (float*)malloc((size_t)m * n * sizeof(float));
  glqo_trellis_decode_f32(p1, K1, p2, K2, s2, m, n, W);
  glqo_linear_forward(x, B, n, W, m, n, su, sv, wscale, blocks_n, nbn, blocks_m, nbm, m, y);
  free(W);
}

void glqo_e8_linear(const float* x, int B, int in_f, const uint16_t* const* q, const uint32_t* const* table,
                    const int* entries, const float* scale, int n_stages, int m, int n, const uint16_t* su,
                    const uint16_t* sv, float wscale, const int* blocks_n, int nbn, const int* blocks_m, int nbm,
                    int out_f, float* y) {
  float* W = (float*)malloc((size_t)m * n * sizeof(float));
  glqo_e8_decode(q, table, entries, scale, n_stages, m, n, W);
  glqo_linear_forward(x, B, in_f, W, m, n, su, sv, wscale, blocks_n, nbn, blocks_m, nbm, out_f, y);
  free(W);
}
