/*
 * CPU restatement, in plain C, of the two tile programs of the hot path, step by
 * step as the reference writes them.  TEST INFRASTRUCTURE ONLY: nothing in the
 * product links or calls this file.
 *
 *  - tile_gemm: reference tests/gemm_baseline_v2.py:62-88 -- zero accumulator;
 *    for each k-tile: load A and B tiles, acc = A_tile * B_tile + acc (MMA
 *    semantics: warpir/ir/ops.py:78-83, bf16 operands, fp32 accumulate); store
 *    the accumulator rounded to bf16.
 *  - tile_attention: reference tests/attention_baseline.py:147-177 -- per KV tile:
 *    S = Q K^T; m_prev = m; m = max(m, rowmax S); P = 2^(S c - m c);
 *    corr = 2^(m_prev c - m c); l = l corr + rowsum P (fp32 P); O = O corr;
 *    O += bf16(P) V; after the loop O / l.  c = scale * log2(e).  Extended, as the
 *    measured workloads need, with a causal mask and LSE = m c ln2 + ln l.
 *
 * bf16 values travel as uint16 bit patterns.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static uint16_t f32_to_bf16(float f) { /* round to nearest even */
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* C[M,N] = A[M,K] * B ; b_layout 0: B[K,N], 1: B[N,K].  tile = k-tile extent. */
void tile_gemm(const uint16_t* A, const uint16_t* B, uint16_t* C, int M, int N, int K, int b_layout, int tile) {
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      float acc = 0.f; /* ZeroOp */
      for (int k0 = 0; k0 < K; k0 += tile) { /* ForOp over k-tiles */
        float part = 0.f;
        int k1 = k0 + tile < K ? k0 + tile : K;
        for (int k = k0; k < k1; ++k) {
          float b = b_layout ? bf16_to_f32(B[(size_t)j * K + k]) : bf16_to_f32(B[(size_t)k * N + j]);
          part += bf16_to_f32(A[(size_t)i * K + k]) * b;
        }
        acc += part; /* MMAOp: a @ b + accum */
      }
      C[(size_t)i * N + j] = f32_to_bf16(acc); /* TMAStoreOp into a bf16 global */
    }
}

/* One head.  Q[S,D], K[S,D], V[S,D] bf16 -> O[S,D] bf16, LSE[S] fp32 (may be NULL). */
void tile_attention(const uint16_t* Q, const uint16_t* K, const uint16_t* V, uint16_t* O, float* LSE, int S, int D,
                    float scale, int causal, int block_q, int block_kv) {
  const float c = scale * 1.44269504089f;
  float* s = (float*)malloc(sizeof(float) * block_kv);
  float* o = (float*)malloc(sizeof(float) * D);
  for (int i = 0; i < S; ++i) {
    (void)block_q; /* rows are independent; the Q tiling does not change the arithmetic */
    float m = -INFINITY, l = 0.f;
    for (int d = 0; d < D; ++d) o[d] = 0.f;
    const int last = causal ? i : S - 1;
    for (int j0 = 0; j0 <= last; j0 += block_kv) {
      const int j1 = j0 + block_kv < S ? j0 + block_kv : S;
      float m_prev = m; /* CopyOp before RowMaxOp */
      for (int j = j0; j < j1; ++j) {
        float acc = 0.f;
        for (int d = 0; d < D; ++d) acc += bf16_to_f32(Q[(size_t)i * D + d]) * bf16_to_f32(K[(size_t)j * D + d]);
        s[j - j0] = (causal && j > i) ? -INFINITY : acc;
        if (s[j - j0] > m) m = s[j - j0]; /* RowMaxOp with prev */
      }
      const float corr = exp2f(m_prev * c - m * c); /* Exp2Op(SubOp(max_prev_sc, max_new_sc)) */
      float rowsum = 0.f;
      for (int d = 0; d < D; ++d) o[d] *= corr; /* MulRowOp */
      for (int j = j0; j < j1; ++j) {
        const float p = exp2f(s[j - j0] * c - m * c); /* SubRowOp + Exp2Op */
        rowsum += p;                                   /* RowSumOp sums the fp32 P */
        const float pb = bf16_to_f32(f32_to_bf16(p));  /* CopyOp fp32 -> bf16 */
        for (int d = 0; d < D; ++d) o[d] += pb * bf16_to_f32(V[(size_t)j * D + d]);
      }
      l = l * corr + rowsum; /* MulOp + RowSumOp(prev) */
    }
    for (int d = 0; d < D; ++d) O[(size_t)i * D + d] = f32_to_bf16(o[d] / l); /* DivRowOp + store */
    if (LSE) LSE[i] = m * c * 0.6931471805599453f + logf(l);
  }
  free(s);
  free(o);
}
