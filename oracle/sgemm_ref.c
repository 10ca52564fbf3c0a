/*
 * TEST INFRASTRUCTURE -- plain-C restatement of the GEMM on the Roller hot path.
 * Built by oracle/gemm_oracle.py (gcc) and used only by tests, the smoke check and the CPU
 * baseline; the product never links or loads it.
 *
 * oracle_sgemm_accumulate: what the reference's generated `gemm_kernel` computes -- the
 *   linalg.matmul payload C += A @ B on fp32 (src/roller.py:47-68, C zeroed by the host at
 *   src/roller.py:534), lowered to fp32 outer products / FMAs (src/roller.py:280-282) with the
 *   reduction walked in blocks of the hint's `rstep` (src/roller.py:93-342).
 * oracle_gemm_3xtf32: the arithmetic of the B200 3xTF32 kernels with an ideal per-chunk
 *   accumulator, to predict their error band on the CPU.
 * oracle_gemm_16bit: the arithmetic of the 16-bit-operand kernels (bf16 or fp16 A and B given as
 *   bit patterns): products exact, an ideal accumulator within a chunk of the reduction, chunk
 *   results rounded to fp32 and added in fp32.
 * Parity unpinned: the reference has no golden outputs for its kernel; both functions are
 *   checked against the fp64 product in tests/.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static float bits_to_float(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static uint32_t float_to_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

/* the 19 bits of an fp32 word the tensor core reads */
static float trunc19(float x) { return bits_to_float(float_to_bits(x) & 0xFFFFE000u); }

/* x - trunc19(x), rounded to nearest on the 19-bit grid; nan for inf/nan (inf - inf) */
float oracle_split_small(float x) {
  float s = x - trunc19(x);
  return bits_to_float((float_to_bits(s) + 0x1000u) & 0xFFFFE000u);
}

void oracle_sgemm_accumulate(const float* A, const float* B, float* C, int M, int N, int K,
                             int rstep) {
  if (rstep < 1) rstep = 1;
  for (int k0 = 0; k0 < K; k0 += rstep) {
    int k1 = k0 + rstep < K ? k0 + rstep : K;
    for (int i = 0; i < M; ++i)
      for (int j = 0; j < N; ++j) {
        float acc = C[(size_t)i * N + j];
        for (int k = k0; k < k1; ++k) acc = fmaf(A[(size_t)i * K + k], B[(size_t)k * N + j], acc);
        C[(size_t)i * N + j] = acc;
      }
  }
}

void oracle_gemm_3xtf32(const float* A, const float* B, float* C, int M, int N, int K, int chunk) {
  if (chunk < 1) chunk = K;
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      float sum = 0.0f;
      for (int k0 = 0; k0 < K; k0 += chunk) {
        int k1 = k0 + chunk < K ? k0 + chunk : K;
        double part = 0.0;
        for (int k = k0; k < k1; ++k) {
          float a = A[(size_t)i * K + k], b = B[(size_t)k * N + j];
          double ab = trunc19(a), bb = trunc19(b);
          double as = oracle_split_small(a), bs = oracle_split_small(b);
          part += as * bb + ab * bs + ab * bb;
        }
        sum += (float)part;
      }
      C[(size_t)i * N + j] = sum;
    }
}

/* bf16 / fp16 bit patterns -> the values they denote */
static float bf16_value(uint16_t b) { return bits_to_float((uint32_t)b << 16); }
static float f16_value(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
  if (exp == 0) return (sign ? -1.0f : 1.0f) * ldexpf((float)man, -24);       /* zero, subnormal */
  if (exp == 31) return bits_to_float(sign | 0x7F800000u | (man << 13));       /* inf, nan */
  return bits_to_float(sign | ((exp + 112u) << 23) | (man << 13));
}

/* kind: 0 = bf16, 1 = fp16 */
void oracle_gemm_16bit(const uint16_t* A, const uint16_t* B, float* C, int M, int N, int K,
                       int kind, int chunk) {
  if (chunk < 1) chunk = K;
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      float sum = 0.0f;
      for (int k0 = 0; k0 < K; k0 += chunk) {
        int k1 = k0 + chunk < K ? k0 + chunk : K;
        double part = 0.0;
        for (int k = k0; k < k1; ++k) {
          uint16_t a = A[(size_t)i * K + k], b = B[(size_t)k * N + j];
          part += (double)(kind ? f16_value(a) : bf16_value(a)) *
                  (double)(kind ? f16_value(b) : bf16_value(b));
        }
        sum += (float)part;
      }
      C[(size_t)i * N + j] = sum;
    }
}
