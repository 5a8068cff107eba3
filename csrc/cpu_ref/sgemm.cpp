// CPU stand-in for the reference's hot kernel, used as an oracle and as a timed CPU baseline.
//
// rust-nn's `blas::sgemm` (src/blas.rs:104-186) is a row-major packed/blocked GEMM: row blocks of MC = 128 run in
// parallel, K is cut into KC = 256 panels and N into NC = 256 panels, both operands are packed (the transposes are
// folded into the packing, and alpha into the packed B), and a 4 x 16 AVX2+FMA micro-kernel does the work
// (src/blas.rs:50-57, 273-339, 429-508); products with m*n*k < 4096 take a plain triple loop (src/blas.rs:147-150).
// The reference cannot be built on a machine without a Rust toolchain, so this file restates that design in C++ with
// the same blocking constants and micro-tile, which keeps the CPU baseline honest: same algorithm class, same ISA.
//
//   C[m x n] = alpha * op(A) * op(B) + beta * C        (row-major, lda/ldb/ldc in elements)
#include <immintrin.h>
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

constexpr int MC = 128, KC = 256, NC = 256, MR = 4, NR = 16;

inline float a_at(const float* A, int lda, bool trans, int i, int p) { return trans ? A[(size_t)p * lda + i] : A[(size_t)i * lda + p]; }
inline float b_at(const float* B, int ldb, bool trans, int p, int j) { return trans ? B[(size_t)j * ldb + p] : B[(size_t)p * ldb + j]; }

// A block [mb x kb] -> panels of MR rows, each panel stored k-major (MR values per k); short panels are zero-padded
void pack_a(const float* A, int lda, bool trans, int i0, int p0, int mb, int kb, float* dst) {
  for (int i = 0; i < mb; i += MR) {
    const int rows = std::min(MR, mb - i);
    for (int p = 0; p < kb; ++p) {
      for (int r = 0; r < rows; ++r) *dst++ = a_at(A, lda, trans, i0 + i + r, p0 + p);
      for (int r = rows; r < MR; ++r) *dst++ = 0.f;
    }
  }
}

// alpha * B block [kb x nb] -> panels of NR columns, each panel stored k-major (NR values per k)
void pack_b(const float* B, int ldb, bool trans, int p0, int j0, int kb, int nb, float alpha, float* dst) {
  for (int j = 0; j < nb; j += NR) {
    const int cols = std::min(NR, nb - j);
    for (int p = 0; p < kb; ++p) {
      for (int c = 0; c < cols; ++c) *dst++ = alpha * b_at(B, ldb, trans, p0 + p, j0 + j + c);
      for (int c = cols; c < NR; ++c) *dst++ = 0.f;
    }
  }
}

// acc[4][16] += Apanel[kb][4] * Bpanel[kb][16]; then C (rows x cols valid) += acc
void micro_4x16(const float* ap, const float* bp, int kb, float* C, int ldc, int rows, int cols) {
  __m256 c00 = _mm256_setzero_ps(), c01 = c00, c10 = c00, c11 = c00, c20 = c00, c21 = c00, c30 = c00, c31 = c00;
  for (int p = 0; p < kb; ++p) {
    const __m256 b0 = _mm256_loadu_ps(bp), b1 = _mm256_loadu_ps(bp + 8);
    __m256 a = _mm256_broadcast_ss(ap + 0); c00 = _mm256_fmadd_ps(a, b0, c00); c01 = _mm256_fmadd_ps(a, b1, c01);
    a = _mm256_broadcast_ss(ap + 1); c10 = _mm256_fmadd_ps(a, b0, c10); c11 = _mm256_fmadd_ps(a, b1, c11);
    a = _mm256_broadcast_ss(ap + 2); c20 = _mm256_fmadd_ps(a, b0, c20); c21 = _mm256_fmadd_ps(a, b1, c21);
    a = _mm256_broadcast_ss(ap + 3); c30 = _mm256_fmadd_ps(a, b0, c30); c31 = _mm256_fmadd_ps(a, b1, c31);
    ap += MR; bp += NR;
  }
  if (rows == MR && cols == NR) {
    float* r = C;
    _mm256_storeu_ps(r, _mm256_add_ps(_mm256_loadu_ps(r), c00)); _mm256_storeu_ps(r + 8, _mm256_add_ps(_mm256_loadu_ps(r + 8), c01)); r += ldc;
    _mm256_storeu_ps(r, _mm256_add_ps(_mm256_loadu_ps(r), c10)); _mm256_storeu_ps(r + 8, _mm256_add_ps(_mm256_loadu_ps(r + 8), c11)); r += ldc;
    _mm256_storeu_ps(r, _mm256_add_ps(_mm256_loadu_ps(r), c20)); _mm256_storeu_ps(r + 8, _mm256_add_ps(_mm256_loadu_ps(r + 8), c21)); r += ldc;
    _mm256_storeu_ps(r, _mm256_add_ps(_mm256_loadu_ps(r), c30)); _mm256_storeu_ps(r + 8, _mm256_add_ps(_mm256_loadu_ps(r + 8), c31));
    return;
  }
  alignas(32) float t[MR][NR];
  _mm256_store_ps(t[0], c00); _mm256_store_ps(t[0] + 8, c01); _mm256_store_ps(t[1], c10); _mm256_store_ps(t[1] + 8, c11);
  _mm256_store_ps(t[2], c20); _mm256_store_ps(t[2] + 8, c21); _mm256_store_ps(t[3], c30); _mm256_store_ps(t[3] + 8, c31);
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c) C[(size_t)r * ldc + c] += t[r][c];
}

void row_block(int i0, int mb, int n, int k, float alpha, const float* A, int lda, bool ta, const float* B, int ldb, bool tb,
               float* C, int ldc) {
  std::vector<float> pa((size_t)((MC + MR - 1) / MR * MR) * KC), pb((size_t)KC * ((NC + NR - 1) / NR * NR));
  for (int p0 = 0; p0 < k; p0 += KC) {
    const int kb = std::min(KC, k - p0);
    pack_a(A, lda, ta, i0, p0, mb, kb, pa.data());
    for (int j0 = 0; j0 < n; j0 += NC) {
      const int nb = std::min(NC, n - j0);
      pack_b(B, ldb, tb, p0, j0, kb, nb, alpha, pb.data());
      for (int i = 0; i < mb; i += MR)
        for (int j = 0; j < nb; j += NR)
          micro_4x16(pa.data() + (size_t)(i / MR) * MR * kb, pb.data() + (size_t)(j / NR) * NR * kb, kb,
                     C + (size_t)(i0 + i) * ldc + j0 + j, ldc, std::min(MR, mb - i), std::min(NR, nb - j));
    }
  }
}

}  // namespace

extern "C" int b200_cpu_sgemm(int trans_a, int trans_b, int m, int n, int k, float alpha, const float* A, int lda, const float* B,
                              int ldb, float beta, float* C, int ldc, int threads) {
  if (m < 0 || n < 0 || k < 0) return -1;
  for (int i = 0; i < m; ++i) {
    float* row = C + (size_t)i * ldc;
    if (beta == 0.f) std::memset(row, 0, sizeof(float) * n);
    else if (beta != 1.f) for (int j = 0; j < n; ++j) row[j] *= beta;
  }
  if (m == 0 || n == 0 || k == 0 || alpha == 0.f) return 0;
  if ((long long)m * n * k < 4096) {                         // small products: i-p-j loop, no packing
    for (int i = 0; i < m; ++i)
      for (int p = 0; p < k; ++p) {
        const float a = alpha * a_at(A, lda, trans_a != 0, i, p);
        for (int j = 0; j < n; ++j) C[(size_t)i * ldc + j] += a * b_at(B, ldb, trans_b != 0, p, j);
      }
    return 0;
  }
  const int blocks = (m + MC - 1) / MC;
  const int nt = std::max(1, std::min(threads > 0 ? threads : (int)std::thread::hardware_concurrency(), blocks));
  auto work = [&](int t) {
    for (int b = t; b < blocks; b += nt)
      row_block(b * MC, std::min(MC, m - b * MC), n, k, alpha, A, lda, trans_a != 0, B, ldb, trans_b != 0, C, ldc);
  };
  if (nt == 1) { work(0); return 0; }
  std::vector<std::thread> pool;
  for (int t = 0; t < nt; ++t) pool.emplace_back(work, t);
  for (auto& th : pool) th.join();
  return 0;
}
