// GEMM on the CUDA cores for the element types the tensor-core path does not cover:
// double (dgemm), complex<float> (cgemm), complex<double> (zgemm) -- and, with one operand read through a
// triangular mask, the triangular products strmm / dtrmm / ctrmm / ztrmm.
//
//   C[m,n] = alpha * op(A) * op(B) + beta * C       op = N, T or C (conjugate transpose)
//   trmm:  C = alpha * op(tri(A)) * B   (left)   or   C = alpha * B * op(tri(A))   (right)
//
// Row-major, any leading dimension and alignment.  64 x 64 output tile per 256-thread CTA, 4 x 4 outputs
// per thread, k-slices of 8 double buffered through shared memory in k-major order (an operand whose
// contiguous dimension is K is transposed on the way in, conjugation is applied on the way in too), so
// that the inner loop is the same for every op(A), op(B) combination.  Products and sums are IEEE in the
// operand's own precision; a complex multiply-add is four real FMAs.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace fb {

struct cfloat { float x, y; };
struct cdouble { double x, y; };

template <class T> struct XNum;
template <> struct XNum<float> {
  using Real = float;
  static __device__ __forceinline__ float zero() { return 0.f; }
  static __device__ __forceinline__ float one() { return 1.f; }
  static __device__ __forceinline__ float make(double re, double) { return static_cast<float>(re); }
  static __device__ __forceinline__ float conj(float a) { return a; }
  static __device__ __forceinline__ float fma(float a, float b, float c) { return fmaf(a, b, c); }
  static __device__ __forceinline__ float mul(float a, float b) { return a * b; }
  static __device__ __forceinline__ bool is_zero(float a) { return a == 0.f; }
};
template <> struct XNum<double> {
  using Real = double;
  static __device__ __forceinline__ double zero() { return 0.0; }
  static __device__ __forceinline__ double one() { return 1.0; }
  static __device__ __forceinline__ double make(double re, double) { return re; }
  static __device__ __forceinline__ double conj(double a) { return a; }
  static __device__ __forceinline__ double fma(double a, double b, double c) { return ::fma(a, b, c); }
  static __device__ __forceinline__ double mul(double a, double b) { return a * b; }
  static __device__ __forceinline__ bool is_zero(double a) { return a == 0.0; }
};
template <> struct XNum<cfloat> {
  using Real = float;
  static __device__ __forceinline__ cfloat zero() { return cfloat{0.f, 0.f}; }
  static __device__ __forceinline__ cfloat one() { return cfloat{1.f, 0.f}; }
  static __device__ __forceinline__ cfloat make(double re, double im) { return cfloat{static_cast<float>(re), static_cast<float>(im)}; }
  static __device__ __forceinline__ cfloat conj(cfloat a) { return cfloat{a.x, -a.y}; }
  static __device__ __forceinline__ cfloat fma(cfloat a, cfloat b, cfloat c) {
    c.x = fmaf(a.x, b.x, c.x); c.x = fmaf(-a.y, b.y, c.x);
    c.y = fmaf(a.x, b.y, c.y); c.y = fmaf(a.y, b.x, c.y);
    return c;
  }
  static __device__ __forceinline__ cfloat mul(cfloat a, cfloat b) { return fma(a, b, zero()); }
  static __device__ __forceinline__ bool is_zero(cfloat a) { return a.x == 0.f && a.y == 0.f; }
};
template <> struct XNum<cdouble> {
  using Real = double;
  static __device__ __forceinline__ cdouble zero() { return cdouble{0.0, 0.0}; }
  static __device__ __forceinline__ cdouble one() { return cdouble{1.0, 0.0}; }
  static __device__ __forceinline__ cdouble make(double re, double im) { return cdouble{re, im}; }
  static __device__ __forceinline__ cdouble conj(cdouble a) { return cdouble{a.x, -a.y}; }
  static __device__ __forceinline__ cdouble fma(cdouble a, cdouble b, cdouble c) {
    c.x = ::fma(a.x, b.x, c.x); c.x = ::fma(-a.y, b.y, c.x);
    c.y = ::fma(a.x, b.y, c.y); c.y = ::fma(a.y, b.x, c.y);
    return c;
  }
  static __device__ __forceinline__ cdouble mul(cdouble a, cdouble b) { return fma(a, b, zero()); }
  static __device__ __forceinline__ bool is_zero(cdouble a) { return a.x == 0.0 && a.y == 0.0; }
};

struct XgemmParams {
  int m, n, k;
  double alpha_re, alpha_im, beta_re, beta_im;
  const void* A;
  long long lda;
  const void* B;
  long long ldb;
  void* C;
  long long ldc;
  int transa, transb;  // 0 = N, 1 = T, 2 = C
  int tiles_n;
  // Triangular operand (trmm): 0 = none, 1 = A (left product), 2 = B (right product).  The mask applies to
  // the matrix as STORED (before op()): `tri_upper` keeps col >= row, else col <= row; `tri_unit` reads the
  // diagonal as 1 without touching memory.
  int tri_operand, tri_upper, tri_unit;
};

struct TriMask {
  bool on, upper, unit;
};

constexpr int kXTile = 64, kXK = 8;

// This thread's two elements of a (64 x 8) operand slice, op() applied.
//   K-contiguous storage [mn][k] (A with trans = N, B with trans = T / C): thread -> (mn = tid / 4, k = 2 * (tid % 4))
//   MN-contiguous storage [k][mn] (A with trans = T / C, B with trans = N): thread -> (k = tid / 32, mn = 2 * (tid % 32))
template <class T>
__device__ __forceinline__ void xgemm_fetch(const T* __restrict__ base, long long ld, bool k_contig, bool conj, int mn0,
                                            int k0, int mn_lim, int k_lim, int tid, TriMask tri, T (&r)[2]) {
  using N = XNum<T>;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    int mn, kk;
    if (k_contig) { mn = mn0 + tid / 4; kk = k0 + 2 * (tid % 4) + j; }
    else { kk = k0 + tid / 32; mn = mn0 + 2 * (tid % 32) + j; }
    T v = N::zero();
    bool read = mn < mn_lim && kk < k_lim;
    if (tri.on && read) {
      const int row = k_contig ? mn : kk, col = k_contig ? kk : mn;  // position in the stored matrix
      if (row == col && tri.unit) { v = N::one(); read = false; }
      else if (tri.upper ? col < row : col > row) read = false;
    }
    if (read) v = k_contig ? base[static_cast<long long>(mn) * ld + kk] : base[static_cast<long long>(kk) * ld + mn];
    r[j] = conj ? N::conj(v) : v;
  }
}

template <class T>
__device__ __forceinline__ void xgemm_stash(T* __restrict__ s, bool k_contig, int tid, const T (&r)[2]) {
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    if (k_contig) s[(2 * (tid % 4) + j) * kXTile + tid / 4] = r[j];
    else s[(tid / 32) * kXTile + 2 * (tid % 32) + j] = r[j];
  }
}

template <class T>
__global__ void __launch_bounds__(256) xgemm_simt_kernel(const XgemmParams p) {
  using N = XNum<T>;
  __shared__ __align__(16) T As[2][kXK * kXTile];
  __shared__ __align__(16) T Bs[2][kXK * kXTile];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = (blockIdx.x / p.tiles_n) * kXTile, n0 = (blockIdx.x % p.tiles_n) * kXTile;
  const T* A = static_cast<const T*>(p.A);
  const T* B = static_cast<const T*>(p.B);
  const bool a_kc = p.transa == 0, b_kc = p.transb != 0;
  const bool a_cj = p.transa == 2, b_cj = p.transb == 2;
  const TriMask tri_a{p.tri_operand == 1, p.tri_upper != 0, p.tri_unit != 0};
  const TriMask tri_b{p.tri_operand == 2, p.tri_upper != 0, p.tri_unit != 0};
  // k range in which this tile's slice of the triangular operand can be non-zero.  op(A) is upper
  // triangular when the stored matrix is upper and not transposed, or lower and transposed.
  int k_begin = 0, k_end = p.k;
  if (p.tri_operand == 1) {          // op(A)(i, kk): upper keeps kk >= i
    const bool up = (p.tri_upper != 0) != (p.transa != 0);
    if (up) k_begin = m0 / kXK * kXK; else k_end = min(p.k, m0 + kXTile);
  } else if (p.tri_operand == 2) {   // op(A)(kk, j): upper keeps kk <= j
    const bool up = (p.tri_upper != 0) != (p.transb != 0);
    if (up) k_end = min(p.k, n0 + kXTile); else k_begin = n0 / kXK * kXK;
  }

  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = N::zero();

  T ra[2], rb[2];
  const int k_iters = k_end > k_begin ? (k_end - k_begin + kXK - 1) / kXK : 0;
  xgemm_fetch<T>(A, p.lda, a_kc, a_cj, m0, k_begin, p.m, k_end, tid, tri_a, ra);
  xgemm_fetch<T>(B, p.ldb, b_kc, b_cj, n0, k_begin, p.n, k_end, tid, tri_b, rb);
  xgemm_stash<T>(As[0], a_kc, tid, ra);
  xgemm_stash<T>(Bs[0], b_kc, tid, rb);
  __syncthreads();
  for (int it = 0; it < k_iters; ++it) {
    const int cur = it & 1;
    if (it + 1 < k_iters) {
      xgemm_fetch<T>(A, p.lda, a_kc, a_cj, m0, k_begin + (it + 1) * kXK, p.m, k_end, tid, tri_a, ra);
      xgemm_fetch<T>(B, p.ldb, b_kc, b_cj, n0, k_begin + (it + 1) * kXK, p.n, k_end, tid, tri_b, rb);
    }
    const T* as = As[cur];
    const T* bs = Bs[cur];
#pragma unroll
    for (int kk = 0; kk < kXK; ++kk) {
      T af[4], bf[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) af[i] = as[kk * kXTile + ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bf[j] = bs[kk * kXTile + tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = N::fma(af[i], bf[j], acc[i][j]);
    }
    if (it + 1 < k_iters) {
      xgemm_stash<T>(As[cur ^ 1], a_kc, tid, ra);
      xgemm_stash<T>(Bs[cur ^ 1], b_kc, tid, rb);
    }
    __syncthreads();
  }

  const T alpha = N::make(p.alpha_re, p.alpha_im), beta = N::make(p.beta_re, p.beta_im);
  const bool beta_zero = N::is_zero(beta);
  T* C = static_cast<T*>(p.C);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = m0 + ty * 4 + i;
    if (row >= p.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = n0 + tx * 4 + j;
      if (col >= p.n) continue;
      T* dst = C + static_cast<long long>(row) * p.ldc + col;
      T v = N::mul(alpha, acc[i][j]);
      if (!beta_zero) v = N::fma(beta, *dst, v);   // C is never read when beta == 0
      *dst = v;
    }
  }
}

// C[m, n] block <- beta * C (zero-fill when beta == 0): the k == 0 / alpha == 0 case.
template <class T>
__global__ void xgemm_scale_kernel(T* c, long long ldc, int m, int n, double beta_re, double beta_im) {
  using N = XNum<T>;
  const T beta = N::make(beta_re, beta_im);
  const bool zero = N::is_zero(beta);
  const long long total = static_cast<long long>(m) * n;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / n, col = i - r * n;
    T* q = c + r * ldc + col;
    *q = zero ? N::zero() : N::mul(beta, *q);
  }
}

}  // namespace fb
