// fp64 GEMM on the fp64 tensor path: mma.sync m8n8k4 (DMMA).  tcgen05 has no fp64 kind, so this warp-level
// instruction is the only tensor route for doubles; it does the same IEEE fused multiply-adds as the CUDA-core
// kernel but needs an eighth of the shared-memory traffic per FMA, which is what bounds that kernel.
//
//   C[m,n] = alpha * op(A) * op(B) + beta * C      (row-major; 16-byte aligned A, B: base and leading dimension)
//
// 128 x 64 tile per 256-thread CTA, 8 warps as 4 (M) x 2 (N), 32 x 32 per warp = 4 x 4 MMA blocks of 8 x 8.
// k-slices of 16 travel global -> shared memory with cp.async, three in flight, in the layout of the operand's
// storage; the paddings (+4 doubles) make every fragment load (one double per thread: 8 rows x 4 k) hit 32
// distinct banks per half warp.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "fb_xgemm_simt.cuh"

namespace fb {

constexpr int kDmBM = 128, kDmBN = 64, kDmK = 16, kDmStages = 3;
constexpr int kDmLdk = kDmK + 4;  // row pitch (doubles) of a K-contiguous tile

template <int TILE, bool KMAJ>
struct DmTile {
  static constexpr int kLd = KMAJ ? kDmLdk : TILE + 4;
  static constexpr int kDoubles = KMAJ ? TILE * kDmLdk : kDmK * (TILE + 4);
};

__device__ __forceinline__ void cp_async16_d(double* dst, const double* src, int src_bytes) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}

template <int TILE, bool KMAJ>
__device__ __forceinline__ void dm_load(double* __restrict__ s, const double* __restrict__ base, long long ld, int mn0,
                                        int k0, int mn_lim, int k_lim, int tid) {
  constexpr int kChunks = TILE * kDmK / 2;
#pragma unroll
  for (int c = tid; c < kChunks; c += 256) {
    if (KMAJ) {
      const int r = c / (kDmK / 2), k2 = (c % (kDmK / 2)) * 2;
      const int valid = (mn0 + r < mn_lim) ? min(2, max(0, k_lim - (k0 + k2))) : 0;
      const double* src = valid ? base + static_cast<long long>(mn0 + r) * ld + k0 + k2 : base;
      cp_async16_d(s + r * kDmLdk + k2, src, valid * 8);
    } else {
      const int kk = c / (TILE / 2), q = (c % (TILE / 2)) * 2;
      const int valid = (k0 + kk < k_lim) ? min(2, max(0, mn_lim - (mn0 + q))) : 0;
      const double* src = valid ? base + static_cast<long long>(k0 + kk) * ld + mn0 + q : base;
      cp_async16_d(s + kk * (TILE + 4) + q, src, valid * 8);
    }
  }
}

__device__ __forceinline__ void dmma_m8n8k4(double (&d)[2], double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
               : "+d"(d[0]), "+d"(d[1])
               : "d"(a), "d"(b));
}

template <bool AK, bool BKM>
__global__ void __launch_bounds__(256) dgemm_mma_kernel(const XgemmParams p) {
  constexpr int kAD = DmTile<kDmBM, AK>::kDoubles, kBD = DmTile<kDmBN, BKM>::kDoubles;
  constexpr int kLdA = DmTile<kDmBM, AK>::kLd, kLdB = DmTile<kDmBN, BKM>::kLd;
  extern __shared__ __align__(16) double dm_smem[];
  double* As = dm_smem;
  double* Bs = dm_smem + kDmStages * kAD;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 1, wn = warp & 1;         // warp's 32 x 32 block inside the tile
  const int fr = lane >> 2, fk = lane & 3;         // fragment row (or column) and k inside an 8 x 4 block
  const int m0 = (blockIdx.x / p.tiles_n) * kDmBM, n0 = (blockIdx.x % p.tiles_n) * kDmBN;
  const double* A = static_cast<const double*>(p.A);
  const double* B = static_cast<const double*>(p.B);

  double acc[4][4][2];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

  const int k_iters = (p.k + kDmK - 1) / kDmK;
#pragma unroll
  for (int s = 0; s < kDmStages - 1; ++s) {
    if (s < k_iters) {
      dm_load<kDmBM, AK>(As + s * kAD, A, p.lda, m0, s * kDmK, p.m, p.k, tid);
      dm_load<kDmBN, BKM>(Bs + s * kBD, B, p.ldb, n0, s * kDmK, p.n, p.k, tid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }

  for (int it = 0; it < k_iters; ++it) {
    asm volatile("cp.async.wait_group %0;" ::"n"(kDmStages - 2) : "memory");
    __syncthreads();
    {
      const int nx = it + kDmStages - 1;
      if (nx < k_iters) {
        const int slot = nx % kDmStages;
        dm_load<kDmBM, AK>(As + slot * kAD, A, p.lda, m0, nx * kDmK, p.m, p.k, tid);
        dm_load<kDmBN, BKM>(Bs + slot * kBD, B, p.ldb, n0, nx * kDmK, p.n, p.k, tid);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const double* as = As + (it % kDmStages) * kAD;
    const double* bs = Bs + (it % kDmStages) * kBD;
#pragma unroll
    for (int k4 = 0; k4 < kDmK / 4; ++k4) {
      const int kk = k4 * 4 + fk;
      double af[4], bf[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = wm * 32 + i * 8 + fr;
        af[i] = AK ? as[r * kLdA + kk] : as[kk * kLdA + r];
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = wn * 32 + j * 8 + fr;
        bf[j] = BKM ? bs[c * kLdB + kk] : bs[kk * kLdB + c];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) dmma_m8n8k4(acc[i][j], af[i], bf[j]);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  // epilogue: thread holds C[row][col], C[row][col + 1] of every 8 x 8 block
  const double alpha = p.alpha_re, beta = p.beta_re;
  double* C = static_cast<double*>(p.C);
  const bool c_vec = ((reinterpret_cast<uintptr_t>(C) | static_cast<uintptr_t>(p.ldc * 8)) & 15) == 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = m0 + wm * 32 + i * 8 + fr;
    if (row >= p.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = n0 + wn * 32 + j * 8 + 2 * fk;
      if (col >= p.n) continue;
      double* dst = C + static_cast<long long>(row) * p.ldc + col;
      double v0 = alpha * acc[i][j][0], v1 = alpha * acc[i][j][1];
      if (c_vec && col + 1 < p.n) {
        if (beta != 0.0) {
          const double2 c = *reinterpret_cast<const double2*>(dst);
          v0 = fma(beta, c.x, v0); v1 = fma(beta, c.y, v1);
        }
        *reinterpret_cast<double2*>(dst) = make_double2(v0, v1);
      } else {
        if (beta != 0.0) v0 = fma(beta, dst[0], v0);
        dst[0] = v0;
        if (col + 1 < p.n) {
          if (beta != 0.0) v1 = fma(beta, dst[1], v1);
          dst[1] = v1;
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// complex<double> GEMM on the same fp64 tensor path: a complex multiply-add is four real DMMAs on the real and
// imaginary parts of the fragments (re += ar*br, re += (-ai)*bi, im += ar*bi, im += ai*br), i.e. exactly the
// four real FMAs of the CUDA-core kernel.  Matrices stay interleaved (re, im); one 128-bit shared load
// fetches both parts of a fragment element.  64 x 64 tile per CTA, 8 warps as 2 (M) x 4 (N), 32 x 16 per warp;
// k-slices of 8, three in flight.  op = C flips the sign of the imaginary fragment part.
constexpr int kZmT = 64, kZmK = 8, kZmStages = 3;
constexpr int kZmLdk = kZmK + 4;   // row pitch (complex) of a K-contiguous tile
constexpr int kZmLdm = kZmT + 2;   // row pitch (complex) of an MN-contiguous tile

template <bool KMAJ>
struct ZmTile {
  static constexpr int kLd = KMAJ ? kZmLdk : kZmLdm;
  static constexpr int kElems = KMAJ ? kZmT * kZmLdk : kZmK * kZmLdm;
};

template <bool KMAJ>
__device__ __forceinline__ void zm_load(cdouble* __restrict__ s, const cdouble* __restrict__ base, long long ld, int mn0,
                                        int k0, int mn_lim, int k_lim, int tid) {
#pragma unroll
  for (int c = tid; c < kZmT * kZmK; c += 256) {
    int r, kk;
    if (KMAJ) { r = c / kZmK; kk = c % kZmK; } else { kk = c / kZmT; r = c % kZmT; }
    const bool valid = mn0 + r < mn_lim && k0 + kk < k_lim;
    const cdouble* src = !valid ? base
                         : (KMAJ ? base + static_cast<long long>(mn0 + r) * ld + k0 + kk
                                 : base + static_cast<long long>(k0 + kk) * ld + mn0 + r);
    cdouble* dst = KMAJ ? s + r * kZmLdk + kk : s + kk * kZmLdm + r;
    cp_async16_d(reinterpret_cast<double*>(dst), reinterpret_cast<const double*>(src), valid ? 16 : 0);
  }
}

template <bool AK, bool BKM>
__global__ void __launch_bounds__(256) zgemm_mma_kernel(const XgemmParams p) {
  constexpr int kAE = ZmTile<AK>::kElems, kBE = ZmTile<BKM>::kElems;
  constexpr int kLdA = ZmTile<AK>::kLd, kLdB = ZmTile<BKM>::kLd;
  extern __shared__ __align__(16) double dm_smem[];
  cdouble* As = reinterpret_cast<cdouble*>(dm_smem);
  cdouble* Bs = As + kZmStages * kAE;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 2, wn = warp & 3;         // warp's 32 x 16 block inside the tile
  const int fr = lane >> 2, fk = lane & 3;
  const int m0 = (blockIdx.x / p.tiles_n) * kZmT, n0 = (blockIdx.x % p.tiles_n) * kZmT;
  const cdouble* A = static_cast<const cdouble*>(p.A);
  const cdouble* B = static_cast<const cdouble*>(p.B);
  const double sa = p.transa == 2 ? -1.0 : 1.0, sb = p.transb == 2 ? -1.0 : 1.0;  // conjugation

  double acc_re[4][2][2], acc_im[4][2][2];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) acc_re[i][j][0] = acc_re[i][j][1] = acc_im[i][j][0] = acc_im[i][j][1] = 0.0;

  const int k_iters = (p.k + kZmK - 1) / kZmK;
#pragma unroll
  for (int s = 0; s < kZmStages - 1; ++s) {
    if (s < k_iters) {
      zm_load<AK>(As + s * kAE, A, p.lda, m0, s * kZmK, p.m, p.k, tid);
      zm_load<BKM>(Bs + s * kBE, B, p.ldb, n0, s * kZmK, p.n, p.k, tid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int it = 0; it < k_iters; ++it) {
    asm volatile("cp.async.wait_group %0;" ::"n"(kZmStages - 2) : "memory");
    __syncthreads();
    {
      const int nx = it + kZmStages - 1;
      if (nx < k_iters) {
        const int slot = nx % kZmStages;
        zm_load<AK>(As + slot * kAE, A, p.lda, m0, nx * kZmK, p.m, p.k, tid);
        zm_load<BKM>(Bs + slot * kBE, B, p.ldb, n0, nx * kZmK, p.n, p.k, tid);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const cdouble* as = As + (it % kZmStages) * kAE;
    const cdouble* bs = Bs + (it % kZmStages) * kBE;
#pragma unroll
    for (int k4 = 0; k4 < kZmK / 4; ++k4) {
      const int kk = k4 * 4 + fk;
      double ar[4], ai[4], nai[4], br[2], bi[2];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = wm * 32 + i * 8 + fr;
        const double2 v = *reinterpret_cast<const double2*>(AK ? as + r * kLdA + kk : as + kk * kLdA + r);
        ar[i] = v.x; ai[i] = sa * v.y; nai[i] = -ai[i];
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int c = wn * 16 + j * 8 + fr;
        const double2 v = *reinterpret_cast<const double2*>(BKM ? bs + c * kLdB + kk : bs + kk * kLdB + c);
        br[j] = v.x; bi[j] = sb * v.y;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          dmma_m8n8k4(acc_re[i][j], ar[i], br[j]);
          dmma_m8n8k4(acc_re[i][j], nai[i], bi[j]);
          dmma_m8n8k4(acc_im[i][j], ar[i], bi[j]);
          dmma_m8n8k4(acc_im[i][j], ai[i], br[j]);
        }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  const double alr = p.alpha_re, ali = p.alpha_im, ber = p.beta_re, bei = p.beta_im;
  const bool beta_zero = ber == 0.0 && bei == 0.0;
  cdouble* C = static_cast<cdouble*>(p.C);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = m0 + wm * 32 + i * 8 + fr;
    if (row >= p.m) continue;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int col = n0 + wn * 16 + j * 8 + 2 * fk + e;
        if (col >= p.n) continue;
        cdouble* dst = C + static_cast<long long>(row) * p.ldc + col;
        const double xr = acc_re[i][j][e], xi = acc_im[i][j][e];
        // alpha * acc (+ beta * C), the same FMA sequence as the CUDA-core kernel's epilogue
        double vr = fma(-ali, xi, alr * xr), vi = fma(ali, xr, alr * xi);
        if (!beta_zero) {
          const cdouble c = *dst;
          vr = fma(ber, c.x, vr); vr = fma(-bei, c.y, vr);
          vi = fma(ber, c.y, vi); vi = fma(bei, c.x, vi);
        }
        *dst = cdouble{vr, vi};
      }
    }
  }
}

}  // namespace fb
