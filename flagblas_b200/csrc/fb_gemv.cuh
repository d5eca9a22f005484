// Matrix-vector products (sgemv / hgemv / bfgemv): the M -> 1 limit of the GEMM path.
//
//   trans = N:  y[m] = alpha * A[m, n] * x[n] + beta * y        (A row-major, lda >= n)
//   trans = T:  y[n] = alpha * A[m, n]^T * x[m] + beta * y
//
// These are HBM-bound (A is read once, 2 FLOP per element), so the kernels are organised around
// 16-byte coalesced loads of A and enough independent loads in flight, not around the math:
//   N: a group of up to 256 threads sweeps four rows together, 16 bytes per thread and row at a time (a wide
//      matrix is read in contiguous 4 KB runs), and reduces with shuffles and shared memory; for matrices
//      with few rows the columns are split in `splits` ranges handled by different CTAs.
//   T: a thread owns 16 bytes' worth of consecutive columns and walks down a range of rows; up to 256
//      threads sit side by side along a row (4 KB runs again); for narrow matrices the spare threads take
//      other rows; the rows are split in `splits` ranges.
// With splits == 1 the result is written directly (alpha, beta and the output cast fused); otherwise
// fp32 partial sums go to a workspace [splits][len_y] and a small second kernel finishes -- the order
// of the additions is fixed, so results are reproducible run to run.
#pragma once

#include <cuda_fp8.h>

#include "fb_gemm_tc.cuh"

namespace fb {

__device__ __forceinline__ float to_f32(__nv_fp8_e4m3 v) { return static_cast<float>(v); }
__device__ __forceinline__ float to_f32(__nv_fp8_e5m2 v) { return static_cast<float>(v); }

// One element through the read-only path, as fp32.
template <class T> __device__ __forceinline__ float ld_f32(const T* p) { return to_f32(__ldg(p)); }
template <> __device__ __forceinline__ float ld_f32<__nv_fp8_e4m3>(const __nv_fp8_e4m3* p) {
  __nv_fp8_e4m3 v;
  v.__x = __ldg(reinterpret_cast<const unsigned char*>(p));
  return to_f32(v);
}
template <> __device__ __forceinline__ float ld_f32<__nv_fp8_e5m2>(const __nv_fp8_e5m2* p) {
  __nv_fp8_e5m2 v;
  v.__x = __ldg(reinterpret_cast<const unsigned char*>(p));
  return to_f32(v);
}

struct GemvParams {
  int m, n;
  long long lda;
  const void* A;
  const void* x;
  void* y;
  long long incx, incy;
  float alpha, beta;
  int splits;
  long long chunk;    // elements of the reduced dimension per split (multiple of the vector width)
  float* partial;     // [splits][len_y] when splits > 1
  int a_vec;          // A base and lda are 16-byte aligned
  int x_vec;          // incx == 1 and x is 16-byte aligned
  int tx;             // threads along the columns (power of two, <= 256)
};

// Load up to kElems consecutive elements starting at `p` (first `valid` are in range) as floats.
template <class T>
__device__ __forceinline__ void load_vec(const T* __restrict__ p, int valid, bool vec, float (&out)[16 / sizeof(T)]) {
  constexpr int E = 16 / sizeof(T);
  if (vec && valid >= E) {
    const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(p));  // streamed once: do not keep in cache
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < E; ++j) out[j] = to_f32(e[j]);
  } else {
#pragma unroll
    for (int j = 0; j < E; ++j) out[j] = j < valid ? to_f32(p[j]) : 0.f;
  }
}

// acc[j] += element j of the 16-byte vector `raw` (type T) * xs, in fp32.
template <class T>
__device__ __forceinline__ void fma_vec(const uint4& raw, float xs, float (&acc)[16 / sizeof(T)]) {
  constexpr int E = 16 / sizeof(T);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int j = 0; j < E; ++j) acc[j] = fmaf(to_f32(e[j]), xs, acc[j]);
}

// fp32 += fp16 * fp16 in one instruction (the product of two fp16 values is exact in fp32).
__device__ __forceinline__ float fma_f32_f16(unsigned short a, unsigned short b, float c) {
  float d;
  asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(d) : "h"(a), "h"(b), "f"(c));
  return d;
}

// FP8: converting 16 elements one by one to fp32 costs more issue slots than the memory system leaves
// room for.  Pairs are converted to fp16x2 (exact) and fed to the mixed-precision FMA together with x
// as fp16 (x comes from an FP8 value, so that conversion is exact too).
template <__nv_fp8_interpretation_t FMT>
__device__ __forceinline__ void fma_vec_fp8(const uint4& raw, float xs, float (&acc)[16]) {
  const unsigned short xh = __half_as_ushort(__float2half_rn(xs));
  const unsigned short* pairs = reinterpret_cast<const unsigned short*>(&raw);
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2(pairs[q], FMT);
    acc[2 * q] = fma_f32_f16(h2.x, xh, acc[2 * q]);
    acc[2 * q + 1] = fma_f32_f16(h2.y, xh, acc[2 * q + 1]);
  }
}
template <>
__device__ __forceinline__ void fma_vec<__nv_fp8_e4m3>(const uint4& raw, float xs, float (&acc)[16]) {
  fma_vec_fp8<__NV_E4M3>(raw, xs, acc);
}
template <>
__device__ __forceinline__ void fma_vec<__nv_fp8_e5m2>(const uint4& raw, float xs, float (&acc)[16]) {
  fma_vec_fp8<__NV_E5M2>(raw, xs, acc);
}

// Dot product of two 16-byte vectors of T, accumulated in fp32.
template <class T>
__device__ __forceinline__ float dot16(const uint4& a, const uint4& b, float acc) {
  constexpr int E = 16 / sizeof(T);
  const T* ea = reinterpret_cast<const T*>(&a);
  const T* eb = reinterpret_cast<const T*>(&b);
#pragma unroll
  for (int j = 0; j < E; ++j) acc = fmaf(to_f32(ea[j]), to_f32(eb[j]), acc);
  return acc;
}

// ---------------------------------------------------------------- trans = N
// 256 threads as (tx, g): p.tx threads (a power of two, 4..256) sweep the columns of kGemvRows
// consecutive rows together, 16 bytes per thread and row at a time, so that the x vector is fetched once
// for all of them and a wide matrix is read in contiguous runs of p.tx * 16 bytes per row; the 256 / p.tx
// groups of a CTA work on different row blocks.  grid: (row-block groups, splits over columns); row blocks
// are dealt grid-stride.  Sums are combined by shuffles inside a warp and, when a group spans several
// warps, by a fixed-order pass over shared memory.
constexpr int kGemvRows = 4;

template <class T, int UNR, int MINB>
__global__ void __launch_bounds__(256, MINB) gemv_n_kernel(const GemvParams p) {
  if (p.partial) grid_launch_dependents();  // the kernel that adds the partial sums may start its prologue
  constexpr int E = 16 / sizeof(T);
  constexpr int R = kGemvRows;
  __shared__ float red[8][R];
  const int lanes = p.tx;
  const int tx = threadIdx.x & (lanes - 1);
  const int g = threadIdx.x / lanes;
  const int groups = 256 / lanes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wpg = lanes > 32 ? lanes / 32 : 1;  // warps per group
  const long long step = static_cast<long long>(lanes) * E;
  const long long c0 = static_cast<long long>(blockIdx.y) * p.chunk;
  const long long c1 = min(static_cast<long long>(p.n), c0 + p.chunk);
  const T* A = static_cast<const T*>(p.A);
  const T* x = static_cast<const T*>(p.x);
  const bool fast = p.a_vec != 0 && p.x_vec != 0;
  const long long rows_per_cta = static_cast<long long>(groups) * R;
  for (long long base = static_cast<long long>(blockIdx.x) * rows_per_cta; base < p.m;
       base += static_cast<long long>(gridDim.x) * rows_per_cta) {
    const long long row = base + static_cast<long long>(g) * R;
    const T* arow[R];
#pragma unroll
    for (int r = 0; r < R; ++r)  // rows past the end re-read the last row; their sums are dropped
      arow[r] = A + min(row + r, static_cast<long long>(p.m) - 1) * p.lda;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
    long long c = c0 + static_cast<long long>(tx) * E;
    if (fast) {
#pragma unroll UNR
      for (; c + E <= c1; c += step) {
        uint4 a[R];
#pragma unroll
        for (int r = 0; r < R; ++r) a[r] = __ldcs(reinterpret_cast<const uint4*>(arow[r] + c));
        const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + c));  // shared by all rows: keep cached
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = dot16<T>(a[r], xv, acc[r]);
      }
    }
    for (; c < c1; c += step) {
      float xv[E];
      const int valid = static_cast<int>(min(static_cast<long long>(E), c1 - c));
#pragma unroll
      for (int j = 0; j < E; ++j) xv[j] = j < valid ? ld_f32(x + (c + j) * p.incx) : 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float a[E];
        load_vec<T>(arow[r] + c, valid, p.a_vec != 0, a);
#pragma unroll
        for (int j = 0; j < E; ++j) acc[r] = fmaf(a[j], xv[j], acc[r]);
      }
    }
    for (int off = (lanes < 32 ? lanes : 32) / 2; off > 0; off >>= 1) {
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], off);
    }
    if (wpg > 1) {
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) red[warp][r] = acc[r];
      }
      __syncthreads();
      if (warp % wpg == 0 && lane < R) {
        float t = 0.f;
        for (int w = 0; w < wpg; ++w) t += red[warp + w][lane];
        acc[0] = t;  // lane r now holds the sum of row `row + r`
      }
    }
    // writer of row `row + r`: the group's first thread for r (single-warp groups) or lane r of the
    // group's first warp (multi-warp groups)
    if (wpg > 1) {
      if (warp % wpg == 0 && lane < R && row + lane < p.m) {
        const long long orow = row + lane;
        if (p.splits > 1) {
          p.partial[static_cast<long long>(blockIdx.y) * p.m + orow] = acc[0];
        } else {
          T* yp = static_cast<T*>(p.y) + orow * p.incy;
          float v = p.alpha * acc[0];
          if (p.beta != 0.f) v += p.beta * to_f32(*yp);
          *yp = from_f32<T>(v);
        }
      }
      __syncthreads();  // red is reused by the next row block
    } else if (tx == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (row + r < p.m) {
          if (p.splits > 1) {
            p.partial[static_cast<long long>(blockIdx.y) * p.m + row + r] = acc[r];
          } else {
            T* yp = static_cast<T*>(p.y) + (row + r) * p.incy;
            float v = p.alpha * acc[r];
            if (p.beta != 0.f) v += p.beta * to_f32(*yp);
            *yp = from_f32<T>(v);
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------- trans = T
// 256 threads as (tx, ty): tx over p.tx 16-byte column vectors (a power of two), ty over 256 / p.tx
// rows at a time -- a warp reads 512 contiguous bytes when the matrix is wide, and several whole rows
// when it is narrow.  grid: (column panels of p.tx * E columns, splits over rows).  The ty partial sums
// are combined through shared memory by a fixed-shape tree.
template <class T, int U, int MINB, class TX = T, class TY = T>
__global__ void __launch_bounds__(256, MINB) gemv_t_kernel(const GemvParams p) {
  if (p.partial) grid_launch_dependents();  // the kernel that adds the partial sums may start its prologue
  constexpr int E = 16 / sizeof(T);
  __shared__ float red[256 * E];
  const int tx = threadIdx.x & (p.tx - 1);
  const int ty = threadIdx.x / p.tx;
  const int ny = 256 / p.tx;
  const long long col = (static_cast<long long>(blockIdx.x) * p.tx + tx) * E;
  const long long r0 = static_cast<long long>(blockIdx.y) * p.chunk;
  const long long r1 = min(static_cast<long long>(p.m), r0 + p.chunk);
  const bool live = col < p.n;
  const int valid = live ? static_cast<int>(min(static_cast<long long>(E), p.n - col)) : 0;
  const T* A = static_cast<const T*>(p.A) + col;
  const TX* x = static_cast<const TX*>(p.x);
  const bool vec = p.a_vec != 0;
  float acc[E];
#pragma unroll
  for (int j = 0; j < E; ++j) acc[j] = 0.f;
  if (live) {
    long long r = r0 + ty;
    if (vec && valid == E) {
      // U rows per trip: U independent 16-byte loads in flight per thread
      for (; r + static_cast<long long>(U - 1) * ny < r1; r += static_cast<long long>(U) * ny) {
        uint4 a[U];
        float xs[U];
#pragma unroll
        for (int u = 0; u < U; ++u) a[u] = __ldcs(reinterpret_cast<const uint4*>(A + (r + u * ny) * p.lda));
#pragma unroll
        for (int u = 0; u < U; ++u) xs[u] = ld_f32(x + (r + u * ny) * p.incx);
#pragma unroll
        for (int u = 0; u < U; ++u) fma_vec<T>(a[u], xs[u], acc);
      }
    }
    for (; r < r1; r += ny) {
      float a0[E];
      load_vec<T>(A + r * p.lda, valid, vec, a0);
      const float x0 = ld_f32(x + r * p.incx);
#pragma unroll
      for (int j = 0; j < E; ++j) acc[j] = fmaf(a0[j], x0, acc[j]);
    }
  }
  if (ny > 1) {
    // red[j][thread]: consecutive threads write consecutive words
#pragma unroll
    for (int j = 0; j < E; ++j) red[j * 256 + threadIdx.x] = acc[j];
    __syncthreads();
    for (int s = ny / 2; s > 0; s >>= 1) {
      if (ty < s) {
#pragma unroll
        for (int j = 0; j < E; ++j) red[j * 256 + threadIdx.x] += red[j * 256 + threadIdx.x + s * p.tx];
      }
      __syncthreads();
    }
    if (ty == 0) {
#pragma unroll
      for (int j = 0; j < E; ++j) acc[j] = red[j * 256 + threadIdx.x];
    }
  }
  if (ty != 0 || !live) return;
#pragma unroll
  for (int j = 0; j < E; ++j) {
    if (j < valid) {
      if (p.splits > 1) {
        p.partial[static_cast<long long>(blockIdx.y) * p.n + col + j] = acc[j];
      } else {
        TY* yp = static_cast<TY*>(p.y) + (col + j) * p.incy;
        float v = p.alpha * acc[j];
        if (p.beta != 0.f) v += p.beta * to_f32(*yp);
        *yp = from_f32<TY>(v);
      }
    }
  }
}

// y[i] = alpha * sum_s partial[s][i] + beta * y[i]
// 256 threads = 32 outputs x 8 slices of the split index: a thread adds every eighth partial sum of its
// output (independent loads, all in flight together), the eight slice sums are then added in slice
// order.  The association is fixed by (splits, slice count) alone: results repeat bit for bit.
constexpr int kFinishSlices = 8;

template <class T>
__global__ void __launch_bounds__(256) gemv_finish_kernel(const float* __restrict__ partial, int splits, long long len,
                                                          T* y, long long incy, float alpha, float beta) {
  __shared__ float red[kFinishSlices][33];
  grid_dependency_wait();  // launched as a programmatic dependent of the kernel that writes the partial sums
  const int o = threadIdx.x & 31, sl = threadIdx.x >> 5;
  const long long i = static_cast<long long>(blockIdx.x) * 32 + o;
  float acc = 0.f;
  if (i < len) {
#pragma unroll 4
    for (int s = sl; s < splits; s += kFinishSlices) acc += __ldcs(partial + static_cast<long long>(s) * len + i);
  }
  red[sl][o] = acc;
  __syncthreads();
  if (sl == 0 && i < len) {
    float t = red[0][o];
#pragma unroll
    for (int q = 1; q < kFinishSlices; ++q) t += red[q][o];
    T* yp = y + i * incy;
    float r = alpha * t;
    if (beta != 0.f) r += beta * to_f32(*yp);
    *yp = from_f32<T>(r);
  }
}

// y[i] = beta * y[i]  (alpha == 0)
template <class T>
__global__ void gemv_scale_kernel(T* y, long long len, long long incy, float beta) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= len) return;
  T* yp = y + i * incy;
  *yp = beta == 0.f ? from_f32<T>(0.f) : from_f32<T>(beta * to_f32(*yp));
}

}  // namespace fb
