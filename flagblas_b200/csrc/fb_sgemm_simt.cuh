// IEEE fp32 GEMM on the CUDA cores (FFMA), for the `sgemm` entry point whose
// contract is true single precision (no TF32 rounding of the inputs).
//
//   C[m,n] = alpha * op(A) * op(B) + beta * C      (row-major, any ld / alignment)
//
// Classic register-tiled design: a BM x BN tile per 256-thread CTA, BK-deep
// k-slices double buffered through shared memory (k-major, so each thread
// reads its A and B fragments with 128-bit loads), (BM/16) x (BN/16) outputs
// per thread.  Operands are read in whichever orientation they are stored:
// an operand whose contiguous dimension is M/N goes straight to shared memory
// with 128-bit stores, one whose contiguous dimension is K is transposed on
// the way in.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace fb {

struct SimtParams {
  int m, n, k;
  float alpha, beta;
  const float* A;
  long long lda;
  const float* B;
  long long ldb;
  float* C;
  long long ldc;
  int a_mn_contig;  // 1: A stored [k, lda] (transa = T); 0: stored [m, lda]
  int b_mn_contig;  // 1: B stored [k, ldb] (transb = N); 0: stored [n, ldb]
  int a_vec, b_vec, c_vec;  // 16-byte aligned base and leading dimension
  int tiles_n;
  // 2: the launch uses clusters of two CTAs that share an output tile, each taking half of k; the second hands its
  // sums to the first through distributed shared memory (pipelined kernel only; small problems with few tiles).
  int ksplit;
};

// Fetch this thread's 4 elements of a (TILE_MN x BK) operand slice.
//  mn-contiguous storage [k][mn]: thread -> (k = tid / (TILE_MN/4), mn = 4*(tid % (TILE_MN/4)))
//  k-contiguous  storage [mn][k]: thread -> (mn = tid / (BK/4),     k  = 4*(tid % (BK/4)))
template <int TILE_MN, int BK>
__device__ __forceinline__ void simt_fetch(const float* __restrict__ base, long long ld, int mn_contig, int vec,
                                           int mn0, int k0, int mn_lim, int k_lim, int tid, float (&r)[4]) {
  if (mn_contig) {
    const int kk = k0 + tid / (TILE_MN / 4);
    const int mn = mn0 + 4 * (tid % (TILE_MN / 4));
    const float* src = base + static_cast<long long>(kk) * ld + mn;
    if (kk < k_lim && mn + 3 < mn_lim && vec) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(src));
      r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) r[j] = (kk < k_lim && mn + j < mn_lim) ? __ldg(src + j) : 0.f;
    }
  } else {
    const int mn = mn0 + tid / (BK / 4);
    const int kk = k0 + 4 * (tid % (BK / 4));
    const float* src = base + static_cast<long long>(mn) * ld + kk;
    if (mn < mn_lim && kk + 3 < k_lim && vec) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(src));
      r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) r[j] = (mn < mn_lim && kk + j < k_lim) ? __ldg(src + j) : 0.f;
    }
  }
}

template <int TILE_MN, int BK, int LDS>
__device__ __forceinline__ void simt_stash(float* __restrict__ s, int mn_contig, int tid, const float (&r)[4]) {
  if (mn_contig) {
    const int kk = tid / (TILE_MN / 4);
    const int mn = 4 * (tid % (TILE_MN / 4));
    *reinterpret_cast<float4*>(s + kk * LDS + mn) = make_float4(r[0], r[1], r[2], r[3]);
  } else {
    const int mn = tid / (BK / 4);
    const int kk = 4 * (tid % (BK / 4));
#pragma unroll
    for (int j = 0; j < 4; ++j) s[(kk + j) * LDS + mn] = r[j];
  }
}

template <int BM, int BN, int BK>
__global__ void __launch_bounds__(256) sgemm_simt_kernel(const SimtParams p) {
  static_assert(BM * BK == 1024 && BN * BK == 1024, "each thread moves exactly 4 elements per operand");
  constexpr int TM = BM / 16, TN = BN / 16;  // outputs per thread
  constexpr int RG = TM / 4, CG = TN / 4;    // 4-wide fragment groups
  constexpr int LDA = BM + 4, LDB = BN + 4;  // padded so the transposing stores spread over banks
  __shared__ __align__(16) float As[2][BK * LDA];
  __shared__ __align__(16) float Bs[2][BK * LDB];

  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int tile_m = blockIdx.x / p.tiles_n, tile_n = blockIdx.x % p.tiles_n;
  const int m0 = tile_m * BM, n0 = tile_n * BN;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  float ra[4], rb[4];
  const int k_iters = (p.k + BK - 1) / BK;
  simt_fetch<BM, BK>(p.A, p.lda, p.a_mn_contig, p.a_vec, m0, 0, p.m, p.k, tid, ra);
  simt_fetch<BN, BK>(p.B, p.ldb, p.b_mn_contig, p.b_vec, n0, 0, p.n, p.k, tid, rb);
  simt_stash<BM, BK, LDA>(As[0], p.a_mn_contig, tid, ra);
  simt_stash<BN, BK, LDB>(Bs[0], p.b_mn_contig, tid, rb);
  __syncthreads();

  for (int it = 0; it < k_iters; ++it) {
    const int cur = it & 1;
    if (it + 1 < k_iters) {
      simt_fetch<BM, BK>(p.A, p.lda, p.a_mn_contig, p.a_vec, m0, (it + 1) * BK, p.m, p.k, tid, ra);
      simt_fetch<BN, BK>(p.B, p.ldb, p.b_mn_contig, p.b_vec, n0, (it + 1) * BK, p.n, p.k, tid, rb);
    }
    const float* as = As[cur];
    const float* bs = Bs[cur];
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float af[TM], bf[TN];
#pragma unroll
      for (int g = 0; g < RG; ++g) {
        const float4 v = *reinterpret_cast<const float4*>(as + kk * LDA + g * (BM / RG) + ty * 4);
        af[g * 4 + 0] = v.x; af[g * 4 + 1] = v.y; af[g * 4 + 2] = v.z; af[g * 4 + 3] = v.w;
      }
#pragma unroll
      for (int g = 0; g < CG; ++g) {
        const float4 v = *reinterpret_cast<const float4*>(bs + kk * LDB + g * (BN / CG) + tx * 4);
        bf[g * 4 + 0] = v.x; bf[g * 4 + 1] = v.y; bf[g * 4 + 2] = v.z; bf[g * 4 + 3] = v.w;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(af[i], bf[j], acc[i][j]);
    }
    if (it + 1 < k_iters) {
      simt_stash<BM, BK, LDA>(As[cur ^ 1], p.a_mn_contig, tid, ra);
      simt_stash<BN, BK, LDB>(Bs[cur ^ 1], p.b_mn_contig, tid, rb);
    }
    __syncthreads();
  }

  // epilogue: alpha * acc + beta * C, C never read when beta == 0
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int row = m0 + (i / 4) * (BM / RG) + ty * 4 + (i % 4);
    if (row >= p.m) continue;
#pragma unroll
    for (int g = 0; g < CG; ++g) {
      const int col = n0 + g * (BN / CG) + tx * 4;
      if (col >= p.n) continue;
      float* dst = p.C + static_cast<long long>(row) * p.ldc + col;
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = p.alpha * acc[i][g * 4 + j];
      if (p.c_vec && col + 3 < p.n) {
        if (p.beta != 0.f) {
          const float4 c = *reinterpret_cast<const float4*>(dst);
          v[0] += p.beta * c.x; v[1] += p.beta * c.y; v[2] += p.beta * c.z; v[3] += p.beta * c.w;
        }
        *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (col + j < p.n) {
            float r = v[j];
            if (p.beta != 0.f) r += p.beta * dst[j];
            dst[j] = r;
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Pipelined variant for 16-byte aligned operands: the k-slices travel global -> shared memory with
// cp.async (no register staging), four slices deep, so that the load latency of a slice is hidden
// behind the FFMAs of the three before it -- what the double-buffered kernel above cannot do when
// few CTAs share an SM (a 512^3 problem is 64 CTAs on 148 SMs).
//
// Shared-memory layout of a slice follows the operand's storage, so that every 16-byte piece is one
// cp.async: an operand stored with M (or N) contiguous lands as [16 k][tile] and is read back as float4
// fragments; one stored with K contiguous lands as [tile][16 k + 4 pad] and is read back two k at a time
// (float2).  For a K-contiguous B the thread's columns are interleaved (tx, tx + 16, ...) to keep those
// reads spread over the banks.
constexpr int kPipeK = 16;      // k per slice
constexpr int kPipeStages = 4;
constexpr int kPipeLdk = 20;    // floats per row of a K-contiguous tile (80 bytes: 16-byte aligned rows)

template <int TILE, bool KMAJ>
struct PipeTile {
  static constexpr int kFloats = KMAJ ? TILE * kPipeLdk : kPipeK * TILE;
};

// A K-contiguous B tile stored for packed FMAs: neighbouring columns (2 p, 2 p + 1) interleaved along k,
// [pair p][k][2] with 34 floats per pair, so that one 64-bit shared load yields the two B values of a packed FMA in
// an aligned register pair and the 16 threads that differ in tx (pairs p, p + 1, ...) cover all 32 banks.
constexpr int kPipePairLd = 2 * kPipeK + 2;
template <int TILE>
struct PipePairTile {
  static constexpr int kFloats = (TILE / 2) * kPipePairLd;
};

__device__ __forceinline__ void cp_async4(float* dst, const float* src, int src_bytes) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}

// This thread's share of the copies of one (TILE x 16) slice of a K-contiguous operand into the pair-interleaved
// layout: 4-byte copies (the scatter is finer than 16 bytes), 16 consecutive threads reading 64 consecutive bytes.
template <int TILE>
__device__ __forceinline__ void pipe_load_pairs(float* __restrict__ s, const float* __restrict__ base, long long ld, int mn0,
                                                int k0, int mn_lim, int k_lim, int tid) {
#pragma unroll
  for (int e = tid; e < TILE * kPipeK; e += 256) {
    const int kk = e & (kPipeK - 1), c = e >> 4;
    const bool valid = mn0 + c < mn_lim && k0 + kk < k_lim;
    const float* src = valid ? base + static_cast<long long>(mn0 + c) * ld + k0 + kk : base;
    cp_async4(s + (c >> 1) * kPipePairLd + kk * 2 + (c & 1), src, valid ? 4 : 0);
  }
}

__device__ __forceinline__ void cp_async16(float* dst, const float* src, int src_bytes) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}

// Issue this thread's share of the copies of one (TILE x 16) slice.  `kmaj`: stored [mn][k].
template <int TILE, bool KMAJ>
__device__ __forceinline__ void pipe_load(float* __restrict__ s, const float* __restrict__ base, long long ld, int mn0,
                                          int k0, int mn_lim, int k_lim, int tid) {
  constexpr int kChunks = TILE * kPipeK / 4;
#pragma unroll
  for (int c = tid; c < kChunks; c += 256) {
    if (KMAJ) {
      const int r = c >> 2, k4 = (c & 3) * 4;
      const int valid = (mn0 + r < mn_lim) ? min(4, max(0, k_lim - (k0 + k4))) : 0;
      const float* src = valid ? base + static_cast<long long>(mn0 + r) * ld + k0 + k4 : base;
      cp_async16(s + r * kPipeLdk + k4, src, valid * 4);
    } else {
      const int kk = c / (TILE / 4), q = (c % (TILE / 4)) * 4;
      const int valid = (k0 + kk < k_lim) ? min(4, max(0, mn_lim - (mn0 + q))) : 0;
      const float* src = valid ? base + static_cast<long long>(k0 + kk) * ld + mn0 + q : base;
      cp_async16(s + kk * TILE + q, src, valid * 4);
    }
  }
}

// PACK: the FMAs are issued as packed pairs (fma.rn.f32x2, two IEEE fp32 FMAs per instruction on sm_100):
// the same arithmetic in half the issue slots, which leaves room for the shared-memory loads next to them.
// 1 = pairs of neighbouring columns (B fragments arrive as float4: the pair is already adjacent in registers),
// 2 = pairs of neighbouring rows (the same for A), 3 = pairs of neighbouring columns of a K-contiguous B, whose tile
// is then stored pair-interleaved (PipePairTile), 0 = scalar FMAs.
template <int BM, int BN, bool AK, bool BKM, int PACK>
__global__ void __launch_bounds__(256, 2) sgemm_pipe_kernel(const SimtParams p) {
  constexpr int TM = BM / 16, TN = BN / 16;
  constexpr int RG = TM / 4, CG = TN / 4;
  constexpr bool BPAIR = BKM && PACK == 3;  // K-contiguous B in the pair-interleaved layout, FMAs packed over column pairs
  constexpr int kAFloats = PipeTile<BM, AK>::kFloats, kBFloats = BPAIR ? PipePairTile<BN>::kFloats : PipeTile<BN, BKM>::kFloats;
  extern __shared__ __align__(16) float pipe_smem[];
  float* As = pipe_smem;
  float* Bs = pipe_smem + kPipeStages * kAFloats;

  // launched as a programmatic dependent of whatever precedes it on the stream: its own dependents may be scheduled
  // from here on, and nothing is read or written before the predecessor has completed (the wait comes after the tile
  // arithmetic, just before the first load: its divisions overlap the predecessor's tail)
  grid_launch_dependents();
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int parts = (p.ksplit == 2 || p.ksplit == 4) ? p.ksplit : 1;  // CTAs of one cluster that share the tile's k range
  const int tile = static_cast<int>(blockIdx.x) / parts, part = static_cast<int>(blockIdx.x) % parts;
  const int tile_m = tile / p.tiles_n, tile_n = tile % p.tiles_n;
  const int m0 = tile_m * BM, n0 = tile_n * BN;
  // this CTA's k range (whole slices)
  const int k_per = ((p.k + parts - 1) / parts + kPipeK - 1) / kPipeK * kPipeK;
  const int k_begin = part * k_per, k_end = min(p.k, k_begin + k_per);

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // row / column of output (i, j) of this thread inside the tile
  auto row_of = [&](int i) { return (i / 4) * (BM / RG) + ty * 4 + (i % 4); };
  auto col_of = [&](int j) {
    if (BPAIR) return (j / 2) * 32 + tx * 2 + (j % 2);  // pairs of neighbouring columns, 32 columns apart
    return BKM ? tx + 16 * j : (j / 4) * (BN / CG) + tx * 4 + (j % 4);
  };

  const int k_iters = k_end > k_begin ? (k_end - k_begin + kPipeK - 1) / kPipeK : 0;
  grid_dependency_wait();
#pragma unroll
  for (int s = 0; s < kPipeStages - 1; ++s) {
    if (s < k_iters) {
      pipe_load<BM, AK>(As + s * kAFloats, p.A, p.lda, m0, k_begin + s * kPipeK, p.m, k_end, tid);
      if constexpr (BPAIR) pipe_load_pairs<BN>(Bs + s * kBFloats, p.B, p.ldb, n0, k_begin + s * kPipeK, p.n, k_end, tid);
      else pipe_load<BN, BKM>(Bs + s * kBFloats, p.B, p.ldb, n0, k_begin + s * kPipeK, p.n, k_end, tid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }

  for (int it = 0; it < k_iters; ++it) {
    asm volatile("cp.async.wait_group %0;" ::"n"(kPipeStages - 2) : "memory");
    __syncthreads();  // slice `it` has landed for everyone; slice it-1's slot is free for the next copy
    {
      const int nx = it + kPipeStages - 1;
      if (nx < k_iters) {
        const int slot = nx % kPipeStages;
        pipe_load<BM, AK>(As + slot * kAFloats, p.A, p.lda, m0, k_begin + nx * kPipeK, p.m, k_end, tid);
        if constexpr (BPAIR) pipe_load_pairs<BN>(Bs + slot * kBFloats, p.B, p.ldb, n0, k_begin + nx * kPipeK, p.n, k_end, tid);
        else pipe_load<BN, BKM>(Bs + slot * kBFloats, p.B, p.ldb, n0, k_begin + nx * kPipeK, p.n, k_end, tid);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const float* as = As + (it % kPipeStages) * kAFloats;
    const float* bs = Bs + (it % kPipeStages) * kBFloats;
#pragma unroll
    for (int kb = 0; kb < kPipeK / 2; ++kb) {
      float af[2][TM], bf[2][TN];
      if (AK) {
#pragma unroll
        for (int i = 0; i < TM; ++i) {
          const float2 v = *reinterpret_cast<const float2*>(as + row_of(i) * kPipeLdk + 2 * kb);
          af[0][i] = v.x; af[1][i] = v.y;
        }
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int g = 0; g < RG; ++g) {
            const float4 v = *reinterpret_cast<const float4*>(as + (2 * kb + h) * BM + g * (BM / RG) + ty * 4);
            af[h][g * 4 + 0] = v.x; af[h][g * 4 + 1] = v.y; af[h][g * 4 + 2] = v.z; af[h][g * 4 + 3] = v.w;
          }
      }
      if (BPAIR) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int jp = 0; jp < TN / 2; ++jp) {
            const float2 v = *reinterpret_cast<const float2*>(bs + (jp * 16 + tx) * kPipePairLd + (2 * kb + h) * 2);
            bf[h][2 * jp] = v.x; bf[h][2 * jp + 1] = v.y;
          }
      } else if (BKM) {
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          const float2 v = *reinterpret_cast<const float2*>(bs + col_of(j) * kPipeLdk + 2 * kb);
          bf[0][j] = v.x; bf[1][j] = v.y;
        }
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int g = 0; g < CG; ++g) {
            const float4 v = *reinterpret_cast<const float4*>(bs + (2 * kb + h) * BN + g * (BN / CG) + tx * 4);
            bf[h][g * 4 + 0] = v.x; bf[h][g * 4 + 1] = v.y; bf[h][g * 4 + 2] = v.z; bf[h][g * 4 + 3] = v.w;
          }
      }
      if (PACK == 1 || PACK == 3) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int i = 0; i < TM; ++i) {
            const float2 a2 = make_float2(af[h][i], af[h][i]);
#pragma unroll
            for (int j = 0; j < TN; j += 2) {
              const float2 r = __ffma2_rn(a2, make_float2(bf[h][j], bf[h][j + 1]), make_float2(acc[i][j], acc[i][j + 1]));
              acc[i][j] = r.x; acc[i][j + 1] = r.y;
            }
          }
      } else if (PACK == 2) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int j = 0; j < TN; ++j) {
            const float2 b2 = make_float2(bf[h][j], bf[h][j]);
#pragma unroll
            for (int i = 0; i < TM; i += 2) {
              const float2 r = __ffma2_rn(make_float2(af[h][i], af[h][i + 1]), b2, make_float2(acc[i][j], acc[i + 1][j]));
              acc[i][j] = r.x; acc[i + 1][j] = r.y;
            }
          }
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(af[h][i], bf[h][j], acc[i][j]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  if (parts > 1) {
    // The first CTA of the cluster has one mailbox per other part behind its ring, each laid out
    // [16-byte unit][thread] so that a warp's accesses cover 512 consecutive bytes; the others write their sums into
    // theirs over distributed shared memory, and the first adds them in part order (the same order every run).
    constexpr int kBoxFloats = BM * BN;
    float* mailbox = pipe_smem + kPipeStages * (kAFloats + kBFloats);
    if (part > 0) {
      const uint32_t theirs = mapa_shared(smem_u32(mailbox + (part - 1) * kBoxFloats) + static_cast<uint32_t>(tid) * 16u, 0);
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; j += 4)
          st_cluster_v4(theirs + static_cast<uint32_t>((i * TN + j) / 4) * 4096u,
                        make_float4(acc[i][j], acc[i][j + 1], acc[i][j + 2], acc[i][j + 3]));
    }
    cluster_arrive_release();
    cluster_wait_acquire();
    if (part > 0) return;
    for (int q = 1; q < parts; ++q) {
      const float* box = mailbox + (q - 1) * kBoxFloats;
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; j += 4) {
          const float4 v = *reinterpret_cast<const float4*>(box + ((i * TN + j) / 4) * 1024 + tid * 4);
          acc[i][j] += v.x; acc[i][j + 1] += v.y; acc[i][j + 2] += v.z; acc[i][j + 3] += v.w;
        }
    }
  }

  // epilogue: alpha * acc + beta * C, C never read when beta == 0
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int row = m0 + row_of(i);
    if (row >= p.m) continue;
    float* crow = p.C + static_cast<long long>(row) * p.ldc;
    if (!BKM) {
#pragma unroll
      for (int g = 0; g < CG; ++g) {
        const int col = n0 + g * (BN / CG) + tx * 4;
        if (col >= p.n) continue;
        float* dst = crow + col;
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = p.alpha * acc[i][g * 4 + j];
        if (p.c_vec && col + 3 < p.n) {
          if (p.beta != 0.f) {
            const float4 c = *reinterpret_cast<const float4*>(dst);
            v[0] += p.beta * c.x; v[1] += p.beta * c.y; v[2] += p.beta * c.z; v[3] += p.beta * c.w;
          }
          *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (col + j < p.n) {
              float r = v[j];
              if (p.beta != 0.f) r += p.beta * dst[j];
              dst[j] = r;
            }
          }
        }
      }
    } else if (BPAIR) {
#pragma unroll
      for (int j = 0; j < TN; j += 2) {
        const int col = n0 + col_of(j);
        float* dst = crow + col;
        float v0 = p.alpha * acc[i][j], v1 = p.alpha * acc[i][j + 1];
        if (col + 1 < p.n && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
          if (p.beta != 0.f) {
            const float2 c = *reinterpret_cast<const float2*>(dst);
            v0 += p.beta * c.x; v1 += p.beta * c.y;
          }
          *reinterpret_cast<float2*>(dst) = make_float2(v0, v1);
        } else {
          if (col < p.n) { if (p.beta != 0.f) v0 += p.beta * dst[0]; dst[0] = v0; }
          if (col + 1 < p.n) { if (p.beta != 0.f) v1 += p.beta * dst[1]; dst[1] = v1; }
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        const int col = n0 + col_of(j);
        if (col < p.n) {
          float r = p.alpha * acc[i][j];
          if (p.beta != 0.f) r += p.beta * crow[col];
          crow[col] = r;
        }
      }
    }
  }
}

}  // namespace fb
