// Persistent, warp-specialised tcgen05 GEMM for sm_100a (one CTA per SM).
//
//   C[m,n] = alpha * op(A)[m,k] * op(B)[k,n] + beta * Cin[m,n]      (row-major)
//
// Roles inside a 256-thread CTA
//   warp 0      : TMA producer  (global -> 128B-swizzled shared memory ring)
//   warp 1      : MMA issuer    (one thread, tcgen05.mma into TMEM)
//   warp 2      : TMEM allocator / deallocator
//   warp 3      : idle
//   warps 4..7  : epilogue      (tcgen05.ld -> alpha/beta -> cast -> global)
//
// The accumulator is double buffered in TMEM (2 x BLOCK_N fp32 columns), so the
// epilogue of tile i overlaps the main loop of tile i+1.  Transposed operands
// are never physically transposed: an operand whose contiguous dimension is
// M (or N) is fetched with MN-contiguous TMA boxes and described to the tensor
// core as "MN-major".
//
// The same kernel serves the dense entry points (one problem, tiles walked in
// grouped-M order) and the grouped entry points (a device-side table maps a
// linear tile index to group + tile coordinates and per-group tensor maps).
#pragma once

#include "fb_ptx.cuh"

namespace fb {

constexpr int kBlockM = 128;        // rows of C per tile == TMEM lanes
constexpr int kSwizzleBytes = 128;  // bytes of the contiguous dimension per smem row
constexpr int kNumThreads = 256;
constexpr int kEpiWarp0 = 4;        // first epilogue warp (must be a multiple of 4)
constexpr int kSmemLimit = 232448;  // 227 KB opt-in dynamic shared memory

// How one operand's pipeline stage is fetched and described to the MMA.
struct OperandGeom {
  uint32_t boxes;        // TMA boxes per stage
  uint32_t box_bytes;    // bytes per box
  uint32_t box_mn_step;  // MN elements between successive boxes (MN-major only)
  uint32_t mn_major;     // 1: tensor-map x is the MN coordinate; 0: x is K
  uint32_t lbo, sbo;     // descriptor byte offsets
  uint32_t k_adv_bytes;  // descriptor start-address advance per MMA K step
  uint32_t layout;       // descriptor swizzle/layout code (kLayoutSw128 or kLayoutSw128Base32)
};

// One GEMM problem as the epilogue sees it.
struct Problem {
  int m, n;
  void* out;
  long long ldo;
  const void* cin;
  long long ldcin;
  int vec_ok;  // out/cin bases and leading dimensions are 16-byte aligned
};

// Per-group record of the grouped GEMM tile table (built on the device).
struct GroupRec {
  int m, n, k;
  int tile_start;  // first linear tile index of this group
  int tiles_n;
  int vec_ok;
  void* out;
  long long ldo;
  const void* cin;
  long long ldcin;
};

struct TcGemmParams {
  // dense: the single problem.  grouped: unused (see `groups`).
  Problem prob;
  int k;
  int tiles_m, tiles_n;
  int group_m;  // grouped-M swizzle width (tiles)
  float alpha, beta;
  uint32_t idesc;
  uint32_t block_k;  // elements of K per pipeline stage
  OperandGeom a, b;
  // grouped mode (num_groups > 0): table + per-group tensor maps in global memory
  int num_groups;
  const GroupRec* groups;
  const int* total_tiles;        // device scalar written by the table builder
  const CUtensorMap* group_maps;  // [2 * num_groups]: A_g, B_g
};

template <int KIND> struct OutOf { using T = float; };
template <> struct OutOf<0> { using T = __half; };
template <> struct OutOf<1> { using T = __nv_bfloat16; };

__device__ __forceinline__ uint32_t pack2(__half lo, __half hi) {
  __half2 v = __halves2half2(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack2(__nv_bfloat16 lo, __nv_bfloat16 hi) {
  __nv_bfloat162 v = __halves2bfloat162(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <class T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Grouped-M raster: walk `group_m` row-tiles down before stepping one column-tile right.
__device__ __forceinline__ void swizzled_tile(int t, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  const int width = group_m * tiles_n;
  const int gid = t / width;
  const int first_m = gid * group_m;
  const int gsz = min(tiles_m - first_m, group_m);
  const int r = t - gid * width;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

// Epilogue for 32 consecutive columns of one row held in `acc` (fp32 bits).
template <class OutT>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&acc)[32], const Problem& pr, int row, int col0,
                                               float alpha, float beta) {
  if (row >= pr.m || col0 >= pr.n) return;
  const int valid = min(32, pr.n - col0);
  OutT* orow = reinterpret_cast<OutT*>(pr.out) + static_cast<size_t>(row) * pr.ldo + col0;
  const OutT* crow = reinterpret_cast<const OutT*>(pr.cin) + static_cast<size_t>(row) * pr.ldcin + col0;
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = alpha * __uint_as_float(acc[j]);

  constexpr int kPerVec = 16 / sizeof(OutT);  // elements per 16-byte access
  constexpr int kVecs = 32 / kPerVec;
  if (pr.vec_ok && valid == 32) {
    if (beta != 0.f) {
#pragma unroll
      for (int q = 0; q < kVecs; ++q) {
        uint4 raw = __ldg(reinterpret_cast<const uint4*>(crow) + q);
        const OutT* e = reinterpret_cast<const OutT*>(&raw);
#pragma unroll
        for (int j = 0; j < kPerVec; ++j) v[q * kPerVec + j] += beta * to_f32(e[j]);
      }
    }
#pragma unroll
    for (int q = 0; q < kVecs; ++q) {
      uint4 raw;
      if constexpr (sizeof(OutT) == 4) {
        raw.x = __float_as_uint(v[q * 4 + 0]);
        raw.y = __float_as_uint(v[q * 4 + 1]);
        raw.z = __float_as_uint(v[q * 4 + 2]);
        raw.w = __float_as_uint(v[q * 4 + 3]);
      } else {
        raw.x = pack2(from_f32<OutT>(v[q * 8 + 0]), from_f32<OutT>(v[q * 8 + 1]));
        raw.y = pack2(from_f32<OutT>(v[q * 8 + 2]), from_f32<OutT>(v[q * 8 + 3]));
        raw.z = pack2(from_f32<OutT>(v[q * 8 + 4]), from_f32<OutT>(v[q * 8 + 5]));
        raw.w = pack2(from_f32<OutT>(v[q * 8 + 6]), from_f32<OutT>(v[q * 8 + 7]));
      }
      *(reinterpret_cast<uint4*>(orow) + q) = raw;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < valid) {
        float r = v[j];
        if (beta != 0.f) r += beta * to_f32(crow[j]);
        orow[j] = from_f32<OutT>(r);
      }
    }
  }
}

template <int KIND, int BLOCK_N>
struct TcCfg {
  static constexpr int kABytes = kBlockM * kSwizzleBytes;
  static constexpr int kBBytes = BLOCK_N * kSwizzleBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kCtlBytes = 1024;
  static constexpr int kStages = (kSmemLimit - 1024 - kCtlBytes) / kStageBytes > 8
                                     ? 8
                                     : (kSmemLimit - 1024 - kCtlBytes) / kStageBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + kCtlBytes + 1024;
  static constexpr int kTmemCols = 2 * BLOCK_N < 32 ? 32 : 2 * BLOCK_N;
};

// g_fb_status (the device status word) is defined by the including translation unit.

template <int KIND, int BLOCK_N>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const TcGemmParams p) {
  using Cfg = TcCfg<KIND, BLOCK_N>;
  using OutT = typename OutOf<KIND>::T;
  constexpr bool kTf32 = (KIND == 2);
  constexpr int kStages = Cfg::kStages;

  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled TMA/UMMA tiles want 1024-byte aligned stage bases.
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * Cfg::kABytes;
  uint8_t* ctl = smem + kStages * Cfg::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctl);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full_bar = empty_bar + kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtl wctl{abort_flag, &g_fb_status};
  const bool grouped = p.num_groups > 0;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], 4);
    }
    fence_mbar_init();
    if (!grouped) {
      prefetch_tensormap(&tmA);
      prefetch_tensormap(&tmB);
    }
  }
  if (warp == 2) {
    tmem_alloc(tmem_holder, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int num_tiles = grouped ? *p.total_tiles : p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int g = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn, kk_total;
        const CUtensorMap* ma = &tmA;
        const CUtensorMap* mb = &tmB;
        if (grouped) {
          while (g + 1 < p.num_groups && t >= p.groups[g + 1].tile_start) ++g;
          const GroupRec& gr = p.groups[g];
          const int lt = t - gr.tile_start;
          tm = lt / gr.tiles_n;
          tn = lt - tm * gr.tiles_n;
          kk_total = gr.k;
          ma = &p.group_maps[2 * g];
          mb = &p.group_maps[2 * g + 1];
          fence_tensormap_acquire(ma);
          fence_tensormap_acquire(mb);
        } else {
          swizzled_tile(t, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
          kk_total = p.k;
        }
        const int m0 = tm * kBlockM, n0 = tn * BLOCK_N;
        const int k_blocks = (kk_total + static_cast<int>(p.block_k) - 1) / static_cast<int>(p.block_k);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, wctl, DEV_TIMEOUT_PRODUCER_EMPTY)) { ok = false; break; }
          mbar_arrive_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          const int k0 = kb * static_cast<int>(p.block_k);
          uint8_t* sa = smem_a + stage * Cfg::kABytes;
          uint8_t* sb = smem_b + stage * Cfg::kBBytes;
          for (uint32_t bx = 0; bx < p.a.boxes; ++bx) {
            if (p.a.mn_major) tma_load_2d(sa + bx * p.a.box_bytes, ma, &full_bar[stage], m0 + bx * p.a.box_mn_step, k0);
            else tma_load_2d(sa, ma, &full_bar[stage], k0, m0);
          }
          for (uint32_t bx = 0; bx < p.b.boxes; ++bx) {
            if (p.b.mn_major) tma_load_2d(sb + bx * p.b.box_bytes, mb, &full_bar[stage], n0 + bx * p.b.box_mn_step, k0);
            else tma_load_2d(sb, mb, &full_bar[stage], k0, n0);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      int g = 0;
      bool ok = true;
      const int mma_per_stage = kSwizzleBytes / 32;  // 32 bytes of K per MMA for every dtype
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int kk_total = p.k;
        if (grouped) {
          while (g + 1 < p.num_groups && t >= p.groups[g + 1].tile_start) ++g;
          kk_total = p.groups[g].k;
        }
        const int k_blocks = (kk_total + static_cast<int>(p.block_k) - 1) / static_cast<int>(p.block_k);
        if (!mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1u, wctl, DEV_TIMEOUT_MMA_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BLOCK_N);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, wctl, DEV_TIMEOUT_MMA_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem_a + stage * Cfg::kABytes);
          const uint32_t b_addr = smem_u32(smem_b + stage * Cfg::kBBytes);
          const uint64_t a_desc = make_smem_desc(a_addr, p.a.lbo, p.a.sbo, p.a.layout);
          const uint64_t b_desc = make_smem_desc(b_addr, p.b.lbo, p.b.sbo, p.b.layout);
#pragma unroll
          for (int kk = 0; kk < mma_per_stage; ++kk) {
            umma<kTf32>(d_tmem, a_desc + ((kk * p.a.k_adv_bytes) >> 4), b_desc + ((kk * p.b.k_adv_bytes) >> 4),
                        p.idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&tmem_full_bar[acc]);  // accumulator complete -> epilogue
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else if (warp >= kEpiWarp0) {
    // ---------------------------------------------------------------- epilogue
    const int lane_group = warp & 3;  // TMEM lanes [32*lane_group, +32) belong to this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    int g = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int tm, tn;
      Problem pr;
      bool k_is_zero = false;  // a group with k == 0 contributes beta * C only
      if (grouped) {
        while (g + 1 < p.num_groups && t >= p.groups[g + 1].tile_start) ++g;
        const GroupRec& gr = p.groups[g];
        const int lt = t - gr.tile_start;
        tm = lt / gr.tiles_n;
        tn = lt - tm * gr.tiles_n;
        pr.m = gr.m; pr.n = gr.n; pr.out = gr.out; pr.ldo = gr.ldo; pr.cin = gr.cin; pr.ldcin = gr.ldcin;
        pr.vec_ok = gr.vec_ok;
        k_is_zero = gr.k == 0;
      } else {
        swizzled_tile(t, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
        pr = p.prob;
      }
      // warp-uniform outcome: tcgen05.ld below needs the whole warp
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full_bar[acc], acc_phase, wctl, DEV_TIMEOUT_EPI_TMEM_FULL))) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = tm * kBlockM + lane_group * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) +
                             static_cast<uint32_t>(acc * BLOCK_N);
#pragma unroll 1
      for (int c = 0; c < BLOCK_N / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        if (k_is_zero) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (c == BLOCK_N / 32 - 1) {
          // every column of this accumulator is in registers: hand TMEM back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
        }
        epilogue_chunk<OutT>(r, pr, row, tn * BLOCK_N + c * 32, p.alpha, p.beta);
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A wait ran out: give copies and MMAs still in flight time to land
    // before shared memory and TMEM are released.
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

}  // namespace fb
