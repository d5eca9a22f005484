// Device-side preparation for grouped GEMM.
//
// The grouped entry points receive every pointer, size and leading dimension
// as *device* arrays and must not read them on the host.  One small kernel
// turns them into
//   (a) a tile table: per group its sizes, epilogue pointers and the linear
//       index of its first output tile (exclusive prefix sum of tile counts),
//       plus the total tile count, and
//   (b) one TMA tensor map per group and operand, made by patching a host-
//       encoded template (address, extents, row stride) in shared memory and
//       publishing it to global memory with a tensormap-proxy release.
// The persistent GEMM kernel then walks linear tile indices and looks its
// group up in the table.
#pragma once

#include "fb_gemm_tc.cuh"

namespace fb {

enum : int {
  DEV_GROUP_MISALIGNED = 201,  // a group's A/B base or leading dimension is not 16-byte aligned
};

// One pass over the groups = one launch of the GEMM kernel with one tile shape.  The grouped
// entry points use two: CTA-pair tiles (256 rows) for every whole 256-row block of a group, and
// single-CTA tiles (128 rows) for what is left over, so that a group of 300 rows costs
// 256 + 128 rows of tensor work instead of 512.
struct GroupPass {
  int enabled;
  int tile_m;     // rows per tile of this pass (256 or 128)
  int rows_mod;   // 0: the pass covers every row; else: pass covers the first floor(m / rows_mod) * rows_mod
                  // rows (`leading` = 1) or the rows after them (`leading` = 0)
  int leading;
  int block_n;
  GroupRec* recs;       // [num_groups]
  int* total_tiles;     // device scalar
  CUtensorMap* maps;    // [2 * num_groups]: A_g, B_g
  CUtensorMap tmpl_a, tmpl_b, tmpl_a3, tmpl_b3;  // templates: 2-D A, 2-D B, 3-D A, 3-D B
};

struct GroupSetupArgs {
  // mode 0: explicit per-group arrays (group_{bf,h,tf32}gemm)
  const long long* a_ptrs;
  const long long* b_ptrs;
  const long long* c_ptrs;
  const long long* out_ptrs;
  const int* m_sizes;
  const int* n_sizes;
  const int* k_sizes;
  const int* ldas;
  const int* ldbs;
  const int* ldcs;
  // mode 1: cumulative row offsets into one A / out (group_mm)
  const int* offs;
  const void* a_base;
  const void* b_base;
  void* out_base;
  long long mm_lda, mm_ldb, mm_b_group_stride, mm_ldo;
  int mm_n, mm_k;
  int mode;
  int num_groups;
  int b_k_contig;  // 1: B_g stored [n_g, ldb] (K contiguous); 0: stored [k_g, ldb] (N contiguous)
  int esz;         // bytes per element
  int span;        // elements per 128 bytes
  int allow3d;     // build 3-D views where a group's extents allow it
};

__device__ __forceinline__ void tensormap_patch(uint32_t smem_map, const void* gaddr, uint32_t dim0, uint32_t dim1,
                                                uint64_t stride_bytes) {
  asm volatile("tensormap.replace.tile.global_address.shared::cta.b1024.b64 [%0], %1;" ::"r"(smem_map),
               "l"(reinterpret_cast<uint64_t>(gaddr))
               : "memory");
  asm volatile("tensormap.replace.tile.global_dim.shared::cta.b1024.b32 [%0], 0, %1;" ::"r"(smem_map), "r"(dim0)
               : "memory");
  asm volatile("tensormap.replace.tile.global_dim.shared::cta.b1024.b32 [%0], 1, %1;" ::"r"(smem_map), "r"(dim1)
               : "memory");
  asm volatile("tensormap.replace.tile.global_stride.shared::cta.b1024.b64 [%0], 0, %1;" ::"r"(smem_map),
               "l"(stride_bytes)
               : "memory");
}

// 3-D view {128-byte row, dim1, dim2}: only the address, the two outer extents and the pitch of dim1 change.
__device__ __forceinline__ void tensormap_patch3(uint32_t smem_map, const void* gaddr, uint32_t dim1, uint32_t dim2,
                                                 uint64_t stride_bytes) {
  asm volatile("tensormap.replace.tile.global_address.shared::cta.b1024.b64 [%0], %1;" ::"r"(smem_map),
               "l"(reinterpret_cast<uint64_t>(gaddr))
               : "memory");
  asm volatile("tensormap.replace.tile.global_dim.shared::cta.b1024.b32 [%0], 1, %1;" ::"r"(smem_map), "r"(dim1)
               : "memory");
  asm volatile("tensormap.replace.tile.global_dim.shared::cta.b1024.b32 [%0], 2, %1;" ::"r"(smem_map), "r"(dim2)
               : "memory");
  asm volatile("tensormap.replace.tile.global_stride.shared::cta.b1024.b64 [%0], 0, %1;" ::"r"(smem_map),
               "l"(stride_bytes)
               : "memory");
}

// Whole-warp: copy the 128-byte map from shared to global with release semantics
// towards the tensormap proxy.
__device__ __forceinline__ void tensormap_publish(CUtensorMap* gdst, uint32_t smem_map) {
  asm volatile(
      "tensormap.cp_fenceproxy.global.shared::cta.tensormap::generic.release.gpu.sync.aligned [%0], [%1], 128;"
      ::"l"(reinterpret_cast<uint64_t>(gdst)), "r"(smem_map)
      : "memory");
}

// 32 warps: building and publishing one tensor map is a chain of ~1 us steps, so the groups are spread
// over as many warps as one CTA can hold (measured: 25.6 us with 8 warps for 64 groups).
constexpr int kSetupThreads = 1024;

__global__ void __launch_bounds__(kSetupThreads)
group_setup_kernel(const __grid_constant__ GroupPass pass0, const __grid_constant__ GroupPass pass1,
                   const GroupSetupArgs ga) {
  __shared__ __align__(128) uint8_t map_slot[kSetupThreads / 32][128];
  __shared__ int chunk_sum[kSetupThreads];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = ga.num_groups;

  for (int pi = 0; pi < 2; ++pi) {
    const GroupPass& ps = pi == 0 ? pass0 : pass1;
    if (!ps.enabled) continue;

    // ---- per-group records + tensor maps (one warp per group, strided)
    for (int g = warp; g < G; g += kSetupThreads / 32) {
      long long m, n, k, lda, ldb, ldo, ldcin;
      const uint8_t* a;
      const uint8_t* b;
      const void* cin;
      void* out;
      if (ga.mode == 0) {
        m = ga.m_sizes[g]; n = ga.n_sizes[g]; k = ga.k_sizes[g];
        lda = ga.ldas[g]; ldb = ga.ldbs[g]; ldo = ga.ldcs[g]; ldcin = ldo;
        a = reinterpret_cast<const uint8_t*>(ga.a_ptrs[g]);
        b = reinterpret_cast<const uint8_t*>(ga.b_ptrs[g]);
        cin = reinterpret_cast<const void*>(ga.c_ptrs[g]);
        out = reinterpret_cast<void*>(ga.out_ptrs[g]);
      } else {
        const long long start = g == 0 ? 0 : ga.offs[g - 1];
        const long long end = ga.offs[g];
        m = end > start ? end - start : 0;
        n = ga.mm_n; k = ga.mm_k;
        lda = ga.mm_lda; ldb = ga.mm_ldb; ldo = ga.mm_ldo; ldcin = ldo;
        a = reinterpret_cast<const uint8_t*>(ga.a_base) + start * lda * ga.esz;
        b = reinterpret_cast<const uint8_t*>(ga.b_base) + static_cast<long long>(g) * ga.mm_b_group_stride * ga.esz;
        out = reinterpret_cast<uint8_t*>(ga.out_base) + start * ldo * ga.esz;
        cin = out;
      }
      if (m < 0) m = 0;
      if (n < 0) n = 0;
      if (k < 0) k = 0;
      const bool empty = (m == 0 || n == 0);
      const bool aligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0 &&
                           ((lda * ga.esz) & 15) == 0 && ((ldb * ga.esz) & 15) == 0;
      const bool usable = !empty && (aligned || k == 0);
      if (!empty && !usable && lane == 0) atomicCAS(&g_fb_status, 0, DEV_GROUP_MISALIGNED);
      // a 3-D view tiles its third dimension in whole 128-byte rows: that extent must divide evenly
      const bool a3d = ga.allow3d && usable && k > 0 && (k % ga.span) == 0;
      const bool b3d = ga.allow3d && usable && k > 0 && ((ga.b_k_contig ? k : n) % ga.span) == 0;
      // rows of the group this pass is responsible for: [row_base, row_base + rows)
      long long row_base = 0, rows = m;
      if (ps.rows_mod > 0) {
        const long long lead = m / ps.rows_mod * ps.rows_mod;
        if (ps.leading) rows = lead;
        else { row_base = lead; rows = m - lead; }
      }

      if (lane == 0) {
        GroupRec r;
        r.m = static_cast<int>(m); r.n = static_cast<int>(n); r.k = static_cast<int>(k);
        r.tiles_n = static_cast<int>((n + ps.block_n - 1) / ps.block_n);
        // tile_start temporarily holds this group's tile count
        r.tile_start = usable ? static_cast<int>((rows + ps.tile_m - 1) / ps.tile_m) * r.tiles_n : 0;
        r.a3d = a3d ? 1 : 0;
        r.b3d = b3d ? 1 : 0;
        r.row_base = static_cast<int>(row_base);
        r.out = out; r.ldo = ldo; r.cin = cin; r.ldcin = ldcin;
        r.vec_ok = (((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(cin)) & 15) == 0 &&
                    ((ldo * ga.esz) & 15) == 0) ? 1 : 0;
        ps.recs[g] = r;
      }

      const uint32_t slot = smem_u32(map_slot[warp]);
      // A_g: stored [m, lda], K contiguous -> 2-D extents {k, m}, or 3-D {128 B, m, k / span}
      reinterpret_cast<uint32_t*>(map_slot[warp])[lane] =
          reinterpret_cast<const uint32_t*>(a3d ? &ps.tmpl_a3 : &ps.tmpl_a)[lane];
      __syncwarp();
      if (lane == 0 && usable && k > 0) {
        if (a3d) tensormap_patch3(slot, a, static_cast<uint32_t>(m), static_cast<uint32_t>(k / ga.span),
                                  static_cast<uint64_t>(lda * ga.esz));
        else tensormap_patch(slot, a, static_cast<uint32_t>(k), static_cast<uint32_t>(m), static_cast<uint64_t>(lda * ga.esz));
      }
      __syncwarp();
      tensormap_publish(&ps.maps[2 * g], slot);
      __syncwarp();
      reinterpret_cast<uint32_t*>(map_slot[warp])[lane] =
          reinterpret_cast<const uint32_t*>(b3d ? &ps.tmpl_b3 : &ps.tmpl_b)[lane];
      __syncwarp();
      if (lane == 0 && usable && k > 0) {
        const uint64_t pitch = static_cast<uint64_t>(ldb * ga.esz);
        if (ga.b_k_contig) {  // stored [n, ldb]: K contiguous
          if (b3d) tensormap_patch3(slot, b, static_cast<uint32_t>(n), static_cast<uint32_t>(k / ga.span), pitch);
          else tensormap_patch(slot, b, static_cast<uint32_t>(k), static_cast<uint32_t>(n), pitch);
        } else {              // stored [k, ldb]: N contiguous
          if (b3d) tensormap_patch3(slot, b, static_cast<uint32_t>(k), static_cast<uint32_t>(n / ga.span), pitch);
          else tensormap_patch(slot, b, static_cast<uint32_t>(n), static_cast<uint32_t>(k), pitch);
        }
      }
      __syncwarp();
      tensormap_publish(&ps.maps[2 * g + 1], slot);
      __syncwarp();
    }
    __threadfence();
    __syncthreads();

    // ---- exclusive prefix sum of tile counts (each thread owns a contiguous chunk of groups)
    const int per = (G + kSetupThreads - 1) / kSetupThreads;
    const int g0 = tid * per;
    const int g1 = min(G, g0 + per);
    int s = 0;
    for (int g = g0; g < g1; ++g) s += ps.recs[g].tile_start;
    chunk_sum[tid] = s;
    __syncthreads();
    if (tid == 0) {
      int run = 0;
      const int chunks = min(kSetupThreads, (G + per - 1) / per);  // later chunks are empty
      for (int i = 0; i < chunks; ++i) {
        const int c = chunk_sum[i];
        chunk_sum[i] = run;
        run += c;
      }
      *ps.total_tiles = run;
    }
    __syncthreads();
    int run = g0 < G ? chunk_sum[tid] : 0;
    for (int g = g0; g < g1; ++g) {
      const int c = ps.recs[g].tile_start;
      ps.recs[g].tile_start = run;
      run += c;
    }
    __syncthreads();
  }
}

}  // namespace fb
