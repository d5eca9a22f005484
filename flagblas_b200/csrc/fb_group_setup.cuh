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
  DEV_GROUP_MISALIGNED = 201,  // a group's A / B address or pitch is not even a multiple of the element size
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
  int keep_over;  // > 0: a trailing remainder of more than `keep_over` rows stays with the leading pass
  int swap_partial;  // 1 (CTA-pair tiles covering every row): a group's last, partial 256-row block is computed
                     // transposed (see GroupRec::swap_rows); a third tensor map per group fetches its rows
  int block_n;
  GroupRec* recs;       // [num_groups]
  int* starts;          // [num_groups]: first tile index of every group (the same as recs[g].tile_start, densely packed)
  int* total_tiles;     // device: [0] = tile count of the pass, [1] = 1 when some operand has no tensor map
  CUtensorMap* maps;    // [3 * num_groups]: A_g, B_g, and A_g with the box of the partial block's rows
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
  int force_by_hand;  // 1: fetch every operand with ordinary loads, aligned or not (tests, comparisons)
  int publish_each;  // 1: publish every map with its own copy-and-fence instruction (profiling comparison)
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

// Whole-warp: copy the 128-byte map from shared to global memory (plain stores; tensormap_release_all()
// orders them towards the tensormap proxy afterwards).
// Rows per box (dimension 1 of both the 2-D and the 3-D view of a K-contiguous operand).
__device__ __forceinline__ void tensormap_patch_box_rows(uint32_t smem_map, uint32_t rows) {
  asm volatile("tensormap.replace.tile.box_dim.shared::cta.b1024.b32 [%0], 1, %1;" ::"r"(smem_map), "r"(rows) : "memory");
}

__device__ __forceinline__ void tensormap_store(CUtensorMap* gdst, const uint8_t* smem_map, int lane) {
  reinterpret_cast<uint32_t*>(gdst)[lane] = reinterpret_cast<const uint32_t*>(smem_map)[lane];
}

// Whole-warp: copy the 128-byte map from shared to global with release semantics towards the tensormap proxy.
__device__ __forceinline__ void tensormap_publish(CUtensorMap* gdst, uint32_t smem_map) {
  asm volatile(
      "tensormap.cp_fenceproxy.global.shared::cta.tensormap::generic.release.gpu.sync.aligned [%0], [%1], 128;"
      ::"l"(reinterpret_cast<uint64_t>(gdst)), "r"(smem_map)
      : "memory");
}

// Release every tensor map this thread wrote to global memory to later readers through the tensormap
// proxy (they acquire with fence.proxy.tensormap::generic.acquire).  One fence for all maps of a warp:
// the per-map copy-with-fence instruction costs a full fence round trip per map.
__device__ __forceinline__ void tensormap_release_all() {
  asm volatile("fence.proxy.tensormap::generic.release.gpu;" ::: "memory");
}

// CTAs of 32 warps, one group per warp at a time.  Building a tensor map is a chain of dependent steps (argument
// loads, eight tensormap.replace, the proxy release), so the kernel is organised to keep that chain short:
// the four templates are staged in shared memory once (lane-indexed reads of kernel parameters are
// serialised by the constant cache), the arguments of a warp's next group are loaded while the current one is
// being built, and the tile counts are scanned with shuffles out of shared memory instead of being re-read
// from global memory.  64 groups take about 11 us (25.6 us for the first, 8-warp version).
constexpr int kSetupThreads = 1024;
constexpr int kSetupSmemGroups = 1024;  // up to this many groups the tile counts stay in shared memory

struct GroupIn {
  long long m, n, k, lda, ldb, ldo;
  const uint8_t* a;
  const uint8_t* b;
  const void* cin;
  void* out;
};

__device__ __forceinline__ GroupIn load_group(const GroupSetupArgs& ga, int g) {
  GroupIn in;
  if (ga.mode == 0) {
    in.m = ga.m_sizes[g]; in.n = ga.n_sizes[g]; in.k = ga.k_sizes[g];
    in.lda = ga.ldas[g]; in.ldb = ga.ldbs[g]; in.ldo = ga.ldcs[g];
    in.a = reinterpret_cast<const uint8_t*>(ga.a_ptrs[g]);
    in.b = reinterpret_cast<const uint8_t*>(ga.b_ptrs[g]);
    in.cin = reinterpret_cast<const void*>(ga.c_ptrs[g]);
    in.out = reinterpret_cast<void*>(ga.out_ptrs[g]);
  } else {
    const long long start = g == 0 ? 0 : ga.offs[g - 1];
    const long long end = ga.offs[g];
    in.m = end > start ? end - start : 0;
    in.n = ga.mm_n; in.k = ga.mm_k;
    in.lda = ga.mm_lda; in.ldb = ga.mm_ldb; in.ldo = ga.mm_ldo;
    in.a = reinterpret_cast<const uint8_t*>(ga.a_base) + start * in.lda * ga.esz;
    in.b = reinterpret_cast<const uint8_t*>(ga.b_base) + static_cast<long long>(g) * ga.mm_b_group_stride * ga.esz;
    in.out = reinterpret_cast<uint8_t*>(ga.out_base) + start * in.ldo * ga.esz;
    in.cin = in.out;
  }
  if (in.m < 0) in.m = 0;
  if (in.n < 0) in.n = 0;
  if (in.k < 0) in.k = 0;
  return in;
}

// Exclusive prefix sum of one int per thread over the whole CTA (kSetupThreads threads); returns this thread's
// prefix and stores the grand total in *total.  `warp_tot` is 32 ints of shared memory.
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_tot, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, off);
    if (lane >= off) inc += t;
  }
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = warp_tot[lane];
    int winc = w;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, winc, off);
      if (lane >= off) winc += t;
    }
    warp_tot[lane] = winc - w;  // exclusive prefix of the warp totals
    if (lane == 31) *total = winc;
  }
  __syncthreads();
  return warp_tot[warp] + inc - v;
}

// What the table builder decides about one group in one pass (the same function serves the CTAs that build the
// group's record and tensor maps and the CTA that scans the tile counts, so the two always agree).
struct GroupPlan {
  bool usable;           // contributes tiles
  bool bad_alignment;    // non-empty, but an address or pitch is not a multiple of the element size
  bool a_tma, b_tma;     // fetched through a tensor map (otherwise by hand)
  bool a3d, b3d;         // ... a 3-D one
  int a_align, b_align;  // bytes every 16-byte unit of the operand is aligned to (<= 16)
  long long row_base, rows;
  int tiles_n, tiles;
  int swap_rows;
};

__device__ __forceinline__ GroupPlan plan_group(const GroupSetupArgs& ga, const GroupPass& ps, const GroupIn& in) {
  GroupPlan pl;
  const long long m = in.m, n = in.n, k = in.k;
  const bool empty = (m == 0 || n == 0);
  // What base and pitch guarantee for every 16-byte unit of the operand: 16 = TMA can address it; less = the
  // GEMM's producer warps fetch it with loads of that width; less than an element = not a matrix of this type.
  const uintptr_t a_bits = reinterpret_cast<uintptr_t>(in.a) | static_cast<uintptr_t>(in.lda * ga.esz) | 16u;
  const uintptr_t b_bits = reinterpret_cast<uintptr_t>(in.b) | static_cast<uintptr_t>(in.ldb * ga.esz) | 16u;
  pl.a_align = static_cast<int>(a_bits & (~a_bits + 1));
  pl.b_align = static_cast<int>(b_bits & (~b_bits + 1));
  pl.usable = !empty && (k == 0 || (pl.a_align >= ga.esz && pl.b_align >= ga.esz));
  pl.bad_alignment = !empty && !pl.usable;
  pl.a_tma = pl.a_align == 16 && !ga.force_by_hand;
  pl.b_tma = pl.b_align == 16 && !ga.force_by_hand;
  // a 3-D view tiles its third dimension in whole 128-byte rows: that extent must divide evenly
  pl.a3d = ga.allow3d && pl.usable && pl.a_tma && k > 0 && (k % ga.span) == 0;
  pl.b3d = ga.allow3d && pl.usable && pl.b_tma && k > 0 && ((ga.b_k_contig ? k : n) % ga.span) == 0;
  // rows of the group this pass is responsible for: [row_base, row_base + rows)
  pl.row_base = 0;
  pl.rows = m;
  if (ps.rows_mod > 0) {
    long long lead = m / ps.rows_mod * ps.rows_mod;
    if (ps.keep_over > 0 && m - lead > ps.keep_over) lead = m;  // a long remainder is one more (padded) tile of the leading pass
    if (ps.leading) pl.rows = lead;
    else { pl.row_base = lead; pl.rows = m - lead; }
  }
  pl.tiles_n = static_cast<int>((n + ps.block_n - 1) / ps.block_n);
  pl.tiles = pl.usable ? static_cast<int>((pl.rows + ps.tile_m - 1) / ps.tile_m) * pl.tiles_n : 0;
  // the last row block of the group, when it is not a whole one, runs transposed with its row count (rounded up
  // to the MMA's granularity of 16) in the instruction's N slot
  const int part_rows = ps.swap_partial ? static_cast<int>(m % ps.tile_m) : 0;
  pl.swap_rows = (part_rows + 15) / 16 * 16;
  return pl;
}

// Grid: `builders` CTAs that each build the records and tensor maps of their share of the groups (one warp per
// group at a time), plus one last CTA that computes every group's tile count itself, scans them and writes the
// groups' first tile indices, the total and the call-wide flags.  The two kinds of CTA write disjoint fields.
__global__ void __launch_bounds__(kSetupThreads)
group_setup_kernel(const __grid_constant__ GroupPass pass0, const __grid_constant__ GroupPass pass1,
                   const GroupSetupArgs ga) {
  __shared__ __align__(128) uint8_t map_slot[kSetupThreads / 32][3][128];  // per warp: A, B and partial-block A map under construction
  __shared__ __align__(128) uint8_t tmpl[4][128];                           // 2-D A, 2-D B, 3-D A, 3-D B of the pass
  __shared__ int counts[kSetupSmemGroups];
  __shared__ int warp_tot[32];
  __shared__ int total_sh;
  __shared__ int by_hand_sh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = ga.num_groups;
  constexpr int kWarps = kSetupThreads / 32;
  const int builders = static_cast<int>(gridDim.x) - 1;
  const bool scanner = static_cast<int>(blockIdx.x) == builders;
  // the GEMM kernel queued behind this one may start its prologue now; it waits for this grid's completion
  // before reading the table (grid_dependency_wait)
  grid_launch_dependents();
  // this kernel may itself have been launched while its predecessor (the previous call's GEMM, which reads the
  // tables this one rewrites) was still running: nothing is written before that one has completed
  grid_dependency_wait();

  if (scanner) {
    for (int pi = 0; pi < 2; ++pi) {
      const GroupPass& ps = pi == 0 ? pass0 : pass1;
      if (!ps.enabled) continue;
      if (tid == 0) by_hand_sh = 0;
      __syncthreads();
      // ---- exclusive prefix sum of tile counts (each thread owns a contiguous chunk of groups)
      const int per = (G + kSetupThreads - 1) / kSetupThreads;
      const int g0 = tid * per;
      const int g1 = min(G, g0 + per);
      const bool in_smem = G <= kSetupSmemGroups;  // then per == 1 and a group's count is kept instead of recomputed
      int s = 0, by_hand = 0;
      for (int g = g0; g < g1; ++g) {
        const GroupIn in = load_group(ga, g);
        const GroupPlan pl = plan_group(ga, ps, in);
        if (pl.bad_alignment) atomicCAS(&g_fb_status, 0, DEV_GROUP_MISALIGNED);
        if (pl.usable && in.k > 0 && (!pl.a_tma || !pl.b_tma)) by_hand = 1;
        if (in_smem) counts[g] = pl.tiles;
        s += pl.tiles;
      }
      if (by_hand) by_hand_sh = 1;
      int run = block_exclusive_scan(s, warp_tot, &total_sh);
      if (tid == 0) {
        ps.total_tiles[0] = total_sh;
        ps.total_tiles[1] = by_hand_sh;  // some operand has no tensor map: the GEMM's producers run as whole warps
      }
      for (int g = g0; g < g1; ++g) {
        const int c = in_smem ? counts[g] : plan_group(ga, ps, load_group(ga, g)).tiles;
        ps.recs[g].tile_start = run;
        ps.starts[g] = run;
        run += c;
      }
      __syncthreads();
    }
    return;
  }

  for (int pi = 0; pi < 2; ++pi) {
    const GroupPass& ps = pi == 0 ? pass0 : pass1;
    if (!ps.enabled) continue;

    // first group's arguments are in flight while the templates are staged
    const int first = static_cast<int>(blockIdx.x) * kWarps + warp, stride = builders * kWarps;
    GroupIn cur{};
    if (first < G) cur = load_group(ga, first);
    if (warp < 4) {
      const CUtensorMap* t = warp == 0 ? &ps.tmpl_a : (warp == 1 ? &ps.tmpl_b : (warp == 2 ? &ps.tmpl_a3 : &ps.tmpl_b3));
      reinterpret_cast<uint32_t*>(tmpl[warp])[lane] = reinterpret_cast<const uint32_t*>(t)[lane];
    }
    __syncthreads();

    // ---- per-group records + tensor maps (one warp per group, strided over all builder CTAs)
    for (int g = first; g < G; g += stride) {
      const GroupIn in = cur;
      if (g + stride < G) cur = load_group(ga, g + stride);  // next group's loads overlap this group's build
      const GroupPlan pl = plan_group(ga, ps, in);
      const long long m = in.m, n = in.n, k = in.k, lda = in.lda, ldb = in.ldb, ldo = in.ldo, ldcin = in.ldo;
      const uint8_t* a = in.a;
      const uint8_t* b = in.b;
      const bool usable = pl.usable, a_tma = pl.a_tma, b_tma = pl.b_tma, a3d = pl.a3d, b3d = pl.b3d;
      const int swap_rows = pl.swap_rows;

      if (lane == 0) {
        // every field but tile_start, which the scanning CTA writes
        GroupRec* r = &ps.recs[g];
        r->swap_rows = swap_rows;
        r->m = static_cast<int>(m); r->n = static_cast<int>(n); r->k = static_cast<int>(k);
        r->tiles_n = pl.tiles_n;
        r->a_fetch = a_tma ? (a3d ? kFetch3d : kFetch2d) : pl.a_align;
        r->b_fetch = b_tma ? (b3d ? kFetch3d : kFetch2d) : pl.b_align;
        r->row_base = static_cast<int>(pl.row_base);
        r->out = in.out; r->ldo = ldo; r->cin = in.cin; r->ldcin = ldcin;
        r->a = a; r->b = b; r->lda = lda; r->ldb = ldb;
        r->vec_ok = (((reinterpret_cast<uintptr_t>(in.out) | reinterpret_cast<uintptr_t>(in.cin)) & 15) == 0 &&
                     ((ldo * ga.esz) & 15) == 0) ? 1 : 0;
      }

      const uint32_t slot_a = smem_u32(map_slot[warp][0]), slot_b = smem_u32(map_slot[warp][1]);
      const uint32_t slot_r = smem_u32(map_slot[warp][2]);
      __syncwarp();  // the previous group's copies out of these slots are done
      // A_g: stored [m, lda], K contiguous -> 2-D extents {k, m}, or 3-D {128 B, m, k / span}
      reinterpret_cast<uint32_t*>(map_slot[warp][0])[lane] = reinterpret_cast<const uint32_t*>(tmpl[a3d ? 2 : 0])[lane];
      reinterpret_cast<uint32_t*>(map_slot[warp][1])[lane] = reinterpret_cast<const uint32_t*>(tmpl[b3d ? 3 : 1])[lane];
      reinterpret_cast<uint32_t*>(map_slot[warp][2])[lane] = reinterpret_cast<const uint32_t*>(tmpl[a3d ? 2 : 0])[lane];
      __syncwarp();
      if (lane == 0 && usable && a_tma && k > 0) {
        if (a3d) tensormap_patch3(slot_a, a, static_cast<uint32_t>(m), static_cast<uint32_t>(k / ga.span),
                                  static_cast<uint64_t>(lda * ga.esz));
        else tensormap_patch(slot_a, a, static_cast<uint32_t>(k), static_cast<uint32_t>(m), static_cast<uint64_t>(lda * ga.esz));
      }
      if (lane == 1 && usable && b_tma && k > 0) {  // a second lane patches B's map at the same time
        const uint64_t pitch = static_cast<uint64_t>(ldb * ga.esz);
        if (ga.b_k_contig) {  // stored [n, ldb]: K contiguous
          if (b3d) tensormap_patch3(slot_b, b, static_cast<uint32_t>(n), static_cast<uint32_t>(k / ga.span), pitch);
          else tensormap_patch(slot_b, b, static_cast<uint32_t>(k), static_cast<uint32_t>(n), pitch);
        } else {              // stored [k, ldb]: N contiguous
          if (b3d) tensormap_patch3(slot_b, b, static_cast<uint32_t>(k), static_cast<uint32_t>(n / ga.span), pitch);
          else tensormap_patch(slot_b, b, static_cast<uint32_t>(n), static_cast<uint32_t>(k), pitch);
        }
      }
      // third map (a third lane, at the same time): A_g again, with a box of the rows one CTA of the pair fetches of
      // the partial block
      if (lane == 2 && swap_rows > 0 && usable && a_tma && k > 0) {
        if (a3d) tensormap_patch3(slot_r, a, static_cast<uint32_t>(m), static_cast<uint32_t>(k / ga.span),
                                  static_cast<uint64_t>(lda * ga.esz));
        else tensormap_patch(slot_r, a, static_cast<uint32_t>(k), static_cast<uint32_t>(m), static_cast<uint64_t>(lda * ga.esz));
        tensormap_patch_box_rows(slot_r, static_cast<uint32_t>(swap_rows / 2));
      }
      __syncwarp();
      if (ga.publish_each) {
        tensormap_publish(&ps.maps[3 * g], slot_a);
        tensormap_publish(&ps.maps[3 * g + 1], slot_b);
        if (swap_rows > 0) tensormap_publish(&ps.maps[3 * g + 2], slot_r);
      } else {
        tensormap_store(&ps.maps[3 * g], map_slot[warp][0], lane);
        tensormap_store(&ps.maps[3 * g + 1], map_slot[warp][1], lane);
        if (swap_rows > 0) tensormap_store(&ps.maps[3 * g + 2], map_slot[warp][2], lane);
      }
    }
    if (!ga.publish_each) tensormap_release_all();
    __threadfence();
    __syncthreads();
  }
}

}  // namespace fb
