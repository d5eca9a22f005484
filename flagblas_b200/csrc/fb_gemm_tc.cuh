// Persistent, warp-specialised tcgen05 GEMM for sm_100a (one CTA per SM).
//
//   C[m,n] = alpha * op(A)[m,k] * op(B)[k,n] + beta * Cin[m,n]      (row-major)
//
// Roles inside a 256-thread CTA
//   warp 0      : TMA producer for A (arms each stage's barrier)
//   warp 1      : MMA issuer    (one thread, tcgen05.mma into TMEM)
//   warp 2      : TMEM allocator / deallocator
//   warp 3      : TMA producer for B
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

// Profiling switches that skip the MMAs, the copies or the stores of a launch (its results are then meaningless)
// exist only in builds made with -DFB_PROFILING_SWITCHES; the shipped library contains none of those branches.
#ifdef FB_PROFILING_SWITCHES
#define FB_AND_COPIES_ON(p) && !((p).debug & 2)
#define FB_MMA_ON(p) (!((p).debug & 1))
#define FB_STORES_ON(p) (!((p).debug & 4))
#else
#define FB_AND_COPIES_ON(p)
#define FB_MMA_ON(p) true
#define FB_STORES_ON(p) true
#endif

namespace fb {

constexpr int kBlockM = 128;        // rows of C per tile == TMEM lanes
constexpr int kSwizzleBytes = 128;  // bytes of the contiguous dimension per smem row
constexpr int kNumThreads = 256;
constexpr int kEpiWarp0 = 4;        // first epilogue warp (must be a multiple of 4)
constexpr int kSmemLimit = 232448;  // 227 KB opt-in dynamic shared memory
constexpr int kMaxRing = 12;        // most pipeline stages a launch may use (barriers are laid out for this many)
constexpr int kSmallMRows = 64;     // small-M plan: rows of a group per tile ...
constexpr int kSmallMSlot = 32;     // ... and rows of A per CTA and k-slab in the stage slot (half of them)

// How one operand's pipeline stage is fetched and described to the MMA.
//
// A stage holds `TcGemmParams::ks` k-slabs; a k-slab is the operand tile restricted to the
// 128 bytes of K that one swizzle row spans (64 16-bit or 32 fp32 elements).
//   K-major operand : slab = [tile rows][128 B]; slabs of a stage lie one after the other.
//   MN-major operand: [128-byte chunk of MN][k rows of the whole stage][128 B].
// With `use3d` one 3-D TMA instruction fetches the operand's whole stage; otherwise
// `boxes` 2-D boxes per slab do (the fallback when an extent is not a multiple of the
// slab width, and the grouped path).
struct OperandGeom {
  uint32_t mn_major;      // 1: the operand's contiguous dimension is M (or N), not K
  uint32_t use3d;         // 1: one 3-D copy per stage
  uint32_t boxes;         // 2-D path: boxes per k-slab
  uint32_t box_bytes;     // 2-D path: bytes per box
  uint32_t box_mn_step;   // 2-D path, MN-major: MN elements between successive boxes
  uint32_t span;          // elements per 128 bytes
  uint32_t lbo, sbo;      // descriptor byte offsets
  uint32_t k_adv_bytes;   // descriptor start-address advance per MMA inside a k-slab
  uint32_t slab_adv_bytes;  // descriptor start-address advance from one k-slab to the next
  uint32_t layout;        // descriptor swizzle/layout code (kLayoutSw128 or kLayoutSw128Base32)
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
  // How the producers fetch this group's A / B: kFetch2d / kFetch3d = through the group's tensor map (2-D boxes, or
  // a 3-D view with one copy per stage); 2, 4, 8 or 16 = by hand with loads of that many bytes, for an operand
  // whose base or row pitch is not 16-byte aligned (TMA cannot address it).
  int a_fetch, b_fetch;
  int row_base;  // first row of the group this pass covers (rows before it belong to the other pass)
  // > 0: the group's last row block is partial and is computed transposed by the CTA pair: the 256 columns of
  // the tile sit in the MMA's M slot (B_g is its A operand, fetched exactly as for an ordinary tile), the block's
  // rows, rounded up to this multiple of 16, in its N slot (each CTA fetches half of them), and the accumulator
  // holds the tile transposed.  Tensor time and operand bytes then follow the rows that exist instead of 256.
  int swap_rows;
  void* out;
  long long ldo;
  const void* cin;
  long long ldcin;
  // raw operands, for the hand-filled path
  const void* a;
  const void* b;
  long long lda, ldb;  // elements
};
enum : int { kFetch2d = 0, kFetch3d = 1 };  // >= 2: hand-filled, the value is the load width in bytes

struct TcGemmParams {
  // dense: the single problem.  grouped: unused (see `groups`).
  Problem prob;
  int k;
  int tiles_m, tiles_n;
  int group_m;  // grouped-M swizzle width (tiles)
  float alpha, beta;
  uint32_t idesc;
  uint32_t block_k;  // elements of K per pipeline stage (= ks slabs)
  uint32_t ks;       // k-slabs per stage (1 or 2)
  OperandGeom a, b;
  // grouped mode (num_groups > 0): table + per-group tensor maps in global memory
  int num_groups;
  const GroupRec* groups;
  // first tile index of every group once more, as a dense int array: a worker's next tile is typically several groups
  // further on, and walking there through the 104-byte records costs one dependent L2 round trip per group (measured:
  // that walk, done by the producers, the MMA issuer and the epilogue for every tile, shows in calls with many small
  // groups); here 32 groups share a cache line
  const int* group_starts;
  const int* total_tiles;        // written by the table builder: [0] tile count, [1] some operand is fetched by hand
  const CUtensorMap* group_maps;  // [3 * num_groups]: A_g, B_g, A_g boxed for the partial block
  // Stream-K tail (dense mode only).  When `sk_enabled`, every worker first takes `sk_dp` whole tiles
  // (tile = worker + i * workers); each of the `sk_rem` tiles left over (at most half as many as there are
  // workers) goes to `sk_group` neighbouring workers: the first ("owner") takes the head of the k range and
  // finishes the tile, each of the others takes `sk_share` stages, parks its fp32 partial accumulators in
  // `sk_partials` (one slot per worker) and raises `sk_flags[worker]`.  The owner's part is the longer one, by
  // about the time a contributor needs to park its sums, so that it does not have to wait for them.
  // sk_enabled == 2: stream-K over the whole launch instead (see dense_work_item).
  // sk_enabled == 3: a last wave more than half full: `sk_rem` owners take the heads of its tiles, the other workers
  // the tails of `sk_share` stages each, parked in one slot per tile.
  int sk_enabled, sk_dp, sk_rem, sk_group, sk_share;
  // Grouped mode takes the same tail (`sk_grouped`): the tile count is only known on the device, so the workers
  // derive the split themselves; `sk_head` = the owner's head start in stages.
  int sk_grouped, sk_head;
  // Grouped mode, CTA-pair tiles: compute every group's partial last row block transposed (GroupRec::swap_rows).
  int swap_partial;
  // Grouped mode, small-M plan (the caller's hints say the groups have at most a few dozen rows each): EVERY tile is
  // a transposed block of at most 64 rows of a group (tiles per group = ceil(m / 64) x column tiles), each CTA's A
  // stage slot shrinks to 32 rows per k-slab, and the shared memory that frees -- together with the epilogue's
  // staging blocks, which transposed tiles do not use -- holds more stages: such calls stream every group's weights
  // once and are bound by how many bytes a CTA keeps in flight towards HBM.
  int small_m;
  // Dense mode, one row block of fewer than 128 rows, A with k contiguous: A's copies fetch only `a_rows` rows (a
  // multiple of 8) per k-slab and the slabs lie that close together in the stage, so that the TMA unit moves no
  // rows of zeros.  The MMA still reads 128 rows from each slab's start; what it finds past `a_rows` belongs to
  // other slabs and ends up in accumulator rows past m that nobody reads.  0 = whole 128-row slots.
  int a_rows;
  uint32_t idesc_swapped;  // instruction descriptor of such a block with N = 0 (the block's row count is added per tile)
  float* sk_partials;  // [workers][BLOCK_N / 4 units][tile rows][4]
  int* sk_flags;       // [slots][8]: one word per CTA of the pair and epilogue warp; a contributor's warp stores the
                       // launch's `sk_epoch` there when its rows of the slot are parked (nothing has to be zeroed)
  int sk_epoch;        // differs from launch to launch (and is never what a stale or cleared word holds)
  int c_tma;           // dense, beta = 0: whole tiles leave through TMA stores described by the kernel's third map
  // Split-K (dense mode only, `splitk` > 1): every tile's k range is cut into `splitk` contiguous parts handled
  // by different CTAs; each writes its raw fp32 sums to `splitk_out + part * m * n` (row pitch n) and a second
  // kernel adds the parts in order and applies alpha, beta and the output cast.  For shapes with too few
  // output tiles to occupy the GPU (a handful of tokens against a large weight matrix).
  int splitk;
  float* splitk_out;
  // Dense call whose operands were packed by a kernel queued just before this one: this kernel is launched as its
  // programmatic dependent and must wait for it before the first copy.
  int wait_prior;
  // Cluster split-K (dense mode, 128-row tiles, `cluster_k` = 2, 4 or 8 = the launch's cluster size): the CTAs of a
  // cluster share one output tile and take consecutive parts of its k range, and CTA r finishes the r-th
  // BLOCK_N / cluster_k columns of the tile from everybody's fp32 sums, added in rank order.  No scratch memory, no
  // second kernel.  `cluster_push` != 0: every CTA sends its sums straight from TMEM into a receiving area in the
  // shared memory of the CTA that finishes them (`cluster_rows` rows per 16-byte column unit; the launch keeps the
  // operand ring clear of that area); 0: every CTA parks its sums in its own operand ring and the finishing CTA
  // reads them over distributed shared memory (see cluster_finish_tile).
  int cluster_k;
  int cluster_push;
  int cluster_rows;
  // Profiling switches, honoured only by builds with -DFB_PROFILING_SWITCHES (results are meaningless when set):
  // bit 0 = issue no MMA, bit 1 = issue no TMA copy, bit 2 = store nothing.
  int debug;
  int stages;  // pipeline stages actually used (<= the compiled maximum)
  // 512-wide tiles: 1 = this CTA's B stage is ONE copy of 256 consecutive columns of the tile (CTA r of the pair owns
  // tile columns [256 r, 256 r + 256); the MMA half h reads rows [128 h, +128) of it, so accumulator column
  // 256 h + 128 q + c holds tile column 256 q + 128 h + c); 0 = two copies of 128 columns, one per MMA half
  // (accumulator columns in tile order).  One copy instruction less per stage.
  int wide_merged;
  // 1: the staged epilogue writes C with streaming (evict-first) stores, so that a large output does not displace the
  // operand panels other tiles still need from L2
  int c_streaming;
  // Optional cycle accounting (profiling builds of a call): 16 counters written by CTA 0, or null.
  long long* prof;
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
// Two fp32 values rounded (to nearest even, each on its own) and packed by one conversion instruction.
template <class T> __device__ __forceinline__ uint32_t pack2_f32(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2_f32<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2_f32<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2_f32<float>(float lo, float) { return __float_as_uint(lo); }  // (unused)
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <class T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Grouped-M raster: walk `group_m` row-tiles down before stepping one column-tile right.
__device__ __forceinline__ void swizzled_tile(int t, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  if (tiles_m == 1) {  // one row of tiles: the same answer without the divisions (these sit before a call's first copy)
    tm = 0;
    tn = t;
    return;
  }
  // (integer divisions cost well over a hundred cycles each here; a whole group of a power-of-two height, the
  // usual case, needs only the first)
  const int width = group_m * tiles_n;
  const int gid = t < width ? 0 : t / width;
  const int first_m = gid * group_m;
  const int gsz = min(tiles_m - first_m, group_m);
  const int r = t - gid * width;
  if (gsz == group_m && (group_m & (group_m - 1)) == 0) {
    tm = first_m + (r & (group_m - 1));
    tn = r >> (31 - __clz(group_m));
  } else {
    tm = first_m + r % gsz;
    tn = r / gsz;
  }
}

// x / d and x % d for d = 2, 3 or 4 (the sharers of a stream-K tail tile) without a division instruction.
__device__ __forceinline__ void div_small(int x, int d, int& quot, int& rem) {
  quot = d == 2 ? x >> 1 : (d == 4 ? x >> 2 : (d == 3 ? x / 3 : x / d));
  rem = x - quot * d;
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

// Bytes of shared memory one epilogue warp stages its rows through: 32 rows x 128 bytes.
constexpr int kEpiStageBytes = 32 * 128;

// Epilogue of one warp's 32 rows x BLOCK_N columns of an accumulator whose TMEM address is `t_row`.
// A thread owns a row of the accumulator, so direct stores would touch 32 rows with 16 bytes each per
// instruction.  Instead the warp passes 128 bytes per row at a time through its private staging block
// (16-byte units XOR-swizzled by the row, which keeps both directions free of bank conflicts) and
// reads it back so that eight neighbouring lanes write one whole 128-byte row segment; the C operand
// of a beta term comes in the same way.  Column spans that are ragged or unaligned fall back to the
// per-thread path.  `hand_back` runs once, right after the last TMEM read; `add_parts(c, r)` may add to the 32
// sums `r` of accumulator columns [32 c, 32 c + 32) (a stream-K owner: the parts other workers parked).
template <class T, int BLOCK_N, class HandBack, class AddParts>
__device__ __forceinline__ void epilogue_tile_staged(uint32_t t_row, uint8_t* stage, const Problem& pr, int row0,
                                                     int col_base, float alpha, float beta, int lane, bool zero_acc,
                                                     HandBack hand_back, AddParts add_parts, bool wide_merged = false,
                                                     bool streaming = false, int s_begin = 0, int s_end = -1) {
  constexpr int kW = 128 / static_cast<int>(sizeof(T));  // columns per step
  constexpr int kLoads = kW / 32;
  constexpr int kSteps = BLOCK_N / kW;
  constexpr int kPerVec = 16 / static_cast<int>(sizeof(T));
  const uint32_t stage_addr = smem_u32(stage);
  const uint32_t own_row = stage_addr + static_cast<uint32_t>(lane) * 128u;
  const int sub_row = lane >> 3, unit = lane & 7;  // read-out role: row within a group of four, 16-byte unit
  const bool with_c = beta != 0.f;
  const int s_stop = s_end < 0 ? kSteps : s_end;  // (a stream-K sharer finishes only steps [s_begin, s_end) of the tile)
#pragma unroll 1
  for (int s = s_begin; s < s_stop; ++s) {
    int acc_col = s * kW;  // accumulator column of this step -> column of the tile
    if (BLOCK_N == 512 && wide_merged) acc_col = ((acc_col >> 7) & 1) * 256 + (acc_col >> 8) * 128 + (acc_col & 127);
    const int col0 = col_base + acc_col;
    const bool fast = pr.vec_ok && col0 + kW <= pr.n;
    if (fast && with_c) {
      // the C rows of this step, whole row segments per instruction, into the staging block
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int lr = j * 4 + sub_row;
        if (row0 + lr < pr.m) {
          const uint4 c = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(pr.cin) +
                                                               static_cast<size_t>(row0 + lr) * pr.ldcin + col0) + unit);
          st_shared_v4(stage_addr + static_cast<uint32_t>(lr * 128 + ((unit ^ (lr & 7)) << 4)), c);
        }
      }
      __syncwarp();
    }
    uint32_t r[kLoads][32];
#pragma unroll
    for (int q = 0; q < kLoads; ++q) tmem_ld_32x32(t_row + static_cast<uint32_t>(s * kW + q * 32), r[q]);
    tmem_ld_wait();
    if (s == s_stop - 1) hand_back();
    if (zero_acc) {
#pragma unroll
      for (int q = 0; q < kLoads; ++q)
#pragma unroll
        for (int j = 0; j < 32; ++j) r[q][j] = 0u;
    }
#pragma unroll
    for (int q = 0; q < kLoads; ++q) add_parts(s * kLoads + q, r[q]);
    if (!fast) {
#pragma unroll
      for (int q = 0; q < kLoads; ++q) epilogue_chunk<T>(r[q], pr, row0 + lane, col0 + q * 32, alpha, beta);
      continue;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      float v[kPerVec];
#pragma unroll
      for (int j = 0; j < kPerVec; ++j) {
        const int e = u * kPerVec + j;  // column of this step
        v[j] = alpha * __uint_as_float(r[e >> 5][e & 31]);
      }
      const uint32_t slot = own_row + static_cast<uint32_t>((u ^ (lane & 7)) << 4);
      if (with_c) {
        const uint4 raw = ld_shared_v4(slot);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < kPerVec; ++j) v[j] += beta * to_f32(e[j]);
      }
      uint4 raw;
      if constexpr (sizeof(T) == 4) {
        raw.x = __float_as_uint(v[0]); raw.y = __float_as_uint(v[1]);
        raw.z = __float_as_uint(v[2]); raw.w = __float_as_uint(v[3]);
      } else {
        raw.x = pack2_f32<T>(v[0], v[1]);
        raw.y = pack2_f32<T>(v[2], v[3]);
        raw.z = pack2_f32<T>(v[4], v[5]);
        raw.w = pack2_f32<T>(v[6], v[7]);
      }
      st_shared_v4(slot, raw);
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int lr = j * 4 + sub_row;
      const uint4 raw = ld_shared_v4(stage_addr + static_cast<uint32_t>(lr * 128 + ((unit ^ (lr & 7)) << 4)));
      if (row0 + lr < pr.m) {
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<T*>(pr.out) + static_cast<size_t>(row0 + lr) * pr.ldo + col0) + unit;
        if (streaming) __stcs(dst, raw);  // evict-first: the output is not read again by this kernel
        else *dst = raw;
      }
    }
    __syncwarp();  // the block is rewritten by the next step
  }
}

// The same for beta = 0 when C can be described by a tensor map (`c_map`: base and row pitch multiples of 16 bytes):
// the warp writes its 32 rows x 128 bytes of a step into one of its two staging blocks (the 128-byte swizzle the map
// declares is the XOR the staged path uses anyway) and one lane hands the block to the TMA unit, which writes the row
// segments and clips them at the matrix edge.  The warp neither reads the block back nor issues the global stores,
// and with two blocks it fills one while the other drains: what a tile's epilogue keeps the accumulator busy for is
// about the TMEM reads and the conversion.  `seq` counts this warp's steps over the whole kernel (block = seq & 1).
template <class T, int BLOCK_N, class HandBack, class AddParts>
__device__ __forceinline__ void epilogue_tile_tma(uint32_t t_row, uint8_t* blocks, const void* c_map, int m, int n, int row0,
                                                  int col_base, float alpha, int lane, bool zero_acc, HandBack hand_back,
                                                  AddParts add_parts, bool wide_merged, uint32_t& seq, int c_begin = 0,
                                                  int c_end = BLOCK_N / 32) {
  constexpr int kW = 128 / static_cast<int>(sizeof(T));  // columns per step (one staging block)
  constexpr int kLoads = kW / 32;                        // 32-column chunks (one TMEM load each) per step
  constexpr int kChunks = BLOCK_N / 32;
  constexpr int kPerVec = 16 / static_cast<int>(sizeof(T));
  constexpr int kUnits = 32 / kPerVec;                   // 16-byte units of a row that one chunk fills
  const uint32_t base = smem_u32(blocks);
  // The TMEM load of chunk c + 1 is in flight while chunk c is converted and written to the block: two register
  // sets, which the loop (unrolled in pairs) alternates between.
  // (A stream-K sharer finishes only chunks [c_begin, c_end) of the tile, whole steps.)
  uint32_t ra[32], rb[32];
  tmem_ld_32x32(t_row + static_cast<uint32_t>(c_begin * 32), ra);
  auto chunk = [&](int c, uint32_t (&r)[32], uint32_t (&r_next)[32]) {
    tmem_ld_wait();
    if (c + 1 < c_end) tmem_ld_32x32(t_row + static_cast<uint32_t>((c + 1) * 32), r_next);
    else hand_back();  // the last column of the accumulator is in registers
    if (zero_acc) {
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = 0u;
    }
    add_parts(c, r);
    const int q = c % kLoads;  // which part of the step's 128 bytes per row
    const uint32_t blk = base + (seq & 1u) * static_cast<uint32_t>(kEpiStageBytes);
    if (q == 0) {
      // the store that read this block two steps ago must be done reading it (only lane 0 owns bulk groups)
      if (lane == 0) bulk_wait_group_read<1>();
      __syncwarp();
    }
    const uint32_t own_row = blk + static_cast<uint32_t>(lane) * 128u;
#pragma unroll
    for (int u = 0; u < kUnits; ++u) {
      float v[kPerVec];
#pragma unroll
      for (int j = 0; j < kPerVec; ++j) v[j] = alpha * __uint_as_float(r[u * kPerVec + j]);
      uint4 raw;
      if constexpr (sizeof(T) == 4) {
        raw.x = __float_as_uint(v[0]); raw.y = __float_as_uint(v[1]);
        raw.z = __float_as_uint(v[2]); raw.w = __float_as_uint(v[3]);
      } else {
        raw.x = pack2_f32<T>(v[0], v[1]);
        raw.y = pack2_f32<T>(v[2], v[3]);
        raw.z = pack2_f32<T>(v[4], v[5]);
        raw.w = pack2_f32<T>(v[6], v[7]);
      }
      st_shared_v4(own_row + static_cast<uint32_t>(((q * kUnits + u) ^ (lane & 7)) << 4), raw);
    }
    if (q == kLoads - 1) {
      fence_proxy_async();  // this thread's writes to the block, before the TMA unit reads it
      __syncwarp();
      int acc_col = (c / kLoads) * kW;  // accumulator column of this step -> column of the tile
      if (BLOCK_N == 512 && wide_merged) acc_col = ((acc_col >> 7) & 1) * 256 + (acc_col >> 8) * 128 + (acc_col & 127);
      const int col0 = col_base + acc_col;
      if (lane == 0 && row0 < m && col0 < n) {
        tma_store_2d(c_map, blk, col0, row0);
        bulk_commit_group();
      }
      ++seq;
    }
  };
  static_assert(kChunks % 2 == 0, "chunks are processed in pairs");
#pragma unroll 1
  for (int c = c_begin; c < c_end; c += 2) {
    chunk(c, ra, rb);
    if (c + 1 < c_end) chunk(c + 1, rb, ra);
  }
}

// Cluster split-K, after the k loops.  The CTAs of a cluster hold fp32 sums of different k parts of one
// 128 x BLOCK_N tile in TMEM.  CTA r of the cluster finishes columns [r * BLOCK_N / parts, +BLOCK_N / parts) of it:
//   1. every CTA parks its sums in its own shared memory (the operand ring is idle by now), all eight warps
//      taking part: warp w reads TMEM lanes 32 * (w % 4) .. +32 and the column half w / 4;
//   2. cluster barrier;
//   3. every CTA reads its columns of the valid rows from all CTAs of the cluster over distributed shared
//      memory (the reads of all parts are issued before the first is used), adds them in rank order, applies
//      alpha, beta and the cast, and stores them;
//   4. cluster barrier: nobody leaves while a peer may still read its shared memory.
// Layout of a parked tile: [128 rows][BLOCK_N] fp32, 16-byte units XOR-swizzled by the row.
//
// Push form (p.cluster_push): reads over distributed shared memory are round trips and each cluster barrier waits
// for the slowest CTA, so the sums travel as asynchronous stores that count themselves in at the receiver:
//   1. set-up: every CTA initialises `recv_bar`, expects the bytes of all senders on it and arrives at the
//      cluster barrier; the matching wait here returns at once;
//   2. every CTA reads its sums of the valid rows from TMEM and sends each 16-byte unit (st.async) to the CTA that
//      finishes its column, itself included; the receiving area `recv` lies outside the operand ring, so nobody
//      has to ask whether the receiver is done with its operands;
//   3. every CTA waits (bounded, status 108) until its barrier has counted all bytes in, adds the senders' regions
//      in rank order from its own shared memory, applies alpha, beta and the cast, and stores.
// No CTA touches a peer's memory after its own stores, and none leaves before everything sent to it has landed.
// Layout of the receiving area: [cluster_k senders][BLOCK_N / 4 / cluster_k units][p.cluster_rows rows] x 16 bytes,
// the row XOR-ed with the unit's low bits: a warp's 32 rows of one unit are 512 consecutive bytes on the way in, and
// the eight units of a row fall into different banks on the way out.
template <class OutT, int BLOCK_N>
__device__ __forceinline__ void cluster_finish_tile(const TcGemmParams& p, uint32_t parked, uint32_t recv,
                                                    uint64_t* recv_bar, const WaitCtl& wctl, uint32_t tmem_base,
                                                    int tile, bool store) {
  constexpr int kUnits = BLOCK_N / 4;  // 16-byte units (four fp32 sums) per row
  constexpr uint32_t kPitch = BLOCK_N * 4;
  const int parts = p.cluster_k;
  const uint32_t rank = cluster_ctarank();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  int tm, tn;
  swizzled_tile(tile, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
  const Problem& pr = p.prob;
  // a CTA's share: BLOCK_N / parts columns of every valid row (a column slice spreads the work evenly over the
  // cluster however few of the 128 rows exist)
  const int slice_units = kUnits / parts;
  const int rows_valid = min(kBlockM, pr.m - tm * kBlockM);
  // alpha, beta, the cast and the store of the four sums of unit `u` of local row `lrow`
  auto put_unit = [&](int lrow, int u, float (&v)[4]) {
    const int row = tm * kBlockM + lrow, col = tn * BLOCK_N + u * 4;
    OutT* orow = reinterpret_cast<OutT*>(pr.out) + static_cast<size_t>(row) * pr.ldo + col;
    const OutT* crow = reinterpret_cast<const OutT*>(pr.cin) + static_cast<size_t>(row) * pr.ldcin + col;
    const int valid = min(4, pr.n - col);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[j] *= p.alpha;
      if (p.beta != 0.f && j < valid) v[j] += p.beta * to_f32(crow[j]);
    }
    if (pr.vec_ok && valid == 4) {
      if constexpr (sizeof(OutT) == 4) {
        *reinterpret_cast<float4*>(orow) = make_float4(v[0], v[1], v[2], v[3]);
      } else {
        *reinterpret_cast<uint2*>(orow) = make_uint2(pack2(from_f32<OutT>(v[0]), from_f32<OutT>(v[1])),
                                                     pack2(from_f32<OutT>(v[2]), from_f32<OutT>(v[3])));
      }
    } else {
      for (int j = 0; j < valid; ++j) orow[j] = from_f32<OutT>(v[j]);
    }
  };

  if (p.cluster_push) {
    const int unit_shift = __ffs(slice_units) - 1;  // slice_units is a power of two
    const uint32_t unit_pitch = static_cast<uint32_t>(p.cluster_rows) << 4;
    const uint32_t region = static_cast<uint32_t>(slice_units) * unit_pitch;  // what one sender leaves here
    const uint32_t bar_addr = smem_u32(recv_bar);
    // pairs with the arrival at the end of set-up, long ago: every CTA of the cluster has initialised its barrier
    cluster_wait_acquire();
    tc_fence_after();
    {
      const int quadrant = warp & 3, half = warp >> 2;
      const int lrow = quadrant * 32 + lane;
      constexpr int kChunks = BLOCK_N / 64;  // 32-column chunks per column half
      if (quadrant * 32 < rows_valid) {
#pragma unroll 1
        for (int cc = 0; cc < kChunks; ++cc) {
          const int c = half * kChunks + cc;
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quadrant * 32) << 16) + static_cast<uint32_t>(c * 32), r);
          tmem_ld_wait();
          if (lrow < rows_valid) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const int gu = c * 8 + q, dst = gu >> unit_shift, u = gu & (slice_units - 1);
              const uint32_t local = recv + rank * region + static_cast<uint32_t>(u) * unit_pitch +
                                     static_cast<uint32_t>((lrow ^ (u & 7)) << 4);
              st_async_v4(mapa_shared(local, static_cast<uint32_t>(dst)), mapa_shared(bar_addr, static_cast<uint32_t>(dst)),
                          r[q * 4 + 0], r[q * 4 + 1], r[q * 4 + 2], r[q * 4 + 3]);
            }
          }
        }
      }
    }
    tc_fence_before();
    if (p.prof && blockIdx.x == 0 && threadIdx.x == 0) p.prof[7] = clock64();  // timeline: sums sent
    const bool landed = mbar_wait<true>(recv_bar, 0, wctl, 108);
    if (p.prof && blockIdx.x == 0 && threadIdx.x == 0) p.prof[8] = clock64();  // timeline: sums landed
    if (store && landed) {
#pragma unroll 2
      for (int i = threadIdx.x; i < rows_valid * slice_units; i += kNumThreads) {
        const int lrow = i >> unit_shift, u0 = i & (slice_units - 1);
        const int u = static_cast<int>(rank) * slice_units + u0;
        if (tn * BLOCK_N + u * 4 >= pr.n) continue;
        const uint32_t off = recv + static_cast<uint32_t>(u0) * unit_pitch + static_cast<uint32_t>((lrow ^ (u0 & 7)) << 4);
        float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int q = 0; q < 8; ++q)
          if (q < parts) {
            const uint4 x = ld_shared_v4(off + static_cast<uint32_t>(q) * region);
            v[0] += __uint_as_float(x.x); v[1] += __uint_as_float(x.y);
            v[2] += __uint_as_float(x.z); v[3] += __uint_as_float(x.w);
          }
        put_unit(lrow, u, v);
      }
    }
    if (p.prof && blockIdx.x == 0 && threadIdx.x == 0) p.prof[10] = clock64();  // timeline: rows stored
    return;
  }

  tc_fence_after();
  {
    const int quadrant = warp & 3, half = warp >> 2;
    const int lrow = quadrant * 32 + lane;
    const uint32_t row_addr = parked + static_cast<uint32_t>(lrow) * kPitch;
    constexpr int kChunks = BLOCK_N / 64;  // 32-column chunks per column half
#pragma unroll 1
    for (int cc = 0; cc < kChunks; ++cc) {
      const int c = half * kChunks + cc;
      uint32_t r[32];
      tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quadrant * 32) << 16) + static_cast<uint32_t>(c * 32), r);
      tmem_ld_wait();
#pragma unroll
      for (int q = 0; q < 8; ++q)
        st_shared_v4(row_addr + static_cast<uint32_t>(((c * 8 + q) ^ (lrow & 7)) << 4),
                     make_uint4(r[q * 4 + 0], r[q * 4 + 1], r[q * 4 + 2], r[q * 4 + 3]));
    }
  }
  tc_fence_before();
  if (p.prof && blockIdx.x == 0 && threadIdx.x == 0) p.prof[7] = clock64();  // timeline: parked
  cluster_arrive_release();
  cluster_wait_acquire();
  if (p.prof && blockIdx.x == 0 && threadIdx.x == 0) p.prof[8] = clock64();  // timeline: cluster barrier passed

  if (store) {
    uint32_t peer[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) peer[q] = mapa_shared(parked, static_cast<uint32_t>(q < parts ? q : 0));
#pragma unroll 2
    for (int i = threadIdx.x; i < rows_valid * slice_units; i += kNumThreads) {
      const int lrow = i / slice_units, u = static_cast<int>(rank) * slice_units + i % slice_units;
      if (tn * BLOCK_N + u * 4 >= pr.n) continue;
      const uint32_t off = static_cast<uint32_t>(lrow) * kPitch + static_cast<uint32_t>((u ^ (lrow & 7)) << 4);
      float4 x[8];
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (q < parts) x[q] = ld_cluster_v4(peer[q] + off);
      float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (q < parts) { v[0] += x[q].x; v[1] += x[q].y; v[2] += x[q].z; v[3] += x[q].w; }
      put_unit(lrow, u, v);
    }
  }
  if (p.prof && blockIdx.x == 0 && threadIdx.x == 0) p.prof[10] = clock64();  // timeline: rows stored
  cluster_arrive_release();
  cluster_wait_acquire();
}

// One unit of work of a persistent worker: stages [sb, se) of the k loop of one output tile.
enum : int { ITEM_FULL = 0, ITEM_PARTIAL = 1, ITEM_OWNER = 2, ITEM_SPLIT = 3, ITEM_CLUSTER = 4, ITEM_SHARED = 5 };
struct WorkItem {
  int tile;
  int sb, se;
  int kind;
  int part;  // ITEM_SPLIT: which k part; ITEM_SHARED: this worker's place among the tile's sharers
  int first; // ITEM_SHARED: the first of the workers that share the tile
  int slot;  // stream-K: >= 0 names the partial slot of the tile (one contributor); < 0: slots go by worker
};

// The idx-th work item of `worker` in dense mode (see the stream-K fields of TcGemmParams).
// `stages` = k-stages per tile.  Returns false when the worker has no idx-th item.
__device__ __forceinline__ bool dense_work_item(const TcGemmParams& p, int worker, int workers, int stages, int idx,
                                                WorkItem& it) {
  const int tiles = p.tiles_m * p.tiles_n;
  it.part = 0;
  it.first = 0;
  it.slot = -1;
  if (p.cluster_k > 1) {
    // the grid is exactly tiles x cluster_k CTAs: one work item each, the cluster rank picks the k part
    if (idx > 0) return false;
    const int shift = 31 - __clz(p.cluster_k), mask = p.cluster_k - 1;  // (2, 4 or 8 parts)
    it.tile = worker >> shift;
    it.part = worker & mask;
    const int base = stages >> shift, rem = stages & mask;
    it.sb = it.part * base + min(it.part, rem);
    it.se = it.sb + base + (it.part < rem ? 1 : 0);
    it.kind = ITEM_CLUSTER;
    return true;
  }
  if (p.splitk > 1) {
    const int w = worker + idx * workers;
    if (w >= tiles * p.splitk) return false;
    it.tile = w % tiles;
    it.part = w / tiles;
    const int base = stages / p.splitk, rem = stages % p.splitk;
    it.sb = it.part * base + min(it.part, rem);
    it.se = it.sb + base + (it.part < rem ? 1 : 0);
    it.kind = ITEM_SPLIT;
    return true;
  }
  if (!p.sk_enabled) {
    it.tile = worker + idx * workers;
    it.sb = 0; it.se = stages; it.kind = ITEM_FULL;
    return it.tile < tiles;
  }
  if (p.sk_enabled == 3) {
    // Last wave more than half full ("heads and tails"): after `sk_dp` whole waves the first `sk_rem` workers each own
    // one of the remaining tiles and sweep its first stages, all in step like a whole wave, so the operand panels
    // they share are fetched once.  The other workers are helpers: each takes the last `sk_share` stages of one
    // owner's tile after another (helper h: tiles h, h + helpers, ...; also in step with one another), parks
    // the partial sums in the tile's slot, and the owner adds them in its epilogue.  The owners' share is sized so
    // that a helper's last tail is parked when the owners finish.
    if (idx < p.sk_dp) {
      it.tile = worker + idx * workers;
      it.sb = 0; it.se = stages; it.kind = ITEM_FULL;
      return true;
    }
    const int j = idx - p.sk_dp;
    const int first = p.sk_dp * workers;
    const int owner_len = stages - p.sk_share;
    if (worker < p.sk_rem) {
      if (j > 0) return false;
      it.tile = first + worker;
      it.sb = 0; it.se = owner_len; it.kind = ITEM_OWNER;
      it.slot = worker;
      return true;
    }
    const int tl = worker - p.sk_rem + j * (workers - p.sk_rem);
    if (tl >= p.sk_rem) return false;
    it.tile = first + tl;
    it.sb = owner_len; it.se = stages; it.kind = ITEM_PARTIAL;
    it.slot = tl;
    return true;
  }
  if (p.sk_enabled == 2) {
    // Few waves, the last one more than half full: the first `sk_dp` waves run whole tiles, all workers sweeping k
    // in step (which is what keeps the shared operand panels in L2: dealing out the stages of ALL tiles was measured
    // 19 % slower than whole tiles on 8192 x 1024 x 8192, each panel then being fetched from HBM once per tile that
    // uses it).  The k stages of the remaining tiles, whose operands fit L2 together, form one
    // line of tiles x stages units that is cut into `workers` equal ranges.  A range that starts inside a tile
    // begins with that tile's tail (a partial, parked for the worker before it, which holds the tile's first
    // stages and finishes it); then come whole tiles; a range that ends inside a tile ends with that tile's head,
    // whose worker owns the tile and adds the parts of the workers after it -- parts that were the first thing
    // those workers did, so they are parked long before the owner's epilogue asks for them.
    if (idx < p.sk_dp) {
      it.tile = worker + idx * workers;
      it.sb = 0; it.se = stages; it.kind = ITEM_FULL;
      return true;
    }
    const int first = p.sk_dp * workers;  // first tile of the line
    const long long line = static_cast<long long>(tiles - first) * stages;
    long long lo = worker * line / workers;
    const long long hi = (worker + 1) * line / workers;
    for (int i = p.sk_dp;; ++i) {
      if (lo >= hi) return false;
      const long long t = lo / stages;
      const int sb = static_cast<int>(lo - t * stages);
      const int se = static_cast<int>(min(static_cast<long long>(stages), sb + (hi - lo)));
      if (i == idx) {
        it.tile = first + static_cast<int>(t);
        it.sb = sb; it.se = se;
        it.kind = sb > 0 ? ITEM_PARTIAL : (se == stages ? ITEM_FULL : ITEM_OWNER);
        if (it.kind == ITEM_OWNER) {
          // workers worker + 1 .. v hold the rest of the tile: v = the one whose range contains its last stage
          const long long last = (t + 1) * stages - 1;
          int v = worker + 1;
          while ((v + 1) * line / workers <= last) ++v;
          it.part = v - worker + 1;  // workers that share the tile
        }
        return true;
      }
      lo += se - sb;
    }
  }
  if (idx < p.sk_dp) {
    it.tile = worker + idx * workers;
    it.sb = 0; it.se = stages; it.kind = ITEM_FULL;
    return true;
  }
  if (idx > p.sk_dp) return false;
  // the tail: tile `tl` is shared by workers tl * sk_group .. + sk_group - 1
  int tl, j;
  div_small(worker, p.sk_group, tl, j);
  if (tl >= p.sk_rem) return false;  // more workers than tail parts: this one is done
  it.tile = p.sk_dp * workers + tl;
  if (p.sk_group == 2) {
    // Two sharers: the first owns the tile (the head of the k range, longer by about the time the other needs to
    // park its sums, and the whole epilogue), the second contributes `sk_share` stages.  (Measured against both
    // finishing half of the columns each: 512 x 4096 x 4096 25.2 against 26.9 us, 256 x 8192 x 8192 43.1 / 44.3,
    // 512 x 4096 x 14336 57.4 / 60.7 -- the exchange is bound by L2 bandwidth either way, and the owner's head start
    // hides the other's parking.)
    const int owner_len = stages - p.sk_share;
    if (j == 0) {
      it.sb = 0; it.se = owner_len; it.kind = ITEM_OWNER;
    } else {
      it.sb = owner_len; it.se = stages; it.kind = ITEM_PARTIAL;
    }
    return true;
  }
  // Three or four sharers: equal parts of the k range, and every sharer finishes a part of the tile's columns
  // (1024 x 1536 x 4096, three sharers: 24.3 - 25.5 us against 25.8 - 26.9 with one owner adding two parked parts).
  int base, extra;
  div_small(stages, p.sk_group, base, extra);
  it.sb = j * base + min(j, extra);
  it.se = it.sb + base + (j < extra ? 1 : 0);
  it.kind = ITEM_SHARED;
  it.part = j;
  it.first = worker - j;
  return true;
}

// Grouped mode: the idx-th tile of `worker`, and in the stream-K tail its role (0 = owner, > 0 = contributor,
// -1 = a whole tile) and the number of workers that share the tile.  False when the worker has no idx-th tile.
__device__ __forceinline__ bool grouped_tile(const TcGemmParams& p, int worker, int workers, int num_tiles, int idx,
                                             int& t, int& role, int& sharers) {
  role = -1;
  sharers = 1;
  if (p.sk_grouped) {
    const int dp = num_tiles / workers, rem = num_tiles - dp * workers;
    int grp = rem > 0 ? workers / rem : 1;
    if (grp > 4) grp = 4;
    if (grp >= 2 && idx >= dp) {
      if (idx > dp) return false;
      const int tl = worker / grp;
      if (tl >= rem) return false;
      t = dp * workers + tl;
      role = worker % grp;
      sharers = grp;
      return true;
    }
  }
  t = worker + idx * workers;
  return t < num_tiles;
}

// Stage range and kind of a grouped work item whose tile has `stages` k-stages.  A tail tile too short to be worth
// splitting is done whole by its owner; false tells a contributor that it has nothing to do.
__device__ __forceinline__ bool grouped_range(const TcGemmParams& p, int stages, int role, int sharers, WorkItem& it) {
  it.part = 0;
  it.slot = -1;
  const int share = sharers > 1 ? (stages - p.sk_head) / sharers : 0;
  if (role < 0 || share < 2) {
    it.sb = 0; it.se = stages; it.kind = ITEM_FULL;
    return role <= 0;
  }
  const int owner_len = stages - (sharers - 1) * share;
  if (role == 0) {
    it.sb = 0; it.se = owner_len; it.kind = ITEM_OWNER;
  } else {
    it.sb = owner_len + (role - 1) * share; it.se = it.sb + share; it.kind = ITEM_PARTIAL;
  }
  return true;
}

// ---- operand stages filled by hand (grouped calls: an operand whose base or row pitch is not 16-byte aligned
// cannot be described by a tensor map, and the host never sees the addresses)
//
// One 16-byte unit of a stage holds 16 / ESZ consecutive elements of the operand's contiguous dimension; `valid` of
// them exist (the rest lies beyond the matrix and reads as zero, like a TMA box that crosses the edge).  VEC = bytes
// per load = the alignment that base and pitch guarantee for every unit.
template <int ESZ, int VEC>
__device__ __forceinline__ uint4 load_unit(const uint8_t* src, int valid) {
  constexpr int kPer = 16 / ESZ;
  uint32_t w[4] = {0u, 0u, 0u, 0u};
  if (valid >= kPer) {
    if constexpr (VEC == 16) {
      return __ldg(reinterpret_cast<const uint4*>(src));
    } else if constexpr (VEC == 8) {
      const uint2 lo = __ldg(reinterpret_cast<const uint2*>(src)), hi = __ldg(reinterpret_cast<const uint2*>(src) + 1);
      return make_uint4(lo.x, lo.y, hi.x, hi.y);
    } else if constexpr (VEC == 4) {
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = __ldg(reinterpret_cast<const uint32_t*>(src) + j);
      return make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  if constexpr (ESZ == 4) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (j < valid) w[j] = __ldg(reinterpret_cast<const uint32_t*>(src) + j);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < valid) w[j >> 1] |= static_cast<uint32_t>(__ldg(reinterpret_cast<const unsigned short*>(src) + j)) << ((j & 1) * 16);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Whole warp: writes this CTA's part of one pipeline stage of one operand (`ks` k-slabs of a `tile_mn`-row tile
// starting at row / column `mn0`, k offset `k0`) in exactly the swizzled layout the TMA copies produce, then
// credits the bytes to the stage's barrier (`bar_addr`, a shared::cluster address), each lane for what it wrote.
//   K-major operand (stored [mn, ld], K contiguous):  [slab][tile row][128 B], 16-byte units XORed with row % 8.
//   MN-major operand (stored [k, ld], MN contiguous): [128-byte chunk of MN][k row of the stage][128 B]; units XORed
//     with k row % 8, or for 32-bit elements 32-byte atoms XORed with k row % 4.
template <int ESZ, int VEC>
__device__ __noinline__ void fill_stage_by_hand(uint8_t* dst, uint32_t bar_addr, int mn_major, int ks, int tile_mn,
                                                const uint8_t* base, long long ld, int mn0, int mn_limit, int k0,
                                                int k_limit) {
  constexpr int kPer = 16 / ESZ, kSpan = 128 / ESZ;
  constexpr int kBatch = 16;  // units a lane has in flight: all loads of a batch are issued before the first store
  const int lane = threadIdx.x & 31;
  const int total = ks * tile_mn * 8;  // 16-byte units
  const int k_rows = kSpan * ks;
  const uint32_t dst_addr = smem_u32(dst);
  for (int u0 = lane; u0 < total; u0 += 32 * kBatch) {
    uint4 v[kBatch];
    uint32_t off[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int u = u0 + 32 * i;
      v[i] = make_uint4(0u, 0u, 0u, 0u);
      off[i] = 0xffffffffu;
      if (u < total) {
        const int unit = u & 7, rr = u >> 3;
        long long r_src, c_src;  // row and first column of the unit in the stored matrix
        int valid;
        if (!mn_major) {
          const int slab = rr / tile_mn, row = rr - slab * tile_mn;
          const int r = mn0 + row, kk = k0 + slab * kSpan + unit * kPer;
          valid = r < mn_limit ? k_limit - kk : 0;
          off[i] = static_cast<uint32_t>(rr * 128 + ((unit ^ (row & 7)) << 4));
          r_src = r; c_src = kk;
        } else {
          const int krow = rr % k_rows;
          const int kk = k0 + krow, mn = mn0 + (rr / k_rows) * kSpan + unit * kPer;
          valid = kk < k_limit ? mn_limit - mn : 0;
          const int su = ESZ == 4 ? ((((unit >> 1) ^ (krow & 3)) << 1) | (unit & 1)) : (unit ^ (krow & 7));
          off[i] = static_cast<uint32_t>(rr * 128 + (su << 4));
          r_src = kk; c_src = mn;
        }
        if (valid > 0) v[i] = load_unit<ESZ, VEC>(base + (r_src * ld + c_src) * ESZ, valid);
      }
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i)
      if (off[i] != 0xffffffffu) st_shared_v4(dst_addr + off[i], v[i]);
  }
  fence_proxy_async_all();
  fence_acq_rel_cluster();
  mbar_complete_tx_cluster(bar_addr, static_cast<uint32_t>(total / 32) * 16u);
}

template <int ESZ>
__device__ __forceinline__ void fill_stage_dispatch(int vec, uint8_t* dst, uint32_t bar_addr, int mn_major, int ks,
                                                    int tile_mn, const void* base, long long ld, int mn0, int mn_limit,
                                                    int k0, int k_limit) {
  const uint8_t* b = static_cast<const uint8_t*>(base);
  if (vec >= 16) fill_stage_by_hand<ESZ, 16>(dst, bar_addr, mn_major, ks, tile_mn, b, ld, mn0, mn_limit, k0, k_limit);
  else if (vec == 8) fill_stage_by_hand<ESZ, 8>(dst, bar_addr, mn_major, ks, tile_mn, b, ld, mn0, mn_limit, k0, k_limit);
  else if (vec == 4) fill_stage_by_hand<ESZ, 4>(dst, bar_addr, mn_major, ks, tile_mn, b, ld, mn0, mn_limit, k0, k_limit);
  else if constexpr (ESZ == 2) fill_stage_by_hand<ESZ, 2>(dst, bar_addr, mn_major, ks, tile_mn, b, ld, mn0, mn_limit, k0, k_limit);
}

// PAIR = true: two CTAs of a cluster work on one 256 x BLOCK_N tile with
// tcgen05 cta_group::2.  Each CTA fetches its own 128 rows of A and its own half
// of the B tile into its own shared memory, the leader CTA (cluster rank 0)
// issues every MMA for both, and each CTA's TMEM ends up with its 128 rows of
// the accumulator.  Per CTA that is a third less operand traffic and shared
// memory per K step than a 128 x BLOCK_N tile, so the same shared memory holds a
// deeper prefetch ring.
template <int KIND, int BLOCK_N, bool PAIR>
struct TcCfg {
  static constexpr int kABytes = kBlockM * kSwizzleBytes;
  static constexpr int kBRows = PAIR ? BLOCK_N / 2 : BLOCK_N;  // B-tile rows this CTA holds
  static constexpr int kBBytes = kBRows * kSwizzleBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kCtlBytes = 1024;
  static constexpr int kEpiBytes = 8 * kEpiStageBytes;  // two staging blocks for each of the four epilogue warps
  static constexpr int kStages = (kSmemLimit - 1024 - kCtlBytes - kEpiBytes) / kStageBytes > 8
                                     ? 8
                                     : (kSmemLimit - 1024 - kCtlBytes - kEpiBytes) / kStageBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + kCtlBytes + kEpiBytes + 1024;
  // One MMA instruction covers at most 256 columns; a 512-wide tile is two halves side by side in
  // TMEM and fills all 512 columns, so its accumulator cannot be double buffered.
  static constexpr int kMmaN = BLOCK_N > 256 ? 256 : BLOCK_N;
  static constexpr int kHalves = BLOCK_N / kMmaN;
  static constexpr int kAccBufs = BLOCK_N > 256 ? 1 : 2;
  static constexpr int kTmemCols = kAccBufs * BLOCK_N < 32 ? 32 : kAccBufs * BLOCK_N;
  static constexpr int kHalfBBytes = kBBytes / kHalves;  // bytes of one half of this CTA's B slab
  static constexpr int kTileM = PAIR ? 2 * kBlockM : kBlockM;  // rows of C per scheduled tile
  static_assert(BLOCK_N <= 256 || PAIR, "512-wide tiles exist only as CTA-pair tiles");
};

// g_fb_status (the device status word) is defined by the including translation unit.

template <int KIND, int BLOCK_N, bool PAIR>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const TcGemmParams p) {
  using Cfg = TcCfg<KIND, BLOCK_N, PAIR>;
  using OutT = typename OutOf<KIND>::T;
  constexpr bool kTf32 = (KIND == 2);
  constexpr int kStages = Cfg::kStages;

  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled TMA/UMMA tiles want 1024-byte aligned stage bases.
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  // [control block: barriers][operand ring: A slots of every stage, then B slots][epilogue staging blocks]; the
  // small-M plan lets the ring run on into the staging blocks, which it does not use
  uint8_t* ctl = smem;
  uint8_t* ring = smem + Cfg::kCtlBytes;
  uint8_t* epi_staging = ring + kStages * Cfg::kStageBytes;
  // one k-slab of A in a stage
  const uint32_t a_slot_bytes = p.small_m ? kSmallMSlot * kSwizzleBytes
                                          : (p.a_rows ? static_cast<uint32_t>(p.a_rows) * kSwizzleBytes : Cfg::kABytes);
  uint8_t* smem_a = ring;
  uint8_t* smem_b = ring + static_cast<uint32_t>(p.stages) * p.ks * a_slot_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctl);
  uint64_t* empty_bar = full_bar + kMaxRing;
  uint64_t* tmem_full_bar = empty_bar + kMaxRing;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  uint64_t* recv_bar = reinterpret_cast<uint64_t*>(tmem_holder + 2);  // cluster split-K, push form

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtl wctl{abort_flag, &g_fb_status};
  const bool grouped = p.num_groups > 0;
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;  // 0 = leader of the pair
  const int worker = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int num_workers = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

  if (p.prof && blockIdx.x == 0 && threadIdx.x == 0) p.prof[3] = clock64();  // timeline: entry
  // Whatever is queued behind this kernel as a programmatic dependent (the next GEMM of the caller, the kernel
  // that adds split-K parts) may take SMs as this grid's CTAs leave them and run its prologue; it waits for the
  // whole grid before it touches global memory.
  grid_launch_dependents();
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kMaxRing; ++s) {
      mbar_init(&full_bar[s], 1);   // the (leader's) producer arrival + transaction bytes
      mbar_init(&empty_bar[s], 1);  // one tcgen05.commit arrival
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], PAIR ? 8 : 4);  // epilogue warps of every CTA that reads this accumulator
    }
    mbar_init(recv_bar, 1);  // (one arrival, by the first epilogue warp, which also says how many bytes to expect)
    fence_mbar_init();
    if (!grouped) {
      prefetch_tensormap(&tmA);
      prefetch_tensormap(&tmB);
    }
  }
  if (warp == 2) {
    if constexpr (PAIR) {
      tmem_alloc_pair(tmem_holder, Cfg::kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_holder, Cfg::kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if constexpr (PAIR) {
    // barriers of both CTAs must be initialised before either touches the other's
    cluster_arrive_release();
    cluster_wait_acquire();
  } else {
    __syncthreads();
    // (the barrier initialisations above were released to the cluster by fence_mbar_init; the wait is in
    // cluster_finish_tile)
    if (p.cluster_push) cluster_arrive_relaxed();
  }
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  if (p.prof && blockIdx.x == 0 && threadIdx.x == 0) p.prof[4] = clock64();  // timeline: set-up done

  // Every launch is a programmatic dependent of whatever precedes it on the stream (the table builder, a packing
  // kernel, the caller's previous kernel): all of the above overlapped with its tail, and global memory may be
  // touched only after the wait.  A grouped call reads the builder's table right away.  A dense call puts the wait
  // off: its producer threads work out their first tile first and wait just before the first copy, its epilogue
  // warps wait before they wait for an accumulator, and the other warps touch no global memory (the whole-CTA
  // finish of a cluster split-K call comes after all of these).
  if (grouped) grid_dependency_wait();
  const int num_tiles = grouped ? *p.total_tiles : p.tiles_m * p.tiles_n;
  // k-stages per dense tile (block_k is a power of two: 128 bytes of k times one or two slabs)
  const int dense_stages = (p.k + static_cast<int>(p.block_k) - 1) >> (31 - __clz(static_cast<int>(p.block_k)));

  if (warp == 0 || warp == 3) {
    // ----------------------------------------------------------- producers
    // Two issuing threads so that the copies of one stage are not serialised behind each
    // other: warp 0 arms the stage's barrier and fetches A, warp 3 fetches B.
    // A grouped call in which some operand cannot be addressed by TMA (`by_hand`, found by the table builder) runs
    // the loop with all 32 lanes: lane 0 still issues the copies of the operands that have tensor maps, the whole
    // warp fills the others with ordinary loads and stores and credits the stage's barrier with the same byte count.
    const bool by_hand = grouped && p.total_tiles[1] != 0;
    if (by_hand || lane == 0) {
      const bool load_a = warp == 0;
      const OperandGeom& og = load_a ? p.a : p.b;
      int stage = 0;
      uint32_t phase = 0;
      int g = 0;
      bool ok = true;
      long long prof_wait = 0, prof_issue = 0;
      for (int idx = 0; ok; ++idx) {
        WorkItem item;
        int t, role = -1, sharers = 1;
        if (grouped) {
          if (!grouped_tile(p, worker, num_workers, num_tiles, idx, t, role, sharers)) break;
        } else {
          if (!dense_work_item(p, worker, num_workers, dense_stages, idx, item)) break;
          t = item.tile;
        }
        int tm, tn, kk_total;
        const CUtensorMap* map = load_a ? &tmA : &tmB;
        uint32_t use3d = og.use3d;
        int row_base = 0;
        int swap_half = 0;             // > 0: a transposed block; rows of A_g each CTA of the pair contributes
        int tile_rows = Cfg::kTileM;   // rows of the group per scheduled tile
        int fetch = kFetch2d;          // grouped: how this group's operand is fetched
        const void* raw = nullptr;     // hand-filled operand: base, pitch and extent along M / N
        long long raw_ld = 0;
        int mn_limit = 0;
        if (grouped) {
          while (g + 1 < p.num_groups && t >= __ldg(p.group_starts + g + 1)) ++g;
          const GroupRec& gr = p.groups[g];
          const int lt = t - gr.tile_start;
          tm = lt / gr.tiles_n;
          tn = lt - tm * gr.tiles_n;
          kk_total = gr.k;
          map = &p.group_maps[3 * g + (load_a ? 0 : 1)];
          fetch = load_a ? gr.a_fetch : gr.b_fetch;
          use3d = fetch == kFetch3d;
          row_base = gr.row_base;
          if (PAIR && p.small_m) {
            // small-M plan: every tile is a transposed block of up to 64 rows; a CTA's box is 32 rows high, of which
            // the MMA reads the first swap_half (what the box holds beyond them lies past the group's rows or is not used)
            swap_half = ((min(kSmallMRows, gr.m - tm * kSmallMRows) + 15) >> 4) << 3;
            tile_rows = kSmallMRows;
          } else if (PAIR && p.swap_partial && gr.swap_rows > 0 && tm == gr.m / Cfg::kTileM) {
            // partial last row block, computed transposed: B_g is fetched as ever; of A_g each CTA fetches its half
            // of the block's rows through the group's third map (or by hand)
            swap_half = gr.swap_rows >> 1;
            if (load_a) map = &p.group_maps[3 * g + 2];
          }
          if (fetch > kFetch3d) {
            raw = load_a ? gr.a : gr.b;
            raw_ld = load_a ? gr.lda : gr.ldb;
            mn_limit = load_a ? gr.m : gr.n;
          } else if (lane == 0) {
            fence_tensormap_acquire(map);
          }
        } else {
          swizzled_tile(t, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
          kk_total = p.k;
        }
        // first row (A) / first column (B) of the operand slab this CTA fetches
        const int mn0 = load_a ? row_base + tm * tile_rows + static_cast<int>(cta_rank) * (swap_half ? swap_half : kBlockM)
                               : tn * BLOCK_N + static_cast<int>(cta_rank) * (p.wide_merged ? Cfg::kBRows : Cfg::kBRows / Cfg::kHalves);
        const int k_blocks = (kk_total + static_cast<int>(p.block_k) - 1) >> (31 - __clz(static_cast<int>(p.block_k)));
        if (grouped && !grouped_range(p, k_blocks, role, sharers, item)) break;
        const int kb_begin = item.sb, kb_end = item.se;
        // bytes of A per k-slab that this CTA puts into the stage (fewer rows in a transposed partial block)
        const uint32_t a_slab_bytes = p.small_m ? a_slot_bytes
                                                : (swap_half ? static_cast<uint32_t>(swap_half) * kSwizzleBytes : a_slot_bytes);
        if (!grouped && idx == 0) grid_dependency_wait();
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          const long long c0 = p.prof ? clock64() : 0;
          if (by_hand) {
            if (!mbar_wait_warp<0>(&empty_bar[stage], phase ^ 1u, wctl, DEV_TIMEOUT_PRODUCER_EMPTY)) { ok = false; break; }
          } else if (!mbar_wait(&empty_bar[stage], phase ^ 1u, wctl, DEV_TIMEOUT_PRODUCER_EMPTY)) { ok = false; break; }
          const long long c1 = p.prof ? clock64() : 0;
          prof_wait += c1 - c0;
          const int k0 = kb * static_cast<int>(p.block_k);
          const uint32_t a_stage_bytes = p.ks * a_slot_bytes, b_stage_bytes = p.ks * Cfg::kBBytes;
          uint8_t* dst = load_a ? smem_a + stage * a_stage_bytes : smem_b + stage * b_stage_bytes;
          const uint32_t slab_bytes = load_a ? a_slab_bytes : Cfg::kBBytes;
          uint32_t bar = smem_u32(&full_bar[stage]);
          if constexpr (PAIR) bar = mapa_shared(bar, 0);  // both CTAs' copies are credited to the leader's barrier
          if (load_a && cta_rank == 0 && lane == 0) {
#ifdef FB_PROFILING_SWITCHES
            if (p.debug & 2) mbar_arrive(&full_bar[stage]);
            else
#endif
            mbar_arrive_expect_tx(&full_bar[stage], (PAIR ? 2u : 1u) * (p.ks * a_slab_bytes + b_stage_bytes));
          }
          if (fetch > kFetch3d) {
            // no tensor map for this operand: the whole warp fills the stage
            fill_stage_dispatch<kTf32 ? 4 : 2>(fetch, dst, bar, static_cast<int>(og.mn_major), static_cast<int>(p.ks),
                                               load_a ? (p.small_m ? kSmallMSlot : (swap_half ? swap_half : kBlockM)) : Cfg::kBRows,
                                               raw, raw_ld, mn0, mn_limit, k0, kk_total);
          } else if (lane == 0 FB_AND_COPIES_ON(p)) {
            if (use3d) {
              // x is always 0: the innermost extent of the 3-D view is exactly one 128-byte row.
              // A 512-wide tile's B stage is two halves, each laid out like a 256-wide tile's B stage
              // (this CTA's 128 columns of tile columns [256 h, 256 h + 256)), fetched by one copy each.
              const int halves = (load_a || p.wide_merged) ? 1 : Cfg::kHalves;
              for (int h = 0; h < halves; ++h) {
                const int mn = mn0 + h * Cfg::kMmaN;
                const int y = og.mn_major ? k0 : mn;
                const int z = og.mn_major ? mn / static_cast<int>(og.span) : k0 / static_cast<int>(og.span);
                uint8_t* d = dst + h * p.ks * Cfg::kHalfBBytes;
                if constexpr (PAIR) tma_load_3d_pair(d, map, bar, 0, y, z);
                else tma_load_3d(d, map, &full_bar[stage], 0, y, z);
              }
            } else if (og.mn_major) {
              // one box per 128-byte chunk of MN, each holding every k row of the stage
              for (uint32_t bx = 0; bx < og.boxes; ++bx) {
                uint8_t* d = dst + bx * og.box_bytes;
                const int x = mn0 + static_cast<int>(bx * og.box_mn_step);
                if constexpr (PAIR) tma_load_2d_pair(d, map, bar, x, k0);
                else tma_load_2d(d, map, &full_bar[stage], x, k0);
              }
            } else {
              // one box per k-slab
              for (uint32_t sl = 0; sl < p.ks; ++sl) {
                uint8_t* d = dst + sl * slab_bytes;
                const int x = k0 + static_cast<int>(sl * og.span);
                if constexpr (PAIR) tma_load_2d_pair(d, map, bar, x, mn0);
                else tma_load_2d(d, map, &full_bar[stage], x, mn0);
              }
            }
          }
          if (p.prof) prof_issue += clock64() - c1;
          if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
      }
      if (p.prof && blockIdx.x == 0 && lane == 0) {
        if (load_a) { p.prof[0] = prof_wait; p.prof[1] = prof_issue; }
        else p.prof[10] = prof_wait + prof_issue;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    // The tensor pipe queues next to nothing: issuing an MMA blocks until the pipe takes it, and
    // whatever the issuing thread does between two issues that lasts longer than one MMA leaves the
    // pipe idle.  So this loop is software-pipelined: the bookkeeping of a stage (releasing the
    // stage, probing the next stage's barrier, building its descriptors) is slotted
    // *between* the MMAs of the current stage, and the last MMA of one stage is followed
    // directly by the first MMA of the next.
    if (lane == 0 && cta_rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      int g = 0;
      bool ok = true;
      constexpr int kH = Cfg::kHalves;
      constexpr int kMaxMma = 8 * kH;  // 4 k-steps per k-slab, at most 2 slabs per stage, kH column halves
      const int n_mma = 4 * static_cast<int>(p.ks) * kH;
      uint32_t off_a[kMaxMma], off_b[kMaxMma];  // descriptor start-address offsets (16-byte units) of each MMA of a stage
#pragma unroll
      for (int j = 0; j < kMaxMma; ++j) {
        // j = (slab, k-step, half): both halves of a k-step follow each other and share the A operand
        const int half = j % kH, step = (j / kH) & 3, slab = j / (4 * kH);
        off_a[j] = (slab * p.a.slab_adv_bytes + step * p.a.k_adv_bytes) >> 4;
        // the second half of a 512-wide tile: a block of its own behind the first half's slabs, or (merged copy of a
        // K-major operand) the next 128 rows of every slab
        const uint32_t half_off = (p.wide_merged && !p.b.mn_major) ? Cfg::kHalfBBytes : p.ks * Cfg::kHalfBBytes;
        off_b[j] = (half * half_off + slab * p.b.slab_adv_bytes + step * p.b.k_adv_bytes) >> 4;
      }
      const uint64_t a_desc0 = make_smem_desc(smem_u32(smem_a), p.a.lbo, p.a.sbo, p.a.layout);
      const uint64_t b_desc0 = make_smem_desc(smem_u32(smem_b), p.b.lbo, p.b.sbo, p.b.layout);
      const uint32_t a_stage_units = (p.ks * a_slot_bytes) >> 4, b_stage_units = (p.ks * Cfg::kBBytes) >> 4;
      long long prof_wfull = 0, prof_wtmem = 0, prof_mma_issue = 0;
      const long long cstart = p.prof ? clock64() : 0;
      unsigned long long gstart = 0;
      if (p.prof) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gstart));
      bool data_ready = false;   // the current stage's barrier was already seen complete (and fenced)
      uint64_t a_desc = 0, b_desc = 0;  // descriptors of the current stage
      for (int idx = 0; ok; ++idx) {
        WorkItem item;
        int t, role = -1, sharers = 1;
        if (grouped) {
          if (!grouped_tile(p, worker, num_workers, num_tiles, idx, t, role, sharers)) break;
        } else {
          if (!dense_work_item(p, worker, num_workers, dense_stages, idx, item)) break;
          t = item.tile;
        }
        // A transposed partial block (GroupRec::swap_rows): the MMA's A operand is the B stage, its B operand the
        // A stage (`swap_half` rows per CTA, so its slabs lie closer together), and N is the block's row count.
        int swap_half = 0;
        int slab_rows = 0;  // rows between the k-slabs of the A stage (the box height of its copies)
        uint32_t idesc = p.idesc;
        if (grouped) {
          while (g + 1 < p.num_groups && t >= __ldg(p.group_starts + g + 1)) ++g;
          const GroupRec& gr = p.groups[g];
          const int stages_g = (gr.k + static_cast<int>(p.block_k) - 1) >> (31 - __clz(static_cast<int>(p.block_k)));
          if (PAIR && p.small_m) {
            const int tm = (t - gr.tile_start) / gr.tiles_n;
            swap_half = ((min(kSmallMRows, gr.m - tm * kSmallMRows) + 15) >> 4) << 3;
            slab_rows = kSmallMSlot;
            idesc = p.idesc_swapped | (static_cast<uint32_t>(swap_half >> 2) << 17);
          } else if (PAIR && p.swap_partial && gr.swap_rows > 0 && (t - gr.tile_start) / gr.tiles_n == gr.m / Cfg::kTileM) {
            swap_half = gr.swap_rows >> 1;
            slab_rows = swap_half;
            idesc = p.idesc_swapped | (static_cast<uint32_t>(gr.swap_rows >> 3) << 17);
          }
          if (!grouped_range(p, stages_g, role, sharers, item)) break;
        }
        const int k_blocks = item.se - item.sb;  // stages of this work item
        // PAIR: the peer's epilogue warps arrive remotely -> cluster-scope acquire
        if (!mbar_test_wait(&tmem_empty_bar[acc], acc_phase ^ 1u) || PAIR) {
          const long long ct0 = p.prof ? clock64() : 0;
          if (!mbar_wait<PAIR>(&tmem_empty_bar[acc], acc_phase ^ 1u, wctl, DEV_TIMEOUT_MMA_TMEM_EMPTY)) { ok = false; break; }
          if (p.prof) prof_wtmem += clock64() - ct0;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BLOCK_N);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!data_ready) {
            const long long c0 = p.prof ? clock64() : 0;
            if (!mbar_wait(&full_bar[stage], phase, wctl, DEV_TIMEOUT_MMA_FULL)) { ok = false; break; }
            if (p.prof) prof_wfull += clock64() - c0;
            if (p.prof && blockIdx.x == 0 && idx == 0 && kb == 0) p.prof[12] = clock64();  // timeline: first operands
            tc_fence_after();
            a_desc = a_desc0 + static_cast<uint32_t>(stage) * a_stage_units;
            b_desc = b_desc0 + static_cast<uint32_t>(stage) * b_stage_units;
          }
          int next_stage = stage + 1;
          uint32_t next_phase = phase;
          if (next_stage == p.stages) { next_stage = 0; next_phase ^= 1u; }
          uint64_t a_next = 0, b_next = 0;
          const long long ci0 = p.prof ? clock64() : 0;
#pragma unroll
          for (int j = 0; j < kMaxMma; ++j) {
            if (j < n_mma) {
              if (FB_MMA_ON(p)) {
                const uint32_t accum = (kb | (j / kH)) != 0 ? 1u : 0u;  // first k-step of the tile overwrites
                const uint32_t d_half = d_tmem + static_cast<uint32_t>((j % kH) * Cfg::kMmaN);
                if constexpr (PAIR) {
                  uint64_t da = a_desc + off_a[j], db = b_desc + off_b[j];
                  if (kH == 1 && swap_half) {
                    // slab j / 4 of the A stage starts swap_half rows of 128 bytes after the previous one
                    da = b_desc + off_b[j];
                    db = a_desc + static_cast<uint32_t>((j >> 2) * slab_rows * (kSwizzleBytes >> 4)) + ((p.a.k_adv_bytes >> 4) * (j & 3));
                  }
                  umma_pair<kTf32>(d_half, da, db, idesc, accum);
                } else {
                  umma<kTf32>(d_half, a_desc + off_a[j], b_desc + off_b[j], idesc, accum);
                }
              }
              if (j == n_mma - 2) {
                // Slot before the last MMA: everything the next stage needs, so that its first MMA
                // can follow this stage's last one back to back.
                data_ready = mbar_test_wait(&full_bar[next_stage], next_phase);
                if (data_ready) tc_fence_after();
                a_next = a_desc0 + static_cast<uint32_t>(next_stage) * a_stage_units;
                b_next = b_desc0 + static_cast<uint32_t>(next_stage) * b_stage_units;
              }
              if (j == n_mma - 1) {
                // Release the stage (in both CTAs of a pair) as soon as its last MMA is queued.  With
                // only three stages in the ring the refill latency is on the critical path: releasing
                // even one MMA later measurably starves the next stages.
                if constexpr (PAIR) umma_commit_pair(&empty_bar[stage], 3);
                else umma_commit(&empty_bar[stage]);
              }
            }
          }
          if (p.prof) prof_mma_issue += clock64() - ci0;
          stage = next_stage;
          phase = next_phase;
          a_desc = a_next;
          b_desc = b_next;
        }
        if (!ok) break;
        // Tile done: publish the accumulator to the epilogue (of both CTAs of a pair).
        if constexpr (PAIR) umma_commit_pair(&tmem_full_bar[acc], 3);
        else umma_commit(&tmem_full_bar[acc]);
        if (++acc == Cfg::kAccBufs) { acc = 0; acc_phase ^= 1u; }
      }
      if (p.prof && blockIdx.x == 0) {
        p.prof[2] = prof_wfull; p.prof[5] = prof_wtmem;
        p.prof[9] = prof_mma_issue;
        p.prof[6] = clock64() - cstart;
        unsigned long long gend;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gend));
        p.prof[11] = static_cast<long long>(gend - gstart);  // the same interval in nanoseconds
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
    long long prof_ewait = 0, prof_ebody = 0;
    uint32_t epi_seq = 0;  // steps this warp has passed through its staging blocks (TMA-store epilogue)
    if (!grouped) grid_dependency_wait();
    if (!PAIR && p.cluster_push && threadIdx.x == kEpiWarp0 * 32) {
      // cluster split-K, push form: the fp32 sums of all CTAs of the cluster for this CTA's columns of the valid
      // rows arrive in this CTA's receiving area; the arrival that lets the phase end comes with the byte count
      int tm, tn;
      swizzled_tile(static_cast<int>(blockIdx.x) / p.cluster_k, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
      mbar_arrive_expect_tx(recv_bar, static_cast<uint32_t>(min(kBlockM, p.prob.m - tm * kBlockM)) * BLOCK_N * 4u);
    }
    for (int idx = 0; ok; ++idx) {
      WorkItem item;
      item.kind = ITEM_FULL;
      item.slot = -1;
      int t, role = -1, sharers = p.sk_group;
      if (grouped) {
        if (!grouped_tile(p, worker, num_workers, num_tiles, idx, t, role, sharers)) break;
      } else {
        if (!dense_work_item(p, worker, num_workers, dense_stages, idx, item)) break;
        t = item.tile;
      }
      int tm, tn;
      int row_base = 0;
      Problem pr;
      bool k_is_zero = false;  // a group with k == 0 contributes beta * C only
      int swap_rows = 0;       // > 0: the accumulator holds a row block transposed (lanes = columns of the tile)
      int tile_rows = Cfg::kTileM;
      if (grouped) {
        while (g + 1 < p.num_groups && t >= __ldg(p.group_starts + g + 1)) ++g;
        const GroupRec& gr = p.groups[g];
        const int lt = t - gr.tile_start;
        tm = lt / gr.tiles_n;
        tn = lt - tm * gr.tiles_n;
        pr.m = gr.m; pr.n = gr.n; pr.out = gr.out; pr.ldo = gr.ldo; pr.cin = gr.cin; pr.ldcin = gr.ldcin;
        pr.vec_ok = gr.vec_ok;
        k_is_zero = gr.k == 0;
        row_base = gr.row_base;
        const int stages_g = (gr.k + static_cast<int>(p.block_k) - 1) >> (31 - __clz(static_cast<int>(p.block_k)));
        if (PAIR && p.small_m) {
          swap_rows = ((min(kSmallMRows, gr.m - tm * kSmallMRows) + 15) >> 4) << 4;
          tile_rows = kSmallMRows;
        } else if (PAIR && p.swap_partial && gr.swap_rows > 0 && tm == gr.m / Cfg::kTileM) {
          swap_rows = gr.swap_rows;
        }
        if (!grouped_range(p, stages_g, role, sharers, item)) break;
      } else {
        swizzled_tile(t, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
        pr = p.prob;
      }
      const long long e0 = p.prof ? clock64() : 0;
      // warp-uniform outcome: tcgen05.ld below needs the whole warp
      if (!mbar_wait_warp<64>(&tmem_full_bar[acc], acc_phase, wctl, DEV_TIMEOUT_EPI_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const long long e1 = p.prof ? clock64() : 0;
      prof_ewait += e1 - e0;
      if (p.prof && blockIdx.x == 0 && idx == 0 && threadIdx.x == kEpiWarp0 * 32) p.prof[13] = e1;  // timeline: first accumulator
      const int row = row_base + tm * Cfg::kTileM + static_cast<int>(cta_rank) * kBlockM + lane_group * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) +
                             static_cast<uint32_t>(acc * BLOCK_N);
      // Stream-K: this thread's row inside a partial slot, for an owner the slots (sk_first .. sk_last) that hold
      // the rest of the tile's k range, for a contributor the slot it parks in (its own, or the tile's).
      // Layout of a slot: [16-byte unit of the row][row of the tile], so that the 32 rows of a warp sit side by
      // side and every access of a warp covers 512 consecutive bytes.
      const size_t sk_row = static_cast<size_t>(static_cast<int>(cta_rank) * kBlockM + lane_group * 32 + lane);
      constexpr size_t kSkSlot = static_cast<size_t>(Cfg::kTileM) * BLOCK_N;
      int sk_first = worker + 1, sk_last = worker, sk_park = worker;
      if (item.slot >= 0) { sk_first = sk_park = item.slot; sharers = 2; }
      if (item.kind == ITEM_OWNER) {
        if (!grouped && p.sk_enabled == 2) sharers = item.part;
        sk_last = sk_first + sharers - 2;
        // wait (bounded) until every contributor has parked the rows this warp needs
        uint32_t good = 1;
        if (lane == 0) {
          const long long w0 = clock64();
          for (int v = sk_first; v <= sk_last && good; ++v) {
            const int* flag = p.sk_flags + v * 8 + static_cast<int>(cta_rank) * 4 + lane_group;
            while (true) {
              int f;
              asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(f) : "l"(flag) : "memory");
              if (f == p.sk_epoch) break;
              if (*abort_flag) { good = 0; break; }
              if (clock64() - w0 > FB_WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                atomicCAS(&g_fb_status, 0, DEV_TIMEOUT_STREAMK_PARTIAL);
                good = 0;
                break;
              }
              __nanosleep(64);
            }
          }
        }
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) ok = false;  // still drain TMEM below so that the MMA issuer is not left waiting
      }
      if (item.kind == ITEM_CLUSTER) break;  // the accumulator is complete; the whole CTA finishes the tile below
      if constexpr (PAIR) if (swap_rows && item.kind != ITEM_PARTIAL) {  // (a contributor parks its raw sums further down)
        // Transposed partial block: TMEM lane = column of the tile (this CTA's 128 of its 256), TMEM column = row of
        // the block.  A thread holds 32 consecutive rows of one output column; for each of them the warp's 32 lanes
        // write 32 neighbouring elements of one output row.
        using T = OutT;
        const int col = tn * BLOCK_N + static_cast<int>(cta_rank) * kBlockM + lane_group * 32 + lane;
        const int block_row0 = row_base + tm * tile_rows;
        const int rows_here = min(swap_rows, pr.m - block_row0);
        const int chunks = (rows_here + 31) >> 5;
        T* ocol = reinterpret_cast<T*>(pr.out) + col;
        const T* ccol = reinterpret_cast<const T*>(pr.cin) + col;
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + static_cast<uint32_t>(acc * BLOCK_N);
        for (int c = 0; c < chunks; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_lane + static_cast<uint32_t>(c * 32), r);
          tmem_ld_wait();
          if (item.kind == ITEM_OWNER && ok) {
            // stream-K tail: add the parts of the tile's k range that the next workers parked (raw accumulator
            // words, the same lane / column positions whatever the tile's orientation)
            for (int v = sk_first; v <= sk_last; ++v) {
              const float4* src = reinterpret_cast<const float4*>(p.sk_partials + v * kSkSlot) + sk_row;
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float4 x = __ldcg(src + static_cast<size_t>(c * 8 + q) * Cfg::kTileM);
                r[q * 4 + 0] = __float_as_uint(__uint_as_float(r[q * 4 + 0]) + x.x);
                r[q * 4 + 1] = __float_as_uint(__uint_as_float(r[q * 4 + 1]) + x.y);
                r[q * 4 + 2] = __float_as_uint(__uint_as_float(r[q * 4 + 2]) + x.z);
                r[q * 4 + 3] = __float_as_uint(__uint_as_float(r[q * 4 + 3]) + x.w);
              }
            }
          }
          if (c == chunks - 1) {
            // every row of this accumulator that exists is in registers: hand TMEM back to the MMA issuer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty_bar[acc]), 0));
          }
          if (FB_STORES_ON(p) && ok && col < pr.n) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int lr = c * 32 + j;
              if (lr < rows_here) {
                const size_t row = static_cast<size_t>(block_row0 + lr);
                float v = k_is_zero ? 0.f : p.alpha * __uint_as_float(r[j]);
                if (p.beta != 0.f) v += p.beta * to_f32(ccol[row * pr.ldcin]);
                ocol[row * pr.ldo] = from_f32<T>(v);
              }
            }
          }
        }
        if (chunks == 0) {  // (cannot happen: a swapped block has at least one row) keep the barrier protocol whole
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty_bar[acc]), 0));
        }
        if (p.prof) prof_ebody += clock64() - e1;
        if (++acc == Cfg::kAccBufs) { acc = 0; acc_phase ^= 1u; }
        continue;
      }
      if (item.kind != ITEM_PARTIAL) {
        // the usual case: this warp's 32 rows leave through its staging block as whole row segments
        uint8_t* stage = epi_staging + (warp - kEpiWarp0) * 2 * kEpiStageBytes;  // (this warp's two blocks)
        const int row0 = row - lane;
        auto hand_back = [&]() {
          // every column of this accumulator is in registers: hand TMEM back to the MMA issuer
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (PAIR) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty_bar[acc]), 0));
            else mbar_arrive(&tmem_empty_bar[acc]);
          }
        };
        auto nothing_to_add = [](int, uint32_t (&)[32]) {};
        // Stream-K: adding the parts of the tile's k range that other workers parked (raw accumulator words) to
        // chunks [c_lo, c_hi) of 32 columns.  Read with plain loads the 64 KB to 128 KB of a part cost an L2 latency
        // per batch of eight.  When this is the worker's last item (no copy will touch the operand ring again: its
        // MMAs are complete) the parts come through the ring instead, one chunk of every part at a time with
        // asynchronous 16-byte copies, each thread fetching exactly the words it will read back: three slots, so
        // that the copies of two chunks are in flight while one is added.
        constexpr int kPartSlots = 3, kMaxParts = 3, kChunksTotal = BLOCK_N / 32;
        constexpr uint32_t kPartUnit = kBlockM * 16;                     // one 16-byte unit of every row
        constexpr uint32_t kPartSlotBytes = kMaxParts * 8 * kPartUnit;   // one chunk of every part
        constexpr bool kRingHoldsParts = Cfg::kStages * Cfg::kStageBytes >= kPartSlots * static_cast<int>(kPartSlotBytes);
        // the slots to add: n_parts consecutive ones from part_first on, leaving out slot part_skip
        int part_first = 0, part_skip = -1, n_parts = 0, c_lo = 0, c_hi = kChunksTotal;
        auto part_slot = [&](int j) { const int v = part_first + j; return v >= part_skip && part_skip >= 0 ? v + 1 : v; };
        bool in_ring = false;
        const uint32_t ring_row = smem_u32(ring) + static_cast<uint32_t>(lane_group * 32 + lane) * 16u;
        auto fetch_chunk = [&](int c) {
          const uint32_t dst0 = ring_row + static_cast<uint32_t>(c % kPartSlots) * kPartSlotBytes;
          for (int j = 0; j < n_parts; ++j) {
            const float4* src = reinterpret_cast<const float4*>(p.sk_partials + part_slot(j) * kSkSlot) + sk_row +
                                static_cast<size_t>(c * 8) * Cfg::kTileM;
#pragma unroll
            for (int q = 0; q < 8; ++q)
              asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst0 + static_cast<uint32_t>(j * 8 + q) * kPartUnit),
                           "l"(src + static_cast<size_t>(q) * Cfg::kTileM) : "memory");
          }
          asm volatile("cp.async.commit_group;" ::: "memory");
        };
        auto start_parts = [&]() {  // after part_slot, n_parts, c_lo, c_hi are set (and the parts are known to be parked)
          if constexpr (kRingHoldsParts) {
            WorkItem nxt;
            int t2, role2, sh2;
            const bool last_item = grouped ? !grouped_tile(p, worker, num_workers, num_tiles, idx + 1, t2, role2, sh2)
                                           : !dense_work_item(p, worker, num_workers, dense_stages, idx + 1, nxt);
            if (last_item && !p.small_m && n_parts <= kMaxParts && c_hi > c_lo) {
              fetch_chunk(c_lo);
              if (c_lo + 1 < c_hi) fetch_chunk(c_lo + 1);
              in_ring = true;
            }
          }
        };
        auto add_parked = [&](int c, uint32_t (&r)[32]) {
          if (in_ring) {
            // chunk c has landed (the copies of chunk c + 1 may still be in flight)
            if (c + 1 < c_hi) asm volatile("cp.async.wait_group 1;" ::: "memory");
            else asm volatile("cp.async.wait_group 0;" ::: "memory");
            const uint32_t src0 = ring_row + static_cast<uint32_t>(c % kPartSlots) * kPartSlotBytes;
            for (int j = 0; j < n_parts; ++j) {
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const uint4 x = ld_shared_v4(src0 + static_cast<uint32_t>(j * 8 + q) * kPartUnit);
                r[q * 4 + 0] = __float_as_uint(__uint_as_float(r[q * 4 + 0]) + __uint_as_float(x.x));
                r[q * 4 + 1] = __float_as_uint(__uint_as_float(r[q * 4 + 1]) + __uint_as_float(x.y));
                r[q * 4 + 2] = __float_as_uint(__uint_as_float(r[q * 4 + 2]) + __uint_as_float(x.z));
                r[q * 4 + 3] = __float_as_uint(__uint_as_float(r[q * 4 + 3]) + __uint_as_float(x.w));
              }
            }
            if (c + 2 < c_hi) fetch_chunk(c + 2);  // (into the slot chunk c - 1 was read from)
            return;
          }
          for (int j = 0; j < n_parts; ++j) {
            const float4* src = reinterpret_cast<const float4*>(p.sk_partials + part_slot(j) * kSkSlot) + sk_row;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 x = __ldcg(src + static_cast<size_t>(c * 8 + q) * Cfg::kTileM);
              r[q * 4 + 0] = __float_as_uint(__uint_as_float(r[q * 4 + 0]) + x.x);
              r[q * 4 + 1] = __float_as_uint(__uint_as_float(r[q * 4 + 1]) + x.y);
              r[q * 4 + 2] = __float_as_uint(__uint_as_float(r[q * 4 + 2]) + x.z);
              r[q * 4 + 3] = __float_as_uint(__uint_as_float(r[q * 4 + 3]) + x.w);
            }
          }
        };
        if (item.kind == ITEM_SPLIT) {
          Problem part = pr;
          part.out = p.splitk_out + static_cast<size_t>(item.part) * pr.m * pr.n;
          part.ldo = pr.n; part.cin = nullptr; part.ldcin = 0;
          part.vec_ok = (pr.n & 3) == 0 ? 1 : 0;
          epilogue_tile_staged<float, BLOCK_N>(t_row, stage, part, row0, tn * BLOCK_N, 1.f, 0.f, lane, k_is_zero, hand_back,
                                               nothing_to_add);
        } else if (item.kind == ITEM_SHARED || item.kind == ITEM_OWNER) {
          constexpr int kW = 128 / static_cast<int>(sizeof(OutT)), kLoads = kW / 32, kSteps = BLOCK_N / kW;
          if (item.kind == ITEM_OWNER) {
            // the other workers' parts of the whole tile (their flags were awaited above)
            part_first = sk_first; n_parts = sk_last - sk_first + 1;
          } else {
            // A tile whose k range `sk_group` workers share, all of them finishing a part of its columns: this worker
            // parks its sums of the other workers' columns in its slot, raises its flag, waits for theirs, adds
            // their sums of its own columns to its accumulator and stores those.  Every worker reads 1 / sk_group of
            // what a single owner would, and the k ranges are equal.
            const int g = p.sk_group, mine = item.part;
            const int s_lo = mine * kSteps / g, s_hi = (mine + 1) * kSteps / g;  // the steps (128 bytes of a row) it finishes
            c_lo = s_lo * kLoads; c_hi = s_hi * kLoads;
            float4* park = reinterpret_cast<float4*>(p.sk_partials + worker * kSkSlot) + sk_row;
#pragma unroll 1
            for (int c = 0; c < kChunksTotal; ++c) {
              if (c >= c_lo && c < c_hi) continue;
              uint32_t r[32];
              tmem_ld_32x32(t_row + c * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int q = 0; q < 8; ++q)
                __stcg(park + static_cast<size_t>(c * 8 + q) * Cfg::kTileM,
                       make_float4(__uint_as_float(r[q * 4 + 0]), __uint_as_float(r[q * 4 + 1]), __uint_as_float(r[q * 4 + 2]),
                                   __uint_as_float(r[q * 4 + 3])));
            }
            __threadfence();  // the partial sums are visible GPU-wide before the flag says so
            __syncwarp();
            const int flag_pos = static_cast<int>(cta_rank) * 4 + lane_group;
            uint32_t good = 1;
            if (lane == 0) {
              asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.sk_flags + worker * 8 + flag_pos), "r"(p.sk_epoch) : "memory");
              const long long w0 = clock64();
              for (int v = item.first; v < item.first + g && good; ++v) {
                if (v == worker) continue;
                while (true) {
                  int f;
                  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(f) : "l"(p.sk_flags + v * 8 + flag_pos) : "memory");
                  if (f == p.sk_epoch) break;
                  if (*abort_flag) { good = 0; break; }
                  if (clock64() - w0 > FB_WAIT_LIMIT_CYCLES) {
                    *abort_flag = 1;
                    atomicCAS(&g_fb_status, 0, DEV_TIMEOUT_STREAMK_PARTIAL);
                    good = 0;
                    break;
                  }
                  __nanosleep(64);
                }
              }
            }
            good = __shfl_sync(0xffffffffu, good, 0);
            if (!good) ok = false;
            part_first = item.first; part_skip = worker; n_parts = g - 1;
          }
          if (c_hi > c_lo && FB_STORES_ON(p) && ok) {
            start_parts();
            if (p.c_tma)
              epilogue_tile_tma<OutT, BLOCK_N>(t_row, stage, &tmC, pr.m, pr.n, row0, tn * BLOCK_N, p.alpha, lane, k_is_zero,
                                               hand_back, add_parked, false, epi_seq, c_lo, c_hi);
            else
              epilogue_tile_staged<OutT, BLOCK_N>(t_row, stage, pr, row0, tn * BLOCK_N, p.alpha, p.beta, lane, k_is_zero,
                                                  hand_back, add_parked, false, false, c_lo / kLoads, c_hi / kLoads);
          } else {
            hand_back();
          }
        } else if (!(FB_STORES_ON(p) && ok)) {
          hand_back();
        } else if (p.c_tma) {
          epilogue_tile_tma<OutT, BLOCK_N>(t_row, stage, &tmC, pr.m, pr.n, row0, tn * BLOCK_N, p.alpha, lane, k_is_zero,
                                           hand_back, nothing_to_add, p.wide_merged != 0, epi_seq);
        } else {
          epilogue_tile_staged<OutT, BLOCK_N>(t_row, stage, pr, row0, tn * BLOCK_N, p.alpha, p.beta, lane, k_is_zero, hand_back,
                                              nothing_to_add, p.wide_merged != 0, p.c_streaming != 0);
        }
        if (p.prof) prof_ebody += clock64() - e1;
        if (++acc == Cfg::kAccBufs) { acc = 0; acc_phase ^= 1u; }
        continue;
      }
      // A contributor of a stream-K tile parks its raw fp32 partial sums in a slot.
      // (a transposed block only has as many accumulator columns as it has rows)
      const int n_chunks = (PAIR && swap_rows) ? (swap_rows + 31) >> 5 : BLOCK_N / 32;
#pragma unroll 1
      for (int c = 0; c < n_chunks; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        if (k_is_zero) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (c == n_chunks - 1) {
          // every column of this accumulator is in registers: hand TMEM back to the MMA issuer
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (PAIR) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty_bar[acc]), 0));
            else mbar_arrive(&tmem_empty_bar[acc]);
          }
        }
        float4* dst = reinterpret_cast<float4*>(p.sk_partials + sk_park * kSkSlot) + sk_row;
#pragma unroll
        for (int q = 0; q < 8; ++q)
          __stcg(dst + static_cast<size_t>(c * 8 + q) * Cfg::kTileM,
                 make_float4(__uint_as_float(r[q * 4 + 0]), __uint_as_float(r[q * 4 + 1]), __uint_as_float(r[q * 4 + 2]),
                             __uint_as_float(r[q * 4 + 3])));
      }
      __threadfence();  // the partial sums are visible GPU-wide before the flag says so
      __syncwarp();
      if (lane == 0)
        asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p.sk_flags + sk_park * 8 + static_cast<int>(cta_rank) * 4 + lane_group),
                     "r"(p.sk_epoch) : "memory");
      if (p.prof) prof_ebody += clock64() - e1;
      if (++acc == Cfg::kAccBufs) { acc = 0; acc_phase ^= 1u; }
    }
    if (p.c_tma && lane == 0) bulk_wait_group<0>();  // this warp's stores have left its staging blocks and landed
    if (p.prof && blockIdx.x == 0 && threadIdx.x == kEpiWarp0 * 32) {
      p.prof[7] = prof_ewait; p.prof[8] = prof_ebody;
      p.prof[14] = clock64();  // timeline: last store issued
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
  if constexpr (PAIR) {
    // Neither CTA may retire while its partner can still signal its barriers or read its operands.
    cluster_arrive_release();
    cluster_wait_acquire();
  } else {
    if (p.cluster_k > 1)
      cluster_finish_tile<OutT, BLOCK_N>(p, smem_u32(ring),
                                         smem_u32(epi_staging) + Cfg::kEpiBytes - static_cast<uint32_t>(p.cluster_rows) * BLOCK_N * 4u,
                                         recv_bar, wctl, tmem_base, static_cast<int>(blockIdx.x) / p.cluster_k, !*abort_flag);
  }
  if (warp == 2) {
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
    else tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (p.prof && blockIdx.x == 0 && threadIdx.x == 0) p.prof[15] = clock64();  // timeline: exit
}

// Second kernel of a split-K call: out = alpha * (part 0 + part 1 + ...) + beta * C, parts added in index order.
template <class OutT>
__global__ void splitk_finish_kernel(const float* __restrict__ parts, int splitk, int m, int n, float alpha, float beta,
                                     OutT* out, long long ldo) {
  grid_dependency_wait();  // launched as a programmatic dependent of the kernel that writes the parts
  const long long total = static_cast<long long>(m) * n;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splitk; ++s) acc += __ldcs(parts + static_cast<long long>(s) * total + i);
    const long long r = i / n, c = i - r * n;
    OutT* dst = out + r * ldo + c;
    float v = alpha * acc;
    if (beta != 0.f) v += beta * to_f32(*dst);
    *dst = from_f32<OutT>(v);
  }
}

}  // namespace fb
