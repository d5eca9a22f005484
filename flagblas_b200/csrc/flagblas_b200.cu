// C ABI of the B200 GEMM back end (see include/flagblas_b200.h) and the host
// logic behind it: argument checks, operand geometry, tensor-map encoding,
// tile-shape choice and kernel launches.  Single translation unit.
#include "../../include/flagblas_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <mutex>
#include <cstdio>
#include <type_traits>

namespace fb {
__device__ int g_fb_status = 0;
}

#include "fb_gemm_tc.cuh"
#include "fb_group_setup.cuh"
#include "fb_sgemm_simt.cuh"
#include "fb_gemv.cuh"
#include "fb_xgemm_simt.cuh"
#include "fb_dgemm_mma.cuh"

namespace fb {

static thread_local int t_last_cuda_error = 0;
// Device buffer of 16 cycle counters, set by fb_debug_set_profile_buffer (profiling only).
static long long* g_prof_buffer = nullptr;

#define FB_CUDA_OK(expr)                                   \
  do {                                                     \
    cudaError_t e__ = (expr);                              \
    if (e__ != cudaSuccess) {                              \
      t_last_cuda_error = static_cast<int>(e__);           \
      return FB_ERR_LAUNCH;                                \
    }                                                      \
  } while (0)

// ---------------------------------------------------------------- device info
struct DeviceInfo {
  int sm_count = 0;
  int cc_major = 0;
  bool ready = false;
};
static DeviceInfo g_dev[64];
static std::mutex g_dev_mu;

static const DeviceInfo* device_info() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_dev_mu);
  DeviceInfo& d = g_dev[dev];
  if (!d.ready) {
    if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return nullptr;
    if (cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return nullptr;
    d.ready = true;
  }
  return &d;
}

// ------------------------------------------------------- tensor-map encoding
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    if (q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Integer environment switches (profiling sweeps and opt-in variants), `dflt` when unset or empty.  The
// environment is read once per process and switch: every call site keeps what it read and looks again only
// after fb_reload_env() (tests and sweeps that flip a switch in a running process call it).
static std::atomic<unsigned> g_env_generation{1};
struct EnvSlot {
  std::atomic<unsigned> generation{0};
  std::atomic<int> is_set{0};
  std::atomic<int> value{0};
};
static int env_lookup(EnvSlot& slot, const char* name, int dflt) {
  const unsigned now = g_env_generation.load(std::memory_order_acquire);
  if (slot.generation.load(std::memory_order_acquire) != now) {
    const char* v = getenv(name);
    const bool set = v && *v;
    slot.value.store(set ? atoi(v) : 0, std::memory_order_relaxed);
    slot.is_set.store(set ? 1 : 0, std::memory_order_relaxed);
    slot.generation.store(now, std::memory_order_release);
  }
  return slot.is_set.load(std::memory_order_relaxed) ? slot.value.load(std::memory_order_relaxed) : dflt;
}
#define env_int(name, dflt) ([&]() -> int { static EnvSlot slot_; return env_lookup(slot_, name, (dflt)); }())

// L2 sector promotion of the tensor maps; FLAGBLAS_B200_L2PROMO = 0 (none), 1 (64 B), 2 (128 B), 3 (256 B,
// the default) for profiling sweeps.
static CUtensorMapL2promotion l2_promotion() {
  switch (env_int("FLAGBLAS_B200_L2PROMO", 3)) {
    case 0: return CU_TENSOR_MAP_L2_PROMOTION_NONE;
    case 1: return CU_TENSOR_MAP_L2_PROMOTION_L2_64B;
    case 2: return CU_TENSOR_MAP_L2_PROMOTION_L2_128B;
    default: return CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
  }
}

static int elem_size(int dtype) { return (dtype == FB_F16 || dtype == FB_BF16) ? 2 : 4; }

static CUtensorMapDataType map_dtype(int dtype) {
  switch (dtype) {
    case FB_F16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    case FB_BF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  }
}

// 2-D row-major view: `inner` contiguous elements per row, `outer` rows `pitch_bytes` apart.
// `atom32`: 128-byte swizzle with 32-byte atoms (MN-major operands of 32-bit types).
static int encode_2d(CUtensorMap* map, int dtype, const void* base, uint64_t inner, uint64_t outer,
                     uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer, bool atom32 = false) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return FB_ERR_DRIVER;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, map_dtype(dtype), 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  l2_promotion(),
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    t_last_cuda_error = static_cast<int>(r);
    return FB_ERR_DRIVER;
  }
  return FB_OK;
}

// 3-D view used to fetch several 128-byte-wide slabs with one copy: extents {d0, d1, d2} with d0
// contiguous, byte strides {s1, s2} for d1 and d2.
static int encode_3d(CUtensorMap* map, int dtype, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                     uint64_t s1_bytes, uint64_t s2_bytes, uint32_t b0, uint32_t b1, uint32_t b2, bool atom32) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return FB_ERR_DRIVER;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1_bytes, s2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, map_dtype(dtype), 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  l2_promotion(), CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    t_last_cuda_error = static_cast<int>(r);
    return FB_ERR_DRIVER;
  }
  return FB_OK;
}

// Geometry of one operand's pipeline stage.  `tile_mn` rows/cols of the tile,
// `mn_contig`: the operand's contiguous dimension is M (resp. N), not K.
static OperandGeom make_geom(int esz, int tile_mn, bool mn_contig, int ks, bool use3d) {
  OperandGeom g{};
  const uint32_t span = kSwizzleBytes / esz;  // elements per 128-byte row
  g.span = span;
  g.use3d = use3d ? 1 : 0;
  if (mn_contig) {
    const uint32_t k_rows = span * ks;  // k rows per 128-byte chunk of MN in one stage
    g.mn_major = 1;
    g.boxes = tile_mn / span;
    g.box_bytes = k_rows * kSwizzleBytes;
    g.box_mn_step = span;
    g.lbo = k_rows * kSwizzleBytes;              // next 128-byte chunk of MN
    g.sbo = (esz == 4 ? 4 : 8) * kSwizzleBytes;  // next group of k-rows (4 with 32-byte atoms, else 8)
    g.k_adv_bytes = (32 / esz) * kSwizzleBytes;  // one MMA consumes 32 bytes' worth of K = that many rows
    g.slab_adv_bytes = span * kSwizzleBytes;     // k rows simply continue
    g.layout = esz == 4 ? kLayoutSw128Base32 : kLayoutSw128;
  } else {
    g.mn_major = 0;
    g.boxes = 1;
    g.box_bytes = tile_mn * kSwizzleBytes;
    g.box_mn_step = 0;
    g.lbo = 16;
    g.sbo = 8 * kSwizzleBytes;  // next group of 8 rows
    g.k_adv_bytes = 32;
    g.slab_adv_bytes = tile_mn * kSwizzleBytes;  // slabs are stacked tile after tile
    g.layout = kLayoutSw128;
  }
  return g;
}

static int idesc_fmt(int dtype) { return dtype == FB_F16 ? 0 : (dtype == FB_BF16 ? 1 : 2); }

// ------------------------------------------------------------ small kernels
template <class T>
__global__ void scale_kernel(T* c, long long ldc, int m, int n, float beta) {
  const long long total = static_cast<long long>(m) * n;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / n, col = i - r * n;
    T* p = c + r * ldc + col;
    *p = beta == 0.f ? from_f32<T>(0.f) : from_f32<T>(beta * to_f32(*p));
  }
}

// Both operands of a dense call in one launch: blocks [0, blocks_a) copy A, the rest copy B (either may be empty).
// The GEMM that follows is launched as a programmatic dependent: it may start its prologue right away and waits
// for this grid before its first copy.
struct PackJob {
  const void* src;
  void* dst;
  long long ld_src, ld_dst, rows, cols;
};
template <class T>
__global__ void pack2_kernel(PackJob a, PackJob b, int blocks_a) {
  grid_launch_dependents();
  const bool is_a = static_cast<int>(blockIdx.x) < blocks_a;
  const PackJob& j = is_a ? a : b;
  const long long first = is_a ? blockIdx.x : blockIdx.x - blocks_a;
  const long long nblocks = is_a ? blocks_a : gridDim.x - blocks_a;
  const T* src = static_cast<const T*>(j.src);
  T* dst = static_cast<T*>(j.dst);
  const long long total = j.rows * j.cols;
  for (long long i = first * blockDim.x + threadIdx.x; i < total; i += nblocks * blockDim.x) {
    const long long r = i / j.cols, c = i - r * j.cols;
    dst[r * j.ld_dst + c] = src[r * j.ld_src + c];
  }
}

__global__ void bounded_wait_selftest_kernel(long long limit) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    fence_mbar_init();
    // Same loop shape as mbar_wait, with a caller-chosen limit.
    const long long t0 = clock64();
    bool done = false;
    while (!done) {
      if (mbar_try_wait(&bar, 0)) break;  // never: nothing arrives on this barrier
      if (clock64() - t0 > limit) {
        abort_flag = 1;
        atomicCAS(&g_fb_status, 0, DEV_TIMEOUT_TEST_FLAG);
        done = true;
      }
    }
  }
  __syncthreads();
}

// ------------------------------------------------------------- tile choice
// Pick the tile width that minimises (waves x per-tile time); `workers` = CTAs (or CTA pairs)
// that run concurrently, `tile_m` = rows per tile.
static int choose_block_n(long long m, long long n, int tile_m, int workers, bool allow64) {
  const long long tm = (m + tile_m - 1) / tile_m;
  double best = 1e300;
  int best_bn = 256;
  const int cand[3] = {256, 128, 64};
  // Relative main-loop efficiency of the narrower tiles (measured: per-stage copy and barrier costs do
  // not shrink with the tile, so a 128-wide tile runs at little more than half the rate of a 256-wide one).
  const double eff[3] = {1.0, 0.6, 0.35};
  for (int i = 0; i < (allow64 ? 3 : 2); ++i) {
    const long long tiles = tm * ((n + cand[i] - 1) / cand[i]);
    const long long waves = (tiles + workers - 1) / workers;
    const double cost = static_cast<double>(waves) * cand[i] / eff[i];
    if (cost < best) { best = cost; best_bn = cand[i]; }
  }
  return best_bn;
}


constexpr size_t kStreamKFlagBytes = 8192;  // eight ints per slot (at most 148 slots), padded

// Bytes of stream-K scratch for a dense call: one fp32 partial tile per worker plus the flags.
static size_t streamk_bytes(int sm_count, int block_n) {
  return static_cast<size_t>(sm_count) * kBlockM * block_n * sizeof(float) + kStreamKFlagBytes;
}

// Launch state kept per kernel instantiation and device.
struct KernelState {
  bool attr_set = false;
  int max_clusters = 0;  // PAIR only: CTA pairs that can be co-resident
};

// A last wave of `rem` tiles on `workers` workers that is more than half full leaves workers - rem of them idle for
// a whole tile time.  Those "helpers" can take the tails of the wave's tiles instead: each sweeps the last x k-slabs
// (128-byte chunks of k) of q = ceil(rem / helpers) tiles, one after the other, and parks the sums for the tile's
// owner, which sweeps the first slabs - x.  x balances the two: slabs - x = q * x + head, `head` being the time a
// helper needs to park its last partial tile.  Returns x (even: whole two-slab stages), or 0 where a tail would be
// too short to pay for the owner's fix-up (FLAGBLAS_B200_SK_TAIL_MIN, in slabs) or the plan is switched off
// (FLAGBLAS_B200_STREAMK_TAILS=0).
static long long tail_slabs(long long slabs, long long workers, long long rem);

// Value a stream-K launch stores in its flags: another one for every launch of the process, and neither 0 nor a
// small number that uninitialised or cleared scratch is likely to hold, so that the flags never need zeroing.
static int next_streamk_epoch() {
  static std::atomic<uint32_t> counter{0};
  return static_cast<int>(0x5EED0000u + (counter.fetch_add(1, std::memory_order_relaxed) & 0x0FFFFFFFu) * 2u + 1u);
}

// Stream-K launches have CTAs that wait for other CTAs of the same launch, so two of them must not share the SMs:
// each could hold a part and wait for CTAs that cannot start.  On one stream they run one after the other anyway;
// when a stream-K launch follows one made on ANOTHER stream, it is made to wait for everything submitted to that
// stream so far (an event recorded there now).  Nothing is added on the common path, where the stream is the same.
// Streams being captured into a graph are left alone (the capture fixes the order itself).
static void streamk_gate(cudaStream_t stream) {
  struct Gate { cudaStream_t last = nullptr; bool any = false; cudaEvent_t ev = nullptr; };
  static Gate gates[64];
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return;
  std::lock_guard<std::mutex> lk(mu);
  Gate& g = gates[dev];
  if (g.any && g.last != stream) {
    cudaStreamCaptureStatus a = cudaStreamCaptureStatusNone, b = cudaStreamCaptureStatusNone;
    const bool ok = cudaStreamIsCapturing(stream, &a) == cudaSuccess && cudaStreamIsCapturing(g.last, &b) == cudaSuccess;
    if (ok && a == cudaStreamCaptureStatusNone && b == cudaStreamCaptureStatusNone) {
      if (!g.ev && cudaEventCreateWithFlags(&g.ev, cudaEventDisableTiming) != cudaSuccess) g.ev = nullptr;
      if (g.ev && cudaEventRecord(g.ev, g.last) == cudaSuccess) cudaStreamWaitEvent(stream, g.ev, 0);
    }
    cudaGetLastError();  // (a stream that no longer exists is not an error of this call)
  }
  g.last = stream;
  g.any = true;
}

static long long tail_slabs(long long slabs, long long workers, long long rem) {
  if (rem <= 0 || 2 * rem <= workers || rem >= workers) return 0;
  if (env_int("FLAGBLAS_B200_STREAMK_TAILS", 1) == 0) return 0;
  const long long helpers = workers - rem;
  const long long q = (rem + helpers - 1) / helpers;
  // (measured, fp16 8192 x 1024 x 8192 in a loop: 113.7 / 112.7 / 111.5 us at head = 4 / 12 / 20, whole tiles 114.0)
  const long long head = env_int("FLAGBLAS_B200_SK_TAIL_HEAD", 20);
  long long x = (slabs - head) / (q + 1);
  x &= ~1LL;
  return x >= env_int("FLAGBLAS_B200_SK_TAIL_MIN", 24) ? x : 0;
}

template <int KIND, int BLOCK_N, bool PAIR>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const TcGemmParams& p, long long tiles,
                     int sm_count, cudaStream_t stream) {
  using Cfg = TcCfg<KIND, BLOCK_N, PAIR>;
  auto kern = gemm_tc_kernel<KIND, BLOCK_N, PAIR>;
  static KernelState state[64];
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  KernelState& st = state[dev];
  {
    std::lock_guard<std::mutex> lk(mu);
    if (!st.attr_set) {
      FB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
      if (PAIR) {
        cudaLaunchConfig_t q{};
        q.gridDim = dim3(static_cast<unsigned>(sm_count / 2 * 2));
        q.blockDim = dim3(kNumThreads);
        q.dynamicSmemBytes = Cfg::kSmemBytes;
        cudaLaunchAttribute qa[1];
        qa[0].id = cudaLaunchAttributeClusterDimension;
        qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
        q.attrs = qa; q.numAttrs = 1;
        int n = 0;
        FB_CUDA_OK(cudaOccupancyMaxActiveClusters(&n, kern, &q));
        st.max_clusters = n > 0 ? n : 1;
      }
      st.attr_set = true;
    }
  }
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attrs[2];
  const long long workers = PAIR ? st.max_clusters : sm_count;
  const long long use = tiles < workers ? tiles : workers;
  cfg.gridDim = dim3(static_cast<unsigned>(PAIR ? 2 * use : use));
  cfg.blockDim = dim3(kNumThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  unsigned n_attrs = 0;
  if (!PAIR && p.cluster_k > 1) {
    // cluster split-K: `tiles` counts one CTA per (tile, k part); the CTAs of a tile form one cluster
    cfg.gridDim = dim3(static_cast<unsigned>(tiles));
    attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
    attrs[n_attrs].val.clusterDim.x = static_cast<unsigned>(p.cluster_k);
    attrs[n_attrs].val.clusterDim.y = 1; attrs[n_attrs].val.clusterDim.z = 1;
    ++n_attrs;
  }
  if (PAIR) {
    attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
    attrs[n_attrs].val.clusterDim.x = 2; attrs[n_attrs].val.clusterDim.y = 1; attrs[n_attrs].val.clusterDim.z = 1;
    ++n_attrs;
  }
  if (env_int("FLAGBLAS_B200_PDL", 1) != 0) {
    // grouped: overlap this kernel's launch and prologue with the table builder queued just before it
    attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
    ++n_attrs;
  }
  if (n_attrs) { cfg.attrs = attrs; cfg.numAttrs = n_attrs; }
  TcGemmParams pp = p;
  pp.sk_enabled = 0;
  if (p.num_groups == 0 && p.sk_partials && env_int("FLAGBLAS_B200_STREAMK", 1) != 0) {
    // Stream-K tail (FLAGBLAS_B200_STREAMK=0 switches it off): for a last wave that is at most half full.
    const long long stages = (p.k + static_cast<long long>(p.block_k) - 1) / p.block_k;
    const long long dp = tiles / workers, rem = tiles - dp * workers;
    long long group = rem > 0 ? workers / rem : 0;  // workers per tail tile
    if (group > 4) group = 4;
    // Two sharers: an owner and a contributor of `share` stages; the owner's part is longer by `head`, about the time
    // the contributor needs to park a 128 x 256 fp32 tile per CTA (in 64-deep stages; measured flat between 8 and 16:
    // 4096 x 4096 x 8192 1358 / 1361 / 1355 / 1350 TFLOP/s at 4 / 12 / 20 / 28).  Three or four: equal parts of the
    // k range, every sharer finishing a part of the tile's columns (dense_work_item).
    const long long head = (env_int("FLAGBLAS_B200_SK_HEAD", 12) + p.ks - 1) / p.ks;
    const long long share = group == 2 ? (stages - head) / 2 : (group > 2 ? stages / group : 0);
    if (group >= 2 && share >= 2 && dp < 9) {
      pp.sk_enabled = 1;
      pp.sk_dp = static_cast<int>(dp);
      pp.sk_rem = static_cast<int>(rem);
      pp.sk_group = static_cast<int>(group);
      pp.sk_share = static_cast<int>(share);
    } else if (tail_slabs(stages * p.ks, workers, rem) / p.ks > 0 && BLOCK_N <= 256 &&
               env_int("FLAGBLAS_B200_STREAMK_FULL", 0) == 0) {
      // Last wave more than half full (one rank's share of an 8192^3 GEMM sharded over eight GPUs: 128 tiles on 74 CTA
      // pairs): whole tiles would leave (workers - rem) workers idle for a whole tile time.  The idle workers
      // take the last stages of the wave's tiles instead (dense_work_item, sk_enabled == 3).
      pp.sk_enabled = 3;
      pp.sk_dp = static_cast<int>(dp);
      pp.sk_rem = static_cast<int>(rem);
      pp.sk_share = static_cast<int>(tail_slabs(stages * p.ks, workers, rem) / p.ks);
    } else if (rem > 0 && 2 * rem > workers && dp >= 1 && dp <= 2 && stages >= 16 && BLOCK_N <= 256 &&
               env_int("FLAGBLAS_B200_STREAMK_FULL", 0) != 0) {
      // Two or three waves of which the last is more than half full (one rank's share of a GEMM sharded over eight
      // GPUs: 128 tiles on 74 CTA pairs): whole tiles leave (workers - rem) workers idle for a whole tile time.
      // Opt-in (FLAGBLAS_B200_STREAMK_FULL=1): after the whole waves the k stages of the last wave's tiles are dealt
      // evenly over all workers; =2 deals out the stages of every tile.  Measured slower than whole tiles, so off:
      // fp16 8192 x 1024 x 8192 118.2 (=1) / 134.8 (=2) against 113.6 us, 5120 x 2560 x 4096 91.1 / 95.1 against 82.6 us
      // -- every worker parks and re-reads a 256 KB partial tile, the owners' epilogues all fall at the end of the
      // kernel, and with =2 the workers no longer sweep k in step, so shared operand panels leave L2 between uses.
      pp.sk_enabled = 2;
      pp.sk_dp = env_int("FLAGBLAS_B200_STREAMK_FULL", 0) == 2 ? 0 : static_cast<int>(dp);
    }
  }
  if (pp.sk_enabled) cfg.gridDim = dim3(static_cast<unsigned>(PAIR ? 2 * workers : workers));  // every worker takes part
  if (pp.sk_enabled || pp.sk_grouped) pp.sk_epoch = next_streamk_epoch();
  if (pp.sk_enabled) streamk_gate(stream);  // (grouped calls pass the gate before their table builder)
  if (env_int("FLAGBLAS_B200_PLAN_DEBUG", 0) != 0 && p.num_groups == 0)
    fprintf(stderr, "fb_gemm launch: workers=%lld grid=%u stream-k mode=%d whole waves=%d tail tiles=%d sharers=%d share=%d stages, c_tma=%d\n",
            workers, cfg.gridDim.x, pp.sk_enabled, pp.sk_dp, pp.sk_rem, pp.sk_group, pp.sk_share, pp.c_tma);
#ifdef FB_PROFILING_SWITCHES
  pp.debug = env_int("FLAGBLAS_B200_DEBUG_SKIP", 0);
#else
  pp.debug = 0;
#endif
  int max_stages = Cfg::kStages / static_cast<int>(p.ks);  // a stage holds ks slabs
  if (p.a_rows) {
    // short A slots: more stages fit the ring
    max_stages = Cfg::kStages * Cfg::kStageBytes / (static_cast<int>(p.ks) * (p.a_rows * kSwizzleBytes + Cfg::kBBytes));
    if (max_stages > kMaxRing) max_stages = kMaxRing;
  }
  if (p.small_m) {
    // small-M plan: 32-row A slots, and the ring runs on into the (unused) epilogue staging blocks
    max_stages = (Cfg::kStages * Cfg::kStageBytes + Cfg::kEpiBytes) /
                 (static_cast<int>(p.ks) * (kSmallMSlot * kSwizzleBytes + Cfg::kBBytes));
    if (max_stages > kMaxRing) max_stages = kMaxRing;
  }
  if (pp.cluster_k > 1 && pp.cluster_push) {
    // The receiving area of the push form takes the epilogue staging blocks, which a cluster split-K call does not
    // use, and, where it is larger, the end of the operand ring; with fewer than two stages left the CTAs read
    // each other's parked sums instead.
    pp.cluster_rows = p.prob.m >= kBlockM ? kBlockM : (p.prob.m + 31) / 32 * 32;
    const int recv = BLOCK_N * pp.cluster_rows * 4;
    if (recv > Cfg::kEpiBytes) {
      const int left = (Cfg::kStages * Cfg::kStageBytes - (recv - Cfg::kEpiBytes)) / (static_cast<int>(p.ks) * Cfg::kStageBytes);
      // (measured: 128 x 4096 x 14336 with two stages of three left, 31.4 -> 37.5 us: the shorter ring costs the k
      // loop more than the push saves; FLAGBLAS_B200_CLUSTER_PUSH=2 takes the ring's end regardless)
      if (left >= 2 && pp.cluster_push == 2) max_stages = left < max_stages ? left : max_stages;
      else pp.cluster_push = 0;
    }
  }
  pp.stages = env_int("FLAGBLAS_B200_STAGES", max_stages);
  if (pp.stages < 1 || pp.stages > max_stages) pp.stages = max_stages;
  pp.prof = g_prof_buffer;
  FB_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, ma, mb, mc, pp));
  return FB_OK;
}

// tiles < 0: grouped mode, the tile count lives on the device -> one worker per SM.
static int dispatch_tc(int dtype, int block_n, bool pair, const CUtensorMap& ma, const CUtensorMap& mb,
                       const CUtensorMap& mc, const TcGemmParams& p, long long tiles, int sm_count, cudaStream_t stream) {
  if (tiles < 0) tiles = 1LL << 40;
#define FB_CASE(KIND)                                                                              \
  if (pair) {                                                                                      \
    if (block_n == 512) return launch_tc<KIND, 512, true>(ma, mb, mc, p, tiles, sm_count, stream); \
    if (block_n == 256) return launch_tc<KIND, 256, true>(ma, mb, mc, p, tiles, sm_count, stream); \
    return launch_tc<KIND, 128, true>(ma, mb, mc, p, tiles, sm_count, stream);                     \
  }                                                                                                \
  switch (block_n) {                                                                               \
    case 256: return launch_tc<KIND, 256, false>(ma, mb, mc, p, tiles, sm_count, stream);          \
    case 128: return launch_tc<KIND, 128, false>(ma, mb, mc, p, tiles, sm_count, stream);          \
    default: return launch_tc<KIND, 64, false>(ma, mb, mc, p, tiles, sm_count, stream);            \
  }
  if (dtype == FB_F16) { FB_CASE(0) }
  if (dtype == FB_BF16) { FB_CASE(1) }
  FB_CASE(2)
#undef FB_CASE
}

static bool aligned16(const void* p, long long ld, int esz) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && ((ld * esz) & 15) == 0;
}
static size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct PackPlan {
  bool pack_a = false, pack_b = false;
  long long a_rows = 0, a_cols = 0, a_ld = 0;
  long long b_rows = 0, b_cols = 0, b_ld = 0;
  size_t a_bytes = 0, b_bytes = 0;
};

static PackPlan plan_pack(int dtype, int transa, int transb, long long m, long long n, long long k, const void* A,
                          long long lda, const void* B, long long ldb) {
  PackPlan pl;
  if (dtype == FB_F32) return pl;
  const int esz = elem_size(dtype);
  const long long per16 = 16 / esz;
  pl.a_rows = transa ? k : m; pl.a_cols = transa ? m : k;
  pl.b_rows = transb ? n : k; pl.b_cols = transb ? k : n;
  pl.pack_a = !aligned16(A, lda, esz);
  pl.pack_b = !aligned16(B, ldb, esz);
  pl.a_ld = (pl.a_cols + per16 - 1) / per16 * per16;
  pl.b_ld = (pl.b_cols + per16 - 1) / per16 * per16;
  pl.a_bytes = pl.pack_a ? round_up(static_cast<size_t>(pl.a_rows) * pl.a_ld * esz, 256) : 0;
  pl.b_bytes = pl.pack_b ? round_up(static_cast<size_t>(pl.b_rows) * pl.b_ld * esz, 256) : 0;
  return pl;
}

template <class T>
static int run_scale(void* C, long long ldc, long long m, long long n, float beta, cudaStream_t stream) {
  if (beta == 1.f || m == 0 || n == 0) return FB_OK;
  const long long total = m * n;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  scale_kernel<T><<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<T*>(C), ldc, static_cast<int>(m),
                                                                static_cast<int>(n), beta);
  FB_CUDA_OK(cudaGetLastError());
  return FB_OK;
}

template <int BM, int BN, bool AK, bool BKM, int PACK>
static int launch_sgemm_pipe(const SimtParams& p, long long tiles, cudaStream_t stream) {
  auto kern = sgemm_pipe_kernel<BM, BN, AK, BKM, PACK>;
  constexpr int kBytes = kPipeStages * (PipeTile<BM, AK>::kFloats + PipeTile<BN, BKM>::kFloats) * 4;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    FB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes));
    attr_set[dev] = true;
  }
  if (p.ksplit == 2 || p.ksplit == 4) {
    // clusters of two or four CTAs per tile; the first CTA's mailboxes for the others' sums sit behind the ring
    constexpr int kMailbox = BM * BN * 4;
    if (kBytes + 3 * kMailbox > kSmemLimit) return FB_ERR_UNSUPPORTED;  // (only 64 x 64 tiles are launched this way)
    static bool attr2_set[64] = {};
    if (dev >= 0 && dev < 64 && !attr2_set[dev]) {
      FB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes + 3 * kMailbox));
      attr2_set[dev] = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(p.ksplit * tiles));
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = kBytes + (p.ksplit - 1) * kMailbox;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(p.ksplit); attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = env_int("FLAGBLAS_B200_PDL", 1) != 0 ? 2 : 1;
    FB_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, p));
    return FB_OK;
  }
  // (a programmatic dependent of its predecessor on the stream, like the tensor-core GEMMs: in a sequence of small
  // calls the launch of one overlaps the tail of the one before)
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles));
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = kBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = env_int("FLAGBLAS_B200_PDL", 1) != 0 ? 1 : 0;
  FB_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, p));
  return FB_OK;
}

// Packed FMAs pair outputs along the dimension whose fragments arrive as float4 (an operand stored with M / N
// contiguous); with both operands K-contiguous there is no such dimension and the FMAs stay scalar.
// FLAGBLAS_B200_SGEMM_FFMA2 = 0 forces scalar FMAs everywhere (profiling comparison).
template <int BM, int BN>
static int dispatch_sgemm_pipe(const SimtParams& p, long long tiles, cudaStream_t stream) {
  const bool ak = !p.a_mn_contig, bk = !p.b_mn_contig;  // K-contiguous storage
  const bool pack = env_int("FLAGBLAS_B200_SGEMM_FFMA2", 1) != 0;
  if (ak) {
    // both K-contiguous (a linear layer's x W^T): with 128 x 128 tiles B's tile is stored pair-interleaved so that the
    // FMAs can be packed over neighbouring columns (4096^3 39.8 -> 43.6 TFLOP/s, 8192^3 40.5 -> 44.4, 2048^3 34.4 ->
    // 36.2; the 64 x 64 tiles of small problems lose with it: 1024^3 26.3 -> 24.7, 512^3 17.2 -> 15.6;
    // FLAGBLAS_B200_SGEMM_NT_PAIRS=0: scalar FMAs on plain K-contiguous tiles)
    if (bk) return (pack && BM >= 128 && env_int("FLAGBLAS_B200_SGEMM_NT_PAIRS", 1) != 0)
                       ? launch_sgemm_pipe<BM, BN, true, true, 3>(p, tiles, stream)
                       : launch_sgemm_pipe<BM, BN, true, true, 0>(p, tiles, stream);
    return pack ? launch_sgemm_pipe<BM, BN, true, false, 1>(p, tiles, stream)
                : launch_sgemm_pipe<BM, BN, true, false, 0>(p, tiles, stream);
  }
  if (bk) return pack ? launch_sgemm_pipe<BM, BN, false, true, 2>(p, tiles, stream)
                      : launch_sgemm_pipe<BM, BN, false, true, 0>(p, tiles, stream);
  return pack ? launch_sgemm_pipe<BM, BN, false, false, 1>(p, tiles, stream)
              : launch_sgemm_pipe<BM, BN, false, false, 0>(p, tiles, stream);
}

static int run_sgemm_simt(int transa, int transb, long long m, long long n, long long k, float alpha, const float* A,
                          long long lda, const float* B, long long ldb, float beta, float* C, long long ldc, int sms,
                          cudaStream_t stream) {
  SimtParams p{};
  p.m = static_cast<int>(m); p.n = static_cast<int>(n); p.k = static_cast<int>(k);
  p.alpha = alpha; p.beta = beta;
  p.A = A; p.lda = lda; p.B = B; p.ldb = ldb; p.C = C; p.ldc = ldc;
  p.a_mn_contig = transa ? 1 : 0;
  p.b_mn_contig = transb ? 0 : 1;
  p.a_vec = aligned16(A, lda, 4); p.b_vec = aligned16(B, ldb, 4); p.c_vec = aligned16(C, ldc, 4);
  const long long big_tiles = ((m + 127) / 128) * ((n + 127) / 128);
  // 128 x 128 tiles once they nearly fill the GPU (measured: 144 tiles, 1536^3, 34.5 -> 41.9 TFLOP/s; 256 tiles, 2048^3,
  // 36.1 -> 41.1; but 100 tiles, 1280 x 1280 x 4096, 31.9 -> 29.7 and 64 tiles, 1024^3, 28.7 -> 18.2): below that
  // 64 x 64 tiles, two CTAs per SM.
  const bool big = big_tiles >= env_int("FLAGBLAS_B200_SGEMM_BIG_TILES", sms * 7 / 8);
  p.tiles_n = static_cast<int>(big ? (n + 127) / 128 : (n + 63) / 64);
  const long long tiles = big ? big_tiles : ((m + 63) / 64) * p.tiles_n;
  // 16-byte aligned operands take the cp.async pipeline; FLAGBLAS_B200_SGEMM_PIPE=0 forces the
  // register-staged kernel (profiling sweeps), which also serves everything unaligned.
  // 64 x 64 tiles that do not fill two CTAs per SM, and a k worth halving: two CTAs per tile (768^3 25.1 -> 28.5 TFLOP/s,
  // 896^3 21.8 -> 27.8, 640 x 640 x 2048 19.4 -> 22.6; FLAGBLAS_B200_SGEMM_KSPLIT=0 switches it off).
  p.ksplit = (!big && tiles <= env_int("FLAGBLAS_B200_SGEMM_KSPLIT_TILES", 2 * sms) && k >= 256 &&
              env_int("FLAGBLAS_B200_SGEMM_KSPLIT", 1) != 0) ? 2 : 1;
  // few enough tiles that four CTAs per tile still fit two to an SM: clusters of four, each a quarter of k -- two
  // CTAs (16 warps) per SM hide the shared-memory latency that one CTA of eight warps cannot
  // (FLAGBLAS_B200_SGEMM_KSPLIT=2 keeps clusters of two)
  if (p.ksplit == 2 && 4 * tiles <= 2LL * sms && k >= 512 && env_int("FLAGBLAS_B200_SGEMM_KSPLIT", 1) != 2) p.ksplit = 4;
  if (p.a_vec && p.b_vec && env_int("FLAGBLAS_B200_SGEMM_PIPE", 1) != 0)
    return big ? dispatch_sgemm_pipe<128, 128>(p, tiles, stream) : dispatch_sgemm_pipe<64, 64>(p, tiles, stream);
  if (big) sgemm_simt_kernel<128, 128, 8><<<static_cast<int>(tiles), 256, 0, stream>>>(p);
  else sgemm_simt_kernel<64, 64, 16><<<static_cast<int>(tiles), 256, 0, stream>>>(p);
  FB_CUDA_OK(cudaGetLastError());
  return FB_OK;
}

// Tile plan of a dense tensor-core call (shared by fb_gemm and fb_gemm_workspace_bytes).
struct DensePlan {
  bool pair;
  int tile_m, block_n;
  long long tiles;
  bool want_streamk;  // the call can use stream-K scratch if the caller provides it
  int splitk;         // > 1: cut every tile's k range into that many parts (needs fp32 scratch for the parts)
  int cluster_k;      // > 1: the parts of a tile go to the CTAs of one cluster, which add them up in shared memory
};

// CTAs of 128-row tiles that can run at once when launched in clusters of `size` (a cluster needs `size` free SMs
// in one GPC, so the larger the cluster the more SMs stay empty).  0: clusters of that size cannot run here.
static int cluster_capacity(int size, int sm_count) {
  static int cached[64][9];
  static std::mutex mu;
  if (size < 2 || size > 8) return sm_count;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lk(mu);
  if (cached[dev][size] == 0) {
    using Cfg = TcCfg<1, 256, false>;
    auto kern = gemm_tc_kernel<1, 256, false>;
    int n = 0;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) == cudaSuccess) {
      cudaLaunchConfig_t q{};
      q.gridDim = dim3(static_cast<unsigned>(sm_count / size * size));
      q.blockDim = dim3(kNumThreads);
      q.dynamicSmemBytes = Cfg::kSmemBytes;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = static_cast<unsigned>(size); qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
      q.attrs = qa; q.numAttrs = 1;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &q) != cudaSuccess) n = 0;
    }
    cudaGetLastError();
    cached[dev][size] = n > 0 ? n * size : -1;  // -1: this cluster size cannot be launched here
  }
  return cached[dev][size] > 0 ? cached[dev][size] : 0;
}

static DensePlan plan_dense(long long m, long long n, long long k, int esz, int sm_count) {
  DensePlan pl{};
  // CTA pairs (256-row tiles) whenever there is more than one 128-row block of C;
  // FLAGBLAS_B200_PAIR=0/1 and FLAGBLAS_B200_BLOCK_N override the choice (profiling sweeps).
  pl.pair = m > kBlockM;
  const int force_pair = env_int("FLAGBLAS_B200_PAIR", -1);
  if (force_pair == 0) pl.pair = false;
  if (force_pair == 1) pl.pair = true;
  // Very short k (at most 512 bytes per row: 256 16-bit elements): a tile's epilogue is longer than its k loop, and
  // the two CTAs of a pair share their TPC's path to L2 when both store (8192 x 8192 x 256: 493 -> 535 TFLOP/s with
  // 128-row tiles; from k = 512 on the pair tiles are level or ahead).
  if (pl.pair && force_pair != 1 && k * esz <= 512) pl.pair = false;
  pl.tile_m = pl.pair ? 2 * kBlockM : kBlockM;
  const int workers = pl.pair ? sm_count / 2 : sm_count;
  pl.block_n = choose_block_n(m, n, pl.tile_m, workers, !pl.pair);
  const int force_bn = env_int("FLAGBLAS_B200_BLOCK_N", 0);
  if (force_bn == 256 || force_bn == 128 || (force_bn == 64 && !pl.pair)) pl.block_n = force_bn;
  const long long span = kSwizzleBytes / esz;
  const long long stages = (k + 2 * span - 1) / (2 * span);  // with two k-slabs per stage
  pl.splitk = 1;
  pl.cluster_k = 1;
  // CTA-pair tiles of 256 x 256 that fill at most half the pairs share their k ranges (the stream-K tail: up to four
  // workers per tile, one kernel).  In two-slab stages a shared tile costs stages / sharers + a fix-up (the owner adds
  // one parked part out of the idle operand ring, ~8 stages, or two or three with plain loads, ~12) against
  // 0.83 x stages for the 128-wide tiles choose_block_n prefers when they fit one wave (bf16 NT 256 x 8192 x 8192:
  // 43.1 against 49 us; 512 x 4096 x 14336: 57.4 / 72.2; 512 x 4096 x 4096: 25.2 / 27.3; 1024 x 1536 x 4096: 26.9 / 27.2).
  double pair_shared_cost = 0.0;  // > 0: cost of that plan in the units of the search below (stages x columns)
  if (pl.pair && force_bn == 0 && stages >= 32 && env_int("FLAGBLAS_B200_STREAMK", 1) != 0 &&
      env_int("FLAGBLAS_B200_SPLITK", -1) < 0) {
    const long long t256 = ((m + 2 * kBlockM - 1) / (2 * kBlockM)) * ((n + 255) / 256);
    if (2 * t256 <= workers && 4 * t256 >= workers) {
      const long long g = workers / t256;  // 2 or 3 (4 sharers only when 4 * t256 == workers)
      const double shared = static_cast<double>(stages) / static_cast<double>(g) + (g == 2 ? 8.0 : 12.0);
      pair_shared_cost = (shared + 4.0) * 256.0;
      if (pl.block_n == 128) {
        const long long t128 = ((m + 2 * kBlockM - 1) / (2 * kBlockM)) * ((n + 127) / 128);
        const long long waves128 = (t128 + workers - 1) / workers;
        if (shared < 0.83 * static_cast<double>(stages) * static_cast<double>(waves128)) pl.block_n = 256;
      }
    }
  }
  // Few output tiles and a long k (a handful of rows against a large matrix, or a small square problem): whole-k
  // tiles leave most SMs idle, and a CTA needs the same ~0.3 us per 64-deep stage whatever its tile width.  So the
  // tile width and a split of the k range are picked together over 128-row tiles:
  //   cost = waves x (stages per CTA + fill) x width / efficiency + the cost of adding the parts,
  // where the parts are added either by the CTAs of a cluster in shared memory (2, 4 or 8 parts, cheap) or by a
  // second kernel from fp32 scratch (any count up to 32; pays off only for very long k).
  // FLAGBLAS_B200_SPLITK = 0 / FLAGBLAS_B200_CLUSTER_K = 0 disable a method, N forces N parts.
  const int force_split = env_int("FLAGBLAS_B200_SPLITK", -1);
  const int force_cluster = env_int("FLAGBLAS_B200_CLUSTER_K", -1);
  const long long row_blocks = (m + kBlockM - 1) / kBlockM;
  const bool gpu_is_full = row_blocks * ((n + 255) / 256) >= 2LL * sm_count;  // whole-k tiles already fill it
  // (FLAGBLAS_B200_PLAN_MIN_STAGES: shortest k, in two-slab stages, for which the search runs; profiling sweeps)
  const int min_stages = env_int("FLAGBLAS_B200_PLAN_MIN_STAGES", 1);
  if (force_bn == 0 && force_pair != 1 && stages >= min_stages && !gpu_is_full && (force_split != 0 || force_cluster != 0)) {
    const int cand[3] = {256, 128, 64};
    const double eff[3] = {1.0, 0.6, 0.35};
    const int push_cost = env_int("FLAGBLAS_B200_CLUSTER_PUSH", 1) != 0 ? env_int("FLAGBLAS_B200_PLAN_PUSH_COST", 1) : 0;
    double best = 1e300;
    int best_bn = 0, best_sp = 1, best_ck = 1;
    for (int i = 0; i < 3; ++i) {
      const long long tl = row_blocks * ((n + cand[i] - 1) / cand[i]);
      for (int sp = 1; sp <= 32; ++sp) {
        if (sp > 1 && stages / sp < 2) break;
        for (int in_cluster = 0; in_cluster < 2; ++in_cluster) {
          if (in_cluster && (force_cluster == 0 || (sp != 2 && sp != 4 && sp != 8))) continue;
          if (!in_cluster && sp > 1 && (force_split == 0 || stages / sp < 4)) continue;
          if (sp == 1 && in_cluster) continue;
          const long long at_once = in_cluster ? cluster_capacity(sp, sm_count) : sm_count;
          if (at_once <= 0) continue;
          const long long ctas = tl * sp;
          const long long waves = (ctas + at_once - 1) / at_once;
          const double per_cta = static_cast<double>((stages + sp - 1) / sp + 4);
          double cost = waves * per_cta * cand[i] / eff[i];
          // measured: two cluster barriers and parking the sums ~0.8 us more than a plain epilogue, and the
          // reads over distributed shared memory run at ~16 bytes per clock per SM
          const double rows = static_cast<double>(m < kBlockM ? m : kBlockM);
          // (sent instead of read where the receiving area fits the idle epilogue staging blocks, see launch_tc:
          // 64 x 4096 x 4096, 3.8 k cycles from the last MMA to the exit against 6.7 k)
          // (only up to 32 rows: charging less for 33 to 128 rows moved 96 .. 128 x 28672 x 8192 to 64-wide tiles,
          // 91 -> 98 us)
          const bool pushed = m <= 32 && 32 * cand[i] * 4 <= 8 * kEpiStageBytes && push_cost != 0;
          const double in_cluster_cost = pushed ? 200.0 + 0.03 * rows * cand[i] : 350.0 + 0.054 * rows * cand[i];
          if (sp > 1) cost += in_cluster ? in_cluster_cost : 2300.0 + 2.1e-4 * static_cast<double>(m) * n * sp * 4.0;
          if (cost < best) { best = cost; best_bn = cand[i]; best_sp = in_cluster ? 1 : sp; best_ck = in_cluster ? sp : 1; }
        }
      }
    }
    bool take = !pl.pair;
    if (pl.pair) {
      // more than one row block: CTA-pair tiles are the default; 128-row tiles (narrower, or with a split k)
      // take over when the model says they are clearly faster (1024^3: 16 pair tiles on 148 SMs against 128
      // tiles of 128 x 64; 129 x 4096 x 4096: 16 pair tiles against 32 x 4 CTAs)
      const long long pair_tiles = ((m + 2 * kBlockM - 1) / (2 * kBlockM)) * ((n + pl.block_n - 1) / pl.block_n);
      const long long pair_waves = (pair_tiles + workers - 1) / workers;
      double pair_cost = static_cast<double>(pair_waves) * static_cast<double>(stages + 4) * 256.0;
      if (force_split != 0 && stages >= 32 && 2 * pair_tiles <= workers) {
        // the CTA-pair tiles would themselves be split through scratch (the rule further down)
        long long sp = workers / pair_tiles;
        if (sp > stages / 4) sp = stages / 4;
        if (sp > 32) sp = 32;
        const double split_cost = static_cast<double>((stages + sp - 1) / sp + 4) * 256.0 + 2300.0 +
                                  2.1e-4 * static_cast<double>(m) * n * sp * 4.0;
        if (sp >= 2 && split_cost < pair_cost) pair_cost = split_cost;
      }
      // ... or share their k ranges through the stream-K tail (bf16 1024 x 1536 x 4096: cluster split-K of 128 x 256
      // tiles 29.1 us, 24 pair tiles sharing 26.9; 512 x 4096 x 4096: 28.9 / 25.2; 256 x 8192 x 8192: 51.1 / 43.1;
      // 512 x 4096 x 14336: 72.2 / 57.4 -- while 16 pair tiles and fewer lose to the 128-row plans: 256 x 4096 x 4096
      // 19.7 against 25.6 us, 512 x 1536 x 4096 19.3 against 25.9)
      if (pair_shared_cost > 0.0 && pl.block_n == 256) {
        take = best_sp == 1 && best < 0.95 * pair_shared_cost;
      } else {
        take = best_sp == 1 && best < 0.8 * pair_cost;
      }
    }
    if (take) {
      pl.pair = false;
      pl.tile_m = kBlockM;
      pl.block_n = best_bn; pl.splitk = best_sp; pl.cluster_k = best_ck;
    }
  }
  const int split_workers = pl.pair ? sm_count / 2 : sm_count;
  pl.tiles = ((m + pl.tile_m - 1) / pl.tile_m) * ((n + pl.block_n - 1) / pl.block_n);
  // CTA-pair tiles with a deep k and few output tiles (200 x 200 x 20000: one tile; 129 x 4096 x 4096: 16): give the
  // idle pairs a part of every tile's k range, as long as a part keeps four stages and the fp32 parts stay small.
  // (Measured: below 32 stages the second kernel costs more than the shorter k loop saves.)
  // With at least a quarter as many tiles as pairs the stream-K tail (up to four workers per tile, one kernel) keeps
  // every pair busy and is the faster of the two (1024 x 1536 x 4096: 26.9 against 33.2 us; 512 x 4096 x 4096: 25.2 /
  // 38.9; 256 x 8192 x 8192: 43.1 / 58.5; 256 x 8192 x 28672: 116 / 127), so the split through scratch is for fewer.
  const bool tail_covers = 4 * pl.tiles >= split_workers && env_int("FLAGBLAS_B200_STREAMK", 1) != 0 && force_split < 0;
  if (pl.pair && force_split != 0 && stages >= 32 && 2 * pl.tiles <= split_workers && !tail_covers) {
    long long sp = split_workers / pl.tiles;
    if (sp > stages / 4) sp = stages / 4;
    if (sp > 32) sp = 32;
    while (sp > 1 && sp * m * n * 4 > (64LL << 20)) --sp;
    if (sp >= 2) pl.splitk = static_cast<int>(sp);
  }
  if (force_split > 1 && stages >= 2LL * force_split) { pl.splitk = force_split; pl.cluster_k = 1; }
  if ((force_cluster == 2 || force_cluster == 4 || force_cluster == 8) && !pl.pair && stages >= force_cluster &&
      cluster_capacity(force_cluster, sm_count) > 0) {
    pl.cluster_k = force_cluster;
    pl.splitk = 1;
  }
  const long long dp = pl.tiles / split_workers, rem = pl.tiles - dp * split_workers;
  pl.want_streamk = rem > 0 && dp < 9 && 2 * rem <= split_workers && stages >= 16 && pl.cluster_k == 1 && pl.splitk == 1 &&
                    stages >= env_int("FLAGBLAS_B200_SK_MIN_STAGES", 32) && env_int("FLAGBLAS_B200_STREAMK", 1) != 0;
  // ... or, for a last wave more than half full, its tiles' last stages go to the workers it leaves idle
  if (tail_slabs((k + span - 1) / span, split_workers, rem) > 0 && pl.cluster_k == 1 && pl.splitk == 1 && pl.block_n <= 256 &&
      env_int("FLAGBLAS_B200_STREAMK", 1) != 0)
    pl.want_streamk = true;
  // ... or stream-K over the whole launch: two or three waves, the last more than half full (see launch_tc)
  if (rem > 0 && 2 * rem > split_workers && dp >= 1 && dp <= 2 && stages >= 16 && pl.cluster_k == 1 && pl.splitk == 1 &&
      pl.block_n <= 256 && env_int("FLAGBLAS_B200_STREAMK", 1) != 0 && env_int("FLAGBLAS_B200_STREAMK_FULL", 0) != 0)
    pl.want_streamk = true;
  return pl;
}

// Launch `kern` as a programmatic dependent of the kernel queued before it on `stream`: it may become resident
// while that kernel still runs and must call griddepcontrol.wait before touching its results.
template <class... KArgs, class... Args>
static cudaError_t launch_dependent(void (*kern)(KArgs...), unsigned grid, unsigned block, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ------------------------------------------------------------------- gemv
// How a matrix-vector call is spread over the GPU (shared by fb_gemv and fb_gemv_workspace_bytes).
struct GemvPlan {
  int lanes;        // threads along the columns (per row block for N)
  int threads;
  int grid_x;
  int splits;       // ranges of the reduced dimension; > 1 needs the fp32 partial buffer
  long long chunk;  // reduced-dimension elements per range
};

static GemvPlan plan_gemv(int trans, long long m, long long n, int esz, int sms) {
  GemvPlan pl{};
  const long long E = 16 / esz;
  const long long vec_cols = (n + E - 1) / E;
  pl.threads = 256;
  pl.splits = 1;
  // FLAGBLAS_B200_GEMV_TX / _GEMV_SPLITS override the choices below (profiling sweeps).
  const int force_tx = env_int("FLAGBLAS_B200_GEMV_TX", 0);
  const int force_splits = env_int("FLAGBLAS_B200_GEMV_SPLITS", 0);
  if (trans == FB_OP_N) {
    int tx = 4;
    while (tx < 256 && tx < vec_cols) tx *= 2;
    if (force_tx >= 4 && force_tx <= 256 && (force_tx & (force_tx - 1)) == 0) tx = force_tx;
    pl.lanes = tx;
    const long long rows_per_cta = (256 / tx) * kGemvRows;
    const long long row_ctas = (m + rows_per_cta - 1) / rows_per_cta;
    pl.grid_x = static_cast<int>(row_ctas < 32LL * sms ? row_ctas : 32LL * sms);
    pl.chunk = n;
    const long long step = tx * E;  // columns one pass of a group covers
    long long s = 1;
    // Few row blocks and long rows: split the columns so that every SM gets work, as long as a
    // range keeps at least eight passes.
    if (row_ctas < sms) {
      const long long by_work = (n + 8 * step - 1) / (8 * step);
      const long long by_fill = (4LL * sms + row_ctas - 1) / row_ctas;
      s = by_work < by_fill ? by_work : by_fill;
    }
    if (force_splits > 0) s = force_splits;
    if (s > 1) {
      long long chunk = (n + s - 1) / s;
      chunk = (chunk + step - 1) / step * step;
      pl.chunk = chunk;
      pl.splits = static_cast<int>((n + chunk - 1) / chunk);
    }
  } else {
    int tx = 1;
    while (tx < 256 && tx < vec_cols) tx *= 2;
    if (force_tx >= 1 && force_tx <= 256 && (force_tx & (force_tx - 1)) == 0) tx = force_tx;
    pl.lanes = tx;
    const long long ny = 256 / tx;
    const long long col_ctas = (vec_cols + tx - 1) / tx;
    pl.grid_x = static_cast<int>(col_ctas);
    // measured on B200: 4 CTAs per SM are best for 16-bit types, 16 per SM for fp32
    const long long want_t = (esz == 4 ? 16LL : 4LL) * sms;
    const long long by_fill = (want_t + col_ctas - 1) / col_ctas;
    const long long by_work = (m + 32 * ny - 1) / (32 * ny);  // at least 32 rows per thread
    long long s = by_work < by_fill ? by_work : by_fill;
    if (force_splits > 0) s = force_splits;
    if (s < 1) s = 1;
    if (s > 65535) s = 65535;
    long long chunk = (m + s - 1) / s;
    chunk = (chunk + ny - 1) / ny * ny;
    pl.chunk = chunk;
    pl.splits = static_cast<int>((m + chunk - 1) / chunk);
  }
  if (pl.splits < 1) pl.splits = 1;
  return pl;
}

template <class T>
static int run_gemv(int trans, long long m, long long n, float alpha, const void* A, long long lda, const void* x,
                    long long incx, float beta, void* y, long long incy, void* workspace, size_t workspace_bytes,
                    int sms, cudaStream_t stream) {
  const long long len_y = trans == FB_OP_N ? m : n;
  if (alpha == 0.f) {
    if (beta == 1.f) return FB_OK;
    gemv_scale_kernel<T><<<static_cast<unsigned>((len_y + 255) / 256), 256, 0, stream>>>(static_cast<T*>(y), len_y,
                                                                                         incy, beta);
    FB_CUDA_OK(cudaGetLastError());
    return FB_OK;
  }
  const GemvPlan pl = plan_gemv(trans, m, n, sizeof(T), sms);
  GemvParams p{};
  p.m = static_cast<int>(m); p.n = static_cast<int>(n); p.lda = lda;
  p.A = A; p.x = x; p.y = y; p.incx = incx; p.incy = incy;
  p.alpha = alpha; p.beta = beta;
  p.splits = pl.splits; p.chunk = pl.chunk; p.tx = pl.lanes;
  p.a_vec = aligned16(A, lda, sizeof(T)) ? 1 : 0;
  p.x_vec = (incx == 1 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) ? 1 : 0;
  if (pl.splits > 1) {
    const size_t need = static_cast<size_t>(pl.splits) * static_cast<size_t>(len_y) * sizeof(float);
    if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15)) return FB_ERR_WORKSPACE;
    p.partial = static_cast<float*>(workspace);
  }
  const dim3 grid(static_cast<unsigned>(pl.grid_x), static_cast<unsigned>(pl.splits));
  if (trans == FB_OP_N) {
    // variant = unroll * 10 + min CTAs per SM; FLAGBLAS_B200_GEMV_NV overrides (profiling sweeps)
    switch (env_int("FLAGBLAS_B200_GEMV_NV", 24)) {
      case 16: gemv_n_kernel<T, 1, 6><<<grid, 256, 0, stream>>>(p); break;
      case 18: gemv_n_kernel<T, 1, 8><<<grid, 256, 0, stream>>>(p); break;
      case 25: gemv_n_kernel<T, 2, 5><<<grid, 256, 0, stream>>>(p); break;
      case 26: gemv_n_kernel<T, 2, 6><<<grid, 256, 0, stream>>>(p); break;
      default: gemv_n_kernel<T, 2, 4><<<grid, 256, 0, stream>>>(p); break;
    }
  } else {
    // variant = rows in flight per thread * 10 + min CTAs per SM; FLAGBLAS_B200_GEMV_TV overrides
    switch (env_int("FLAGBLAS_B200_GEMV_TV", sizeof(T) == 4 ? 46 : 85)) {
      case 46: gemv_t_kernel<T, 4, 6><<<grid, pl.threads, 0, stream>>>(p); break;
      case 48: gemv_t_kernel<T, 4, 8><<<grid, pl.threads, 0, stream>>>(p); break;
      case 28: gemv_t_kernel<T, 2, 8><<<grid, pl.threads, 0, stream>>>(p); break;
      case 86: gemv_t_kernel<T, 8, 6><<<grid, pl.threads, 0, stream>>>(p); break;
      default: gemv_t_kernel<T, 8, 5><<<grid, pl.threads, 0, stream>>>(p); break;
    }
  }
  FB_CUDA_OK(cudaGetLastError());
  if (pl.splits > 1) {
    FB_CUDA_OK(launch_dependent(gemv_finish_kernel<T>, static_cast<unsigned>((len_y + 31) / 32), 256, stream, p.partial,
                                pl.splits, len_y, static_cast<T*>(y), incy, alpha, beta));
  }
  return FB_OK;
}

// fp8 matrix and vector, trans = T only: y[n] (TY) = alpha * A^T x + beta * y.
template <class TA, class TX, class TY>
static int run_gemv_fp8(long long m, long long n, float alpha, const void* A, long long lda, const void* x,
                        long long incx, float beta, void* y, long long incy, void* workspace, size_t workspace_bytes,
                        int sms, cudaStream_t stream) {
  if (alpha == 0.f) {
    if (beta == 1.f) return FB_OK;
    gemv_scale_kernel<TY><<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(static_cast<TY*>(y), n, incy, beta);
    FB_CUDA_OK(cudaGetLastError());
    return FB_OK;
  }
  const GemvPlan pl = plan_gemv(FB_OP_T, m, n, 1, sms);
  GemvParams p{};
  p.m = static_cast<int>(m); p.n = static_cast<int>(n); p.lda = lda;
  p.A = A; p.x = x; p.y = y; p.incx = incx; p.incy = incy;
  p.alpha = alpha; p.beta = beta;
  p.splits = pl.splits; p.chunk = pl.chunk; p.tx = pl.lanes;
  p.a_vec = aligned16(A, lda, 1) ? 1 : 0;
  p.x_vec = 0;
  if (pl.splits > 1) {
    const size_t need = static_cast<size_t>(pl.splits) * static_cast<size_t>(n) * sizeof(float);
    if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15)) return FB_ERR_WORKSPACE;
    p.partial = static_cast<float*>(workspace);
  }
  const dim3 grid(static_cast<unsigned>(pl.grid_x), static_cast<unsigned>(pl.splits));
  gemv_t_kernel<TA, 8, 4, TX, TY><<<grid, pl.threads, 0, stream>>>(p);
  FB_CUDA_OK(cudaGetLastError());
  if (pl.splits > 1) {
    FB_CUDA_OK(launch_dependent(gemv_finish_kernel<TY>, static_cast<unsigned>((n + 31) / 32), 256, stream, p.partial,
                                pl.splits, n, static_cast<TY*>(y), incy, alpha, beta));
  }
  return FB_OK;
}

template <class TA, class TX>
static int run_gemv_fp8_y(int y_dtype, long long m, long long n, float alpha, const void* A, long long lda,
                          const void* x, long long incx, float beta, void* y, long long incy, void* ws, size_t ws_bytes,
                          int sms, cudaStream_t stream) {
  switch (y_dtype) {
    case FB_F16: return run_gemv_fp8<TA, TX, __half>(m, n, alpha, A, lda, x, incx, beta, y, incy, ws, ws_bytes, sms, stream);
    case FB_BF16: return run_gemv_fp8<TA, TX, __nv_bfloat16>(m, n, alpha, A, lda, x, incx, beta, y, incy, ws, ws_bytes, sms, stream);
    default: return run_gemv_fp8<TA, TX, float>(m, n, alpha, A, lda, x, incx, beta, y, incy, ws, ws_bytes, sms, stream);
  }
}

// A GEMM with one output row or column is a matrix-vector product: it goes to the HBM-bound gemv kernels (fp32
// accumulate and one rounding, like the tensor-core path) instead of a tile that is 127/128 padding.
// FB_TF32 stays on the tensor cores (its contract is TF32 products).
struct GemvView {
  bool ok;
  int trans;
  long long m, n, lda, incx, incy;
  const void* A;
  const void* x;
};

static GemvView gemm_as_gemv(int dtype, int transa, int transb, long long m, long long n, long long k, const void* A,
                             long long lda, const void* B, long long ldb, long long ldc) {
  GemvView v{};
  if (dtype == FB_TF32 || env_int("FLAGBLAS_B200_GEMM_AS_GEMV", 1) == 0) return v;
  if (m == 1) {
    // C[1, n] = a[k] * op(B): B stored [n, k] (transb = T) -> y = B a;  stored [k, n] -> y = B^T a
    v.ok = true; v.A = B; v.lda = ldb; v.x = A;
    v.incx = transa ? lda : 1;  // a is a row of A[1, k], or a column of A stored [k, 1]
    v.incy = 1;
    if (transb) { v.trans = FB_OP_N; v.m = n; v.n = k; } else { v.trans = FB_OP_T; v.m = k; v.n = n; }
  } else if (n == 1) {
    // C[m, 1] = op(A) * b[k]: A stored [m, k] -> y = A b;  stored [k, m] (transa = T) -> y = A^T b
    v.ok = true; v.A = A; v.lda = lda; v.x = B;
    v.incx = transb ? 1 : ldb;  // b is a column of B stored [k, 1] (stride ldb), or the row B[1, k]
    v.incy = ldc;
    if (transa) { v.trans = FB_OP_T; v.m = k; v.n = m; } else { v.trans = FB_OP_N; v.m = m; v.n = k; }
  }
  return v;
}

// --------------------------------------------------- double / complex GEMM on the CUDA cores
template <bool AK, bool BKM>
static int launch_dgemm_mma_t(XgemmParams p, cudaStream_t stream) {
  auto kern = dgemm_mma_kernel<AK, BKM>;
  constexpr int kBytes = kDmStages * (DmTile<kDmBM, AK>::kDoubles + DmTile<kDmBN, BKM>::kDoubles) * 8;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    FB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes));
    attr_set[dev] = true;
  }
  p.tiles_n = (p.n + kDmBN - 1) / kDmBN;
  const long long tiles = static_cast<long long>((p.m + kDmBM - 1) / kDmBM) * p.tiles_n;
  if (tiles > 0x7fffffffLL) return FB_ERR_UNSUPPORTED;
  kern<<<static_cast<unsigned>(tiles), 256, kBytes, stream>>>(p);
  FB_CUDA_OK(cudaGetLastError());
  return FB_OK;
}

template <bool AK, bool BKM>
static int launch_zgemm_mma_t(XgemmParams p, cudaStream_t stream) {
  auto kern = zgemm_mma_kernel<AK, BKM>;
  constexpr int kBytes = kZmStages * (ZmTile<AK>::kElems + ZmTile<BKM>::kElems) * 16;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    FB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes));
    attr_set[dev] = true;
  }
  p.tiles_n = (p.n + kZmT - 1) / kZmT;
  const long long tiles = static_cast<long long>((p.m + kZmT - 1) / kZmT) * p.tiles_n;
  if (tiles > 0x7fffffffLL) return FB_ERR_UNSUPPORTED;
  kern<<<static_cast<unsigned>(tiles), 256, kBytes, stream>>>(p);
  FB_CUDA_OK(cudaGetLastError());
  return FB_OK;
}

static int launch_zgemm_mma(const XgemmParams& p, bool a_kc, bool b_kc, cudaStream_t stream) {
  if (a_kc) return b_kc ? launch_zgemm_mma_t<true, true>(p, stream) : launch_zgemm_mma_t<true, false>(p, stream);
  return b_kc ? launch_zgemm_mma_t<false, true>(p, stream) : launch_zgemm_mma_t<false, false>(p, stream);
}

// fp64 tensor path for 16-byte aligned operands; a_kc / b_kc: the operand is stored with K contiguous.
static int launch_dgemm_mma(const XgemmParams& p, bool a_kc, bool b_kc, cudaStream_t stream) {
  if (a_kc) return b_kc ? launch_dgemm_mma_t<true, true>(p, stream) : launch_dgemm_mma_t<true, false>(p, stream);
  return b_kc ? launch_dgemm_mma_t<false, true>(p, stream) : launch_dgemm_mma_t<false, false>(p, stream);
}

template <class T>
static int run_xgemm(int transa, int transb, long long m, long long n, long long k, const double* alpha, const void* A,
                     long long lda, const void* B, long long ldb, const double* beta, void* C, long long ldc,
                     bool complex_type, cudaStream_t stream, int tri_operand = 0, int tri_upper = 0, int tri_unit = 0) {
  const double ar = alpha[0], ai = complex_type ? alpha[1] : 0.0;
  const double br = beta[0], bi = complex_type ? beta[1] : 0.0;
  if (k == 0 || (ar == 0.0 && ai == 0.0)) {
    if (br == 1.0 && bi == 0.0) return FB_OK;
    long long blocks = (m * n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    xgemm_scale_kernel<T><<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<T*>(C), ldc, static_cast<int>(m),
                                                                        static_cast<int>(n), br, bi);
    FB_CUDA_OK(cudaGetLastError());
    return FB_OK;
  }
  XgemmParams p{};
  p.m = static_cast<int>(m); p.n = static_cast<int>(n); p.k = static_cast<int>(k);
  p.alpha_re = ar; p.alpha_im = ai; p.beta_re = br; p.beta_im = bi;
  p.A = A; p.lda = lda; p.B = B; p.ldb = ldb; p.C = C; p.ldc = ldc;
  p.transa = transa; p.transb = transb;
  p.tri_operand = tri_operand; p.tri_upper = tri_upper; p.tri_unit = tri_unit;
  if (std::is_same<T, double>::value && tri_operand == 0 && aligned16(A, lda, 8) && aligned16(B, ldb, 8) &&
      env_int("FLAGBLAS_B200_DGEMM_MMA", 1) != 0)
    return launch_dgemm_mma(p, transa == 0, transb != 0, stream);
  if (std::is_same<T, cdouble>::value && tri_operand == 0 && ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) == 0 &&
      env_int("FLAGBLAS_B200_DGEMM_MMA", 1) != 0)
    return launch_zgemm_mma(p, transa == 0, transb != 0, stream);
  p.tiles_n = static_cast<int>((n + kXTile - 1) / kXTile);
  const long long tiles = ((m + kXTile - 1) / kXTile) * p.tiles_n;
  if (tiles > 0x7fffffffLL) return FB_ERR_UNSUPPORTED;
  xgemm_simt_kernel<T><<<static_cast<unsigned>(tiles), 256, 0, stream>>>(p);
  FB_CUDA_OK(cudaGetLastError());
  return FB_OK;
}

}  // namespace fb

using namespace fb;

extern "C" {

size_t fb_gemm_workspace_bytes(int dtype, int transa, int transb, int64_t m, int64_t n, int64_t k, const void* A,
                               int64_t lda, const void* B, int64_t ldb) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  {
    const GemvView gv = gemm_as_gemv(dtype, transa, transb, m, n, k, A, lda, B, ldb, n);
    if (gv.ok) return fb_gemv_workspace_bytes(dtype, gv.trans, gv.m, gv.n);
  }
  const PackPlan pl = plan_pack(dtype, transa, transb, m, n, k, A, lda, B, ldb);
  size_t bytes = pl.a_bytes + pl.b_bytes;
  if (dtype != FB_F32) {
    const DeviceInfo* di = device_info();
    if (di) {
      const DensePlan dp = plan_dense(m, n, k, elem_size(dtype), di->sm_count);
      if (dp.want_streamk) bytes += streamk_bytes(di->sm_count, dp.block_n);
      if (dp.splitk > 1) bytes = round_up(bytes, 256) + static_cast<size_t>(dp.splitk) * m * n * sizeof(float);
    }
  }
  return bytes;
}

int fb_gemm(int dtype, int transa, int transb, int64_t m, int64_t n, int64_t k, float alpha, const void* A,
            int64_t lda, const void* B, int64_t ldb, float beta, void* C, int64_t ldc, void* workspace,
            size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (dtype < FB_F32 || dtype > FB_BF16) return FB_ERR_INVALID_ARG;
  if ((transa != FB_OP_N && transa != FB_OP_T) || (transb != FB_OP_N && transb != FB_OP_T)) return FB_ERR_INVALID_ARG;
  if (m < 0 || n < 0 || k < 0) return FB_ERR_INVALID_ARG;
  if (m > 0x7fffffffLL || n > 0x7fffffffLL || k > 0x7fffffffLL) return FB_ERR_UNSUPPORTED;
  if (m == 0 || n == 0) return FB_OK;
  if (!C || ldc < n) return FB_ERR_INVALID_ARG;

  const DeviceInfo* di = device_info();
  if (!di) return FB_ERR_LAUNCH;
  if (di->cc_major != 10) return FB_ERR_UNSUPPORTED;

  if (k == 0 || alpha == 0.f) {
    switch (dtype) {
      case FB_F16: return run_scale<__half>(C, ldc, m, n, beta, stream);
      case FB_BF16: return run_scale<__nv_bfloat16>(C, ldc, m, n, beta, stream);
      default: return run_scale<float>(C, ldc, m, n, beta, stream);
    }
  }
  if (!A || !B) return FB_ERR_INVALID_ARG;
  if (lda < (transa ? m : k) || ldb < (transb ? k : n)) return FB_ERR_INVALID_ARG;

  {
    const GemvView gv = gemm_as_gemv(dtype, transa, transb, m, n, k, A, lda, B, ldb, ldc);
    if (gv.ok)
      return fb_gemv(dtype, gv.trans, gv.m, gv.n, alpha, gv.A, gv.lda, gv.x, gv.incx, beta, C, gv.incy, workspace,
                     workspace_bytes, stream_);
  }
  if (dtype == FB_F32)
    return run_sgemm_simt(transa, transb, m, n, k, alpha, static_cast<const float*>(A), lda,
                          static_cast<const float*>(B), ldb, beta, static_cast<float*>(C), ldc, di->sm_count, stream);

  const int esz = elem_size(dtype);
  size_t ws_used = 0;  // bytes of the workspace taken by packed operands
  bool packed = false; // a packing kernel was queued just before the GEMM
  // Operands that TMA cannot address in place are packed to a 16-byte pitched copy first.
  const PackPlan pl = plan_pack(dtype, transa, transb, m, n, k, A, lda, B, ldb);
  if (pl.pack_a || pl.pack_b) {
    if (!workspace || workspace_bytes < pl.a_bytes + pl.b_bytes || (reinterpret_cast<uintptr_t>(workspace) & 255))
      return FB_ERR_WORKSPACE;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    ws_used = pl.a_bytes + pl.b_bytes;
    PackJob ja{}, jb{};
    int blocks_a = 0, blocks_b = 0;
    auto blocks_for = [](long long total) {
      long long b = (total + 255) / 256;
      return static_cast<int>(b > 148 * 8 ? 148 * 8 : b);
    };
    if (pl.pack_a) {
      ja = PackJob{A, ws, lda, pl.a_ld, pl.a_rows, pl.a_cols};
      blocks_a = blocks_for(pl.a_rows * pl.a_cols);
      A = ws; lda = pl.a_ld; ws += pl.a_bytes;
    }
    if (pl.pack_b) {
      jb = PackJob{B, ws, ldb, pl.b_ld, pl.b_rows, pl.b_cols};
      blocks_b = blocks_for(pl.b_rows * pl.b_cols);
      B = ws; ldb = pl.b_ld;
    }
    if (blocks_a + blocks_b > 0) {
      if (esz == 2) pack2_kernel<uint16_t><<<blocks_a + blocks_b, 256, 0, stream>>>(ja, jb, blocks_a);
      else pack2_kernel<uint32_t><<<blocks_a + blocks_b, 256, 0, stream>>>(ja, jb, blocks_a);
      FB_CUDA_OK(cudaGetLastError());
      packed = true;
    }
  }

  const DensePlan dplan = plan_dense(m, n, k, esz, di->sm_count);
  const bool pair = dplan.pair;
  const int tile_m = dplan.tile_m;
  int block_n = dplan.block_n;
  const uint32_t span = kSwizzleBytes / esz;
  const bool a_mn = transa == FB_OP_T;  // stored [k, m]: M contiguous
  const bool b_mn = transb == FB_OP_N;  // stored [k, n]: N contiguous

  // One 3-D copy per operand and stage where the operand's extents allow it (the 3-D view's
  // innermost extent is a full 128-byte row, so the dimension it tiles must be a multiple of
  // `span`); then a stage can also hold two k-slabs, which halves barrier traffic and lets each
  // copy instruction move twice the bytes.
  const bool a3d = (a_mn ? (m % span == 0) : (k % span == 0)) && env_int("FLAGBLAS_B200_TMA3D", 1) != 0;
  const bool b3d = (b_mn ? (n % span == 0) : (k % span == 0)) && env_int("FLAGBLAS_B200_TMA3D", 1) != 0;
  int ks = (a3d && b3d && k > static_cast<long long>(span)) ? 2 : 1;
  const int force_ks = env_int("FLAGBLAS_B200_KS", 0);
  if (force_ks == 1 || (force_ks == 2 && a3d && b3d)) ks = force_ks;
  // 256 x 512 pair tiles (FLAGBLAS_B200_BLOCK_N=512): a quarter less operand traffic per FLOP than
  // 256 x 256, paid for with a single-buffered accumulator (all 512 TMEM columns hold one tile).
  // They need the one-copy-per-stage 3-D views of both operands.
  // Chosen by itself for large beta = 0 calls: with random data the GPU is power-limited, the smaller operand stream
  // leaves more of the budget to the tensor pipe (8192^3, 300 launches back to back: 0.955 -> 0.884 ms, SM clock
  // 1312 -> 1365 MHz; with all-zero operands, which do not throttle, it is 2 % slower).  It needs at least one full
  // wave of tiles, and a wave count that wastes no more than the 256-wide tiling does.
  bool wide = false;
  // with the merged B copy and one-slab stages (bf16 8192 x 8192 x k: k = 4096 +3.1 %, 2048 -1.2 %, 1024 -15 %; TF32 TN:
  // k = 8192 +9 %, 4096 +8 %, 2048 +1.4 %)
  // beta != 0: the epilogue also reads C and every tile's is exposed, which only a four times longer k loop pays for,
  // and for 16-bit types only (bf16 NT beta = 1: 8192 x 8192 x 16384 +4.6 %, fp16 8192^3 +0.9 %, 16384 x 14336 x 4096
  // -11 %; TF32 TN beta = 0.5: 8192^3 +2.6 %, but 16384^3 -4 to +7 % from run to run and 8192 x 8192 x 4096 -3.5 %)
  const bool long_k = beta == 0.f ? (esz == 4 ? k >= 2048 : k >= 4096) : (esz == 2 && k >= 16384);
  if (pair && a3d && b3d && block_n == 256 && dplan.splitk == 1 && long_k &&
      env_int("FLAGBLAS_B200_BLOCK_N", 0) == 0 && env_int("FLAGBLAS_B200_WIDE_TILES", 1) != 0) {
    const long long pairs = di->sm_count / 2;
    const long long rows = (m + 2 * kBlockM - 1) / (2 * kBlockM);
    const long long t256 = rows * ((n + 255) / 256), t512 = rows * ((n + 511) / 512);
    const double e256 = static_cast<double>(t256) / static_cast<double>((t256 + pairs - 1) / pairs * pairs);
    const double e512 = static_cast<double>(t512) / static_cast<double>((t512 + pairs - 1) / pairs * pairs);
    // (at least one full wave of wide tiles: 4096^3 = 1.73 waves +3.7 %, 16384 x 1536 x 4096 = 2.6 waves +3.8 %)
    wide = t512 >= pairs && e512 >= e256 - 0.02 && n % 512 == 0;
    // ... or a single wave of them more than three quarters full, where 256-wide tiles make two waves of which the
    // second is more than half full (one rank's share of 8192^3 over eight GPUs, fp16 8192 x 1024 x 8192: 103.0 us
    // against 112.8 with the narrow tiles' last stages dealt to the idle workers and 114.6 with whole narrow tiles;
    // 4096 x 2048 x 8192 100.9 against 109.3; 8192 x 1024 x 4096 55.6 against 59.4).  Less full than that the
    // narrow tiles' stream-K tail wins (6144 x 1024 x 8192, 48 wide tiles: 94.4 against 89.8 us).
    if (t512 < pairs && 4 * t512 > 3 * pairs && n % 512 == 0) wide = true;
  }
  if (pair && a3d && b3d && (wide || env_int("FLAGBLAS_B200_BLOCK_N", 0) == 512)) block_n = 512;
  // A 512-wide tile holds four k-slabs of 48 KB: as four one-slab stages the refill of a stage has three stages'
  // MMAs to hide behind (two two-slab stages leave one), and with the B stage fetched by ONE copy the two copies per
  // slab stay below the slab's MMA time (8192^3 fp16: 1463-1472 against 1425-1427 TFLOP/s with two slabs per stage;
  // with two B copies per stage one slab per stage loses, 1403 against 1415)
  if (block_n == 512 && force_ks == 0 && env_int("FLAGBLAS_B200_WIDE_MERGED", 1) != 0) ks = 1;
  // 512-wide tiles fetch this CTA's 256 columns of B with one copy (FLAGBLAS_B200_WIDE_MERGED=0: one copy of 128
  // columns per MMA half, the accumulator then holds the tile's columns in order)
  const bool wide_merged = block_n > 256 && env_int("FLAGBLAS_B200_WIDE_MERGED", 1) != 0;
  const int halves = (block_n > 256 && !wide_merged) ? 2 : 1;
  const int b_rows = (pair ? block_n / 2 : block_n) / halves;  // rows of B per copy

  CUtensorMap ma, mb;
  const bool atom32 = esz == 4;  // MN-major fp32 operands use the 32-byte-atom swizzle
  const uint64_t kslabs = (static_cast<uint64_t>(k) + span - 1) / span;
  // A single row block of few rows of a k-contiguous A: copies of only those rows, rounded up to the 8 rows of a
  // swizzle pattern, and slots to match (TcGemmParams::a_rows).  The TMA unit is what bounds the k loop of such
  // calls (~250 cycles + bytes / 120 per copy), and half or more of a 128-row box would be zeros.
  const int a_rows = (!pair && !a_mn && m < kBlockM - 8 && env_int("FLAGBLAS_B200_A_ROWS", 1) != 0)
                         ? static_cast<int>((m + 7) / 8 * 8) : kBlockM;
  auto encode_maps = [&](bool a3, bool b3, int nks) -> int {
    int rc;
    if (a3) {
      if (a_mn) rc = encode_3d(&ma, dtype, A, span, k, m / span, lda * esz, kSwizzleBytes, span, span * nks, kBlockM / span, atom32);
      else rc = encode_3d(&ma, dtype, A, span, m, kslabs, lda * esz, kSwizzleBytes, span, a_rows, nks, false);
    } else if (a_mn) rc = encode_2d(&ma, dtype, A, m, k, lda * esz, span, span, atom32);
    else rc = encode_2d(&ma, dtype, A, k, m, lda * esz, span, a_rows);
    if (rc) return rc;
    if (b3) {
      if (b_mn) rc = encode_3d(&mb, dtype, B, span, k, n / span, ldb * esz, kSwizzleBytes, span, span * nks, b_rows / span, atom32);
      else rc = encode_3d(&mb, dtype, B, span, n, kslabs, ldb * esz, kSwizzleBytes, span, b_rows, nks, false);
    } else if (b_mn) rc = encode_2d(&mb, dtype, B, n, k, ldb * esz, span, span, atom32);
    else rc = encode_2d(&mb, dtype, B, k, n, ldb * esz, span, b_rows);
    return rc;
  };
  bool use_a3d = a3d, use_b3d = b3d;
  int rc = encode_maps(use_a3d, use_b3d, ks);
  if (rc && (use_a3d || use_b3d)) {
    // the driver refused a 3-D view: fall back to plain 2-D boxes, one k-slab per stage
    if (block_n > 256) return rc;  // (512-wide tiles are only chosen on request)
    use_a3d = use_b3d = false;
    ks = 1;
    rc = encode_maps(false, false, 1);
  }
  if (rc) return rc;

  TcGemmParams p{};
  p.prob.m = static_cast<int>(m); p.prob.n = static_cast<int>(n);
  p.prob.out = C; p.prob.ldo = ldc; p.prob.cin = C; p.prob.ldcin = ldc;
  p.prob.vec_ok = aligned16(C, ldc, esz) ? 1 : 0;
  p.k = static_cast<int>(k);
  p.tiles_m = static_cast<int>((m + tile_m - 1) / tile_m);
  p.tiles_n = static_cast<int>((n + block_n - 1) / block_n);
  // raster: row tiles walked down before stepping one column tile right (measured at 8192^3: 256-wide pair tiles
  // 4 / 8 / 16 -> 1187 / 1307 / 1086 TFLOP/s; 512-wide 8 / 12 / 16 / 32 -> 1407 / 1418 / 1431 / 1412)
  p.group_m = env_int("FLAGBLAS_B200_GROUP_M", pair ? (block_n == 512 ? 16 : 8) : 16);
  if (p.group_m < 1) p.group_m = 1;
  p.alpha = alpha; p.beta = beta;
  p.idesc = make_idesc(idesc_fmt(dtype), a_mn, b_mn, tile_m, block_n > 256 ? 256 : block_n);
  p.block_k = span * ks;
  p.ks = ks;
  p.a = make_geom(esz, a_rows, a_mn, ks, use_a3d);
  p.a_rows = a_rows < kBlockM ? a_rows : 0;
  p.b = make_geom(esz, b_rows, b_mn, ks, use_b3d);
  p.num_groups = 0;
  p.wide_merged = wide_merged ? 1 : 0;
  p.c_streaming = env_int("FLAGBLAS_B200_C_STREAMING", 0) != 0 ? 1 : 0;
  p.wait_prior = packed ? 1 : 0;
  // Optional stream-K scratch behind the packed operands: used only when the caller provided it.
  if (dplan.want_streamk && block_n <= 256 && workspace && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0 &&
      workspace_bytes >= ws_used + streamk_bytes(di->sm_count, block_n)) {
    uint8_t* sk = static_cast<uint8_t*>(workspace) + ws_used;
    p.sk_flags = reinterpret_cast<int*>(sk);
    p.sk_partials = reinterpret_cast<float*>(sk + kStreamKFlagBytes);
  }
  long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
  // Split-K for skinny calls: used only when the caller provided the scratch fb_gemm_workspace_bytes asked for.
  int splitk = dplan.splitk;
  const long long k_stages = (k + p.block_k - 1) / p.block_k;
  while (splitk > 1 && k_stages / splitk < 2) --splitk;
  const size_t split_off = round_up(ws_used, 256);
  if (splitk > 1 && !p.sk_partials && workspace && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0 &&
      workspace_bytes >= split_off + static_cast<size_t>(splitk) * m * n * sizeof(float)) {
    p.splitk = splitk;
    p.splitk_out = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + split_off);
    tiles *= splitk;
  }
  if (p.splitk <= 1 && !p.sk_partials && !pair && block_n <= 256) {
    // Cluster split-K: needs no scratch.  Every part must own at least one stage.
    int ck = dplan.cluster_k;
    while (ck > 1 && k_stages < ck) ck /= 2;
    if (ck > 1) {
      p.cluster_k = ck;
      p.cluster_push = env_int("FLAGBLAS_B200_CLUSTER_PUSH", 1);
      tiles *= ck;
    }
  }
  if (env_int("FLAGBLAS_B200_PLAN_DEBUG", 0) != 0)
    fprintf(stderr, "fb_gemm plan: %lld x %lld x %lld pair=%d block_n=%d ks=%d stages=%lld split=%d cluster=%d ctas=%lld\n",
            static_cast<long long>(m), static_cast<long long>(n), static_cast<long long>(k), pair ? 1 : 0, block_n, ks,
            k_stages, p.splitk, p.cluster_k, tiles);
  // beta = 0 and whole tiles: C leaves through TMA stores when a tensor map can describe it (FLAGBLAS_B200_C_TMA=0:
  // through the epilogue warps' own stores)
  CUtensorMap mc = ma;  // (unused unless c_tma)
  p.c_tma = 0;
  if (beta == 0.f && p.splitk <= 1 && p.cluster_k <= 1 && (reinterpret_cast<uintptr_t>(C) & 15) == 0 &&
      (static_cast<uint64_t>(ldc) * esz) % 16 == 0 && env_int("FLAGBLAS_B200_C_TMA", 1) != 0 &&
      encode_2d(&mc, dtype, C, static_cast<uint64_t>(n), static_cast<uint64_t>(m), static_cast<uint64_t>(ldc) * esz,
                kSwizzleBytes / esz, 32) == FB_OK)
    p.c_tma = 1;
  rc = dispatch_tc(dtype, block_n, pair, ma, mb, mc, p, tiles, di->sm_count, stream);
  if (rc || p.splitk <= 1) return rc;
  long long blocks = (m * n + 255) / 256;
  if (blocks > 4LL * di->sm_count) blocks = 4LL * di->sm_count;
  cudaLaunchConfig_t fcfg{};
  fcfg.gridDim = dim3(static_cast<unsigned>(blocks));
  fcfg.blockDim = dim3(256);
  fcfg.stream = stream;
  cudaLaunchAttribute fattr[1];
  fattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  fattr[0].val.programmaticStreamSerializationAllowed = 1;
  fcfg.attrs = fattr;
  fcfg.numAttrs = 1;
  const float* parts = p.splitk_out;
  const int im = static_cast<int>(m), in = static_cast<int>(n);
  const long long ldo = ldc;
  switch (dtype) {
    case FB_F16:
      FB_CUDA_OK(cudaLaunchKernelEx(&fcfg, splitk_finish_kernel<__half>, parts, p.splitk, im, in, alpha, beta,
                                    static_cast<__half*>(C), ldo));
      break;
    case FB_BF16:
      FB_CUDA_OK(cudaLaunchKernelEx(&fcfg, splitk_finish_kernel<__nv_bfloat16>, parts, p.splitk, im, in, alpha, beta,
                                    static_cast<__nv_bfloat16*>(C), ldo));
      break;
    default:
      FB_CUDA_OK(cudaLaunchKernelEx(&fcfg, splitk_finish_kernel<float>, parts, p.splitk, im, in, alpha, beta,
                                    static_cast<float*>(C), ldo));
      break;
  }
  FB_CUDA_OK(cudaGetLastError());
  return FB_OK;
}

// Workspace of one pass: records, the tile count, tensor maps.
static constexpr size_t group_pass_bytes(size_t groups) {
  return (sizeof(GroupRec) * groups + 255) / 256 * 256 + 256 + (sizeof(int) * groups + 255) / 256 * 256 +
         sizeof(CUtensorMap) * 3 * groups;
}
static constexpr size_t group_ws_bytes(size_t groups) { return 2 * group_pass_bytes(groups); }

// Behind the two passes' tables: flags and partial-sum slots of the stream-K tail (optional: a caller that passes
// only the tables' bytes gets whole tiles).
static size_t group_tail_offset(size_t groups) { return round_up(group_ws_bytes(groups), 256); }

size_t fb_group_min_workspace_bytes(int group_count) {
  return group_count <= 0 ? 0 : group_ws_bytes(static_cast<size_t>(group_count));
}

size_t fb_group_workspace_bytes(int group_count) {
  if (group_count <= 0) return 0;
  const size_t base = group_ws_bytes(static_cast<size_t>(group_count));
  const DeviceInfo* di = device_info();
  if (!di || env_int("FLAGBLAS_B200_GROUP_STREAMK", 1) == 0) return base;
  return group_tail_offset(static_cast<size_t>(group_count)) + streamk_bytes(di->sm_count, 256);
}

// `phases`: kGroupBuild = run the table builder, kGroupRun = launch the GEMM over tables already in the workspace;
// a plain call does both.
enum : int { kGroupBuild = 1, kGroupRun = 2 };
static int run_grouped(int dtype, int b_k_contig, GroupSetupArgs ga, float alpha, float beta, long long m_hint,
                       long long n_hint, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                       int phases = kGroupBuild | kGroupRun) {
  const DeviceInfo* di = device_info();
  if (!di) return FB_ERR_LAUNCH;
  if (di->cc_major != 10) return FB_ERR_UNSUPPORTED;
  const int G = ga.num_groups;
  if (!workspace || workspace_bytes < group_ws_bytes(static_cast<size_t>(G)) || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return FB_ERR_WORKSPACE;
  const int esz = elem_size(dtype);
  const uint32_t span = kSwizzleBytes / esz;
  const bool atom32 = esz == 4;
  // Tile plan: one pass of CTA-pair tiles (256 x block_n, two k-slabs per stage).  With
  // FLAGBLAS_B200_GROUP_SPLIT=1 the pair pass takes only the whole 256-row blocks of each group and a
  // second pass of single-CTA tiles (128 x block_n) takes the remaining rows; on the MoE benchmark
  // shape that saves padded rows but loses as much to the slower single-CTA kernel, so it is off by
  // default.  FLAGBLAS_B200_PAIR=0 runs everything in a single-CTA pass; _KS / _TMA3D as in the dense path.
  int block_n = (n_hint > 0 && n_hint <= 64) ? 64 : ((n_hint > 0 && n_hint <= 128) ? 128 : 256);
  const bool pair = env_int("FLAGBLAS_B200_PAIR", 1) != 0 && block_n >= 128;
  const bool split = pair && env_int("FLAGBLAS_B200_GROUP_SPLIT", 0) != 0;
  ga.span = static_cast<int>(span);
  ga.allow3d = env_int("FLAGBLAS_B200_TMA3D", 1) != 0 ? 1 : 0;
  ga.b_k_contig = b_k_contig;
  ga.publish_each = env_int("FLAGBLAS_B200_GROUP_PUBLISH", 1);
  // FLAGBLAS_B200_GROUP_BY_HAND=1: no tensor maps at all, every operand goes through the producers' load / store
  // path that otherwise serves only operands TMA cannot address (tests and comparisons)
  ga.force_by_hand = env_int("FLAGBLAS_B200_GROUP_BY_HAND", 0) != 0 ? 1 : 0;
  ga.esz = esz;

  uint8_t* ws = static_cast<uint8_t*>(workspace);
  GroupPass pass[2] = {};
  int pass_ks[2] = {1, 1};
  bool pass_pair[2] = {false, false};
  for (int i = 0; i < 2; ++i) {
    GroupPass& ps = pass[i];
    uint8_t* base = ws + i * group_pass_bytes(G);
    ps.recs = reinterpret_cast<GroupRec*>(base);
    ps.total_tiles = reinterpret_cast<int*>(base + round_up(sizeof(GroupRec) * static_cast<size_t>(G), 256));
    ps.starts = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(ps.total_tiles) + 256);
    ps.maps = reinterpret_cast<CUtensorMap*>(reinterpret_cast<uint8_t*>(ps.starts) + round_up(sizeof(int) * static_cast<size_t>(G), 256));
    ps.block_n = block_n;
  }
  // One pass of CTA-pair tiles: every whole 256-row block of a group is an ordinary tile, its last, partial block is
  // computed transposed with its row count in the MMA's N slot (FLAGBLAS_B200_GROUP_SWAP=0: an ordinary, padded tile).
  // Small-M plan when the hint says the groups average at most 64 rows (the reference's callers promise that with
  // use_small_m, runtime/backend/_nvidia/hopper/ops/group_gemm.py:717-721; here it only steers the plan, any m_g is
  // still computed): every tile a transposed block of up to 64 rows, deeper operand ring.
  // FLAGBLAS_B200_GROUP_SMALL_M = 0 / 1 forces it off / on.
  const int force_small = env_int("FLAGBLAS_B200_GROUP_SMALL_M", -1);
  const bool small_m = pair && !split && block_n == 256 && env_int("FLAGBLAS_B200_GROUP_SWAP", 1) != 0 &&
                       (force_small == 1 || (force_small != 0 && m_hint > 0 && m_hint <= 64LL * G));
  const bool swap_partial = pair && !split && block_n == 256 && !small_m && env_int("FLAGBLAS_B200_GROUP_SWAP", 1) != 0;
  if (pair) {
    pass[0].enabled = 1; pass[0].tile_m = small_m ? kSmallMRows : 2 * kBlockM; pass_pair[0] = true;
    pass[0].swap_partial = swap_partial ? 1 : 0;
    pass_ks[0] = env_int("FLAGBLAS_B200_KS", 2) == 1 ? 1 : 2;
    if (split) {
      pass[0].rows_mod = 2 * kBlockM; pass[0].leading = 1;
      pass[1].enabled = 1; pass[1].tile_m = kBlockM; pass[1].rows_mod = 2 * kBlockM; pass[1].leading = 0;
      // FLAGBLAS_B200_GROUP_SPLIT=2: only remainders of at most 128 rows go to the single-CTA pass
      if (env_int("FLAGBLAS_B200_GROUP_SPLIT", 0) == 2) pass[0].keep_over = pass[1].keep_over = kBlockM;
    }
  } else {
    pass[0].enabled = 1; pass[0].tile_m = kBlockM;
  }
  // Templates carry everything the device does not patch: dtype, box, swizzle (and, for the 3-D
  // views, the 128-byte innermost extent and the 128-byte pitch of the slab dimension).
  // Their address / extents are placeholders (the workspace itself, a valid 256-byte aligned range).
  for (int i = 0; i < 2; ++i) {
    GroupPass& ps = pass[i];
    if (!ps.enabled) continue;
    const int ks = pass_ks[i];
    const int b_rows = pass_pair[i] ? block_n / 2 : block_n;
    const uint32_t a_box_rows = (small_m && i == 0) ? kSmallMSlot : kBlockM;  // rows of A_g one copy fetches
    int rc = encode_2d(&ps.tmpl_a, dtype, ws, span, kBlockM, kSwizzleBytes, span, a_box_rows);
    if (rc) return rc;
    if (b_k_contig) rc = encode_2d(&ps.tmpl_b, dtype, ws, span, b_rows, kSwizzleBytes, span, b_rows);
    else rc = encode_2d(&ps.tmpl_b, dtype, ws, span, span * ks, kSwizzleBytes, span, span * ks, atom32);
    if (rc) return rc;
    rc = encode_3d(&ps.tmpl_a3, dtype, ws, span, kBlockM, ks, kSwizzleBytes, kSwizzleBytes, span, a_box_rows, ks, false);
    if (!rc) {
      if (b_k_contig)
        rc = encode_3d(&ps.tmpl_b3, dtype, ws, span, b_rows, ks, kSwizzleBytes, kSwizzleBytes, span, b_rows, ks, false);
      else
        rc = encode_3d(&ps.tmpl_b3, dtype, ws, span, span * ks, b_rows / span, kSwizzleBytes, kSwizzleBytes, span,
                       span * ks, b_rows / span, atom32);
    }
    if (rc) {  // no 3-D views on this driver: every group uses 2-D boxes
      ga.allow3d = 0;
      ps.tmpl_a3 = ps.tmpl_a;
      ps.tmpl_b3 = ps.tmpl_b;
    }
  }

  // Stream-K tail of the (single) pass: when the last wave of tiles is at most half full, each of its tiles is
  // shared by 2-4 neighbouring workers (the split is derived on the device, where the tile count is known).  Needs
  // the scratch behind the tables; FLAGBLAS_B200_GROUP_STREAMK=0 switches it off.
  uint8_t* tail = nullptr;
  if (!split && env_int("FLAGBLAS_B200_GROUP_STREAMK", 1) != 0 &&
      workspace_bytes >= group_tail_offset(static_cast<size_t>(G)) + streamk_bytes(di->sm_count, block_n)) {
    tail = ws + group_tail_offset(static_cast<size_t>(G));
  }
  if (tail) streamk_gate(stream);

  // The builder is itself a programmatic dependent of whatever precedes it on the stream (typically the previous
  // grouped GEMM, which reads the same tables): it becomes resident as that kernel drains and waits for its
  // completion before writing anything.
  // builder CTAs (32 groups at a time each, at most 16 of them) + the CTA that scans the tile counts
  int builders = (G + kSetupThreads / 32 - 1) / (kSetupThreads / 32);
  if (builders > 16) builders = 16;
  const unsigned setup_ctas = static_cast<unsigned>(builders + 1);
  if (phases & kGroupBuild) {
    if (env_int("FLAGBLAS_B200_PDL", 1) != 0) {
      FB_CUDA_OK(launch_dependent(group_setup_kernel, setup_ctas, kSetupThreads, stream, pass[0], pass[1], ga));
    } else {
      group_setup_kernel<<<setup_ctas, kSetupThreads, 0, stream>>>(pass[0], pass[1], ga);
      FB_CUDA_OK(cudaGetLastError());
    }
  }
  if (!(phases & kGroupRun)) return FB_OK;

  for (int i = 0; i < 2; ++i) {
    const GroupPass& ps = pass[i];
    if (!ps.enabled) continue;
    const int ks = pass_ks[i];
    const int b_rows = pass_pair[i] ? block_n / 2 : block_n;
    TcGemmParams p{};
    p.alpha = alpha; p.beta = beta;
    p.idesc = make_idesc(idesc_fmt(dtype), 0, b_k_contig ? 0 : 1, ps.tile_m, block_n);
    p.block_k = span * ks;
    p.ks = ks;
    p.a = make_geom(esz, kBlockM, false, ks, false);
    p.b = make_geom(esz, b_rows, !b_k_contig, ks, false);
    p.num_groups = G;
    p.swap_partial = ps.swap_partial;
    p.small_m = (small_m && i == 0) ? 1 : 0;
    p.idesc_swapped = make_idesc(idesc_fmt(dtype), b_k_contig ? 0 : 1, 0, block_n, 0);  // M slot = the tile's columns
    p.groups = ps.recs;
    p.group_starts = ps.starts;
    p.total_tiles = ps.total_tiles;
    p.group_maps = ps.maps;
    if (tail) {
      p.sk_grouped = 1;
      p.sk_head = (env_int("FLAGBLAS_B200_SK_HEAD", 12) + ks - 1) / ks;
      p.sk_flags = reinterpret_cast<int*>(tail);
      p.sk_partials = reinterpret_cast<float*>(tail + kStreamKFlagBytes);
    }
    const int rc = dispatch_tc(dtype, block_n, pass_pair[i], ps.tmpl_a, ps.tmpl_b, ps.tmpl_a, p, /*tiles=*/-1, di->sm_count, stream);
    if (rc) return rc;
  }
  return FB_OK;
}

int fb_group_gemm(int dtype, int b_k_contiguous, const int64_t* d_a, const int64_t* d_b, const int64_t* d_c,
                  const int64_t* d_out, const int32_t* d_m, const int32_t* d_n, const int32_t* d_k,
                  const int32_t* d_lda, const int32_t* d_ldb, const int32_t* d_ldc, int group_count, int64_t m_hint,
                  int64_t n_hint, int64_t k_hint, float alpha, float beta, void* workspace, size_t workspace_bytes,
                  void* stream) {
  (void)k_hint;
  if (dtype != FB_TF32 && dtype != FB_F16 && dtype != FB_BF16) return FB_ERR_INVALID_ARG;
  if (group_count < 0) return FB_ERR_INVALID_ARG;
  if (group_count == 0) return FB_OK;
  if (!d_a || !d_b || !d_out || !d_m || !d_n || !d_k || !d_lda || !d_ldb || !d_ldc) return FB_ERR_INVALID_ARG;
  if (beta != 0.f && !d_c) return FB_ERR_INVALID_ARG;
  GroupSetupArgs ga{};
  ga.mode = 0;
  ga.a_ptrs = reinterpret_cast<const long long*>(d_a);
  ga.b_ptrs = reinterpret_cast<const long long*>(d_b);
  ga.c_ptrs = reinterpret_cast<const long long*>(d_c ? d_c : d_out);
  ga.out_ptrs = reinterpret_cast<const long long*>(d_out);
  ga.m_sizes = d_m; ga.n_sizes = d_n; ga.k_sizes = d_k;
  ga.ldas = d_lda; ga.ldbs = d_ldb; ga.ldcs = d_ldc;
  ga.num_groups = group_count;
  return run_grouped(dtype, b_k_contiguous ? 1 : 0, ga, alpha, beta, m_hint, n_hint, workspace, workspace_bytes,
                     static_cast<cudaStream_t>(stream));
}

int fb_group_gemm_prepare(int dtype, int b_k_contiguous, const int64_t* d_a, const int64_t* d_b, const int64_t* d_c,
                          const int64_t* d_out, const int32_t* d_m, const int32_t* d_n, const int32_t* d_k,
                          const int32_t* d_lda, const int32_t* d_ldb, const int32_t* d_ldc, int group_count,
                          int64_t m_hint, int64_t n_hint, int64_t k_hint, void* workspace, size_t workspace_bytes,
                          void* stream) {
  (void)k_hint;
  if (dtype != FB_TF32 && dtype != FB_F16 && dtype != FB_BF16) return FB_ERR_INVALID_ARG;
  if (group_count < 0) return FB_ERR_INVALID_ARG;
  if (group_count == 0) return FB_OK;
  if (!d_a || !d_b || !d_out || !d_m || !d_n || !d_k || !d_lda || !d_ldb || !d_ldc) return FB_ERR_INVALID_ARG;
  GroupSetupArgs ga{};
  ga.mode = 0;
  ga.a_ptrs = reinterpret_cast<const long long*>(d_a);
  ga.b_ptrs = reinterpret_cast<const long long*>(d_b);
  ga.c_ptrs = reinterpret_cast<const long long*>(d_c ? d_c : d_out);
  ga.out_ptrs = reinterpret_cast<const long long*>(d_out);
  ga.m_sizes = d_m; ga.n_sizes = d_n; ga.k_sizes = d_k;
  ga.ldas = d_lda; ga.ldbs = d_ldb; ga.ldcs = d_ldc;
  ga.num_groups = group_count;
  return run_grouped(dtype, b_k_contiguous ? 1 : 0, ga, 1.f, 0.f, m_hint, n_hint, workspace, workspace_bytes,
                     static_cast<cudaStream_t>(stream), kGroupBuild);
}

int fb_group_gemm_run(int dtype, int b_k_contiguous, int group_count, int64_t m_hint, int64_t n_hint, int64_t k_hint,
                      float alpha, float beta, void* workspace, size_t workspace_bytes, void* stream) {
  (void)k_hint;
  if (dtype != FB_TF32 && dtype != FB_F16 && dtype != FB_BF16) return FB_ERR_INVALID_ARG;
  if (group_count < 0) return FB_ERR_INVALID_ARG;
  if (group_count == 0) return FB_OK;
  GroupSetupArgs ga{};
  ga.num_groups = group_count;
  return run_grouped(dtype, b_k_contiguous ? 1 : 0, ga, alpha, beta, m_hint, n_hint, workspace, workspace_bytes,
                     static_cast<cudaStream_t>(stream), kGroupRun);
}

int fb_group_mm(int dtype, int b_k_contiguous, const void* A, int64_t lda, const void* B, int64_t ldb,
                int64_t b_group_stride, void* C, int64_t ldc, const int32_t* d_offs, int group_count, int64_t n,
                int64_t k, void* workspace, size_t workspace_bytes, void* stream) {
  if (dtype != FB_F16 && dtype != FB_BF16 && dtype != FB_TF32) return FB_ERR_INVALID_ARG;
  if (group_count < 0 || n < 0 || k < 0) return FB_ERR_INVALID_ARG;
  if (n > 0x7fffffffLL || k > 0x7fffffffLL) return FB_ERR_UNSUPPORTED;
  if (group_count == 0 || n == 0) return FB_OK;
  if (!A || !B || !C || !d_offs) return FB_ERR_INVALID_ARG;
  if (lda < k || ldc < n || ldb < (b_k_contiguous ? k : n)) return FB_ERR_INVALID_ARG;
  GroupSetupArgs ga{};
  ga.mode = 1;
  ga.offs = d_offs;
  ga.a_base = A; ga.b_base = B; ga.out_base = C;
  ga.mm_lda = lda; ga.mm_ldb = ldb; ga.mm_b_group_stride = b_group_stride; ga.mm_ldo = ldc;
  ga.mm_n = static_cast<int>(n); ga.mm_k = static_cast<int>(k);
  ga.num_groups = group_count;
  return run_grouped(dtype, b_k_contiguous ? 1 : 0, ga, 1.f, 0.f, /*m_hint=*/0, n, workspace, workspace_bytes,
                     static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------
// Grouped GEMM for callers that must not allocate.
//
// fb_group_gemm needs a little device scratch per call (the tile table and the per-group tensor
// maps that its set-up kernel writes).  Normally the caller passes that in.  Some callers cannot:
// code running inside another runtime's "enqueue" hook whose contract forbids allocation, and
// processes that have already handed every byte of HBM to their own memory pool, where a
// cudaMalloc would fail or stall the device.  For them the scratch lives here, in a fixed
// array that is part of the library image: every GPU that loads the library carries these
// bytes until the process exits, which is why the capacity is kept small.
constexpr int kNoAllocMaxGroups = 256;
constexpr size_t kNoAllocScratchBytes = group_ws_bytes(kNoAllocMaxGroups);
static __device__ __align__(256) unsigned char g_no_alloc_scratch[kNoAllocScratchBytes];

// In host code `g_no_alloc_scratch` is only a handle for the runtime, not an address a kernel can
// use; the device address is looked up once per device and cached here.
static void* g_no_alloc_ptr[64] = {};
static std::mutex g_no_alloc_mu;

static int no_alloc_scratch(void** out) {
  int dev = 0;
  FB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return FB_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lk(g_no_alloc_mu);
  if (!g_no_alloc_ptr[dev]) {
    void* p = nullptr;
    FB_CUDA_OK(cudaGetSymbolAddress(&p, g_no_alloc_scratch));  // address on the current device
    g_no_alloc_ptr[dev] = p;
  }
  *out = g_no_alloc_ptr[dev];
  return FB_OK;
}

int fb_group_gemm_no_alloc(int dtype, int b_k_contiguous, const int64_t* d_a, const int64_t* d_b, const int64_t* d_c,
                           const int64_t* d_out, const int32_t* d_m, const int32_t* d_n, const int32_t* d_k,
                           const int32_t* d_lda, const int32_t* d_ldb, const int32_t* d_ldc, int group_count,
                           int64_t m_hint, int64_t n_hint, int64_t k_hint, float alpha, float beta, void* stream) {
  if (group_count > kNoAllocMaxGroups) return FB_ERR_TOO_LARGE;
  void* scratch = nullptr;
  const int rc = no_alloc_scratch(&scratch);
  if (rc) return rc;
  // Same set-up kernel, same GEMM kernel, same arithmetic as fb_group_gemm; only the scratch differs.
  // The set-up kernel rewrites every record, map and the tile count it later reads, so nothing in the
  // array has to be cleared between calls.
  return fb_group_gemm(dtype, b_k_contiguous, d_a, d_b, d_c, d_out, d_m, d_n, d_k, d_lda, d_ldb, d_ldc, group_count,
                       m_hint, n_hint, k_hint, alpha, beta, scratch, kNoAllocScratchBytes, stream);
}

int fb_no_alloc_max_groups(void) { return kNoAllocMaxGroups; }

size_t fb_gemv_workspace_bytes(int dtype, int trans, int64_t m, int64_t n) {
  if (m <= 0 || n <= 0 || (dtype != FB_F32 && dtype != FB_F16 && dtype != FB_BF16)) return 0;
  const DeviceInfo* di = device_info();
  if (!di) return 0;
  const GemvPlan pl = plan_gemv(trans, m, n, elem_size(dtype), di->sm_count);
  if (pl.splits <= 1) return 0;
  return static_cast<size_t>(pl.splits) * static_cast<size_t>(trans == FB_OP_N ? m : n) * sizeof(float);
}

int fb_gemv(int dtype, int trans, int64_t m, int64_t n, float alpha, const void* A, int64_t lda, const void* x,
            int64_t incx, float beta, void* y, int64_t incy, void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (dtype != FB_F32 && dtype != FB_F16 && dtype != FB_BF16) return FB_ERR_INVALID_ARG;
  if (trans != FB_OP_N && trans != FB_OP_T) return FB_ERR_INVALID_ARG;
  if (m < 0 || n < 0 || incx <= 0 || incy <= 0) return FB_ERR_INVALID_ARG;
  if (m > 0x7fffffffLL || n > 0x7fffffffLL) return FB_ERR_UNSUPPORTED;
  if (m == 0 || n == 0) return FB_OK;
  if (!y) return FB_ERR_INVALID_ARG;
  if (alpha != 0.f && (!A || !x || lda < n)) return FB_ERR_INVALID_ARG;
  const DeviceInfo* di = device_info();
  if (!di) return FB_ERR_LAUNCH;
  if (di->cc_major != 10) return FB_ERR_UNSUPPORTED;
  switch (dtype) {
    case FB_F16:
      return run_gemv<__half>(trans, m, n, alpha, A, lda, x, incx, beta, y, incy, workspace, workspace_bytes,
                              di->sm_count, stream);
    case FB_BF16:
      return run_gemv<__nv_bfloat16>(trans, m, n, alpha, A, lda, x, incx, beta, y, incy, workspace, workspace_bytes,
                                     di->sm_count, stream);
    default:
      return run_gemv<float>(trans, m, n, alpha, A, lda, x, incx, beta, y, incy, workspace, workspace_bytes,
                             di->sm_count, stream);
  }
}

size_t fb_gemv_fp8_workspace_bytes(int64_t m, int64_t n) {
  if (m <= 0 || n <= 0) return 0;
  const DeviceInfo* di = device_info();
  if (!di) return 0;
  const GemvPlan pl = plan_gemv(FB_OP_T, m, n, 1, di->sm_count);
  return pl.splits <= 1 ? 0 : static_cast<size_t>(pl.splits) * static_cast<size_t>(n) * sizeof(float);
}

int fb_gemv_fp8(int a_format, int x_format, int y_dtype, int64_t m, int64_t n, float alpha, const void* A, int64_t lda,
                const void* x, int64_t incx, float beta, void* y, int64_t incy, void* workspace,
                size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if ((a_format != FB_FP8_E4M3 && a_format != FB_FP8_E5M2) || (x_format != FB_FP8_E4M3 && x_format != FB_FP8_E5M2))
    return FB_ERR_INVALID_ARG;
  if (y_dtype != FB_F32 && y_dtype != FB_F16 && y_dtype != FB_BF16) return FB_ERR_INVALID_ARG;
  if (m < 0 || n < 0 || incx <= 0 || incy <= 0) return FB_ERR_INVALID_ARG;
  if (m > 0x7fffffffLL || n > 0x7fffffffLL) return FB_ERR_UNSUPPORTED;
  if (m == 0 || n == 0) return FB_OK;
  if (!y) return FB_ERR_INVALID_ARG;
  if (alpha != 0.f && (!A || !x || lda < n)) return FB_ERR_INVALID_ARG;
  const DeviceInfo* di = device_info();
  if (!di) return FB_ERR_LAUNCH;
  if (di->cc_major != 10) return FB_ERR_UNSUPPORTED;
  const int sms = di->sm_count;
  if (a_format == FB_FP8_E4M3) {
    if (x_format == FB_FP8_E4M3)
      return run_gemv_fp8_y<__nv_fp8_e4m3, __nv_fp8_e4m3>(y_dtype, m, n, alpha, A, lda, x, incx, beta, y, incy, workspace, workspace_bytes, sms, stream);
    return run_gemv_fp8_y<__nv_fp8_e4m3, __nv_fp8_e5m2>(y_dtype, m, n, alpha, A, lda, x, incx, beta, y, incy, workspace, workspace_bytes, sms, stream);
  }
  if (x_format == FB_FP8_E4M3)
    return run_gemv_fp8_y<__nv_fp8_e5m2, __nv_fp8_e4m3>(y_dtype, m, n, alpha, A, lda, x, incx, beta, y, incy, workspace, workspace_bytes, sms, stream);
  return run_gemv_fp8_y<__nv_fp8_e5m2, __nv_fp8_e5m2>(y_dtype, m, n, alpha, A, lda, x, incx, beta, y, incy, workspace, workspace_bytes, sms, stream);
}

int fb_gemm_ex(int dtype, int transa, int transb, int64_t m, int64_t n, int64_t k, const double* alpha, const void* A,
               int64_t lda, const void* B, int64_t ldb, const double* beta, void* C, int64_t ldc, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (dtype != FB_F64 && dtype != FB_C64 && dtype != FB_C128) return FB_ERR_INVALID_ARG;
  const bool cplx = dtype != FB_F64;
  const int max_op = cplx ? FB_OP_C : FB_OP_T;
  if (transa < 0 || transa > max_op || transb < 0 || transb > max_op) return FB_ERR_INVALID_ARG;
  if (m < 0 || n < 0 || k < 0 || !alpha || !beta) return FB_ERR_INVALID_ARG;
  if (m > 0x7fffffffLL || n > 0x7fffffffLL || k > 0x7fffffffLL) return FB_ERR_UNSUPPORTED;
  if (m == 0 || n == 0) return FB_OK;
  if (!C || ldc < n) return FB_ERR_INVALID_ARG;
  const bool scale_only = k == 0 || (alpha[0] == 0.0 && (!cplx || alpha[1] == 0.0));
  if (!scale_only) {
    if (!A || !B) return FB_ERR_INVALID_ARG;
    if (lda < (transa ? m : k) || ldb < (transb ? k : n)) return FB_ERR_INVALID_ARG;
  }
  const DeviceInfo* di = device_info();
  if (!di) return FB_ERR_LAUNCH;
  if (di->cc_major != 10) return FB_ERR_UNSUPPORTED;
  switch (dtype) {
    case FB_F64: return run_xgemm<double>(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, false, stream);
    case FB_C64: return run_xgemm<cfloat>(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, true, stream);
    default: return run_xgemm<cdouble>(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, true, stream);
  }
}

int fb_trmm(int dtype, int side, int uplo, int trans, int diag, int64_t m, int64_t n, const double* alpha, const void* A,
            int64_t lda, const void* B, int64_t ldb, void* C, int64_t ldc, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (dtype != FB_F32 && dtype != FB_F64 && dtype != FB_C64 && dtype != FB_C128) return FB_ERR_INVALID_ARG;
  const bool cplx = dtype == FB_C64 || dtype == FB_C128;
  if ((side != 0 && side != 1) || (uplo != 0 && uplo != 1) || (diag != 0 && diag != 1)) return FB_ERR_INVALID_ARG;
  if (trans < 0 || trans > (cplx ? FB_OP_C : FB_OP_T)) return FB_ERR_INVALID_ARG;
  if (m < 0 || n < 0 || !alpha) return FB_ERR_INVALID_ARG;
  if (m > 0x7fffffffLL || n > 0x7fffffffLL) return FB_ERR_UNSUPPORTED;
  if (m == 0 || n == 0) return FB_OK;
  const int64_t kdim = side == 0 ? m : n;
  if (!C || ldc < n) return FB_ERR_INVALID_ARG;
  const bool zero = alpha[0] == 0.0 && (!cplx || alpha[1] == 0.0);
  if (!zero && (!A || !B || lda < kdim || ldb < n)) return FB_ERR_INVALID_ARG;
  const DeviceInfo* di = device_info();
  if (!di) return FB_ERR_LAUNCH;
  if (di->cc_major != 10) return FB_ERR_UNSUPPORTED;
  const double beta[2] = {0.0, 0.0};
  // left:  C[m,n] = alpha * op(tri A)[m,m] * B[m,n]  -> GEMM operands (A, trans) x (B, N), k = m
  // right: C[m,n] = alpha * B[m,n] * op(tri A)[n,n]  -> GEMM operands (B, N) x (A, trans), k = n
  const void* ga = side == 0 ? A : B;
  const void* gb = side == 0 ? B : A;
  const int64_t glda = side == 0 ? lda : ldb, gldb = side == 0 ? ldb : lda;
  const int ta = side == 0 ? trans : 0, tb = side == 0 ? 0 : trans;
  const int tri = zero ? 0 : (side == 0 ? 1 : 2);
  switch (dtype) {
    case FB_F32: return run_xgemm<float>(ta, tb, m, n, kdim, alpha, ga, glda, gb, gldb, beta, C, ldc, false, stream, tri, uplo, diag);
    case FB_F64: return run_xgemm<double>(ta, tb, m, n, kdim, alpha, ga, glda, gb, gldb, beta, C, ldc, false, stream, tri, uplo, diag);
    case FB_C64: return run_xgemm<cfloat>(ta, tb, m, n, kdim, alpha, ga, glda, gb, gldb, beta, C, ldc, true, stream, tri, uplo, diag);
    default: return run_xgemm<cdouble>(ta, tb, m, n, kdim, alpha, ga, glda, gb, gldb, beta, C, ldc, true, stream, tri, uplo, diag);
  }
}

const char* fb_status_string(int status) {
  switch (status) {
    case FB_OK: return "ok";
    case FB_ERR_INVALID_ARG: return "invalid argument";
    case FB_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case FB_ERR_LAUNCH: return "CUDA error at launch";
    case FB_ERR_UNSUPPORTED: return "unsupported device or size";
    case FB_ERR_DRIVER: return "tensor-map encoding failed";
    case FB_ERR_TOO_LARGE: return "request exceeds a fixed capacity (more groups than the built-in scratch holds)";
    case DEV_TIMEOUT_PRODUCER_EMPTY: return "device: TMA producer timed out waiting for a free stage";
    case DEV_TIMEOUT_MMA_FULL: return "device: MMA issuer timed out waiting for operand data";
    case DEV_TIMEOUT_MMA_TMEM_EMPTY: return "device: MMA issuer timed out waiting for a free accumulator";
    case DEV_TIMEOUT_EPI_TMEM_FULL: return "device: epilogue timed out waiting for an accumulator";
    case DEV_TIMEOUT_TEST_FLAG: return "device: self-test wait timed out (expected)";
    case DEV_TIMEOUT_PEER: return "device: CTA-pair handshake timed out";
    case DEV_TIMEOUT_STREAMK_PARTIAL: return "device: timed out waiting for another worker's partial sums of a shared tile";
    case DEV_TIMEOUT_CLUSTER_SUMS: return "device: timed out waiting for the sums of the other CTAs of a split-k cluster";
    case DEV_GROUP_MISALIGNED: return "device: a group's A / B address or pitch is not a multiple of the element size; group skipped";
    default: return "unknown status";
  }
}

int fb_device_status(int reset) {
  int v = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return FB_ERR_LAUNCH;
  if (cudaMemcpyFromSymbol(&v, g_fb_status, sizeof(int)) != cudaSuccess) return FB_ERR_LAUNCH;
  if (reset && v != 0) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_fb_status, &zero, sizeof(int)) != cudaSuccess) return FB_ERR_LAUNCH;
  }
  return v;
}

int fb_last_cuda_error(void) { return t_last_cuda_error; }

#ifndef FB_BUILD_ID
#define FB_BUILD_ID "unversioned"
#endif
const char* fb_build_id(void) { return FB_BUILD_ID; }

void fb_reload_env(void) { g_env_generation.fetch_add(1, std::memory_order_acq_rel); }

void fb_debug_set_profile_buffer(void* device_buffer_16_int64) {
  g_prof_buffer = static_cast<long long*>(device_buffer_16_int64);
}

int fb_sm_count(void) {
  const DeviceInfo* di = device_info();
  return di ? di->sm_count : 0;
}

int fb_selftest_bounded_wait(int64_t limit_cycles, void* stream) {
  if (limit_cycles <= 0 || limit_cycles > 4000000000LL) return FB_ERR_INVALID_ARG;
  bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_cycles);
  FB_CUDA_OK(cudaGetLastError());
  return fb_device_status(1);
}

}  // extern "C"
