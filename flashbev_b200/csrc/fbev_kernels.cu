// Forward, backward and index kernels of the fused BEV pooling operator for sm_100a,
// and the C ABI declared in include/fbev.h.
//
// Work decomposition (forward and backward alike).  A thread block owns a
// TX x TY tile of BEV cells of one batch sample.  It copies that sample's camera
// matrices into shared memory, drops the cameras that cannot see the tile
// (camera_may_see), and then each warp takes groups of CPW neighbouring cells:
//
//   list phase   the 32 lanes evaluate the group's (cell, camera, z) candidates,
//                one candidate per lane: projection, rejection tests, bilinear
//                weights, depth weight.  Accepted samples are compacted, in the
//                reference's camera-major / z-minor order, into a per-cell record
//                list in shared memory.  Geometry is therefore computed once per
//                sample, not once per channel as in the reference kernel
//                (flash_bevpool_cuda.cu:31-33, one thread per (cell, channel)).
//   channel phase GL lanes share a cell; each owns V 16-byte chunks of the channel
//                vector, walks the cell's record list and gathers the four
//                corner texels with 128-bit loads, accumulating in float32
//                registers.  The result leaves with one 16-byte store per chunk.
//
// No frustum, voxel or sample tensor is ever written to global memory.
//
// Files: fbev_device.cuh (arithmetic of one candidate), fbev_lists.cuh (block state, list phases),
// fbev_forward.cuh, fbev_backward.cuh, fbev_sort.cuh, fbev_misc.cuh (kernels), this file (plans, launches and
// the C ABI).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "fbev.h"
#include "fbev_debug.h"
#include "fbev_device.cuh"
#include "fbev_lists.cuh"
#include "fbev_forward.cuh"
#include "fbev_backward.cuh"
#include "fbev_sort.cuh"
#include "fbev_misc.cuh"
#include "fbev_deterministic.cuh"

namespace fbev {

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
// Launch tuning of experiments and tests (fbev_debug.h).  Per host thread: a launch reads the values its own
// thread set, so one thread's experiments never change the kernels another thread launches.
struct Tuning {
  int tx, ty, v, warps, minb;
};
static thread_local Tuning g_tuning = {0, 0, 0, 0, 0};
static thread_local int g_experiment = 0;  // FBEV_EXP_* bits (fbev_debug.h)

static size_t elem_size(int dtype) { return dtype == FBEV_F32 ? 4 : 2; }
static bool is_categorical(int mode) { return mode == FBEV_DEPTH_CATEGORICAL || mode == FBEV_DEPTH_CATEGORICAL_LOGITS; }

static int validate(const FbevProblem* p) {
  if (p == nullptr) return FBEV_ERR_NULL;
  if (p->struct_size != sizeof(FbevProblem)) return FBEV_ERR_STRUCT;
  if (p->dtype != FBEV_F32 && p->dtype != FBEV_BF16 && p->dtype != FBEV_F16) return FBEV_ERR_DTYPE;
  if (p->out_dtype != p->dtype && p->out_dtype != FBEV_F32) return FBEV_ERR_DTYPE;
  if (p->B <= 0 || p->N <= 0 || p->H <= 0 || p->W <= 0 || p->C <= 0 || p->D <= 0 || p->X <= 0 || p->Y <= 0 ||
      p->Z <= 0)
    return FBEV_ERR_SHAPE;
  if (p->proj_stride != 12 && p->proj_stride != 16) return FBEV_ERR_SHAPE;
  if (p->y_begin < 0 || p->y_end > p->Y || p->y_begin > p->y_end) return FBEV_ERR_SHAPE;
  if (p->mode != FBEV_DEPTH_GAUSSIAN && p->mode != FBEV_DEPTH_LAPLACE && !is_categorical(p->mode)) return FBEV_ERR_MODE;
  if (p->pool != FBEV_POOL_MEAN && p->pool != FBEV_POOL_SUM) return FBEV_ERR_MODE;
  if (is_categorical(p->mode) && !(p->depth_delta > 0.0f)) return FBEV_ERR_MODE;
  if (!is_categorical(p->mode) && p->D != 2) return FBEV_ERR_SHAPE;
  if (p->mode == FBEV_DEPTH_CATEGORICAL_LOGITS && p->depth_stats == nullptr) return FBEV_ERR_NULL;
  if ((uintptr_t)p->depth_stats % 8) return FBEV_ERR_ALIGN;
  if (!p->image_feats || !p->depth || !p->projection || !p->feature_size || !p->image_size) return FBEV_ERR_NULL;
  const size_t es = elem_size(p->dtype);
  if (((uintptr_t)p->image_feats % es) || ((uintptr_t)p->depth % es) || ((uintptr_t)p->projection % 4) ||
      ((uintptr_t)p->feature_size % 4) || ((uintptr_t)p->image_size % 4) || ((uintptr_t)p->roi_range % 4) ||
      ((uintptr_t)p->status % 4) || ((uintptr_t)p->workspace % 16))
    return FBEV_ERR_ALIGN;
  // texel indices are 32-bit inside the kernels; block index is a 31-bit int
  if ((unsigned long long)p->B * p->N * p->H * p->W >= (1ull << 31)) return FBEV_ERR_RANGE;
  if ((unsigned long long)p->B * p->Y * p->X >= (1ull << 31)) return FBEV_ERR_RANGE;
  if (p->N > 1024) return FBEV_ERR_RANGE;
  return FBEV_OK;
}

static void fill_dev(const FbevProblem* p, Dev& d) {
  d = Dev{};
  d.feats = p->image_feats;
  d.depth = p->depth;
  d.proj = p->projection;
  d.fsize = p->feature_size;
  d.isize = p->image_size;
  d.roi = p->roi_range;
  d.status = p->status;
  d.sched = reinterpret_cast<unsigned*>(p->workspace);
  d.exp = g_experiment;
  d.saved = reinterpret_cast<uint4*>(p->saved_state);
  d.saved_bytes = p->saved_state_bytes;
  d.saved_B = p->B;
  d.saved_b0 = 0;
  d.out_f32 = (p->out_dtype == FBEV_F32 && p->dtype != FBEV_F32) ? 1 : 0;
  d.B = p->B; d.N = p->N; d.H = p->H; d.W = p->W; d.C = p->C; d.D = p->D;
  d.X = p->X; d.Y = p->Y; d.Z = p->Z;
  d.pstride = p->proj_stride;
  // inside the kernels logits are the categorical mode with per-texel softmax statistics at hand
  d.mode = is_categorical(p->mode) ? (int)FBEV_DEPTH_CATEGORICAL : p->mode;
  d.dstat = p->mode == FBEV_DEPTH_CATEGORICAL_LOGITS ? reinterpret_cast<const float2*>(p->depth_stats) : nullptr;
  d.pool = p->pool;
  d.y0 = p->y_begin; d.y1 = p->y_end;
  d.out_rows = p->compact_rows ? p->y_end - p->y_begin : p->Y;
  d.out_y0 = p->compact_rows ? p->y_begin : 0;
  d.eps = p->epsilon; d.thr = p->threshold; d.d0 = p->depth_d0; d.delta = p->depth_delta;
  for (int i = 0; i < 3; ++i) {
    d.vs[i] = p->voxel_size[i];
    d.vmin[i] = p->voxel_min[i];
  }
}

struct Plan {
  bool chunked;
  int V, GL, CPW, warps, cap;
  size_t smem;
  int blocks;
};

// Chooses the lane layout.  chunks = 16-byte chunks per texel.  A lane owns V of
// them; GL = chunks / V lanes share a cell; CPW = 32 / GL cells per warp.
// wide_ok: four chunks per lane may be chosen for float32 (measured: better everywhere but in the categorical
// depth-gradient kernel on small grids, see wide_depth_pays).
static Plan make_plan(const FbevProblem* p, Dev& d, bool bwd, const void* a, const void* b2, const void* c,
                      bool wide_ok = true) {
  Plan pl{};
  const size_t es = elem_size(p->dtype);
  const size_t row = (size_t)p->C * es;
  const bool aligned = (row % 16 == 0) && ((uintptr_t)a % 16 == 0) && ((uintptr_t)b2 % 16 == 0) &&
                       ((uintptr_t)c % 16 == 0);
  const int chunks = aligned ? (int)(row / 16) : 0;
  // the chunked kernels index texels, feature chunks and depth elements with 32 bits
  pl.chunked = aligned && chunks <= 128 && (unsigned long long)p->B * p->N * p->H * p->W * (unsigned long long)p->D < (1ull << 32);
  pl.warps = g_tuning.warps > 0 ? (g_tuning.warps > kMaxWarps ? kMaxWarps : g_tuning.warps) : (bwd ? 8 : 4);
  pl.cap = 32;
  if (pl.chunked) {
    int bestV = 0;
    double best = -1.0;
    const int vs_[3] = {1, 2, 4};
    for (int i = 0; i < 3; ++i) {
      const int V = vs_[i];
      if (chunks % V) continue;
      const int GL = chunks / V;
      if (GL > 32) continue;
      const int CPW = 32 / GL < kMaxCellsPerWarp ? 32 / GL : kMaxCellsPerWarp;
      // lane utilisation first
      double score = (double)(CPW * GL) / 32.0;
      // at equal utilisation: as many chunks per lane as sixteen float32 accumulators hold (two of a 16-bit
      // type, four of float32) -- more cells per warp share one list phase; beyond that registers run out
      if (V * (es == 4 ? 4 : 8) <= 16 && (V < 4 || wide_ok)) score += 0.01 * V;
      if (score > best) {
        best = score;
        bestV = V;
      }
    }
    if (g_tuning.v > 0 && chunks % g_tuning.v == 0 && chunks / g_tuning.v <= 32 &&
        (g_tuning.v == 1 || g_tuning.v == 2 || g_tuning.v == 4))
      bestV = g_tuning.v;
    if (bestV == 0) pl.chunked = false;
    pl.V = bestV;
  }
  if (pl.chunked) {
    pl.GL = chunks / pl.V;
    pl.CPW = 32 / pl.GL < kMaxCellsPerWarp ? 32 / pl.GL : kMaxCellsPerWarp;
  } else {
    pl.V = 0;
    pl.GL = 32;
    pl.CPW = 1;
  }
  d.GL = pl.GL;
  d.CPW = pl.CPW;
  d.cpt = pl.chunked ? pl.GL * pl.V : 0;
  d.cap = pl.cap;
  // backward: tile = 16 groups of CPW cells, two passes for eight warps.  forward: small tiles of about 24
  // cells for four warps: a single sample has only some 10^4 cells, and the tail of the last tiles is what
  // a launch waits for.
  int tx = 4 * pl.CPW, ty = 4;
  if (tx > 16) {
    tx /= 2;
    ty *= 2;
  }
  if (!bwd && pl.chunked) {
    tx = pl.CPW * (6 / pl.CPW > 1 ? 6 / pl.CPW : 1);
    ty = 4;
  }
  const bool tile_tuned = g_tuning.minb != 9 && g_tuning.minb != 10 && g_tuning.minb != 16;  // 9 / 10: tile_x / tile_y steer the gather / scatter kernel instead
  d.TX = tile_tuned && g_tuning.tx > 0 ? g_tuning.tx : tx;
  d.TY = tile_tuned && g_tuning.ty > 0 ? g_tuning.ty : ty;
  d.tiles_x = (p->X + d.TX - 1) / d.TX;
  d.tiles_y = (p->y_end - p->y_begin + d.TY - 1) / d.TY;
  pl.blocks = d.tiles_x * d.tiles_y * p->B;
  if (!bwd && pl.chunked &&
      (p->N > 32 ||
       (unsigned long long)p->B * p->N * p->H * p->W * (unsigned long long)(pl.GL * pl.V) >= (1ull << 32))) {
    // the forward keeps the visible cameras in a 32-bit mask and 32-bit chunk indices into the feature
    // tensor in its records: more cameras or a larger tensor take the scalar kernel
    pl.chunked = false;
    pl.V = 0;
    d.GL = pl.GL = 32;
    d.CPW = pl.CPW = 1;
    d.cpt = 0;
  }
  const size_t wb = bwd ? warp_bytes<3>(pl.CPW, pl.cap)
                        : (pl.chunked ? fwd_warp_bytes(pl.CPW, pl.cap) : warp_bytes<2>(pl.CPW, pl.cap));
  pl.smem = header_bytes(p->N) + (size_t)pl.warps * wb;
  return pl;
}

// Four 16-byte chunks per lane in the categorical depth-gradient kernel (and in a training forward, which runs in
// that kernel's layout).  Only float32 is affected: make_plan gives the 16-bit types no bonus for it.  Twice the cells
// per warp then share one list phase, which pays as long as one sample still has enough groups of cells to fill the
// GPU.  Measured: 200 x 200 cells of 80 channels (cfg3) 480 -> 428 us, 128 x 128 cells of 64 channels (cfg1) 58 -> 63 us.
// Decided per sample, so that forward and backward agree whatever slice of the batch a launch covers.
static bool wide_depth_pays(const FbevProblem* p) {
  const size_t row = (size_t)p->C * elem_size(p->dtype);
  if (p->dtype != FBEV_F32 || row % 64 != 0 || row / 64 > 32) return false;
  const int GL = (int)(row / 64);
  const int CPW = 32 / GL < kMaxCellsPerWarp ? 32 / GL : kMaxCellsPerWarp;
  return (size_t)p->X * (size_t)(p->y_end - p->y_begin) / (size_t)CPW >= 4096;
}

// Lays the saved list state (include/fbev.h: FbevProblem.saved_state) out for a launch whose plan is in d: directory
// size, data capacity, plan key, first unit.  Leaves d.saved null when there is no state or it cannot even hold the
// directory.  Forward and backward call this with the same plan, so they agree on every field.
static void setup_saved(Dev& d, int CPW) {
  uint4* base = d.saved;
  d.saved = nullptr;
  if (base == nullptr || CPW <= 0 || CPW > 8 || d.cap <= 0 || d.cap > 16) return;  // counts are packed in 6 / 5 bits
  const unsigned long long ngroups = (unsigned long long)(d.TX * d.TY + CPW - 1) / CPW;
  const unsigned long long per_sample = (unsigned long long)d.tiles_x * d.tiles_y * ngroups;
  const unsigned long long passes = ((unsigned long long)d.N * d.Z + d.cap - 1) / d.cap;
  const unsigned long long dir = per_sample * (unsigned long long)d.saved_B * passes;
  const unsigned long long units16 = d.saved_bytes / 16;
  const unsigned long long dir16 = dir;  // one 16-byte entry per (unit, pass)
  if (dir == 0 || dir >= (1ull << 32) || units16 < 1 + dir16 + 64) return;
  unsigned long long cap16 = units16 - 1 - dir16;
  if (cap16 > 0xfffffff0ull - dir16) cap16 = 0xfffffff0ull - dir16;  // offsets are 32-bit
  d.saved = base;
  d.saved_dir = (unsigned)dir;
  d.saved_cap = (unsigned)cap16;
  d.saved_passes = (int)passes;
  d.saved_unit0 = (unsigned)(per_sample * (unsigned long long)d.saved_b0);
  // the saved indices count from the first sample of the forward's batch; this launch's tensors start at sample b0
  const unsigned long long tex0 = (unsigned long long)d.saved_b0 * d.N * d.H * d.W;
  d.saved_sub_rec = (unsigned)(tex0 * (unsigned long long)d.cpt);
  d.saved_sub_dep = (unsigned)(tex0 * (unsigned long long)d.D);
  unsigned key = 2166136261u;  // FNV-1a over what fixes the layout of the lists
  const int fields[] = {CPW, d.GL, d.cap, d.TX, d.TY, d.tiles_x, d.tiles_y, d.N, d.Z, d.y0, d.y1, d.X, d.saved_B, d.mode};
  for (int f : fields) {
    key ^= (unsigned)f;
    key *= 16777619u;
  }
  d.saved_key = key | 1u;  // never 0: a cleared header matches nothing
}

static int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Resident blocks per SM of a kernel at a block size and dynamic shared memory size; the runtime's answer is
// remembered (per device: the library is sm_100a only, but the query needs a current device), because asking costs
// about as much as a launch and every launch asks.
static int resident_blocks(const void* kernel, int threads, size_t smem) {
  struct Entry {
    const void* kernel;
    int threads, dev, per_sm;
    size_t smem;
  };
  static Entry cache[64];
  static int used = 0;
  static std::mutex lock;
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> g(lock);
    for (int i = 0; i < used; ++i)
      if (cache[i].kernel == kernel && cache[i].threads == threads && cache[i].smem == smem && cache[i].dev == dev)
        return cache[i].per_sm;
  }
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess || per_sm <= 0) {
    cudaGetLastError();
    per_sm = 1;
  }
  std::lock_guard<std::mutex> g(lock);
  if (used < 64) cache[used++] = Entry{kernel, threads, dev, per_sm, smem};
  return per_sm;
}

// One resident wave when the blocks can draw tiles from the scheduler word or stride over the work themselves
// (static_units), else one block per tile.  static_units is decided here, where the wave is known.
template <typename K>
static int launch(K kernel, const Plan& pl, Dev d, cudaStream_t st, int groups_per_tile = 0) {
  if (pl.blocks <= 0) return FBEV_OK;
  if (pl.smem > 200 * 1024) return FBEV_ERR_RANGE;
  if (pl.smem > 48 * 1024) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem) != cudaSuccess) {
      cudaGetLastError();
      return FBEV_ERR_LAUNCH;
    }
  }
  int blocks = pl.blocks;
  if (d.sched != nullptr || groups_per_tile > 0) {
    // one resident wave
    const int per_sm = resident_blocks(reinterpret_cast<const void*>(kernel), pl.warps * 32, pl.smem);
    const long long wave = (long long)per_sm * sm_count();
    // forward: a single sample with at most three units of work per resident warp takes the barrier-free
    // static order (measured ahead there, behind the counter on larger problems)
    const long long units = (long long)pl.blocks * groups_per_tile;
    const bool few = groups_per_tile > 0 && d.B == 1 && units <= 3 * wave * pl.warps && g_tuning.minb != 14;
    if (few || (groups_per_tile > 0 && g_tuning.minb == 15)) d.static_units = d.B == 1 ? 1 : 0;
    if (d.sched == nullptr && !d.static_units) {
      // no scheduler word and too much work for the static order: one block per tile
    } else if (wave < blocks) {
      blocks = (int)wave;
    }
  }
  kernel<<<blocks, pl.warps * 32, pl.smem, st>>>(d);
  return cudaGetLastError() == cudaSuccess ? FBEV_OK : FBEV_ERR_LAUNCH;
}

// Launch that may overlap the tail of the kernel before it in the stream (programmatic dependent launch); the
// kernel calls grid_dependency_wait() before it touches anything that kernel wrote.
template <typename... KArgs, typename... Args>
static cudaError_t launch_after(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem, cudaStream_t st,
                                Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename T>
static int forward_t(const Plan& pl, const Dev& d, cudaStream_t st) {
  if (!pl.chunked) return launch(fwd_generic_kernel<T>, pl, d, st);
  if (d.saved != nullptr) {  // training forward: also writes the lists the backward needs
    const int gpt = (d.TX * d.TY + pl.CPW - 1) / pl.CPW;
    switch (pl.V) {
      case 1: return launch(fwd_kernel<T, 1, 3, false, kMaxWarps * 32, true>, pl, d, st, gpt);
      case 2: return launch(fwd_kernel<T, 2, 3, false, kMaxWarps * 32, true>, pl, d, st, gpt);
      default: return launch(fwd_kernel<T, 4, 2, false, kMaxWarps * 32, true>, pl, d, st, gpt);
    }
  }
  const bool two = g_tuning.minb == 2;  // compiled for two resident blocks per SM (128 registers) instead of three (80)
  const int gpt = (d.TX * d.TY + pl.CPW - 1) / pl.CPW;  // groups of CPW cells per tile
  switch (pl.V) {
    case 1: return two ? launch(fwd_kernel<T, 1, 2>, pl, d, st, gpt) : launch(fwd_kernel<T, 1, 3>, pl, d, st, gpt);
    case 2:
      if (d.exp != 0 && !two) return launch(fwd_kernel<T, 2, 3, true>, pl, d, st, gpt);
      // experiment: five resident blocks of four warps (96 registers, no spills) instead of six (80)
      if (g_tuning.minb == 3 && pl.warps <= 4) return launch(fwd_kernel<T, 2, 5, false, 128>, pl, d, st, gpt);
      return two ? launch(fwd_kernel<T, 2, 2>, pl, d, st, gpt) : launch(fwd_kernel<T, 2, 3>, pl, d, st, gpt);
    default: return launch(fwd_kernel<T, 4, 2>, pl, d, st, gpt);
  }
}

template <typename T>
static int sort_finish_t(const Plan& pl, const Dev& d, cudaStream_t st, bool fixed = false);

// Feature gradient through the global sort: emission (list phase only), scan, scatter, gather.
template <typename T>
static int backward_feats_sort_t(const Plan& pl, const Dev& d_in, cudaStream_t st) {
  Dev d = d_in;
  d.ent_d = d.ent_d_sorted = nullptr;  // this emitter writes no depth values
  d.flags &= ~FBEV_BWD_DEPTH;
  int rc;
  switch (pl.V) {
    case 1: rc = launch(bwd_feats_kernel<T, 1, true>, pl, d, st, (d.TX * d.TY + pl.CPW - 1) / pl.CPW); break;
    case 2: rc = launch(bwd_feats_kernel<T, 2, true>, pl, d, st, (d.TX * d.TY + pl.CPW - 1) / pl.CPW); break;
    default: rc = launch(bwd_feats_kernel<T, 4, true>, pl, d, st, (d.TX * d.TY + pl.CPW - 1) / pl.CPW); break;
  }
  if (rc != FBEV_OK) return rc;
  return sort_finish_t<T>(pl, d, st);
}

// Scan, scatter and gather of the sorted gradients, after a kernel that called emit_entries.
// fixed: the reproducible backward's gather (64-bit fixed-point sums in d.gfeat).
template <typename T>
static int sort_finish_t(const Plan& pl, const Dev& d, cudaStream_t st, bool fixed) {
  const unsigned texels = (unsigned)((size_t)d.B * d.N * d.H * d.W);
  const int sms = sm_count();
  unsigned* total = d.ent_count + 1;  // second word of the counter block
  if (texels <= kScanInBlock) {
    // experiments: fbev_set_tuning(blocks per SM, threads, 0, 0, 10)
    const unsigned sb = g_tuning.minb == 10 && g_tuning.tx > 0 ? (unsigned)g_tuning.tx : 2u;
    const unsigned stt = g_tuning.minb == 10 && g_tuning.ty > 0 ? (unsigned)g_tuning.ty : 1024u;
    launch_after(ent_scatter_kernel<true>, sms * sb, stt, (size_t)(texels + 1) * 4, st, d, texels, total);
  } else {
    // at most 128 blocks of 1024 threads, `per` counters per thread
    const unsigned per = (texels + 1024u * 128u - 1u) / (1024u * 128u);
    const unsigned sblocks = (texels + per * 1024u - 1u) / (per * 1024u);
    launch_after(tex_scan_kernel, sblocks, 1024, 0, st, (const unsigned*)d.tex_count, d.tex_start, texels, per);
    Dev ds = d;
    ds.tex_count = d.tex_start;  // what the scatter kernel reads as segment starts
    launch_after(ent_scatter_kernel<false>, sms * 8, 256, 0, st, ds, texels, (unsigned*)nullptr);
    total = d.tex_start + texels;
  }
  // entries one lane group walks per run, blocks per SM (experiments: fbev_set_tuning tile_y / tile_x with min_blocks 9)
  const unsigned run_len = g_tuning.minb == 9 && g_tuning.ty > 0 ? (unsigned)g_tuning.ty : 32u;
  const int gb = sms * (g_tuning.minb == 9 && g_tuning.tx > 0 ? g_tuning.tx : 8);
  const bool pd = d.ent_d_sorted != nullptr;
  // The entries do not depend on the lane layout that emitted them.  A float32 list phase that ran with four
  // chunks per lane is gathered with two: eight accumulators per texel side instead of sixteen, and twice the
  // lane groups (measured on the training shape: 94 against 102 us).
  const bool narrow = !fixed && sizeof(T) == 4 && pl.V == 4 && g_tuning.minb != 9;
  int gather_v = narrow ? 2 : pl.V;
  if (!fixed && g_tuning.minb == 16 && (g_tuning.tx == 1 || g_tuning.tx == 2 || g_tuning.tx == 4)) gather_v = g_tuning.tx;  // experiments
  Dev dn = d;
  const int cpt = d.GL * pl.V;
  if (gather_v != pl.V && cpt % gather_v == 0 && cpt / gather_v <= 32) {
    dn.GL = cpt / gather_v;
    dn.CPW = 32 / dn.GL < kMaxCellsPerWarp ? 32 / dn.GL : kMaxCellsPerWarp;
  } else {
    gather_v = pl.V;
  }
  if (fixed) {
#define FBEV_GATHER_FIXED(VV, GF) launch_after(feats_gather_fixed_kernel<T, VV, GF>, gb, 128, 0, st, d, (const unsigned*)total, run_len)
    switch (pl.V) {
      case 1: if (d.out_f32) FBEV_GATHER_FIXED(1, true); else FBEV_GATHER_FIXED(1, false); break;
      case 2: if (d.out_f32) FBEV_GATHER_FIXED(2, true); else FBEV_GATHER_FIXED(2, false); break;
      default: if (d.out_f32) FBEV_GATHER_FIXED(4, true); else FBEV_GATHER_FIXED(4, false); break;
    }
#undef FBEV_GATHER_FIXED
    return cudaGetLastError() == cudaSuccess ? FBEV_OK : FBEV_ERR_LAUNCH;
  }
#define FBEV_GATHER(VV, GF, PD) launch_after(feats_gather_kernel<T, VV, GF, PD>, gb, 128, 0, st, dn, (const unsigned*)total, run_len)
#define FBEV_GATHER_V(GF, PD)                 \
  switch (gather_v) {                         \
    case 1: FBEV_GATHER(1, GF, PD); break;    \
    case 2: FBEV_GATHER(2, GF, PD); break;    \
    default: FBEV_GATHER(4, GF, PD); break;   \
  }
  if (d.out_f32) {
    if (pd) { FBEV_GATHER_V(true, true) } else { FBEV_GATHER_V(true, false) }
  } else {
    if (pd) { FBEV_GATHER_V(false, true) } else { FBEV_GATHER_V(false, false) }
  }
#undef FBEV_GATHER_V
#undef FBEV_GATHER
  return cudaGetLastError() == cudaSuccess ? FBEV_OK : FBEV_ERR_LAUNCH;
}

template <typename T>
static int backward_feats_t(const Plan& pl, const Dev& d, cudaStream_t st) {
  if (d.ent != nullptr) return backward_feats_sort_t<T>(pl, d, st);
  // measured: ahead of the direct kernel on small feature maps with many cells per texel, behind it otherwise
  if (g_tuning.minb != 1 && (g_tuning.minb == 6 || ((long long)d.H * d.W <= 1024 && (long long)d.X * (d.y1 - d.y0) >= 30000)) &&
      (long long)d.H * d.W < (1 << 21)) {
    // texel-stationary kernel: eight warps, 12 x 8 tiles, block-wide entry array
    Plan ps = pl;
    Dev ds = d;
    ps.warps = g_tuning.warps > 0 ? pl.warps : 8;
    // about 20 (small feature maps) to 35 (large ones) entries per cell: keep a tile within the entry array
    ds.TX = g_tuning.tx > 0 ? g_tuning.tx : 12;
    ds.TY = g_tuning.ty > 0 ? g_tuning.ty : 4;
    ds.tiles_x = (d.X + ds.TX - 1) / ds.TX;
    ds.tiles_y = (d.y1 - d.y0 + ds.TY - 1) / ds.TY;
    ps.blocks = ds.tiles_x * ds.tiles_y * d.B;
    ps.smem = header_bytes(d.N) + (size_t)ps.warps * fwd_warp_bytes(ps.CPW, ps.cap) + feats_block_bytes();
    switch (ps.V) {
      case 1: return launch(bwd_feats_sorted_kernel<T, 1>, ps, ds, st);
      case 2: return launch(bwd_feats_sorted_kernel<T, 2>, ps, ds, st);
      default: return launch(bwd_feats_sorted_kernel<T, 4>, ps, ds, st);
    }
  }
  switch (pl.V) {
    case 1: return launch(bwd_feats_kernel<T, 1, false>, pl, d, st, (d.TX * d.TY + pl.CPW - 1) / pl.CPW);
    case 2: return launch(bwd_feats_kernel<T, 2, false>, pl, d, st, (d.TX * d.TY + pl.CPW - 1) / pl.CPW);
    default: return launch(bwd_feats_kernel<T, 4, false>, pl, d, st, (d.TX * d.TY + pl.CPW - 1) / pl.CPW);
  }
}

// Launches the record-based depth-gradient kernel for plan pld / problem dd.  With a saved state to offer, the
// instantiation that reads the forward's lists goes first and the rebuilding one after it; each looks at the state
// (saved_usable) and exactly one of them does the work, so an incomplete or foreign state costs one empty launch.
template <typename T, int V, bool EMIT>
static int launch_depth_v(const Plan& pld, const Dev& dd, cudaStream_t st) {
  const int gpt = (dd.TX * dd.TY + pld.CPW - 1) / pld.CPW;
  const bool cat = dd.mode == FBEV_DEPTH_CATEGORICAL;
  if (dd.saved != nullptr) {
    const int rc = cat ? launch(bwd_depth_kernel<T, V, EMIT, true>, pld, dd, st, gpt)
                       : launch(bwd_depth_param_kernel<T, V, EMIT, true>, pld, dd, st, gpt);
    if (rc != FBEV_OK) return rc;
  }
  return cat ? launch(bwd_depth_kernel<T, V, EMIT, false>, pld, dd, st, gpt)
             : launch(bwd_depth_param_kernel<T, V, EMIT, false>, pld, dd, st, gpt);
}
// The reproducible backward's instantiations: entries for the feature gradient, fixed-point depth sums, lists rebuilt.
template <typename T, int V>
static int launch_depth_fixed_v(const Plan& pld, const Dev& dd, cudaStream_t st) {
  const int gpt = (dd.TX * dd.TY + pld.CPW - 1) / pld.CPW;
  return dd.mode == FBEV_DEPTH_CATEGORICAL ? launch(bwd_depth_kernel<T, V, true, false, true>, pld, dd, st, gpt)
                                           : launch(bwd_depth_param_kernel<T, V, true, false, true>, pld, dd, st, gpt);
}
template <typename T>
static int launch_depth_fixed(const Plan& pld, const Dev& dd, cudaStream_t st) {
  switch (pld.V) {
    case 1: return launch_depth_fixed_v<T, 1>(pld, dd, st);
    case 2: return launch_depth_fixed_v<T, 2>(pld, dd, st);
    default: return launch_depth_fixed_v<T, 4>(pld, dd, st);
  }
}

template <typename T, bool EMIT>
static int launch_depth(const Plan& pld, const Dev& dd, cudaStream_t st) {
  switch (pld.V) {
    case 1: return launch_depth_v<T, 1, EMIT>(pld, dd, st);
    case 2: return launch_depth_v<T, 2, EMIT>(pld, dd, st);
    default: return launch_depth_v<T, 4, EMIT>(pld, dd, st);
  }
}

// pl / d: plan of the per-sample kernel (depth gradient, or both gradients when the feature-gradient kernel cannot
// take the shape); plf / df: plan of the feature-gradient kernel.
template <typename T>
static int backward_t(const Plan& pl, Dev d, const Plan& plf, const Dev& df, cudaStream_t st) {
  if (!pl.chunked) return launch(bwd_generic_kernel<T>, pl, d, st);
  // the record-based depth kernel: categorical depth always; the parametric modes (two gradient slots per texel,
  // where one lane per sample firing at them contends more than the per-group issue of bwd_kernel) when their
  // per-record sums can ride on the entry lists or leave as one atomic per record texel beside them
  const bool depth_on_records = (d.flags & FBEV_BWD_DEPTH) && plf.chunked &&
                                (d.mode == FBEV_DEPTH_CATEGORICAL || g_tuning.minb == 5 || df.ent != nullptr) &&
                                (unsigned long long)df.B * df.N * df.H * df.W * (unsigned long long)df.D < (1ull << 32);
  Plan pld = plf;
  Dev dd = df;
  // 16 candidates per cell and pass: half the shared memory of the forward's 32, twice the resident warps, which
  // this latency-bound kernel needs more than it minds a second pass on tiles that three cameras see
  pld.cap = dd.cap = 16;
  pld.smem = header_bytes(dd.N) + (size_t)pld.warps * depth_warp_bytes(pld.CPW, pld.cap);
  setup_saved(dd, pld.CPW);  // lists of a training forward, when the caller kept them
  if ((d.flags & FBEV_BWD_FEATS) && plf.chunked) {
    if (depth_on_records && df.ent != nullptr) {
      // both gradients from one list phase: the depth kernel also emits the entries of the sorted feature gradient
      // parametric depth without room in the entries: per-record sums leave as atomics (sort_carries_depth)
      dd.flags = d.flags | (d.mode != FBEV_DEPTH_CATEGORICAL && df.ent_d == nullptr ? kBwdRecordAtomics : 0);
      const int rc = launch_depth<T, true>(pld, dd, st);
      return rc != FBEV_OK ? rc : sort_finish_t<T>(pld, dd, st);
    }
    const int rc = backward_feats_t<T>(plf, df, st);
    if (rc != FBEV_OK) return rc;
    d.flags &= ~FBEV_BWD_FEATS;
    if (!(d.flags & FBEV_BWD_DEPTH)) return FBEV_OK;
  }
  if (depth_on_records && df.ent_d != nullptr) {
    // parametric depth gradient alone: its per-texel sums travel through the entry lists
    dd.flags = d.flags;
    const int rc = launch_depth<T, true>(pld, dd, st);
    return rc != FBEV_OK ? rc : sort_finish_t<T>(pld, dd, st);
  }
  if (depth_on_records) {
    // depth gradient alone: per-texel dot products on the forward's row records
    dd.flags = d.flags;
    return launch_depth<T, false>(pld, dd, st);
  }
  switch (pl.V) {
    case 1: return launch(bwd_kernel<T, 1>, pl, d, st);
    case 2: return launch(bwd_kernel<T, 2>, pl, d, st);
    default: return launch(bwd_kernel<T, 4>, pl, d, st);
  }
}

}  // namespace fbev

using namespace fbev;

// Per-texel softmax statistics of a logits depth tensor into p->depth_stats (no-op in the other modes).
static int launch_softmax_stats(const FbevProblem* p, cudaStream_t st) {
  if (p->mode != FBEV_DEPTH_CATEGORICAL_LOGITS) return FBEV_OK;
  const size_t texels = (size_t)p->B * p->N * p->H * p->W;
  const unsigned blocks = (unsigned)((texels * 32 + 255) / 256);
  float2* stats = reinterpret_cast<float2*>(p->depth_stats);
  switch (p->dtype) {
    case FBEV_F32: softmax_stats_kernel<float><<<blocks, 256, 0, st>>>(reinterpret_cast<const float*>(p->depth), stats, texels, p->D); break;
    case FBEV_BF16: softmax_stats_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(p->depth), stats, texels, p->D); break;
    default: softmax_stats_kernel<__half><<<blocks, 256, 0, st>>>(reinterpret_cast<const __half*>(p->depth), stats, texels, p->D); break;
  }
  return cudaGetLastError() == cudaSuccess ? FBEV_OK : FBEV_ERR_LAUNCH;
}

// unknown_hw: the caller could not tell the tensor's H and W (reference launcher signature); the
// kernels then trust feature_size, as the reference does.
static int forward_impl(const FbevProblem* p, void* out, int32_t* valid_count, void* stream, bool unknown_hw,
                        void* const* peers = nullptr, int n_peers = 0, void* out_multicast = nullptr) {
  const int rc = validate(p);
  if (rc != FBEV_OK) return rc;
  if (out == nullptr) return FBEV_ERR_NULL;
  if (((uintptr_t)out % elem_size(p->out_dtype)) || ((uintptr_t)valid_count % 4)) return FBEV_ERR_ALIGN;
  if (n_peers < 0 || n_peers > 7 || (n_peers > 0 && peers == nullptr)) return FBEV_ERR_SHAPE;
  if (p->compact_rows && (n_peers > 0 || out_multicast != nullptr)) return FBEV_ERR_SHAPE;  // peers hold whole grids
  Dev d;
  fill_dev(p, d);
  d.out = out;
  d.count = valid_count;
  d.n_peers = n_peers;
  if (out_multicast != nullptr && ((uintptr_t)out_multicast % 16 || (uintptr_t)out % 16)) return FBEV_ERR_ALIGN;
  d.out_mc = out_multicast;
  for (int k = 0; k < n_peers; ++k) {
    if (peers[k] == nullptr) return FBEV_ERR_NULL;
    if ((uintptr_t)peers[k] % 16 != (uintptr_t)out % 16) return FBEV_ERR_ALIGN;  // same kernel, same store width
    d.out_peers[k] = peers[k];
  }
  if (unknown_hw) d.H = d.W = 46340;  // feature_size entries up to 2^31 texels pass the in-kernel bound
  if ((uintptr_t)p->saved_state % 16) return FBEV_ERR_ALIGN;
  const bool train = p->saved_state != nullptr && !unknown_hw;
  // a training forward runs in the depth-gradient kernel's layout (see backward_t) so that its lists can be reused
  Plan pl = make_plan(p, d, false, p->image_feats, out, nullptr, !(train && is_categorical(p->mode)) || wide_depth_pays(p));
  if (out_multicast != nullptr && !pl.chunked) return FBEV_ERR_RANGE;  // only the 16-byte-chunk kernel stores to it
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (train && pl.chunked) {
    pl.cap = d.cap = 16;
    pl.smem = header_bytes(p->N) + (size_t)pl.warps * depth_warp_bytes(pl.CPW, pl.cap);
    setup_saved(d, pl.CPW);
  } else {
    d.saved = nullptr;
  }
  if (train && d.saved == nullptr) {
    pl = make_plan(p, d, false, p->image_feats, out, nullptr);  // no usable state after all: the ordinary forward
  } else if (d.saved != nullptr && cudaMemsetAsync(d.saved, 0, 16, st) != cudaSuccess) {  // cursor and key
    cudaGetLastError();
    return FBEV_ERR_LAUNCH;
  }
  const int src = launch_softmax_stats(p, st);
  if (src != FBEV_OK) return src;
  switch (p->dtype) {
    case FBEV_F32: return forward_t<float>(pl, d, st);
    case FBEV_BF16: return forward_t<__nv_bfloat16>(pl, d, st);
    default: return forward_t<__half>(pl, d, st);
  }
}

extern "C" {

int fbev_version(void) { return FBEV_ABI_VERSION; }

#ifndef FBEV_SOURCE_HASH
#define FBEV_SOURCE_HASH "unknown"
#endif
const char* fbev_source_hash(void) { return FBEV_SOURCE_HASH; }

const char* fbev_strerror(int status) {
  switch (status) {
    case FBEV_OK: return "ok";
    case FBEV_ERR_NULL: return "a required pointer is NULL";
    case FBEV_ERR_STRUCT: return "FbevProblem.struct_size does not match this library";
    case FBEV_ERR_SHAPE: return "a size is non-positive or inconsistent (depth last dim must be 2 for the parametric modes; proj_stride 12 or 16; 0 <= y_begin <= y_end <= Y)";
    case FBEV_ERR_DTYPE: return "unknown element type";
    case FBEV_ERR_MODE: return "unknown depth model or pooling, or depth_delta <= 0 in a categorical mode";
    case FBEV_ERR_ALIGN: return "a pointer is not aligned to its element size";
    case FBEV_ERR_RANGE: return "sizes exceed kernel indexing: B*N*H*W and B*Y*X must be below 2^31, N <= 1024, shared memory per block <= 200 KiB";
    case FBEV_ERR_SCRATCH: return "scratch buffer missing, misaligned or smaller than fbev_backward_min_scratch_bytes()";
    case FBEV_ERR_LAUNCH: return "the CUDA runtime refused a launch or memset (cudaGetLastError)";
    case FBEV_ERR_NO_DEVICE: return "no usable sm_100 device";
    case FBEV_ERR_STATIC_LIMIT: return "the problem needs more float32 scratch than fbev_backward_static_scratch holds (FBEV_STATIC_SCRATCH_BYTES); use fbev_backward with caller scratch";
    default: return "unknown status";
  }
}

void fbev_set_tuning(int tile_x, int tile_y, int chunks_per_lane, int warps, int min_blocks) {
  g_tuning = Tuning{tile_x, tile_y, chunks_per_lane, warps, min_blocks};
}

void fbev_set_experiment(int bits) { g_experiment = bits; }

int fbev_forward(const FbevProblem* p, void* out, int32_t* valid_count, void* stream) {
  return forward_impl(p, out, valid_count, stream, false);
}

// Side stream and events of fbev_forward_to_host: one set per (device, caller stream), created on first use
// under a lock and kept for the life of the process.  Calls on different streams therefore share nothing;
// calls on one stream are ordered by that stream.
struct HostPipe {
  int dev = -1;
  cudaStream_t caller = nullptr;
  cudaStream_t side = nullptr;
  cudaEvent_t ready[16] = {};
  cudaEvent_t done = nullptr;
};
constexpr int kMaxHostPipes = 256;
static HostPipe g_host_pipe[kMaxHostPipes];
static int g_host_pipes = 0;
static std::mutex g_host_pipe_lock;

static HostPipe* host_pipe(int dev, cudaStream_t caller) {
  std::lock_guard<std::mutex> g(g_host_pipe_lock);
  for (int i = 0; i < g_host_pipes; ++i)
    if (g_host_pipe[i].dev == dev && g_host_pipe[i].caller == caller) return &g_host_pipe[i];
  if (g_host_pipes == kMaxHostPipes) return nullptr;
  HostPipe hp;
  hp.dev = dev;
  hp.caller = caller;
  bool good = cudaStreamCreateWithFlags(&hp.side, cudaStreamNonBlocking) == cudaSuccess;
  for (int k = 0; k < 16 && good; ++k) good = cudaEventCreateWithFlags(&hp.ready[k], cudaEventDisableTiming) == cudaSuccess;
  good = good && cudaEventCreateWithFlags(&hp.done, cudaEventDisableTiming) == cudaSuccess;
  if (!good) {
    cudaGetLastError();
    return nullptr;
  }
  g_host_pipe[g_host_pipes] = hp;
  return &g_host_pipe[g_host_pipes++];
}

int fbev_forward_to_host(const FbevProblem* p, void* out_dev, void* out_host, int row_chunks, void* stream) {
  const int rc = validate(p);
  if (rc != FBEV_OK) return rc;
  if (out_dev == nullptr || out_host == nullptr) return FBEV_ERR_NULL;
  if (row_chunks < 1 || row_chunks > 16 || p->compact_rows) return FBEV_ERR_SHAPE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) {
    cudaGetLastError();
    return FBEV_ERR_NO_DEVICE;
  }
  HostPipe* hpp = host_pipe(dev, reinterpret_cast<cudaStream_t>(stream));
  if (hpp == nullptr) return FBEV_ERR_LAUNCH;
  HostPipe& hp = *hpp;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int y0 = p->y_begin, rows = p->y_end - p->y_begin;
  const size_t row_bytes = (size_t)p->X * p->C * elem_size(p->out_dtype);
  const size_t pitch = (size_t)p->Y * row_bytes;  // one batch sample
  // bands are whole rows of tiles: the launches then work on exactly the tiles of one launch over all rows, and
  // the result is bit-identical to it (which candidates share a sweep, and so which weights are summed before
  // they meet the features, depends on the tiling)
  Dev probe;
  fill_dev(p, probe);
  (void)make_plan(p, probe, false, p->image_feats, out_dev, nullptr);
  const int ty = probe.TY > 0 ? probe.TY : 1;
  const int tile_rows = (rows + ty - 1) / ty;
  for (int k = 0; k < row_chunks; ++k) {
    FbevProblem q = *p;
    q.y_begin = y0 + (int)((long long)tile_rows * k / row_chunks) * ty;
    q.y_end = y0 + (int)((long long)tile_rows * (k + 1) / row_chunks) * ty;
    if (q.y_end > p->y_end) q.y_end = p->y_end;
    if (q.y_end <= q.y_begin) continue;
    const int frc = forward_impl(&q, out_dev, nullptr, stream, false);
    if (frc != FBEV_OK) return frc;
    // the copy engine takes the rows of this launch while the next launch computes
    const size_t off = (size_t)q.y_begin * row_bytes;
    if (cudaEventRecord(hp.ready[k], st) != cudaSuccess || cudaStreamWaitEvent(hp.side, hp.ready[k], 0) != cudaSuccess ||
        cudaMemcpy2DAsync(reinterpret_cast<unsigned char*>(out_host) + off, pitch,
                          reinterpret_cast<const unsigned char*>(out_dev) + off, pitch,
                          (size_t)(q.y_end - q.y_begin) * row_bytes, (size_t)p->B, cudaMemcpyDeviceToHost,
                          hp.side) != cudaSuccess) {
      cudaGetLastError();
      return FBEV_ERR_LAUNCH;
    }
  }
  // the caller's stream continues when the last rows have landed
  if (cudaEventRecord(hp.done, hp.side) != cudaSuccess || cudaStreamWaitEvent(st, hp.done, 0) != cudaSuccess) {
    cudaGetLastError();
    return FBEV_ERR_LAUNCH;
  }
  return FBEV_OK;
}

// float32 accumulation targets of the 16-bit types: what fbev_backward cannot do without
// Reproducible backward: a 256-byte head (DetHeader), 64-bit fixed-point sums for both gradients (the kernels always
// form both; only the requested ones are converted) and, for logits, the float32 gradient with respect to the
// probabilities that the softmax backward consumes.
static size_t round256(size_t n) { return ((n + 255) / 256) * 256; }
static size_t det_scratch_bytes(const FbevProblem* p) {
  const size_t tex = (size_t)p->B * p->N * p->H * p->W;
  size_t n = 256 + round256(tex * p->C * 8) + round256(tex * p->D * 8);
  if (p->mode == FBEV_DEPTH_CATEGORICAL_LOGITS) n += round256(tex * p->D * 4);
  return n;
}

static size_t scratch_min_bytes(const FbevProblem* p, int flags) {
  if (flags & FBEV_BWD_DETERMINISTIC) return det_scratch_bytes(p);
  if (p->dtype == FBEV_F32) return 0;
  size_t n = 0;
  const size_t tex = (size_t)p->B * p->N * p->H * p->W;
  if (flags & FBEV_BWD_FEATS) n += ((tex * p->C * 4 + 255) / 256) * 256;
  if (flags & FBEV_BWD_DEPTH) n += ((tex * p->D * 4 + 255) / 256) * 256;
  return n;
}

// Entry lists of the sorted gradients.  One entry per two candidates is a little over twice what the benchmark
// rigs emit (one per row record); warps that find the list full add directly instead.  The lists are transient
// scratch, so their size is bounded: at most kSortBudgetBytes, whatever the batch.  A batch whose lists would
// not fit is processed in runs of as many samples as do (sort_batch_run); one sample that does not fit by itself
// gets the capped list and its overflow takes the direct path.
constexpr size_t kSortBudgetBytes = FBEV_SORT_BUDGET_BYTES;
// The parametric depth gradient (two values per texel) rides on the same entries, 16 more bytes in each list, when
// the feature map is small: few texels mean many records per texel, and their sums as atomics on two words per
// texel queue up.  From 8192 texels per sample on the sums leave the depth kernel as one atomic per record texel
// instead (measured, both gradients: 16x44 maps 121 us on the entries against 159 us by atomics; 32x88 maps 571
// against 574 us on a 200x200x8 grid and 2393 against 1841 us on a 512x512x16 grid with 256 channels).
static bool sort_carries_depth(const FbevProblem* p, int flags) {
  if (!(flags & FBEV_BWD_DEPTH) || is_categorical(p->mode)) return false;
  if (g_tuning.minb == 12) return false;  // experiments: never / (13) always
  return g_tuning.minb == 13 || (size_t)p->N * p->H * p->W < 8192;
}
static size_t sort_entry_bytes(const FbevProblem* p, int flags) {
  // entry and its grouped copy, position, and for the parametric depth gradient four floats in either list
  return 16 + 16 + 4 + (sort_carries_depth(p, flags) ? 32 : 0);
}
static size_t sort_entries_per_sample(const FbevProblem* p) {
  return (size_t)p->X * (size_t)(p->y_end - p->y_begin) * p->N * p->Z / 2;
}
// samples of the batch that share one set of entry lists
static int sort_batch_run(const FbevProblem* p, int flags) {
  const size_t per = sort_entries_per_sample(p) * sort_entry_bytes(p, flags);
  if (per == 0 || per * (size_t)p->B <= kSortBudgetBytes) return p->B;
  const size_t fit = kSortBudgetBytes / per;
  return fit < 1 ? 1 : (int)fit;
}
static size_t sort_capacity(const FbevProblem* p, int flags) {
  if (g_tuning.minb == 8) return 4096;  // tests: nearly every warp finds the list full
  const size_t cand = sort_entries_per_sample(p) * (size_t)sort_batch_run(p, flags);
  size_t top = kSortBudgetBytes / sort_entry_bytes(p, flags);
  if (top > ((size_t)1 << 26)) top = (size_t)1 << 26;
  return cand < top ? (cand < 4096 ? 4096 : cand) : top;
}
static size_t sort_bytes(const FbevProblem* p, int flags) {
  if (flags & FBEV_BWD_DETERMINISTIC) flags = FBEV_BWD_FEATS;  // entries of the feature gradient only, whatever was asked for
  if (!(flags & FBEV_BWD_FEATS) && !sort_carries_depth(p, flags)) return 0;
  const size_t tex = (size_t)sort_batch_run(p, flags) * p->N * p->H * p->W;
  if (tex >= 0xfffffff0ull || (size_t)p->B * p->Y * p->X >= 0xfffffff0ull) return 0;
  const size_t cnt = (((tex + 1) * 4 + 255) / 256) * 256;
  // feature maps too large for the in-block scan keep the segment starts in an array of their own
  return cnt + 256 + sort_capacity(p, flags) * sort_entry_bytes(p, flags) + (tex > kScanInBlock ? cnt : 0);
}

int fbev_forward_peers(const FbevProblem* p, void* out, void* const* peer_outs, int n_peers, int32_t* valid_count,
                       void* stream) {
  return forward_impl(p, out, valid_count, stream, false, peer_outs, n_peers);
}

int fbev_forward_multicast(const FbevProblem* p, void* out, void* out_multicast, int32_t* valid_count, void* stream) {
  if (out_multicast == nullptr) return FBEV_ERR_NULL;
  return forward_impl(p, out, valid_count, stream, false, nullptr, 0, out_multicast);
}

size_t fbev_saved_state_bytes(const FbevProblem* p) {
  if (p == nullptr || validate(p) != FBEV_OK) return 0;
  // directory: 16 bytes per (group of cells, pass), sized for the smallest groups and passes the kernels use;
  // data: 24 bytes per candidate covers the benchmark rigs (about 17 are used) with room to spare, at most 1 GiB
  const unsigned long long cells = (unsigned long long)p->B * p->X * (unsigned long long)(p->y_end - p->y_begin);
  const unsigned long long cand = cells * p->N * p->Z;
  const unsigned long long dir = (cells / 2 + (unsigned long long)p->B * 4096) * (((unsigned long long)p->N * p->Z + 15) / 16);
  unsigned long long data = cand * 24;
  if (data > (1ull << 30)) data = 1ull << 30;
  return (size_t)(16 + dir * 16 + data + 4096);
}

size_t fbev_backward_min_scratch_bytes(const FbevProblem* p, int flags) {
  return p == nullptr ? 0 : scratch_min_bytes(p, flags);
}

size_t fbev_backward_scratch_bytes(const FbevProblem* p, int flags) {
  if (p == nullptr) return 0;
  return scratch_min_bytes(p, flags) + sort_bytes(p, flags);
}

// FBEV_BWD_DETERMINISTIC (fbev_deterministic.cuh): bounds of the inputs, scale, accumulation, conversion.  Shapes the
// chunked kernels take, given room for the entry lists, accumulate through the default pipeline's kernels in their
// fixed-point instantiations (list phase + entries + depth sums, scatter, gather); everything else through the
// one-cell-per-warp kernel.
struct DetLayout {
  DetHeader* hdr;
  long long* gf;
  long long* gd;
  float* dprob;          // logits only
  unsigned char* sort;   // entry lists, or null
};

extern "C++" {
template <typename T>
static int backward_deterministic_t(const FbevProblem* p, const void* grad_out, void* grad_feats, void* grad_depth,
                                    const DetLayout& L, int flags, cudaStream_t st) {
  const size_t tex_sample = (size_t)p->N * p->H * p->W, tex_all = tex_sample * p->B;
  const size_t nf = tex_all * p->C, nd = tex_all * p->D;
  const size_t out_rows = p->compact_rows ? (size_t)(p->y_end - p->y_begin) : (size_t)p->Y;
  const size_t es = elem_size(p->dtype), eso = elem_size(p->out_dtype);
  const bool cat = is_categorical(p->mode);
  const int work = (flags & FBEV_BWD_LEGACY_DEPTH) | FBEV_BWD_FEATS | FBEV_BWD_DEPTH;  // both gradients are always formed
  const int sort_flags = FBEV_BWD_FEATS;
  // 2^bits above the number of contributions one element can receive: four corners of every candidate of its camera
  const unsigned long long cnt = 4ull * (unsigned long long)(p->y_end - p->y_begin) * p->X * p->Z;
  int bits = 0;
  while (bits < 48 && (1ull << bits) < cnt) ++bits;
  const int shift = 62 - bits;

  // which way: the plan of the first run of samples decides for all of them
  const int run = L.sort != nullptr ? sort_batch_run(p, sort_flags) : p->B;
  bool fast = false;
  if (L.sort != nullptr) {
    FbevProblem q = *p;
    q.B = run < p->B ? run : p->B;
    Dev probe;
    fill_dev(&q, probe);
    const Plan plf = make_plan(&q, probe, false, q.image_feats, grad_out, L.gf, !cat);
    fast = plf.chunked;
  }

  const int kind = p->mode == FBEV_DEPTH_CATEGORICAL_LOGITS ? 1 : (cat ? 0 : ((flags & FBEV_BWD_LEGACY_DEPTH) ? 3 : 2));
  // the chunked depth kernel sums up to a warp's worth of equal (texel, bin) neighbours before it adds them
  det_bounds_kernel<T><<<sm_count() * 8, 256, 0, st>>>(L.hdr, grad_out, (p->out_dtype == FBEV_F32 && p->dtype != FBEV_F32) ? 1 : 0,
                                                       (size_t)p->B * out_rows * p->X, reinterpret_cast<const T*>(p->image_feats),
                                                       tex_all, p->C, reinterpret_cast<const T*>(p->depth), p->D, cat ? 1 : 0,
                                                       p->epsilon, shift, p->Z, kind, fast ? 32 : 1);
  if (cudaGetLastError() != cudaSuccess) return FBEV_ERR_LAUNCH;

  if (!fast) {
    Dev d;
    fill_dev(p, d);
    d.saved = nullptr;
    d.gout = grad_out;
    d.flags = work;
    d.gfeat = reinterpret_cast<float*>(L.gf);   // read as int64 arrays by the kernel
    d.gdepth = reinterpret_cast<float*>(L.gd);
    d.det = L.hdr;
    d.GL = 32;
    d.CPW = 1;
    d.cpt = 1;  // record texel fields are plain texel indices
    d.cap = 32;
    d.TX = 8;
    d.TY = 4;
    d.tiles_x = (p->X + d.TX - 1) / d.TX;
    d.tiles_y = (p->y_end - p->y_begin + d.TY - 1) / d.TY;
    Plan pl{};
    pl.chunked = false;
    pl.GL = 32;
    pl.CPW = 1;
    pl.warps = kMaxWarps;
    pl.cap = d.cap;
    pl.smem = header_bytes(p->N) + (size_t)pl.warps * depth_warp_bytes(1, pl.cap);
    pl.blocks = d.tiles_x * d.tiles_y * p->B;
    const int rc = launch(bwd_det_kernel<T>, pl, d, st);
    if (rc != FBEV_OK) return rc;
  } else {
    const size_t tex_run = (size_t)run * tex_sample;
    const size_t cnt_bytes = round256((tex_run + 1) * 4);
    for (int b0 = 0; b0 < p->B; b0 += run) {
      FbevProblem q = *p;  // the samples [b0, b0 + run) as a problem of their own
      q.B = p->B - b0 < run ? p->B - b0 : run;
      q.image_feats = reinterpret_cast<const unsigned char*>(p->image_feats) + (size_t)b0 * tex_sample * p->C * es;
      q.depth = reinterpret_cast<const unsigned char*>(p->depth) + (size_t)b0 * tex_sample * p->D * es;
      q.projection = p->projection + (size_t)b0 * p->N * p->proj_stride;
      q.feature_size = p->feature_size + (size_t)b0 * p->N * 2;
      if (p->mode == FBEV_DEPTH_CATEGORICAL_LOGITS) q.depth_stats = p->depth_stats + (size_t)b0 * tex_sample * 2;
      const void* gout = reinterpret_cast<const unsigned char*>(grad_out) + (size_t)b0 * out_rows * p->X * p->C * eso;
      Dev d;
      fill_dev(&q, d);
      d.saved = nullptr;
      d.gout = gout;
      d.flags = work;
      d.gfeat = reinterpret_cast<float*>(L.gf + (size_t)b0 * tex_sample * p->C);
      d.gdepth = reinterpret_cast<float*>(L.gd + (size_t)b0 * tex_sample * p->D);
      d.det = L.hdr;
      if (cudaMemsetAsync(L.sort, 0, cnt_bytes + 256, st) != cudaSuccess) {
        cudaGetLastError();
        return FBEV_ERR_LAUNCH;
      }
      d.tex_count = reinterpret_cast<unsigned*>(L.sort);
      d.ent_count = reinterpret_cast<unsigned*>(L.sort + cnt_bytes);
      d.ent_cap = (unsigned)sort_capacity(p, sort_flags);
      d.ent = reinterpret_cast<uint4*>(L.sort + cnt_bytes + 256);
      d.ent_sorted = d.ent + d.ent_cap;
      d.ent_pos = reinterpret_cast<unsigned*>(d.ent_sorted + d.ent_cap);
      d.tex_start = d.ent_pos + d.ent_cap;
      Plan pld = make_plan(&q, d, false, q.image_feats, gout, d.gfeat, !cat);
      if (!pld.chunked) return FBEV_ERR_RANGE;  // cannot happen: a slice of the batch fits where the first run did
      pld.cap = d.cap = 16;  // as the default backward: half the shared memory, twice the resident warps
      pld.smem = header_bytes(d.N) + (size_t)pld.warps * depth_warp_bytes(pld.CPW, pld.cap);
      int rc = launch_depth_fixed<T>(pld, d, st);
      if (rc == FBEV_OK) rc = sort_finish_t<T>(pld, d, st, true);
      if (rc != FBEV_OK) return rc;
    }
  }
  const size_t na = (flags & FBEV_BWD_FEATS) ? nf : 0, nb = (flags & FBEV_BWD_DEPTH) ? nd : 0;
  const size_t want = (na + nb + 255) / 256;
  const int blocks = (int)(want < (size_t)sm_count() * 16 ? (want ? want : 1) : (size_t)sm_count() * 16);
  if (L.dprob != nullptr)
    det_finish_kernel<T, float><<<blocks, 256, 0, st>>>(L.hdr, L.gf, reinterpret_cast<T*>(grad_feats), na, L.gd, L.dprob, nb);
  else
    det_finish_kernel<T, T><<<blocks, 256, 0, st>>>(L.hdr, L.gf, reinterpret_cast<T*>(grad_feats), na, L.gd,
                                                    reinterpret_cast<T*>(grad_depth), nb);
  return cudaGetLastError() == cudaSuccess ? FBEV_OK : FBEV_ERR_LAUNCH;
}
}  // extern "C++"

static int backward_deterministic(const FbevProblem* p, const void* grad_out, void* grad_feats, void* grad_depth,
                                  void* scratch, size_t scratch_bytes, int flags, cudaStream_t st) {
  const size_t tex_all = (size_t)p->B * p->N * p->H * p->W;
  const size_t nf = tex_all * p->C, nd = tex_all * p->D;
  // the row-record list phase keeps the visible cameras in a 32-bit mask and 32-bit depth element indices
  if (p->N > 32 || (unsigned long long)nd >= (1ull << 32)) return FBEV_ERR_RANGE;
  const size_t need = det_scratch_bytes(p);
  if (scratch == nullptr || scratch_bytes < need || ((uintptr_t)scratch % 256)) return FBEV_ERR_SCRATCH;
  const bool logits = p->mode == FBEV_DEPTH_CATEGORICAL_LOGITS;
  unsigned char* s = reinterpret_cast<unsigned char*>(scratch);
  DetLayout L{};
  L.hdr = reinterpret_cast<DetHeader*>(s);
  s += 256;
  L.gf = reinterpret_cast<long long*>(s);
  s += round256(nf * 8);
  L.gd = reinterpret_cast<long long*>(s);
  s += round256(nd * 8);
  if (logits && (flags & FBEV_BWD_DEPTH)) L.dprob = reinterpret_cast<float*>(s);
  // the entry lists of the sort by texel lie beyond, when the caller gave that much and the problem is large enough
  // for three more launches to pay (the default path's rule)
  const size_t sortb = sort_bytes(p, flags);
  const bool want_sort = g_tuning.minb == 7 || g_tuning.minb == 8 ||
                         (g_tuning.minb == 0 && (size_t)p->B * p->X * (size_t)(p->y_end - p->y_begin) * p->N * p->Z >= 200000);
  if (want_sort && sortb != 0 && scratch_bytes >= need + sortb) L.sort = reinterpret_cast<unsigned char*>(scratch) + need;
  if (cudaMemsetAsync(scratch, 0, 256 + round256(nf * 8) + round256(nd * 8), st) != cudaSuccess) {
    cudaGetLastError();
    return FBEV_ERR_LAUNCH;
  }
  int rc;
  switch (p->dtype) {
    case FBEV_F32: rc = backward_deterministic_t<float>(p, grad_out, grad_feats, grad_depth, L, flags, st); break;
    case FBEV_BF16: rc = backward_deterministic_t<__nv_bfloat16>(p, grad_out, grad_feats, grad_depth, L, flags, st); break;
    default: rc = backward_deterministic_t<__half>(p, grad_out, grad_feats, grad_depth, L, flags, st); break;
  }
  if (rc != FBEV_OK) return rc;
  if (L.dprob != nullptr) {
    // dL/dprob -> dL/dlogit through the folded softmax: one thread order per texel, nothing is drawn
    const unsigned blocks = (unsigned)((tex_all * 32 + 255) / 256);
    const float2* stats = reinterpret_cast<const float2*>(p->depth_stats);
    switch (p->dtype) {
      case FBEV_F32: launch_after(softmax_bwd_kernel<float>, blocks, 256, 0, st, reinterpret_cast<const float*>(p->depth), stats, (const float*)L.dprob, reinterpret_cast<float*>(grad_depth), tex_all, p->D); break;
      case FBEV_BF16: launch_after(softmax_bwd_kernel<__nv_bfloat16>, blocks, 256, 0, st, reinterpret_cast<const __nv_bfloat16*>(p->depth), stats, (const float*)L.dprob, reinterpret_cast<__nv_bfloat16*>(grad_depth), tex_all, p->D); break;
      default: launch_after(softmax_bwd_kernel<__half>, blocks, 256, 0, st, reinterpret_cast<const __half*>(p->depth), stats, (const float*)L.dprob, reinterpret_cast<__half*>(grad_depth), tex_all, p->D); break;
    }
    if (cudaGetLastError() != cudaSuccess) return FBEV_ERR_LAUNCH;
  }
  return FBEV_OK;
}

int fbev_backward(const FbevProblem* p, const void* grad_out, void* grad_feats, void* grad_depth, void* scratch,
                  size_t scratch_bytes, int flags, void* stream) {
  const int rc = validate(p);
  if (rc != FBEV_OK) return rc;
  if ((flags & (FBEV_BWD_FEATS | FBEV_BWD_DEPTH)) == 0) return FBEV_OK;
  if (grad_out == nullptr) return FBEV_ERR_NULL;
  if ((uintptr_t)p->saved_state % 16) return FBEV_ERR_ALIGN;
  if ((flags & FBEV_BWD_FEATS) && grad_feats == nullptr) return FBEV_ERR_NULL;
  if ((flags & FBEV_BWD_DEPTH) && grad_depth == nullptr) return FBEV_ERR_NULL;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t tex_all = (size_t)p->B * p->N * p->H * p->W;
  const size_t nf = tex_all * p->C, nd = tex_all * p->D;
  const bool f32 = p->dtype == FBEV_F32;
  const bool logits = p->mode == FBEV_DEPTH_CATEGORICAL_LOGITS;
  if (logits && (flags & FBEV_BWD_DEPTH) && ((uintptr_t)grad_depth % elem_size(p->dtype))) return FBEV_ERR_ALIGN;
  {
    const int src = launch_softmax_stats(p, st);
    if (src != FBEV_OK) return src;
  }
  if (flags & FBEV_BWD_DETERMINISTIC)
    return backward_deterministic(p, grad_out, grad_feats, grad_depth, scratch, scratch_bytes, flags, st);
  // float32 accumulation targets of the whole batch: the gradient tensors themselves, or the head of the scratch
  float* gfeat_all = nullptr;
  float* gdepth_all = nullptr;
  if (f32) {
    if (((uintptr_t)grad_feats % 4) || ((uintptr_t)grad_depth % 4)) return FBEV_ERR_ALIGN;
    gfeat_all = reinterpret_cast<float*>(grad_feats);
    gdepth_all = reinterpret_cast<float*>(grad_depth);
  } else {
    const size_t need = scratch_min_bytes(p, flags);
    if (scratch == nullptr || scratch_bytes < need || ((uintptr_t)scratch % 256)) return FBEV_ERR_SCRATCH;
    unsigned char* s = reinterpret_cast<unsigned char*>(scratch);
    if (flags & FBEV_BWD_FEATS) {
      gfeat_all = reinterpret_cast<float*>(s);
      s += ((nf * 4 + 255) / 256) * 256;
    }
    if (flags & FBEV_BWD_DEPTH) gdepth_all = reinterpret_cast<float*>(s);
  }
  // what lies beyond the accumulation targets holds the entry lists of the sorted gradients, when the caller gave
  // that much (fbev_backward_scratch_bytes asks for it); small problems keep the single-launch kernels: three more
  // launches cost more than they save there
  const size_t sortb = sort_bytes(p, flags), minb = scratch_min_bytes(p, flags);
  const bool want_sort = g_tuning.minb == 7 || g_tuning.minb == 8 || g_tuning.minb == 9 || g_tuning.minb == 10 || g_tuning.minb == 12 || g_tuning.minb == 13 || g_tuning.minb == 16 ||
                         (g_tuning.minb == 0 && (size_t)p->B * p->X * (size_t)(p->y_end - p->y_begin) * p->N * p->Z >= 200000);
  const bool sorted = want_sort && sortb != 0 && scratch != nullptr && ((uintptr_t)scratch % 256) == 0 &&
                      scratch_bytes >= minb + sortb;
  const int run = sorted ? sort_batch_run(p, flags) : p->B;  // samples per pass over the entry lists
  const size_t tex_run = (size_t)run * p->N * p->H * p->W;
  const size_t cnt_bytes = (((tex_run + 1) * 4 + 255) / 256) * 256;
  unsigned char* sort_base = sorted ? reinterpret_cast<unsigned char*>(scratch) + minb : nullptr;
  // clears: the accumulation targets and, for the first run, the sort's counters; one memset when they are
  // neighbours in the scratch
  if (!f32 && sorted) {
    if (cudaMemsetAsync(scratch, 0, minb + cnt_bytes + 256, st) != cudaSuccess) {
      cudaGetLastError();
      return FBEV_ERR_LAUNCH;
    }
  } else {
    if (sorted && cudaMemsetAsync(sort_base, 0, cnt_bytes + 256, st) != cudaSuccess) {
      cudaGetLastError();
      return FBEV_ERR_LAUNCH;
    }
    if ((flags & FBEV_BWD_FEATS) && cudaMemsetAsync(gfeat_all, 0, nf * 4, st) != cudaSuccess) {
      cudaGetLastError();
      return FBEV_ERR_LAUNCH;
    }
    if ((flags & FBEV_BWD_DEPTH) && cudaMemsetAsync(gdepth_all, 0, nd * 4, st) != cudaSuccess) {
      cudaGetLastError();
      return FBEV_ERR_LAUNCH;
    }
  }
  const size_t es = elem_size(p->dtype), eso = elem_size(p->out_dtype);
  const size_t tex_sample = (size_t)p->N * p->H * p->W;
  for (int b0 = 0; b0 < p->B; b0 += run) {
    // the samples [b0, b0 + run) as a problem of their own: every tensor is indexed by the sample first
    FbevProblem q = *p;
    q.B = p->B - b0 < run ? p->B - b0 : run;
    q.image_feats = reinterpret_cast<const unsigned char*>(p->image_feats) + (size_t)b0 * tex_sample * p->C * es;
    q.depth = reinterpret_cast<const unsigned char*>(p->depth) + (size_t)b0 * tex_sample * p->D * es;
    q.projection = p->projection + (size_t)b0 * p->N * p->proj_stride;
    q.feature_size = p->feature_size + (size_t)b0 * p->N * 2;
    if (logits) q.depth_stats = p->depth_stats + (size_t)b0 * tex_sample * 2;
    const size_t out_rows = p->compact_rows ? (size_t)(p->y_end - p->y_begin) : (size_t)p->Y;
    const void* gout = reinterpret_cast<const unsigned char*>(grad_out) + (size_t)b0 * out_rows * p->X * p->C * eso;
    Dev d;
    fill_dev(&q, d);
    d.gout = gout;
    d.flags = flags;
    d.saved_B = p->B;  // the saved lists were written for the whole batch
    d.saved_b0 = b0;
    d.gfeat = gfeat_all ? gfeat_all + (size_t)b0 * tex_sample * p->C : nullptr;
    d.gdepth = gdepth_all ? gdepth_all + (size_t)b0 * tex_sample * p->D : nullptr;
    const Plan pl = make_plan(&q, d, true, q.image_feats, gout, f32 ? (const void*)d.gfeat : (const void*)nullptr);
    if (sorted) {
      if (b0 > 0 && cudaMemsetAsync(sort_base, 0, cnt_bytes + 256, st) != cudaSuccess) {  // counters of the run before
        cudaGetLastError();
        return FBEV_ERR_LAUNCH;
      }
      d.tex_count = reinterpret_cast<unsigned*>(sort_base);
      d.ent_count = reinterpret_cast<unsigned*>(sort_base + cnt_bytes);
      d.ent_cap = (unsigned)sort_capacity(p, flags);
      d.ent = reinterpret_cast<uint4*>(sort_base + cnt_bytes + 256);
      d.ent_sorted = d.ent + d.ent_cap;
      unsigned char* after = reinterpret_cast<unsigned char*>(d.ent_sorted + d.ent_cap);
      if (sort_carries_depth(p, flags)) {
        d.ent_d = reinterpret_cast<float4*>(after);
        d.ent_d_sorted = d.ent_d + d.ent_cap;
        after = reinterpret_cast<unsigned char*>(d.ent_d_sorted + d.ent_cap);
      }
      d.ent_pos = reinterpret_cast<unsigned*>(after);
      d.tex_start = d.ent_pos + d.ent_cap;
    }
    // the feature gradient has a kernel of its own, laid out like the forward
    Dev df = d;
    const bool wide_ok = !((flags & FBEV_BWD_DEPTH) && is_categorical(p->mode)) || wide_depth_pays(p);
    const Plan plf = make_plan(&q, df, false, q.image_feats, gout, d.gfeat, wide_ok);
    int lrc;
    switch (p->dtype) {
      case FBEV_F32: lrc = backward_t<float>(pl, d, plf, df, st); break;
      case FBEV_BF16: lrc = backward_t<__nv_bfloat16>(pl, d, plf, df, st); break;
      default: lrc = backward_t<__half>(pl, d, plf, df, st); break;
    }
    if (lrc != FBEV_OK) return lrc;
  }
  if (logits && (flags & FBEV_BWD_DEPTH)) {
    // what was accumulated is dL/dprob; through the folded softmax it becomes dL/dlogit, written in the tensor's
    // own type (so the conversion below has only the feature gradient left)
    const unsigned blocks = (unsigned)((tex_all * 32 + 255) / 256);
    const float2* stats = reinterpret_cast<const float2*>(p->depth_stats);
    switch (p->dtype) {
      case FBEV_F32: launch_after(softmax_bwd_kernel<float>, blocks, 256, 0, st, reinterpret_cast<const float*>(p->depth), stats, (const float*)gdepth_all, reinterpret_cast<float*>(grad_depth), tex_all, p->D); break;
      case FBEV_BF16: launch_after(softmax_bwd_kernel<__nv_bfloat16>, blocks, 256, 0, st, reinterpret_cast<const __nv_bfloat16*>(p->depth), stats, (const float*)gdepth_all, reinterpret_cast<__nv_bfloat16*>(grad_depth), tex_all, p->D); break;
      default: launch_after(softmax_bwd_kernel<__half>, blocks, 256, 0, st, reinterpret_cast<const __half*>(p->depth), stats, (const float*)gdepth_all, reinterpret_cast<__half*>(grad_depth), tex_all, p->D); break;
    }
    if (cudaGetLastError() != cudaSuccess) return FBEV_ERR_LAUNCH;
  }
  if (!f32) {
    // float32 accumulation targets -> gradient tensors, both in one launch
    const float* sa = (flags & FBEV_BWD_FEATS) ? gfeat_all : nullptr;
    const float* sb = ((flags & FBEV_BWD_DEPTH) && !logits) ? gdepth_all : nullptr;
    const size_t na = sa ? nf : 0, nb = sb ? nd : 0;
    const size_t units = (na + 3) / 4 + (nb + 3) / 4;
    const int threads = 256;
    const int blocks = (int)((units + threads - 1) / threads < 148 * 16 ? (units + threads - 1) / threads : 148 * 16);
    if (p->dtype == FBEV_BF16)
      launch_after(convert2_kernel<__nv_bfloat16>, blocks, threads, 0, st, sa, reinterpret_cast<__nv_bfloat16*>(grad_feats), na,
                   sb, reinterpret_cast<__nv_bfloat16*>(grad_depth), nb);
    else
      launch_after(convert2_kernel<__half>, blocks, threads, 0, st, sa, reinterpret_cast<__half*>(grad_feats), na, sb,
                   reinterpret_cast<__half*>(grad_depth), nb);
    if (cudaGetLastError() != cudaSuccess) return FBEV_ERR_LAUNCH;
  }
  return FBEV_OK;
}

int fbev_debug_indices(const FbevProblem* p, int32_t* u0, int32_t* v0, int32_t* kbin, uint8_t* valid, int32_t* count,
                       void* stream) {
  const int rc = validate(p);
  if (rc != FBEV_OK) return rc;
  if (!u0 || !v0 || !kbin || !valid || !count) return FBEV_ERR_NULL;
  if (p->compact_rows) return FBEV_ERR_SHAPE;  // the index dump covers whole grids
  Dev d;
  fill_dev(p, d);
  d.count = count;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int src = launch_softmax_stats(p, st);
  if (src != FBEV_OK) return src;
  const size_t cells = (size_t)p->B * p->Y * p->X;
  const int threads = 128;
  const int blocks = (int)((cells + threads - 1) / threads);
  switch (p->dtype) {
    case FBEV_F32: indices_kernel<float><<<blocks, threads, 0, st>>>(d, u0, v0, kbin, valid); break;
    case FBEV_BF16: indices_kernel<__nv_bfloat16><<<blocks, threads, 0, st>>>(d, u0, v0, kbin, valid); break;
    default: indices_kernel<__half><<<blocks, threads, 0, st>>>(d, u0, v0, kbin, valid); break;
  }
  return cudaGetLastError() == cudaSuccess ? FBEV_OK : FBEV_ERR_LAUNCH;
}

int fbev_flash_bevpool(int total_threads, int num_channels, int num_cameras, int batch_size, int num_extrinsic_params,
                       int num_intrinsic_params, int depth_distribution, int use_shared_memory,
                       int optimize_z_precompute, int use_warp_kernel, int use_vectorized_load, float epsilon,
                       float depth_weight_threshold, const float* depth_params, const float* image_feats,
                       const float* projection_matrices, const int* feature_size, const int* image_size, int grid_x,
                       int grid_y, int grid_z, float voxel_size_x, float voxel_size_y, float voxel_size_z,
                       float voxel_x_min, float voxel_y_min, float voxel_z_min, float* out, void* stream) {
  (void)total_threads; (void)num_extrinsic_params; (void)num_intrinsic_params; (void)use_shared_memory;
  (void)optimize_z_precompute; (void)use_warp_kernel; (void)use_vectorized_load;
  FbevProblem p{};
  p.struct_size = sizeof(FbevProblem);
  p.dtype = FBEV_F32;
  p.out_dtype = FBEV_F32;
  p.B = batch_size; p.N = num_cameras; p.C = num_channels;
  // The launcher is not told the tensor's H and W; like the reference it addresses with feature_size alone.
  p.H = 1; p.W = 1;
  p.D = 2;
  p.X = grid_x; p.Y = grid_y; p.Z = grid_z;
  p.proj_stride = 12;
  p.mode = depth_distribution == 1 ? FBEV_DEPTH_LAPLACE : FBEV_DEPTH_GAUSSIAN;
  p.pool = FBEV_POOL_MEAN;
  p.epsilon = epsilon; p.threshold = depth_weight_threshold;
  p.y_begin = 0; p.y_end = grid_y;
  p.voxel_size[0] = voxel_size_x; p.voxel_size[1] = voxel_size_y; p.voxel_size[2] = voxel_size_z;
  p.voxel_min[0] = voxel_x_min; p.voxel_min[1] = voxel_y_min; p.voxel_min[2] = voxel_z_min;
  p.image_feats = image_feats; p.depth = depth_params; p.projection = projection_matrices;
  p.feature_size = feature_size; p.image_size = image_size;
  return forward_impl(&p, out, nullptr, stream, true);
}

int fbev_flash_bevpool_grad(int total_threads, int num_channels, int num_cameras, int batch_size,
                            int num_extrinsic_params, int num_intrinsic_params, int depth_distribution, float epsilon,
                            float depth_weight_threshold, const float* out_grad, const float* depth_params,
                            const float* image_feats, const float* projection_matrices, const int* feature_size,
                            const int* image_size, const float* roi_range, int grid_x, int grid_y, int grid_z,
                            float* depth_params_grad, float* image_feats_grad, int feat_h, int feat_w, void* stream) {
  (void)total_threads; (void)num_extrinsic_params; (void)num_intrinsic_params;
  FbevProblem p{};
  p.struct_size = sizeof(FbevProblem);
  p.dtype = FBEV_F32;
  p.out_dtype = FBEV_F32;
  p.B = batch_size; p.N = num_cameras; p.C = num_channels; p.H = feat_h; p.W = feat_w; p.D = 2;
  p.X = grid_x; p.Y = grid_y; p.Z = grid_z;
  p.proj_stride = 12;
  p.mode = depth_distribution == 1 ? FBEV_DEPTH_LAPLACE : FBEV_DEPTH_GAUSSIAN;
  p.pool = FBEV_POOL_MEAN;
  p.epsilon = epsilon; p.threshold = depth_weight_threshold;
  p.y_begin = 0; p.y_end = grid_y;
  p.image_feats = image_feats; p.depth = depth_params; p.projection = projection_matrices;
  p.feature_size = feature_size; p.image_size = image_size; p.roi_range = roi_range;
  if (roi_range == nullptr) return FBEV_ERR_NULL;
  return fbev_backward(&p, out_grad, image_feats_grad, depth_params_grad, nullptr, 0,
                       FBEV_BWD_FEATS | FBEV_BWD_DEPTH | FBEV_BWD_LEGACY_DEPTH, stream);
}

int fbev_projection_matrices(const float* sensor2ego, const float* camera2imgs, const float* post_rots,
                             const float* post_trans, float* out, int count, void* stream) {
  if (!sensor2ego || !camera2imgs || !post_rots || !post_trans || !out) return FBEV_ERR_NULL;
  if (count <= 0) return FBEV_ERR_SHAPE;
  if (((uintptr_t)sensor2ego | (uintptr_t)camera2imgs | (uintptr_t)post_rots | (uintptr_t)post_trans | (uintptr_t)out) % 4)
    return FBEV_ERR_ALIGN;
  projection_kernel<<<(count + 63) / 64, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(sensor2ego, camera2imgs, post_rots,
                                                                                           post_trans, out, count);
  return cudaGetLastError() == cudaSuccess ? FBEV_OK : FBEV_ERR_LAUNCH;
}

int fbev_pillar_pool(int c, int n_intervals, const float* depth, const float* feat, const float* u_coords,
                     const float* v_coords, const float* z_coords, const int* batch_camera_indices, const int* ranks_bev,
                     const int* interval_starts, const int* interval_lengths, int batch_size, int num_cameras, int feat_h,
                     int feat_w, float epsilon, int depth_distribution, float* out, void* stream) {
  (void)batch_size; (void)num_cameras;  // the camera index of a sample already counts batch * cameras + camera
  if (n_intervals == 0) return FBEV_OK;
  if (!depth || !feat || !u_coords || !v_coords || !z_coords || !batch_camera_indices || !ranks_bev || !interval_starts ||
      !interval_lengths || !out)
    return FBEV_ERR_NULL;
  if (c <= 0 || n_intervals < 0 || feat_h <= 0 || feat_w <= 0) return FBEV_ERR_SHAPE;
  if (((uintptr_t)depth % 8) || ((uintptr_t)feat % 4) || ((uintptr_t)out % 4) || ((uintptr_t)u_coords % 4) ||
      ((uintptr_t)v_coords % 4) || ((uintptr_t)z_coords % 4) || ((uintptr_t)batch_camera_indices % 4) ||
      ((uintptr_t)ranks_bev % 4) || ((uintptr_t)interval_starts % 4) || ((uintptr_t)interval_lengths % 4))
    return FBEV_ERR_ALIGN;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool vec = c % 4 == 0 && (uintptr_t)feat % 16 == 0;
  const long long threads = (long long)n_intervals * (vec ? c / 4 : c);
  if ((threads + 255) / 256 >= (1ll << 31)) return FBEV_ERR_RANGE;
  const unsigned blocks = (unsigned)((threads + 255) / 256);
  const int laplace = depth_distribution == 1 ? 1 : 0;
  if (vec)
    pillar_pool_kernel<4><<<blocks, 256, 0, st>>>(c, n_intervals, depth, feat, u_coords, v_coords, z_coords, batch_camera_indices,
                                                  ranks_bev, interval_starts, interval_lengths, feat_h, feat_w, epsilon, laplace, out);
  else
    pillar_pool_kernel<1><<<blocks, 256, 0, st>>>(c, n_intervals, depth, feat, u_coords, v_coords, z_coords, batch_camera_indices,
                                                  ranks_bev, interval_starts, interval_lengths, feat_h, feat_w, epsilon, laplace, out);
  return cudaGetLastError() == cudaSuccess ? FBEV_OK : FBEV_ERR_LAUNCH;
}

int fbev_probe_read(const void* buf, size_t bytes, int repeats, void* sink, void* stream) {
  if (buf == nullptr || sink == nullptr) return FBEV_ERR_NULL;
  if (((uintptr_t)buf % 16) || ((uintptr_t)sink % 4)) return FBEV_ERR_ALIGN;
  probe_read_kernel<<<148 * 8, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(buf), bytes / 16, repeats, reinterpret_cast<unsigned*>(sink));
  return cudaGetLastError() == cudaSuccess ? FBEV_OK : FBEV_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------
// Backward without caller scratch
// ---------------------------------------------------------------------------
// Float32 accumulation area for 16-bit gradients that lives inside the library image.  Every GPU
// that loads libfbev.so carries these bytes until the process exits, which is why the size is kept
// small.  In host code the symbol below is only a handle: the device address must be asked for with
// cudaGetSymbolAddress on the device in use (done once per device in fbev_backward_static_scratch).
#define FBEV_STATIC_SCRATCH_LIMIT ((size_t)FBEV_STATIC_SCRATCH_BYTES)
static __device__ __align__(256) unsigned char g_fbev_static_scratch[FBEV_STATIC_SCRATCH_BYTES];
static void* g_fbev_static_scratch_addr[64] = {nullptr};  // device address of the array, per device ordinal
static std::mutex g_fbev_static_scratch_lock;                // guards the table above

int fbev_backward_static_scratch(const FbevProblem* p, const void* grad_out, void* grad_feats, void* grad_depth,
                                 int flags, void* stream) {
  const int rc = validate(p);
  if (rc != FBEV_OK) return rc;
  const size_t need = scratch_min_bytes(p, flags);  // the entry lists of the sorted gradient are used when they fit too
  if (need > FBEV_STATIC_SCRATCH_LIMIT) return FBEV_ERR_STATIC_LIMIT;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return FBEV_ERR_NO_DEVICE;
  }
  void* addr = nullptr;
  {
    std::lock_guard<std::mutex> g(g_fbev_static_scratch_lock);
    if (g_fbev_static_scratch_addr[dev] == nullptr) {
      // first call on this device: resolve the array's address in this device's copy of the module
      void* found = nullptr;
      if (cudaGetSymbolAddress(&found, g_fbev_static_scratch) != cudaSuccess || found == nullptr) {
        cudaGetLastError();
        return FBEV_ERR_LAUNCH;
      }
      g_fbev_static_scratch_addr[dev] = found;
    }
    addr = g_fbev_static_scratch_addr[dev];
  }
  // fbev_backward clears the part of the scratch it accumulates into, so what an earlier call left
  // behind is never read
  return fbev_backward(p, grad_out, grad_feats, grad_depth, addr, FBEV_STATIC_SCRATCH_LIMIT, flags, stream);
}

}  // extern "C"
