// Backward kernels: feature gradient by direct reductions or entry emission (bwd_feats_kernel), per-tile sort
// (bwd_feats_sorted_kernel), depth gradient on row records (bwd_depth_kernel), the per-sample kernel
// (bwd_kernel), the scalar kernel for any shape (bwd_generic_kernel) and the float32 -> 16-bit conversion.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fbev.h"
#include "fbev_lists.cuh"

namespace fbev {

__device__ __forceinline__ void red_add4(float* addr, float a, float b, float c, float d) {
  // one 16-byte reduction instead of four scalar ones (sm_90+)
  atomicAdd(reinterpret_cast<float4*>(addr), make_float4(a, b, c, d));
}

// Sum over the GL lanes of a group; the result is valid in the group's first lane.
__device__ __forceinline__ float group_sum(float v, int lg, int GL) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float o = __shfl_down_sync(kFull, v, off);
    if (lg + off < GL) v += o;
  }
  return v;
}

// Feature-gradient kernel: the forward kernel run backwards.  It builds the same merged row records
// (texel pair, summed weights with the depth weight folded in) and, instead of gathering, adds
//   d_feats[texel, c] += g_c * inv * weight          (flash_bevpool_cuda.cu:665,676-679)
// with one 16-byte float32 reduction per chunk and texel.  Merging the height bins that share a feature
// row cuts the number of reductions, which is what bounds this kernel, by the same factor as the
// forward's gathers; no feature is read at all.  inv = 1/count for mean pooling, 1 for sum.

// Adds the contributions of one cell's row records to the float32 feature gradient; go holds this lane's
// chunks of the cell's upstream gradient, already times 1/count.
template <typename T, int V>
__device__ __forceinline__ void add_records_direct(const Dev& p, const uint4* rec, int n, const float* go, float* gl) {
  constexpr int E = Chunk<T>::E;
  for (int i = 0; i < n; ++i) {
    const uint4 r = rec[i];
    const float w0 = __uint_as_float(r.z), w1 = __uint_as_float(r.w);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      float* d0 = gl + (size_t)(r.x + j * p.GL) * E;
      float* d1 = gl + (size_t)(r.x + r.y + j * p.GL) * E;
#pragma unroll
      for (int e4 = 0; e4 < E; e4 += 4) {
        const float g0 = go[j * E + e4], g1 = go[j * E + e4 + 1], g2 = go[j * E + e4 + 2], g3 = go[j * E + e4 + 3];
        red_add4(d0 + e4, g0 * w0, g1 * w0, g2 * w0, g3 * w0);
        if (r.y != 0u) {
          red_add4(d1 + e4, g0 * w1, g1 * w1, g2 * w1, g3 * w1);
        } else {  // u1 == u0 (last column): both weights belong to the same texel
          red_add4(d0 + e4, g0 * w1, g1 * w1, g2 * w1, g3 * w1);
        }
      }
    }
  }
}

// The contributions of one cell's row records as 64-bit fixed-point integers (reproducible backward, for the warps
// that find the entry list full): p.gfeat holds int64 sums, go the lane's chunks of the cell's upstream gradient as
// loaded, lg the lane's position in its group, scale the fixed-point scale of d_feats.  Every term is formed exactly
// as the entry path forms it -- emit_entries' weight (times 1 / count, both weights merged when the record has one
// texel), times the scale, times g, rounded to an integer -- because which warps end up here depends on the order
// the warps drew their slots in, and the result must not.
template <typename T, int V>
__device__ __forceinline__ void add_records_fixed(const Dev& p, const uint4* rec, int n, const float* go, float inv_cell,
                                                  int lg, float scale) {
  constexpr int E = Chunk<T>::E;
  unsigned long long* gf = reinterpret_cast<unsigned long long*>(p.gfeat);
  for (int i = 0; i < n; ++i) {
    const uint4 r = rec[i];
    const float a = __uint_as_float(r.z) * inv_cell, b = __uint_as_float(r.w) * inv_cell;
    const bool two = r.y != 0u;
    const float w0 = (two ? a : a + b) * scale, w1 = (two ? b : 0.0f) * scale;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const size_t e0 = (size_t)(r.x + j * p.GL + lg) * E, e1 = (size_t)(r.x + r.y + j * p.GL + lg) * E;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        atomicAdd(gf + e0 + e, (unsigned long long)__float2ll_rn(w0 * go[j * E + e]));
        if (two) atomicAdd(gf + e1 + e, (unsigned long long)__float2ll_rn(w1 * go[j * E + e]));
      }
    }
  }
}

// Entry emission of the sorted gradients, for the whole warp: every row record of the warp's cells leaves one
// entry {texel of (row, u0), cell, weight of u0 * inv, weight of u1 * inv} in p.ent and, in p.ent_pos, the
// position it drew inside its texel's segment.  Slots come from p.ent_count (one atomic per call), positions
// from p.tex_count.  rec / n / cell / inv_cell describe this lane's cell (n = 0 for lanes without one), sLen the
// list lengths of all cells of the warp.  first_slot: record i of the lane's cell owns slot first_slot + i.
// Returns false, having stored nothing, when the list is full.
__device__ __forceinline__ bool emit_entries(const Dev& p, const uint4* rec, int n, int g, int lg, int lane, unsigned cell,
                                             float inv_cell, const int* sLen, unsigned ucpt, unsigned* first_slot = nullptr) {
  int before = 0, total = 0;  // records of the cells before mine in this warp, and of the whole warp
  for (int c = 0; c < p.CPW; ++c) {
    const int lc = sLen[c];
    before += c < g ? lc : 0;
    total += lc;
  }
  unsigned base = 0;
  if (lane == 0 && total > 0) base = atomicAdd(p.ent_count, (unsigned)total);
  base = __shfl_sync(kFull, base, 0);
  if ((unsigned long long)base + (unsigned)total > (unsigned long long)p.ent_cap) {
    // the slots drawn stay unused: ent_scatter_kernel skips what lies beyond the capacity, and the part of
    // this reservation below it is marked void
    if (lane == 0 && base < p.ent_cap)
      for (unsigned k = base; k < p.ent_cap; ++k) p.ent[k] = make_uint4(0xffffffffu, 0u, 0u, 0u);
    return false;
  }
  const unsigned slot0 = base + (unsigned)before;
  if (first_slot != nullptr) *first_slot = slot0;
  int nmax = n;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) nmax = max(nmax, __shfl_xor_sync(kFull, nmax, off));
  const unsigned lt_mask = (1u << lane) - 1u;
  // lanes with the same group-local index hold the same record of neighbouring cells, which mostly lies on the
  // same texel: lanes with equal texels draw their positions with one atomic between them
  for (int i0 = 0; i0 < nmax; i0 += p.GL) {
    const int i = i0 + lg;
    const bool valid = i < n;
    uint4 r = make_uint4(0u, 0u, 0u, 0u);
    if (valid) r = rec[i];
    const unsigned tex0 = r.x / ucpt;
    const unsigned key = valid ? tex0 : 0xffffffffu - (unsigned)lane;
    const unsigned peers = __match_any_sync(kFull, key);
    const int lead = __ffs((int)peers) - 1;
    unsigned old = 0;
    if (valid && lane == lead) old = atomicAdd(p.tex_count + tex0, (unsigned)__popc(peers));
    old = __shfl_sync(kFull, old, lead) + (unsigned)__popc(peers & lt_mask);
    if (valid) {
      const float w0 = __uint_as_float(r.z) * inv_cell, w1 = __uint_as_float(r.w) * inv_cell;
      const bool two = r.y != 0u;  // u1 == u0 (last column): both weights belong to u0
      p.ent[slot0 + i] = make_uint4(tex0, cell, __float_as_uint(two ? w0 : w0 + w1), __float_as_uint(two ? w1 : 0.0f));
      p.ent_pos[slot0 + i] = old;
    }
  }
  return true;
}

// EMIT: instead of adding to global memory, every record leaves an entry in p.ent (emit_entries) and is counted
// per texel in p.tex_count; tex_scan_kernel, ent_scatter_kernel and feats_gather_kernel finish the job.  A warp whose
// entries do not fit the array any more adds its contributions directly, as without EMIT.
template <typename T, int V, bool EMIT>
__global__ void __launch_bounds__(kMaxWarps * 32, 3) bwd_feats_kernel(const __grid_constant__ Dev p) {
  constexpr int E = Chunk<T>::E;
  extern __shared__ __align__(16) unsigned char smem[];
  const BlockHeader h = carve(smem, p.N);
  __shared__ int s_tile[2];
  float vs[3], vmin[3];
  voxel_frame(p, vs, vmin);
  const int image_h = __ldg(p.isize), image_w = __ldg(p.isize + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  unsigned char* wa = h.warp_area + (size_t)warp * fwd_warp_bytes(p.CPW, p.cap);
  int* sLen = reinterpret_cast<int*>(wa);
  int* sCnt = sLen + 32;
  uint4* recs = reinterpret_cast<uint4*>(wa + 256);
  const int rstride = row_stride(p.cap);

  const int g = lane / p.GL, lg = lane - g * p.GL;
  const bool lane_used = g < p.CPW;
  const int cpt = p.GL * V;
  const int tile_cells = p.TX * p.TY;
  const int ngroups = (tile_cells + p.CPW - 1) / p.CPW;
  float* gl = p.gfeat + (size_t)lg * E;  // this lane's chunk of texel 0 in the float32 gradient
  const bool mean_pool = p.pool == FBEV_POOL_MEAN;
  int loaded_b = -1;
  UnitLoop sched;
  sched.begin(p, s_tile, warp, nwarps);
  if (sched.stat) {  // the sample's matrices, once, by the whole block
    const Tile tt = tile_of(p, 0);
    (void)tile_visibility(p, tt, h, vs, vmin, image_h, image_w, loaded_b);
  }
  int g_first = 0, g_step = 1;
  for (int tile; (tile = sched.current(p, ngroups, warp, nwarps, g_first, g_step)) >= 0; sched.advance(p, nwarps)) {
    const Tile t = tile_of(p, tile);
    const unsigned vis = tile_visibility(p, t, h, vs, vmin, image_h, image_w, loaded_b);
    const int nvis = __popc(vis);
    const int ncand = nvis * p.Z;
    const bool single_pass = ncand <= p.cap;

    for (int grp = g_first; grp < ngroups; grp += g_step) {
      const int t0 = grp * p.CPW;
      const int tc = t0 + g;
      const int ly = tc / p.TX, lx = tc - ly * p.TX;
      const int x = t.x0 + lx, y = t.y0 + ly;
      const bool cell_ok = lane_used && tc < tile_cells && x < t.x1 && y < t.y1;

      float go[V * E];
#pragma unroll
      for (int i = 0; i < V * E; ++i) go[i] = 0.0f;
      const size_t cell = out_cell(p, t.b, y, x);
      if (!EMIT && cell_ok) {
#pragma unroll
        for (int j = 0; j < V; ++j) load_chunk<T>(p.gout, p.out_f32, cell * cpt + lg + j * p.GL, go + j * E);
      }
      float inv_cell = 1.0f;  // EMIT: 1 / count of this lane's cell (mean pooling)
      if (lane < p.CPW) sCnt[lane] = 0;
      __syncwarp();
      if (mean_pool && !single_pass) {
        // the count of all passes is needed before the first contribution leaves
        for (int r0 = 0; r0 < ncand; r0 += p.cap) {
          if (lane < p.CPW) sLen[lane] = 0;
          __syncwarp();
          row_list_phase<T, false>(p, t, h, vis, (unsigned)cpt, t0, r0, min(r0 + p.cap, ncand), vs, vmin, image_h,
                                   image_w, sLen, sCnt, recs, lane);
        }
        const int cnt = lane_used ? sCnt[g] : 0;
        const float inv = cnt > 0 ? __fdiv_rn(1.0f, (float)cnt) : 0.0f;
        inv_cell = inv;
#pragma unroll
        for (int i = 0; i < V * E; ++i) go[i] *= inv;
        __syncwarp();
      }

      for (int r0 = 0; r0 < ncand; r0 += p.cap) {
        if (lane < p.CPW) sLen[lane] = 0;
        __syncwarp();
        row_list_phase<T, true>(p, t, h, vis, (unsigned)cpt, t0, r0, min(r0 + p.cap, ncand), vs, vmin, image_h,
                                image_w, sLen, sCnt, recs, lane);
        if (mean_pool && single_pass) {
          const int cnt = lane_used ? sCnt[g] : 0;
          const float inv = cnt > 0 ? __fdiv_rn(1.0f, (float)cnt) : 0.0f;
          inv_cell = inv;
#pragma unroll
          for (int i = 0; i < V * E; ++i) go[i] *= inv;
        }
        const int n = cell_ok ? sLen[g] : 0;
        const uint4* rec = recs + (size_t)g * rstride;
        if (EMIT) {
          if (emit_entries(p, rec, n, g, lg, lane, (unsigned)cell, inv_cell, sLen, (unsigned)cpt)) {
            __syncwarp();
            continue;
          }
          if (cell_ok) {  // no room left in the entry list: add directly; the upstream gradient was not needed so far
#pragma unroll
            for (int j = 0; j < V; ++j) load_chunk<T>(p.gout, p.out_f32, cell * cpt + lg + j * p.GL, go + j * E);
#pragma unroll
            for (int k = 0; k < V * E; ++k) go[k] *= inv_cell;
          }
        }
        add_records_direct<T, V>(p, rec, n, go, gl);
        __syncwarp();
      }
      __syncwarp();
    }
  }  // tiles
  sched.end(p, nwarps);
  // from here on the next kernel's blocks may move in (they wait for this whole grid before touching its output);
  // triggering at the start instead lets them sit on the SMs for the whole run, which cost 25 % on large maps
  grid_dependency_trigger();
}

// ---------------------------------------------------------------------------
// Feature gradient, texel-stationary
// ---------------------------------------------------------------------------
// d_feats[texel, c] = sum over the cells that sampled the texel of  g_cell[c] * inv_cell * weight.
// A scatter with float atomics is bound by the atomic rate of the L2: neighbouring cells hit the same
// few texels (a 12 x 8 tile of cfg2 makes some 2000 texel updates on fewer than 100 distinct texels
// per camera).  This kernel therefore turns the scatter of a tile into a gather:
//   1. list phase as in the forward (merged row records), every record becomes two entries
//      {texel key, cell of the tile, weight} in a block-wide array;
//   2. the entries are counting-sorted by texel key (shared-memory integer atomics);
//   3. one lane group per texel walks that texel's entries, gathers the cells' upstream gradient
//      chunks (L1-resident: the tile's rows of dO) into float32 registers, and issues ONE 16-byte
//      reduction per chunk for the whole tile.
// Keys index the rectangles camera_rect() predicts per visible camera.  An entry outside its
// rectangle, a camera whose rectangle does not fit the key space, or an entry beyond the array's
// capacity is added to global memory directly by the lane that found it (slow, rare: only tiles right
// next to the rig have footprints that large).
constexpr int kFeatKeys = 3072;     // texel keys per tile (all visible cameras together)
constexpr int kFeatEntries = 4096;  // entries per tile

__host__ __device__ inline size_t feats_block_bytes() {
  return (size_t)kFeatEntries * 8 + (size_t)kFeatEntries * 2 + (size_t)(kFeatKeys + 1) * 4 + 64;
}

// Rectangle of feature texels the cells of a tile can touch in one camera, from the tile's eight box
// corners: u and v are ratios of affine functions of the voxel centre, so over a box on which the
// depth stays positive their extremes sit at the corners.  A hint only: every entry is checked.
__device__ __forceinline__ bool camera_rect(const float* P, int fh, int fw, float bx0, float bx1, float by0, float by1,
                                            float bz0, float bz1, int image_h, int image_w, int& r0, int& r1,
                                            int& c0, int& c1) {
  const float inf = __int_as_float(0x7f800000);
  float umin = inf, umax = -inf, vmin = inf, vmax = -inf;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const float x = (c & 1) ? bx1 : bx0, y = (c & 2) ? by1 : by0, z = (c & 4) ? bz1 : bz0;
    const float ld = fmaf(P[10], z, fmaf(P[9], y, P[8] * x)) + P[11];
    if (!(ld > 1e-2f)) return false;
    const float u = (fmaf(P[2], z, fmaf(P[1], y, P[0] * x)) + P[3]) / ld / (float)image_w * (float)fw;
    const float v = (fmaf(P[6], z, fmaf(P[5], y, P[4] * x)) + P[7]) / ld / (float)image_h * (float)fh;
    umin = fminf(umin, u);
    umax = fmaxf(umax, u);
    vmin = fminf(vmin, v);
    vmax = fmaxf(vmax, v);
  }
  if (!(umax >= -2.0f && umin <= (float)fw + 2.0f && vmax >= -2.0f && vmin <= (float)fh + 2.0f)) return false;
  c0 = max(0, (int)floorf(fmaxf(umin, 0.0f)) - 1);
  c1 = min(fw - 1, (int)floorf(fminf(umax, (float)fw)) + 2);
  r0 = max(0, (int)floorf(fmaxf(vmin, 0.0f)) - 1);
  r1 = min(fh - 1, (int)floorf(fminf(vmax, (float)fh)) + 2);
  return c0 <= c1 && r0 <= r1;
}

template <typename T, int V>
__global__ void __launch_bounds__(kMaxWarps * 32, 3) bwd_feats_sorted_kernel(const __grid_constant__ Dev p) {
  constexpr int E = Chunk<T>::E;
  extern __shared__ __align__(16) unsigned char smem[];
  const BlockHeader h = carve(smem, p.N);
  __shared__ int s_tile[2];
  __shared__ int4 s_rect[32];        // per camera: first row, first column, columns, first key (-1: no keys)
  __shared__ int s_rows[32];         // per camera: rows of the rectangle
  __shared__ unsigned s_texbase[32]; // per camera: texel index of (0, 0)
  __shared__ int s_nent, s_nkeys;
  __shared__ int s_wsum[kMaxWarps];
  float vs[3], vmin[3];
  voxel_frame(p, vs, vmin);
  const int image_h = __ldg(p.isize), image_w = __ldg(p.isize + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
  unsigned char* wa = h.warp_area + (size_t)warp * fwd_warp_bytes(p.CPW, p.cap);
  int* sLen = reinterpret_cast<int*>(wa);
  int* sCnt = sLen + 32;
  uint4* recs = reinterpret_cast<uint4*>(wa + 256);
  const int rstride = row_stride(p.cap);
  unsigned char* blk = h.warp_area + (size_t)nwarps * fwd_warp_bytes(p.CPW, p.cap);
  uint2* ent = reinterpret_cast<uint2*>(blk);                                     // {key | cell << 16, weight}
  unsigned short* order = reinterpret_cast<unsigned short*>(ent + kFeatEntries);  // entries sorted by key
  int* hist = reinterpret_cast<int*>(order + kFeatEntries);                       // counts, then offsets / ends

  const int g = lane / p.GL, lg = lane - g * p.GL;
  const bool lane_used = g < p.CPW;
  const int cpt = p.GL * V;  // 16-byte chunks per texel
  const int tile_cells = p.TX * p.TY;
  const int ngroups = (tile_cells + p.CPW - 1) / p.CPW;
  const float inv_tx = 1.0f / (float)p.TX;
  const bool mean_pool = p.pool == FBEV_POOL_MEAN;
  int loaded_b = -1;
  TileLoop loop;
  loop.begin(p, s_tile);
  for (int tile; (tile = loop.current(p)) >= 0; loop.advance()) {
    const Tile t = tile_of(p, tile);
    const unsigned vis = tile_visibility(p, t, h, vs, vmin, image_h, image_w, loaded_b);
    const int ncand = __popc(vis) * p.Z;
    const bool single_pass = ncand <= p.cap;

    // ---- key space: one rectangle per visible camera (warp 0); clear the counts ----
    if (warp == 0) {
      int r0 = 0, r1 = -1, c0 = 0, c1 = -1;
      bool have = false;
      if (lane < p.N && ((vis >> lane) & 1u)) {
        const float bx0 = centre(t.x0, vs[0], vmin[0]), bx1 = centre(t.x1 - 1, vs[0], vmin[0]);
        const float by0 = centre(t.y0, vs[1], vmin[1]), by1 = centre(t.y1 - 1, vs[1], vmin[1]);
        const float bz0 = centre(0, vs[2], vmin[2]), bz1 = centre(p.Z - 1, vs[2], vmin[2]);
        have = camera_rect(h.P + lane * 12, h.fs[lane * 2], h.fs[lane * 2 + 1], bx0, bx1, by0, by1, bz0, bz1, image_h,
                           image_w, r0, r1, c0, c1);
      }
      const int need = have ? (r1 - r0 + 1) * (c1 - c0 + 1) : 0;
      int base = 0, mine = -1;
      for (int n = 0; n < p.N; ++n) {  // cameras take their keys in index order; one that does not fit gets none
        const int sz = __shfl_sync(kFull, need, n);
        const bool fits = sz > 0 && base + sz <= kFeatKeys;
        if (n == lane && fits) mine = base;
        if (fits) base += sz;
      }
      if (lane < p.N) {
        s_rect[lane] = make_int4(r0, c0, c1 - c0 + 1, mine);
        s_rows[lane] = r1 - r0 + 1;
        s_texbase[lane] = (unsigned)(((size_t)t.b * p.N + lane) * (size_t)h.fs[lane * 2] * h.fs[lane * 2 + 1]);
      }
      if (lane == 0) {
        s_nkeys = base;
        s_nent = 0;
      }
    }
    for (int i = tid; i <= kFeatKeys; i += blockDim.x) hist[i] = 0;
    __syncthreads();

    // ---- list phase per group, records -> entries ----
    for (int grp = warp; grp < ngroups; grp += nwarps) {
      const int t0 = grp * p.CPW;
      if (lane < p.CPW) sCnt[lane] = 0;
      __syncwarp();
      float inv_of_lane = 1.0f;  // lane c keeps 1 / count of cell c of the group (mean pooling)
      if (mean_pool && !single_pass) {
        for (int r0 = 0; r0 < ncand; r0 += p.cap) {
          if (lane < p.CPW) sLen[lane] = 0;
          __syncwarp();
          row_list_phase<T, false>(p, t, h, vis, 1u, t0, r0, min(r0 + p.cap, ncand), vs, vmin, image_h, image_w, sLen,
                                   sCnt, recs, lane);
        }
        if (lane < p.CPW) inv_of_lane = sCnt[lane] > 0 ? __fdiv_rn(1.0f, (float)sCnt[lane]) : 0.0f;
      }
      for (int r0 = 0; r0 < ncand; r0 += p.cap) {
        if (lane < p.CPW) {
          sLen[lane] = 0;
          if (single_pass) sCnt[lane] = 0;
        }
        __syncwarp();
        // cpt = 1: the records hold the texel index and u1 - u0 themselves
        row_list_phase<T, true>(p, t, h, vis, 1u, t0, r0, min(r0 + p.cap, ncand), vs, vmin, image_h, image_w, sLen,
                                sCnt, recs, lane);
        if (mean_pool && single_pass && lane < p.CPW)
          inv_of_lane = sCnt[lane] > 0 ? __fdiv_rn(1.0f, (float)sCnt[lane]) : 0.0f;
        for (int c = 0; c < p.CPW; ++c) {
          const int n = sLen[c];
          const float inv = mean_pool ? __shfl_sync(kFull, inv_of_lane, c) : 1.0f;
          const int tc = t0 + c;  // cell of the tile
          for (int i = lane; i < n; i += 32) {
            const uint4 r = recs[(size_t)c * rstride + i];
            const unsigned tex = r.x, du = r.y;
            float w0 = __uint_as_float(r.z) * inv, w1 = __uint_as_float(r.w) * inv;
            if (du == 0u) {  // u1 == u0: one texel takes both weights
              w0 += w1;
              w1 = 0.0f;
            }
            // camera of the texel, its row and column
            int cam = -1;
            for (unsigned m = vis; m; m &= m - 1u) {
              const int n2 = __ffs((int)m) - 1;
              const unsigned tb = s_texbase[n2];
              if (tex >= tb && tex - tb < (unsigned)(h.fs[n2 * 2] * h.fs[n2 * 2 + 1])) cam = n2;
            }
            int key = -1;
            if (cam >= 0) {
              const int fw = h.fs[cam * 2 + 1];
              const int rel = (int)(tex - s_texbase[cam]);
              const int row = fast_div(rel, 1.0f / (float)fw), col = rel - row * fw;
              const int4 rc = s_rect[cam];
              const int lr = row - rc.x, lc = col - rc.y;
              if (rc.w >= 0 && lr >= 0 && lr < s_rows[cam] && lc >= 0 && lc + (int)du < rc.z) key = rc.w + lr * rc.z + lc;
            }
            const int want = 1 + (int)du;
            int slot = -1;
            if (key >= 0) {
              slot = atomicAdd(&s_nent, want);
              if (slot + want > kFeatEntries) {
                // array full: this record goes the direct way; a slot it reserved below the capacity is
                // marked void so that the sort never reads an unwritten entry
                if (slot < kFeatEntries) ent[slot] = make_uint2(0xffffu, 0u);
                slot = -1;
              }
            }
            if (slot >= 0) {
              ent[slot] = make_uint2((unsigned)key | ((unsigned)tc << 16), __float_as_uint(w0));
              atomicAdd(&hist[key], 1);
              if (du) {
                ent[slot + 1] = make_uint2((unsigned)(key + 1) | ((unsigned)tc << 16), __float_as_uint(w1));
                atomicAdd(&hist[key + 1], 1);
              }
            } else {
              // direct: this lane alone adds g * w to the record's texel(s), chunk by chunk
              const int ly = fast_div(tc, inv_tx), lx = tc - ly * p.TX;
              const size_t cell = out_cell(p, t.b, t.y0 + ly, t.x0 + lx);
              for (int ch = 0; ch < cpt; ++ch) {
                float gv[E];
                load_chunk<T>(p.gout, p.out_f32, cell * cpt + ch, gv);
                float* d0 = p.gfeat + ((size_t)tex * cpt + ch) * E;
#pragma unroll
                for (int e4 = 0; e4 < E; e4 += 4) {
                  red_add4(d0 + e4, gv[e4] * w0, gv[e4 + 1] * w0, gv[e4 + 2] * w0, gv[e4 + 3] * w0);
                  if (du)
                    red_add4(d0 + (size_t)cpt * E + e4, gv[e4] * w1, gv[e4 + 1] * w1, gv[e4 + 2] * w1, gv[e4 + 3] * w1);
                }
              }
            }
          }
        }
        __syncwarp();
      }
    }
    __syncthreads();

    // ---- counting sort of the entries by key ----
    const int nkeys = s_nkeys;
    const int nent = min(s_nent, kFeatEntries);
    {
      const int chunk = (nkeys + (int)blockDim.x - 1) / (int)blockDim.x;
      const int k0 = min(tid * chunk, nkeys), k1 = min(k0 + chunk, nkeys);
      int local = 0;
      for (int k = k0; k < k1; ++k) local += hist[k];
      int incl = local;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int o = __shfl_up_sync(kFull, incl, off);
        if (lane >= off) incl += o;
      }
      if (lane == 31) s_wsum[warp] = incl;
      __syncthreads();
      int run = incl - local;
      for (int w2 = 0; w2 < warp; ++w2) run += s_wsum[w2];
      for (int k = k0; k < k1; ++k) {  // counts -> first position of each key
        const int c = hist[k];
        hist[k] = run;
        run += c;
      }
    }
    __syncthreads();
    for (int e = tid; e < nent; e += blockDim.x) {
      const int key = (int)(ent[e].x & 0xffffu);
      if (key < nkeys) order[atomicAdd(&hist[key], 1)] = (unsigned short)e;  // afterwards hist[key] = end of the key's entries
    }
    __syncthreads();

    // ---- one lane group per texel: gather the cells' gradients, one reduction per chunk ----
    const int G = nwarps * p.CPW;
    for (int k = warp * p.CPW + g; k < nkeys + G; k += G) {  // same trip count for every lane of a warp
      if (!(lane_used && k < nkeys)) continue;
      const int start = k > 0 ? hist[k - 1] : 0, end = hist[k];
      if (end <= start) continue;
      float acc[V * E];
#pragma unroll
      for (int i = 0; i < V * E; ++i) acc[i] = 0.0f;
      for (int e = start; e < end; ++e) {
        const uint2 en = ent[order[e]];
        const int tc = (int)(en.x >> 16);
        const float w = __uint_as_float(en.y);
        const int ly = fast_div(tc, inv_tx), lx = tc - ly * p.TX;
        const size_t cell = out_cell(p, t.b, t.y0 + ly, t.x0 + lx);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          float gv[E];
          load_chunk<T>(p.gout, p.out_f32, cell * cpt + lg + j * p.GL, gv);
#pragma unroll
          for (int e2 = 0; e2 < E; ++e2) acc[j * E + e2] = fmaf(w, gv[e2], acc[j * E + e2]);
        }
      }
      // texel of the key
      unsigned tex = 0;
      for (unsigned m = vis; m; m &= m - 1u) {
        const int n2 = __ffs((int)m) - 1;
        const int4 rc = s_rect[n2];
        if (rc.w >= 0 && k >= rc.w && k < rc.w + s_rows[n2] * rc.z) {
          const int rel = k - rc.w;
          const int lr = fast_div(rel, 1.0f / (float)rc.z), lc = rel - lr * rc.z;
          tex = s_texbase[n2] + (unsigned)((rc.x + lr) * h.fs[n2 * 2 + 1] + rc.y + lc);
        }
      }
#pragma unroll
      for (int j = 0; j < V; ++j) {
        float* d0 = p.gfeat + ((size_t)tex * cpt + lg + j * p.GL) * E;
#pragma unroll
        for (int e4 = 0; e4 < E; e4 += 4)
          red_add4(d0 + e4, acc[j * E + e4], acc[j * E + e4 + 1], acc[j * E + e4 + 2], acc[j * E + e4 + 3]);
      }
    }
  }  // tiles
  loop.end(p);
}

// Depth-gradient kernel.  For every accepted sample
//   parametric, analytic:  d_mean_ij  += inv * S * dwgt/dmean  * w_ij,  d_sigma_ij += inv * S * dwgt/dsigma * w_ij
//   parametric, legacy:    both slots += inv * S * wgt * w_ij                          (flash_bevpool_cuda.cu:667-674)
//   categorical:           d_prob[corner_ij, k] += inv * S * w_ij
// with S = sum_c g_c f_c, f the bilinearly interpolated feature.  S is linear in the four corner
// texels, S = sum_ij w_ij T_ij with T = <g, feature of the texel>, and the samples of a cell share
// their texels exactly as in the forward.  So the kernel builds the forward's row records, computes T
// once per record texel (two gathers, a dot product, a shuffle reduction over the group's lanes) and
// then lets one lane per SAMPLE combine four T values and issue that sample's atomics.  Compared with
// evaluating S per sample this reads 2.7 times fewer texels and spreads the atomics over all lanes.

// EMIT: the kernel also leaves the entries of the sorted feature gradient (emit_entries) from the same row
// records, so that one list phase serves both gradients.
// CAT: categorical depth (compile-time so that each of the two kernels below carries only its own sample pass).
// SAVED: the lists come from the saved state of a training forward (load_pass) and the instantiation carries no
// list-phase code at all, which is most of the other one's registers.  Whether the state is usable is decided once
// per launch (saved_usable); the host launches both instantiations when it has a state to offer and exactly one of
// them does the work: this one when the state is complete and in its layout, the rebuilding one otherwise.
// DET: reproducible sums (fbev_deterministic.cuh): p.gfeat / p.gdepth are int64 fixed-point arrays, every addition to
// them is an integer atomic at the scales in p.det, and the parametric depth gradient takes the per-sample path (the
// per-record one sums in shared memory with float atomics, whose order inside a warp instruction is not specified).
template <typename T, int V, bool EMIT, bool CAT, bool SAVED = false, bool DET = false>
__device__ __forceinline__ void bwd_depth_body(const Dev& p) {
  constexpr int E = Chunk<T>::E;
  if (saved_usable(p) != SAVED) {  // the other instantiation's launch does the work
    grid_dependency_trigger();
    return;
  }
  extern __shared__ __align__(16) unsigned char smem[];
  const BlockHeader h = carve(smem, p.N);
  __shared__ int s_tile[2];
  float vs[3], vmin[3];
  voxel_frame(p, vs, vmin);
  const int image_h = __ldg(p.isize), image_w = __ldg(p.isize + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  unsigned char* wa = h.warp_area + (size_t)warp * depth_warp_bytes(p.CPW, p.cap);
  int* sLen = reinterpret_cast<int*>(wa);  // [32] row records per cell
  int* sCnt = sLen + 32;                    // [32] accepted samples per cell, all passes
  int* sSmp = sCnt + 32;                    // [32] sample records per cell, this pass
  const int rstride = row_stride(p.cap);
  uint4* recs = reinterpret_cast<uint4*>(wa + 512);
  uint4* samp = recs + (size_t)p.CPW * rstride;

  const int g = lane / p.GL, lg = lane - g * p.GL;
  const bool lane_used = g < p.CPW;
  const int cpt = p.GL * V;
  const int tile_cells = p.TX * p.TY;
  const int ngroups = (tile_cells + p.CPW - 1) / p.CPW;
  const uint4* fl = reinterpret_cast<const uint4*>(p.feats) + lg;
  const bool legacy = (p.flags & FBEV_BWD_LEGACY_DEPTH) != 0;
  const bool mean_pool = p.pool == FBEV_POOL_MEAN;
  const bool depth_entries = p.ent_d != nullptr;
  const bool by_record = !DET && (p.flags & FBEV_BWD_DEPTH) != 0 && (!EMIT || depth_entries || (p.flags & kBwdRecordAtomics) != 0);
  const float scale_f = DET ? p.det->scale_f : 0.0f, scale_d = DET ? p.det->scale_d : 0.0f;
  long long* gd64 = reinterpret_cast<long long*>(p.gdepth);
  // categorical: sum equal (texel, bin) neighbours before the atomics.  Pays with six cells per warp (the scan's
  // fixed cost is shared by many samples and the depth tensor is small enough for its atomics to contend);
  // measured a loss with two or three cells per warp on large feature maps
  const bool merge_bins = p.CPW >= 4;
  int* sOff = sSmp + 32;                    // [2 x 9] SAVED: start offsets of the cells' lists in a saved block
  int loaded_b = -1;
  UnitLoop sched;
  sched.begin(p, s_tile, warp, nwarps);
  if (sched.stat) {  // the sample's matrices, once, by the whole block
    const Tile tt = tile_of(p, 0);
    (void)tile_visibility(p, tt, h, vs, vmin, image_h, image_w, loaded_b);
  }
  int g_first = 0, g_step = 1;
  for (int tile; (tile = sched.current(p, ngroups, warp, nwarps, g_first, g_step)) >= 0; sched.advance(p, nwarps)) {
    const Tile t = tile_of(p, tile);
    const unsigned vis = tile_visibility(p, t, h, vs, vmin, image_h, image_w, loaded_b);
    const int ncand = __popc(vis) * p.Z;
    const bool single_pass = ncand <= p.cap;

    for (int grp = g_first; grp < ngroups; grp += g_step) {
      const int t0 = grp * p.CPW;
      const int tc = t0 + g;
      const int ly = tc / p.TX, lx = tc - ly * p.TX;
      const int x = t.x0 + lx, y = t.y0 + ly;
      const bool cell_ok = lane_used && tc < tile_cells && x < t.x1 && y < t.y1;

      float go[V * E];
#pragma unroll
      for (int i = 0; i < V * E; ++i) go[i] = 0.0f;
      if (cell_ok) {
        const size_t cell = out_cell(p, t.b, y, x);
#pragma unroll
        for (int j = 0; j < V; ++j) load_chunk<T>(p.gout, p.out_f32, cell * cpt + lg + j * p.GL, go + j * E);
      }
      if (lane < p.CPW) sCnt[lane] = 0;
      __syncwarp();
      const unsigned unit = (unsigned)(tile * ngroups + grp);
      if (mean_pool && !single_pass) {  // the count of all passes is needed before the first contribution
        for (int r0 = 0; r0 < ncand; r0 += p.cap) {
          if (SAVED) {  // the saved pass knows its sample counts
            const uint4 entry = __ldg(saved_dir_entry(p, unit, r0 / p.cap));
            if (lane < p.CPW) sCnt[lane] += saved_cnt(entry, lane);
            __syncwarp();
            continue;
          }
          if (lane < p.CPW) sLen[lane] = 0;
          __syncwarp();
          if (!SAVED)
            row_list_phase<T, false>(p, t, h, vis, (unsigned)cpt, t0, r0, min(r0 + p.cap, ncand), vs, vmin, image_h,
                                     image_w, sLen, sCnt, recs, lane);
        }
      }
      // inverse count per cell of the group, kept by lane c for cell c
      float inv_of_lane = 1.0f;
      if (mean_pool && !single_pass && lane < p.CPW) {
        const int cnt = sCnt[lane];
        inv_of_lane = cnt > 0 ? __fdiv_rn(1.0f, (float)cnt) : 0.0f;
      }

      for (int r0 = 0; r0 < ncand; r0 += p.cap) {
        if (lane < p.CPW) {
          sLen[lane] = 0;
          sSmp[lane] = 0;
          if (single_pass) sCnt[lane] = 0;
        }
        __syncwarp();
        if (SAVED)
          load_pass(p, unit, r0 / p.cap, sLen, sCnt, sSmp, sOff, recs, samp, lane);
        else
          row_list_phase<T, true, true>(p, t, h, vis, (unsigned)cpt, t0, r0, min(r0 + p.cap, ncand), vs, vmin, image_h,
                                        image_w, sLen, sCnt, recs, lane, samp, sSmp);
        if (mean_pool && single_pass && lane < p.CPW) {
          const int cnt = sCnt[lane];
          inv_of_lane = cnt > 0 ? __fdiv_rn(1.0f, (float)cnt) : 0.0f;
        }
        const int n = cell_ok ? sLen[g] : 0;
        bool emitted = false;       // warp-uniform: this pass's records have slots in the entry list
        unsigned first_slot = 0;    // slots 2i, 2i+1 from here belong to record i of my cell
        if (EMIT) {
          const float inv_cell = __shfl_sync(kFull, inv_of_lane, g < p.CPW ? g : 0);
          const uint4* rec_e = recs + (size_t)g * rstride;
          const size_t cell = out_cell(p, t.b, y, x);
          emitted = emit_entries(p, rec_e, n, g, lg, lane, (unsigned)cell, inv_cell, sLen, (unsigned)cpt, &first_slot);
          if (!emitted && (p.flags & FBEV_BWD_FEATS)) {
            float gs[V * E];
#pragma unroll
            for (int k = 0; k < V * E; ++k) gs[k] = go[k] * inv_cell;
            if (DET)
              add_records_fixed<T, V>(p, rec_e, n, go, inv_cell, lg, scale_f);
            else
              add_records_direct<T, V>(p, rec_e, n, gs, p.gfeat + (size_t)lg * E);
          }
          __syncwarp();
        }
        // ---- T = <g, texel> for the two texels of every row record; stored over the record's weights ----
        int nmax = n;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) nmax = max(nmax, __shfl_xor_sync(kFull, nmax, off));
        uint4* rec = recs + (size_t)g * rstride;
        for (int i = 0; i < nmax; ++i) {
          float d0 = 0.0f, d1 = 0.0f;
          if (i < n) {
            const uint4 r = rec[i];
#pragma unroll
            for (int j = 0; j < V; ++j) {
              float f0[E], f1[E];
              Chunk<T>::unpack(ldg16(fl + (r.x + j * p.GL)), f0);
              Chunk<T>::unpack(ldg16(fl + (r.x + r.y + j * p.GL)), f1);
#pragma unroll
              for (int e = 0; e < E; ++e) {
                d0 = fmaf(go[j * E + e], f0[e], d0);
                d1 = fmaf(go[j * E + e], f1[e], d1);
              }
            }
          }
          d0 = group_sum(d0, lg, p.GL);
          d1 = group_sum(d1, lg, p.GL);
          if (i < n && lg == 0) {
            rec[i].z = __float_as_uint(d0);
            rec[i].w = __float_as_uint(d1);
          }
        }
        __syncwarp();
        if (!CAT && by_record) {
          // ---- parametric depth, per record: the samples of a run share their texels, so their (d mean,
          // d sigma) contributions are summed per record texel in shared memory first; the sums leave as the
          // depth part of the record's entries (summed per texel by feats_gather_kernel) or, without entry
          // slots, as one atomic per record texel ----
          for (int c = 0; c < p.CPW; ++c) {  // S * inv of every sample, kept in its record
            const int ns = sSmp[c];
            const float inv = mean_pool ? __shfl_sync(kFull, inv_of_lane, c) : 1.0f;
            const uint4* rc = recs + (size_t)c * rstride;
            for (int idx = lane; idx < ns; idx += 32) {
              uint4* sr = samp + ((size_t)c * p.cap + idx) * 3;
              const uint4 sw = sr[0];
              const unsigned pos = sr[2].x;
              const uint4 ra = rc[pos & 0xffffu], rb = rc[pos >> 16];
              float S = __uint_as_float(sw.x) * __uint_as_float(ra.z);
              S = fmaf(__uint_as_float(sw.z), __uint_as_float(ra.w), S);
              S = fmaf(__uint_as_float(sw.y), __uint_as_float(rb.z), S);
              S = fmaf(__uint_as_float(sw.w), __uint_as_float(rb.w), S);
              sr[1].x = __float_as_uint(S * inv);
            }
          }
          __syncwarp();
          if (emitted && depth_entries) {
            // the records' texel fields went into the entries already, so all four words of a record can hold
            // sums: d mean / d sigma of u0, d mean / d sigma of u1 -- one walk over the samples instead of two.
            // Which of my records have a second texel is remembered in a register first.
            unsigned two_bits = 0;
            for (int i = lg, k = 0; i < n; i += p.GL, ++k) two_bits |= (rec[i].y != 0u ? 1u : 0u) << k;
            __syncwarp();
            for (int c = 0; c < p.CPW; ++c) {
              uint4* rc = recs + (size_t)c * rstride;
              const int nr = sLen[c];
              for (int i = lane; i < nr; i += 32) rc[i] = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncwarp();
            for (int c = 0; c < p.CPW; ++c) {
              const int ns = sSmp[c];
              uint4* rc = recs + (size_t)c * rstride;
              for (int idx = lane; idx < ns; idx += 32) {
                const uint4* sr = samp + ((size_t)c * p.cap + idx) * 3;
                const uint4 sw = sr[0], sp = sr[2];
                const float sd = __uint_as_float(sr[1].x);
                const float vm = sd * (legacy ? __uint_as_float(sp.y) : __uint_as_float(sp.z));
                const float vs2 = sd * (legacy ? __uint_as_float(sp.y) : __uint_as_float(sp.w));
                float* a = reinterpret_cast<float*>(rc + (sp.x & 0xffffu));
                float* b = reinterpret_cast<float*>(rc + (sp.x >> 16));
                const float w00 = __uint_as_float(sw.x), w01 = __uint_as_float(sw.y), w10 = __uint_as_float(sw.z),
                            w11 = __uint_as_float(sw.w);
                atomicAdd(a + 0, vm * w00);   // (v0, u0)
                atomicAdd(a + 1, vs2 * w00);
                atomicAdd(a + 2, vm * w10);   // (v0, u1)
                atomicAdd(a + 3, vs2 * w10);
                atomicAdd(b + 0, vm * w01);   // (v1, u0)
                atomicAdd(b + 1, vs2 * w01);
                atomicAdd(b + 2, vm * w11);   // (v1, u1)
                atomicAdd(b + 3, vs2 * w11);
              }
            }
            __syncwarp();
            for (int i = lg, k = 0; i < n; i += p.GL, ++k) {
              const uint4 r = rec[i];
              const float m0 = __uint_as_float(r.x), s0 = __uint_as_float(r.y), m1 = __uint_as_float(r.z),
                          s1 = __uint_as_float(r.w);
              const bool two = (two_bits >> k) & 1u;
              p.ent_d[first_slot + (unsigned)i] = two ? make_float4(m0, s0, m1, s1) : make_float4(m0 + m1, s0 + s1, 0.0f, 0.0f);
            }
            __syncwarp();
            continue;
          }
          for (int which = 0; which < 2; ++which) {  // 0: d mean, 1: d sigma (no entry slots: one atomic per record texel)
            for (int c = 0; c < p.CPW; ++c) {
              uint4* rc = recs + (size_t)c * rstride;
              const int nr = sLen[c];
              for (int i = lane; i < nr; i += 32) rc[i].z = rc[i].w = 0u;
            }
            __syncwarp();
            for (int c = 0; c < p.CPW; ++c) {
              const int ns = sSmp[c];
              uint4* rc = recs + (size_t)c * rstride;
              for (int idx = lane; idx < ns; idx += 32) {
                const uint4* sr = samp + ((size_t)c * p.cap + idx) * 3;
                const uint4 sw = sr[0], sp = sr[2];
                const float sd = __uint_as_float(sr[1].x);
                const float coef = legacy ? __uint_as_float(sp.y) : __uint_as_float(which == 0 ? sp.z : sp.w);
                const float v = sd * coef;
                float* a = reinterpret_cast<float*>(rc + (sp.x & 0xffffu));
                float* b = reinterpret_cast<float*>(rc + (sp.x >> 16));
                atomicAdd(a + 2, v * __uint_as_float(sw.x));  // w00 -> (v0, u0)
                atomicAdd(a + 3, v * __uint_as_float(sw.z));  // w10 -> (v0, u1)
                atomicAdd(b + 2, v * __uint_as_float(sw.y));  // w01 -> (v1, u0)
                atomicAdd(b + 3, v * __uint_as_float(sw.w));  // w11 -> (v1, u1)
              }
            }
            __syncwarp();
            for (int i = lg; i < n; i += p.GL) {
              const uint4 r = rec[i];
              const float v0 = __uint_as_float(r.z), v1 = __uint_as_float(r.w);
              const bool two = r.y != 0u;
              if (emitted && depth_entries) {
                float* e = reinterpret_cast<float*>(p.ent_d + first_slot + (unsigned)i);
                e[which] = two ? v0 : v0 + v1;
                e[2 + which] = two ? v1 : 0.0f;
              } else {
                const unsigned tex = r.x / (unsigned)cpt;
                atomicAdd(p.gdepth + (size_t)tex * 2 + which, v0);
                atomicAdd(p.gdepth + (size_t)(tex + (two ? 1u : 0u)) * 2 + which, v1);
              }
            }
            __syncwarp();
          }
          continue;
        }
        // ---- one lane per sample: S from four T values, then the sample's atomics.  The samples of all cells of
        // the warp are walked as one list.  Categorical: neighbouring samples are the height bins of one camera
        // column, which mostly share the texel AND the depth bin (depth barely changes with height), so equal
        // (texel, bin) neighbours are summed with a segmented scan first and one lane adds for the run ----
        int ns_total = 0;
        for (int c = 0; c < p.CPW; ++c) ns_total += sSmp[c];
        const unsigned lt_mask = (1u << lane) - 1u;
        for (int base = 0; base < ns_total; base += 32) {
          int off = base + lane, c = 0;
          bool active = false;
          for (int cc = 0; cc < p.CPW; ++cc) {
            const int nsc = sSmp[cc];
            if (!active) {
              if (off < nsc) {
                c = cc;
                active = true;
              } else {
                off -= nsc;
              }
            }
          }
          const float inv = mean_pool ? __shfl_sync(kFull, inv_of_lane, c) : 1.0f;
          float v00 = 0.0f, v01 = 0.0f, v10 = 0.0f, v11 = 0.0f, cm = 0.0f, cs = 0.0f;
          uint4 sa = make_uint4(0u, 0u, 0u, 0u);
          if (active) {
            const uint4* rc = recs + (size_t)c * rstride;
            const uint4* sr = samp + ((size_t)c * p.cap + off) * 3;
            const uint4 sw = sr[0], sp = sr[2];
            sa = sr[1];
            const float w00 = __uint_as_float(sw.x), w01 = __uint_as_float(sw.y), w10 = __uint_as_float(sw.z),
                        w11 = __uint_as_float(sw.w);
            const uint4 ra = rc[sp.x & 0xffffu], rb = rc[sp.x >> 16];
            float S = w00 * __uint_as_float(ra.z);
            S = fmaf(w10, __uint_as_float(ra.w), S);
            S = fmaf(w01, __uint_as_float(rb.z), S);
            S = fmaf(w11, __uint_as_float(rb.w), S);
            const float sd = S * inv;
            v00 = sd * w00; v01 = sd * w01; v10 = sd * w10; v11 = sd * w11;
            const float wgt = __uint_as_float(sp.y);
            cm = legacy ? wgt : __uint_as_float(sp.z);
            cs = legacy ? wgt : __uint_as_float(sp.w);
          }
          float* d00 = p.gdepth + sa.x;
          float* d10 = d00 + sa.y;
          float* d01 = d00 + sa.z;
          float* d11 = d01 + sa.y;
          // the same four corners as element indices of the fixed-point array
          const size_t e00 = (size_t)sa.x, e10 = e00 + sa.y, e01 = e00 + sa.z, e11 = e01 + sa.y;
          if (CAT && !merge_bins) {
            if (active) {
              const int k = (int)sa.w;
              if (DET) {
                det_add(gd64, e00 + k, v00, scale_d);
                det_add(gd64, e01 + k, v01, scale_d);
                det_add(gd64, e10 + k, v10, scale_d);
                det_add(gd64, e11 + k, v11, scale_d);
              } else {
                atomicAdd(d00 + k, v00);
                atomicAdd(d01 + k, v01);
                atomicAdd(d10 + k, v10);
                atomicAdd(d11 + k, v11);
              }
            }
          } else if (CAT) {
            const unsigned key = active ? sa.x + sa.w : 0xffffffffu - (unsigned)lane;  // element index of (texel, bin)
            const unsigned pkey = __shfl_up_sync(kFull, key, 1);
            const unsigned headm = __ballot_sync(kFull, active && (lane == 0 || pkey != key));
            const int rs = 31 - __clz((int)(headm & (lt_mask | (1u << lane))));
            for (int d = 1; d < 32 && d < p.Z; d <<= 1) {
              const float a = __shfl_up_sync(kFull, v00, d), b = __shfl_up_sync(kFull, v01, d);
              const float e = __shfl_up_sync(kFull, v10, d), f = __shfl_up_sync(kFull, v11, d);
              if (active && lane - d >= rs) {
                v00 += a; v01 += b; v10 += e; v11 += f;
              }
            }
            const unsigned actm = __ballot_sync(kFull, active);
            const bool tail = active && (lane == 31 || ((headm >> (lane + 1)) & 1u) || !((actm >> (lane + 1)) & 1u));
            if (tail) {
              const int k = (int)sa.w;
              if (DET) {  // the run's sums were formed by fixed lanes in a fixed order
                det_add(gd64, e00 + k, v00, scale_d);
                det_add(gd64, e01 + k, v01, scale_d);
                det_add(gd64, e10 + k, v10, scale_d);
                det_add(gd64, e11 + k, v11, scale_d);
              } else {
                atomicAdd(d00 + k, v00);
                atomicAdd(d01 + k, v01);
                atomicAdd(d10 + k, v10);
                atomicAdd(d11 + k, v11);
              }
            }
          } else if (active) {
            if (DET) {
              det_add(gd64, e00, cm * v00, scale_d);
              det_add(gd64, e00 + 1, cs * v00, scale_d);
              det_add(gd64, e01, cm * v01, scale_d);
              det_add(gd64, e01 + 1, cs * v01, scale_d);
              det_add(gd64, e10, cm * v10, scale_d);
              det_add(gd64, e10 + 1, cs * v10, scale_d);
              det_add(gd64, e11, cm * v11, scale_d);
              det_add(gd64, e11 + 1, cs * v11, scale_d);
            } else {
              atomicAdd(d00 + 0, cm * v00);
              atomicAdd(d00 + 1, cs * v00);
              atomicAdd(d01 + 0, cm * v01);
              atomicAdd(d01 + 1, cs * v01);
              atomicAdd(d10 + 0, cm * v10);
              atomicAdd(d10 + 1, cs * v10);
              atomicAdd(d11 + 0, cm * v11);
              atomicAdd(d11 + 1, cs * v11);
            }
          }
        }
        __syncwarp();
      }
      __syncwarp();
    }
  }  // tiles
  sched.end(p, nwarps);
  // from here on the next kernel's blocks may move in (they wait for this whole grid before touching its output);
  // triggering at the start instead lets them sit on the SMs for the whole run, which cost 25 % on large maps
  grid_dependency_trigger();
}

// The two depth-gradient kernels.  Categorical: 96 registers, five resident blocks per SM (no spills; measured 4 %
// ahead of 80 registers / six blocks on the benchmark shape, 9 % on cfg4).  Parametric: 80 registers / six blocks,
// which its shared-memory sample pass prefers (96 registers cost it 8 % on the benchmark shape).
template <typename T, int V, bool EMIT, bool SAVED = false, bool DET = false>
__global__ void __maxnreg__(96) bwd_depth_kernel(const __grid_constant__ Dev p) {
  bwd_depth_body<T, V, EMIT, true, SAVED, DET>(p);
}
template <typename T, int V, bool EMIT, bool SAVED = false, bool DET = false>
__global__ void __launch_bounds__(kMaxWarps * 32, 3) bwd_depth_param_kernel(const __grid_constant__ Dev p) {
  bwd_depth_body<T, V, EMIT, false, SAVED, DET>(p);
}

// Gradient kernel.  Same decomposition as the forward.  For every accepted sample
//   d_feats[corner_ij, c] += g_c * wgt * inv * w_ij          (flash_bevpool_cuda.cu:665,676-679)
//   parametric, analytic:  d_mean_ij  += inv * (sum_c g_c f_c) * dwgt/dmean  * w_ij
//                          d_sigma_ij += inv * (sum_c g_c f_c) * dwgt/dsigma * w_ij
//   parametric, legacy:    both slots += inv * wgt * (sum_c g_c f_c) * w_ij  (:667-674)
//   categorical:           d_prob[corner_ij, k] += inv * (sum_c g_c f_c) * w_ij
// with f_c the bilinearly interpolated feature and inv = 1/count (mean) or 1 (sum).
// Feature gradients leave as 16-byte float32 reductions, depth gradients as scalar
// atomics from the first lane of each group after a shuffle reduction over channels.
template <typename T, int V>
__global__ void __launch_bounds__(kMaxWarps * 32) bwd_kernel(const __grid_constant__ Dev p) {
  constexpr int E = Chunk<T>::E;
  extern __shared__ __align__(16) unsigned char smem[];
  const BlockHeader h = carve(smem, p.N);
  __shared__ int s_tile[2];
  float vs[3], vmin[3];
  voxel_frame(p, vs, vmin);
  const int image_h = __ldg(p.isize), image_w = __ldg(p.isize + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  unsigned char* wa = h.warp_area + (size_t)warp * warp_bytes<3>(p.CPW, p.cap);
  int* sLen = reinterpret_cast<int*>(wa);
  int* sTot = sLen + 32;
  uint4* recs = reinterpret_cast<uint4*>(wa + 256);

  const int g = lane / p.GL, lg = lane - g * p.GL;
  const bool lane_used = g < p.CPW;
  const int cpt = p.GL * V;
  const int tile_cells = p.TX * p.TY;
  const int ngroups = (tile_cells + p.CPW - 1) / p.CPW;
  const uint4* fbase = reinterpret_cast<const uint4*>(p.feats);
  const bool want_feats = (p.flags & FBEV_BWD_FEATS) != 0;
  const bool want_depth = (p.flags & FBEV_BWD_DEPTH) != 0;
  const bool legacy = (p.flags & FBEV_BWD_LEGACY_DEPTH) != 0;
  const bool mean_pool = p.pool == FBEV_POOL_MEAN;
  int loaded_b = -1;
  TileLoop loop;
  loop.begin(p, s_tile);
  for (int tile; (tile = loop.current(p)) >= 0; loop.advance()) {
  const Tile t = tile_of(p, tile);
  block_prologue(p, t, h, vs, vmin, image_h, image_w, loaded_b);
  const int nvis = *h.nvis;
  const int ncand = nvis * p.Z;

  for (int grp = warp; grp < ngroups; grp += nwarps) {
    const int t0 = grp * p.CPW;
    const int tc = t0 + g;
    const int ly = tc / p.TX, lx = tc - ly * p.TX;
    const int x = t.x0 + lx, y = t.y0 + ly;
    const bool cell_ok = lane_used && tc < tile_cells && x < t.x1 && y < t.y1;

    // mean pooling needs the cell's total count before the first contribution
    const bool single_pass = ncand <= p.cap;
    if (mean_pool && !single_pass) {
      if (lane < p.CPW) sTot[lane] = 0;
      for (int r0 = 0; r0 < ncand; r0 += p.cap) {
        list_phase<T, true, true>(p, t, h, nvis, t0, r0, min(r0 + p.cap, ncand), vs, vmin, image_h, image_w, sLen,
                                  recs, lane);
        if (lane < p.CPW) sTot[lane] += sLen[lane];
        __syncwarp();
      }
    }

    float go[V * E];
#pragma unroll
    for (int i = 0; i < V * E; ++i) go[i] = 0.0f;
    if (cell_ok) {
      const size_t cell = out_cell(p, t.b, y, x);
#pragma unroll
      for (int j = 0; j < V; ++j) load_chunk<T>(p.gout, p.out_f32, cell * cpt + lg + j * p.GL, go + j * E);
    }

    for (int r0 = 0; r0 < ncand; r0 += p.cap) {
      list_phase<T, true, false>(p, t, h, nvis, t0, r0, min(r0 + p.cap, ncand), vs, vmin, image_h, image_w, sLen,
                                 recs, lane);
      const int n = cell_ok ? sLen[g] : 0;
      float inv = 1.0f;
      if (mean_pool) {
        const int cnt = lane_used ? (single_pass ? sLen[g] : sTot[g]) : 0;
        inv = cnt > 0 ? __fdiv_rn(1.0f, (float)cnt) : 0.0f;
      }
      // all lanes of the warp run the same trip count so that the shuffles below are converged
      int nmax = n;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) nmax = max(nmax, __shfl_xor_sync(kFull, nmax, off));
      const uint4* rec = recs + (size_t)g * p.cap * 3;
      for (int i = 0; i < nmax; ++i) {
        const bool live = i < n;
        uint4 rw = make_uint4(0, 0, 0, 0), ri = rw, rd = rw;
        if (live) {
          rw = rec[i * 3];
          ri = rec[i * 3 + 1];
          rd = rec[i * 3 + 2];
        }
        const float w00 = __uint_as_float(rw.x), w01 = __uint_as_float(rw.y), w10 = __uint_as_float(rw.z),
                    w11 = __uint_as_float(rw.w);
        const float wgt = __uint_as_float(rd.x);
        const size_t du = (size_t)ri.y * cpt, dv = (size_t)ri.z * cpt;
        const size_t c00 = (size_t)ri.x * cpt + lg;
        float dot = 0.0f;
        if (live) {
          const float s = wgt * inv;
          const float a00 = s * w00, a01 = s * w01, a10 = s * w10, a11 = s * w11;
#pragma unroll
          for (int j = 0; j < V; ++j) {
            if (want_depth) {
              float f00[E], f01[E], f10[E], f11[E];
              Chunk<T>::unpack(ldg16(fbase + c00 + j * p.GL), f00);
              Chunk<T>::unpack(ldg16(fbase + c00 + dv + j * p.GL), f01);
              Chunk<T>::unpack(ldg16(fbase + c00 + du + j * p.GL), f10);
              Chunk<T>::unpack(ldg16(fbase + c00 + du + dv + j * p.GL), f11);
#pragma unroll
              for (int e = 0; e < E; ++e) {
                float f = w00 * f00[e];
                f = fmaf(w01, f01[e], f);
                f = fmaf(w10, f10[e], f);
                f = fmaf(w11, f11[e], f);
                dot = fmaf(go[j * E + e], f, dot);
              }
            }
            if (want_feats) {
              // element offset of this lane's chunk inside the float32 gradient tensor
              const size_t e00 = ((size_t)ri.x * cpt + lg + (size_t)j * p.GL) * E;
              const size_t edu = du * E, edv = dv * E;
#pragma unroll
              for (int e4 = 0; e4 < E; e4 += 4) {
                const float g0 = go[j * E + e4], g1 = go[j * E + e4 + 1], g2 = go[j * E + e4 + 2],
                            g3 = go[j * E + e4 + 3];
                red_add4(p.gfeat + e00 + e4, g0 * a00, g1 * a00, g2 * a00, g3 * a00);
                red_add4(p.gfeat + e00 + edv + e4, g0 * a01, g1 * a01, g2 * a01, g3 * a01);
                red_add4(p.gfeat + e00 + edu + e4, g0 * a10, g1 * a10, g2 * a10, g3 * a10);
                red_add4(p.gfeat + e00 + edu + edv + e4, g0 * a11, g1 * a11, g2 * a11, g3 * a11);
              }
            }
          }
        }
        if (want_depth) {
          dot = group_sum(dot, lg, p.GL);
          if (live && lg == 0) {
            const float sd = dot * inv;
            const size_t D = (size_t)p.D;
            float* d00 = p.gdepth + (size_t)ri.x * D;
            float* d01 = d00 + (size_t)ri.z * D;
            float* d10 = d00 + (size_t)ri.y * D;
            float* d11 = d01 + (size_t)ri.y * D;
            if (p.mode == FBEV_DEPTH_CATEGORICAL) {
              const int k = (int)ri.w;
              atomicAdd(d00 + k, sd * w00);
              atomicAdd(d01 + k, sd * w01);
              atomicAdd(d10 + k, sd * w10);
              atomicAdd(d11 + k, sd * w11);
            } else {
              const float cm = legacy ? wgt : __uint_as_float(rd.y);
              const float cs = legacy ? wgt : __uint_as_float(rd.z);
              atomicAdd(d00 + 0, sd * cm * w00);
              atomicAdd(d00 + 1, sd * cs * w00);
              atomicAdd(d01 + 0, sd * cm * w01);
              atomicAdd(d01 + 1, sd * cs * w01);
              atomicAdd(d10 + 0, sd * cm * w10);
              atomicAdd(d10 + 1, sd * cs * w10);
              atomicAdd(d11 + 0, sd * cm * w11);
              atomicAdd(d11 + 1, sd * cs * w11);
            }
          }
        }
      }
      __syncwarp();
    }
  }
  }  // tiles
  loop.end(p);
}

// Gradient kernel for any channel count and alignment: one cell per warp, lanes stride over the
// channels with scalar loads and scalar float32 atomics.  Slow path, same arithmetic as bwd_kernel.
template <typename T>
__global__ void __launch_bounds__(kMaxWarps * 32) bwd_generic_kernel(const __grid_constant__ Dev p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const BlockHeader h = carve(smem, p.N);
  __shared__ int s_tile[2];
  float vs[3], vmin[3];
  voxel_frame(p, vs, vmin);
  const int image_h = __ldg(p.isize), image_w = __ldg(p.isize + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  unsigned char* wa = h.warp_area + (size_t)warp * warp_bytes<3>(1, p.cap);
  int* sLen = reinterpret_cast<int*>(wa);
  uint4* recs = reinterpret_cast<uint4*>(wa + 256);
  const int tile_cells = p.TX * p.TY;
  const T* fbase = reinterpret_cast<const T*>(p.feats);
  const bool want_feats = (p.flags & FBEV_BWD_FEATS) != 0;
  const bool want_depth = (p.flags & FBEV_BWD_DEPTH) != 0;
  const bool legacy = (p.flags & FBEV_BWD_LEGACY_DEPTH) != 0;
  int loaded_b = -1;
  TileLoop loop;
  loop.begin(p, s_tile);
  for (int tile; (tile = loop.current(p)) >= 0; loop.advance()) {
    const Tile t = tile_of(p, tile);
    block_prologue(p, t, h, vs, vmin, image_h, image_w, loaded_b);
    const int nvis = *h.nvis;
    const int ncand = nvis * p.Z;
    for (int tc = warp; tc < tile_cells; tc += nwarps) {
      const int ly = tc / p.TX, lx = tc - ly * p.TX;
      const int x = t.x0 + lx, y = t.y0 + ly;
      if (!(x < t.x1 && y < t.y1)) continue;  // uniform per warp
      const size_t cell = out_cell(p, t.b, y, x);
      float inv = 1.0f;
      if (p.pool == FBEV_POOL_MEAN) {
        int cnt = 0;
        for (int r0 = 0; r0 < ncand; r0 += p.cap) {
          list_phase<T, true, true>(p, t, h, nvis, tc, r0, min(r0 + p.cap, ncand), vs, vmin, image_h, image_w,
                                    sLen, recs, lane);
          cnt += sLen[0];
          __syncwarp();
        }
        inv = cnt > 0 ? __fdiv_rn(1.0f, (float)cnt) : 0.0f;
      }
      for (int r0 = 0; r0 < ncand; r0 += p.cap) {
        list_phase<T, true, false>(p, t, h, nvis, tc, r0, min(r0 + p.cap, ncand), vs, vmin, image_h, image_w,
                                   sLen, recs, lane);
        const int n = sLen[0];
        for (int i = 0; i < n; ++i) {
          const uint4 rw = recs[i * 3], ri = recs[i * 3 + 1], rd = recs[i * 3 + 2];
          const float w00 = __uint_as_float(rw.x), w01 = __uint_as_float(rw.y), w10 = __uint_as_float(rw.z),
                      w11 = __uint_as_float(rw.w);
          const float wgt = __uint_as_float(rd.x);
          const float sc = wgt * inv;
          const size_t t00 = (size_t)ri.x, t01 = t00 + ri.z, t10 = t00 + ri.y, t11 = t01 + ri.y;
          float dot = 0.0f;
          for (int c = lane; c < p.C; c += 32) {
            const float gc = p.out_f32 ? __ldg(reinterpret_cast<const float*>(p.gout) + cell * p.C + c)
                                       : to_float(__ldg(reinterpret_cast<const T*>(p.gout) + cell * p.C + c));
            if (want_depth) {
              float f = w00 * to_float(__ldg(fbase + t00 * p.C + c));
              f = fmaf(w01, to_float(__ldg(fbase + t01 * p.C + c)), f);
              f = fmaf(w10, to_float(__ldg(fbase + t10 * p.C + c)), f);
              f = fmaf(w11, to_float(__ldg(fbase + t11 * p.C + c)), f);
              dot = fmaf(gc, f, dot);
            }
            if (want_feats) {
              const float a = gc * sc;
              atomicAdd(p.gfeat + t00 * p.C + c, a * w00);
              atomicAdd(p.gfeat + t01 * p.C + c, a * w01);
              atomicAdd(p.gfeat + t10 * p.C + c, a * w10);
              atomicAdd(p.gfeat + t11 * p.C + c, a * w11);
            }
          }
          if (want_depth) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(kFull, dot, off);
            if (lane == 0) {
              const float sd = dot * inv;
              const size_t D = (size_t)p.D;
              float* d00 = p.gdepth + t00 * D;
              float* d01 = p.gdepth + t01 * D;
              float* d10 = p.gdepth + t10 * D;
              float* d11 = p.gdepth + t11 * D;
              if (p.mode == FBEV_DEPTH_CATEGORICAL) {
                const int k = (int)ri.w;
                atomicAdd(d00 + k, sd * w00);
                atomicAdd(d01 + k, sd * w01);
                atomicAdd(d10 + k, sd * w10);
                atomicAdd(d11 + k, sd * w11);
              } else {
                const float cm = legacy ? wgt : __uint_as_float(rd.y);
                const float cs = legacy ? wgt : __uint_as_float(rd.z);
                atomicAdd(d00 + 0, sd * cm * w00);
                atomicAdd(d00 + 1, sd * cs * w00);
                atomicAdd(d01 + 0, sd * cm * w01);
                atomicAdd(d01 + 1, sd * cs * w01);
                atomicAdd(d10 + 0, sd * cm * w10);
                atomicAdd(d10 + 1, sd * cs * w10);
                atomicAdd(d11 + 0, sd * cm * w11);
                atomicAdd(d11 + 1, sd * cs * w11);
              }
            }
          }
        }
        __syncwarp();
      }
    }
  }  // tiles
  loop.end(p);
}

// float32 accumulation buffers -> gradient tensors of a 16-bit type; two arrays (either may be empty) in one
// launch, four elements per step
template <typename T>
__global__ void convert2_kernel(const float* __restrict__ sa, T* __restrict__ da, size_t na, const float* __restrict__ sb,
                                T* __restrict__ db, size_t nb) {
  grid_dependency_wait();
  const size_t ua = (na + 3) / 4, ub = (nb + 3) / 4;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t u = (size_t)blockIdx.x * blockDim.x + threadIdx.x; u < ua + ub; u += stride) {
    const bool first = u < ua;
    const float* src = first ? sa : sb;
    T* dst = first ? da : db;
    const size_t n = first ? na : nb, i = (first ? u : u - ua) * 4;
    if (i + 4 <= n && ((uintptr_t)(dst + i) % 8) == 0) {
      const float4 v = *reinterpret_cast<const float4*>(src + i);
      *reinterpret_cast<uint2*>(dst + i) = make_uint2(Chunk<T>::pack2(v.x, v.y), Chunk<T>::pack2(v.z, v.w));
    } else {
      for (size_t k = i; k < n && k < i + 4; ++k) dst[k] = from_float<T>(src[k]);
    }
  }
}

}  // namespace fbev
