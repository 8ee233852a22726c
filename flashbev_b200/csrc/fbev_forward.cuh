// Forward kernels: fwd_kernel (16-byte channel chunks, merged row records) and fwd_generic_kernel (any channel
// count and alignment).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fbev.h"
#include "fbev_lists.cuh"

namespace fbev {

// EXPERIMENTS: the instantiation that honours the switches of fbev_set_experiment (Dev.exp); the ordinary one
// carries none of their code.
// MAXT: largest block the instantiation is launched with (with MINB it sets the register budget).
// TRAIN: the forward of a training step.  It runs in the lane layout and pass size of the depth-gradient kernel,
// keeps every accepted sample beside the row records (row_list_phase with SAMPLES) and writes both to the saved
// state (save_pass), from which the backward takes them instead of rebuilding them.  Same results as the ordinary
// instantiation up to the grouping of the sums (the passes are half as long).
template <typename T, int V, int MINB, bool EXPERIMENTS = false, int MAXT = kMaxWarps * 32, bool TRAIN = false>
__global__ void __launch_bounds__(MAXT, MINB) fwd_kernel(const __grid_constant__ Dev p) {
  constexpr int E = Chunk<T>::E;
  extern __shared__ __align__(16) unsigned char smem[];
  const BlockHeader h = carve(smem, p.N);
  __shared__ int s_tile[2];
  float vs[3], vmin[3];
  voxel_frame(p, vs, vmin);
  const int image_h = __ldg(p.isize), image_w = __ldg(p.isize + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  unsigned char* wa = h.warp_area + (size_t)warp * (TRAIN ? depth_warp_bytes(p.CPW, p.cap) : fwd_warp_bytes(p.CPW, p.cap));
  int* sLen = reinterpret_cast<int*>(wa);  // [32] records in the list of each cell
  int* sCnt = sLen + 32;                    // [32] accepted samples of each cell
  int* sSmp = sCnt + 32;                    // [32] TRAIN: sample records of each cell, this pass
  uint4* recs = reinterpret_cast<uint4*>(wa + (TRAIN ? 512 : 256));
  const int rstride = row_stride(p.cap);
  uint4* samp = recs + (size_t)p.CPW * rstride;  // TRAIN: three words per accepted sample
  if (TRAIN && blockIdx.x == 0 && threadIdx.x == 0) reinterpret_cast<unsigned*>(p.saved)[1] = p.saved_key;

  const int g = lane / p.GL, lg = lane - g * p.GL;
  const bool lane_used = g < p.CPW;
  const int cpt = p.GL * V;  // 16-byte chunks per texel
  const int tile_cells = p.TX * p.TY;
  const int ngroups = (tile_cells + p.CPW - 1) / p.CPW;
  const uint4* fl = reinterpret_cast<const uint4*>(p.feats) + lg;  // this lane's chunk of texel 0
  int loaded_b = -1;
  if (EXPERIMENTS && (p.exp & FBEV_EXP_PREFETCH)) {
    // one 128-byte line per thread of the feature and depth tensors, the whole grid covering both once
    const size_t tex = (size_t)p.B * p.N * p.H * p.W;
    const size_t lf = (tex * p.C * sizeof(T) + 127) / 128, ld = (tex * p.D * sizeof(T) + 127) / 128;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < lf + ld; i += stride) {
      const unsigned char* a = i < lf ? reinterpret_cast<const unsigned char*>(p.feats) + i * 128
                                      : reinterpret_cast<const unsigned char*>(p.depth) + (i - lf) * 128;
      asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
    }
  }
  UnitLoop sched;  // counter of tiles with a barrier per tile, or the barrier-free static order of units
  sched.begin(p, s_tile, warp, nwarps);
  if (sched.stat) {  // the sample's matrices, once, by the whole block
    const Tile tt = tile_of(p, 0);
    (void)tile_visibility(p, tt, h, vs, vmin, image_h, image_w, loaded_b);
  }
  int g_first = 0, g_step = 1;
  for (int tile; (tile = sched.current(p, ngroups, warp, nwarps, g_first, g_step)) >= 0; sched.advance(p, nwarps)) {
    const Tile t = tile_of(p, tile);
    const unsigned vis_tile = tile_visibility(p, t, h, vs, vmin, image_h, image_w, loaded_b);

    for (int grp = g_first; grp < ngroups; grp += g_step) {
      const int t0 = grp * p.CPW;
      const int tc = t0 + g;
      const int ly = tc / p.TX, lx = tc - ly * p.TX;
      const int x = t.x0 + lx, y = t.y0 + ly;
      const bool cell_ok = lane_used && tc < tile_cells && x < t.x1 && y < t.y1;
      unsigned vis = vis_tile;
      if (EXPERIMENTS && (p.exp & FBEV_EXP_GROUP_CULL)) {
        // the cull again for the box of this group's cells alone (rows ly0..ly1 of the tile; one row: its columns)
        const int last = min(t0 + p.CPW, tile_cells) - 1;
        const int ly0 = t0 / p.TX, ly1 = last / p.TX;
        Tile tg = t;
        tg.y0 = t.y0 + ly0;
        tg.y1 = min(t.y0 + ly1 + 1, t.y1);
        if (ly0 == ly1) {
          tg.x0 = t.x0 + (t0 - ly0 * p.TX);
          tg.x1 = min(t.x0 + (last - ly0 * p.TX) + 1, t.x1);
        }
        vis = (tg.x0 < tg.x1 && tg.y0 < tg.y1) ? (vis_tile & box_visibility(p, tg, h, vs, vmin, image_h, image_w)) : 0u;
      }
      const int nvis = __popc(vis);
      const int ncand = nvis * p.Z;

      // accumulators as pairs: one packed FFMA2 (two independent IEEE fp32 fmas) per pair of channels
      float2 acc2[V * E / 2];
#pragma unroll
      for (int i = 0; i < V * E / 2; ++i) acc2[i] = make_float2(0.0f, 0.0f);
      if (lane < p.CPW) sCnt[lane] = 0;

      for (int r0 = 0; r0 < ncand; r0 += p.cap) {
        if (lane < p.CPW) {
          sLen[lane] = 0;
          if (TRAIN) sSmp[lane] = 0;
        }
        __syncwarp();
        if (TRAIN) {
          row_list_phase<T, true, true>(p, t, h, vis, (unsigned)cpt, t0, r0, min(r0 + p.cap, ncand), vs, vmin, image_h, image_w,
                                        sLen, sCnt, recs, lane, samp, sSmp);
          save_pass(p, (unsigned)(tile * ngroups + grp), r0 / p.cap, sLen, sSmp, recs, samp, lane);
        } else {
          row_list_phase<T>(p, t, h, vis, (unsigned)cpt, t0, r0, min(r0 + p.cap, ncand), vs, vmin, image_h, image_w, sLen, sCnt,
                            recs, lane);
        }
        const int n = cell_ok ? sLen[g] : 0;
        const uint4* rec = recs + (size_t)g * rstride;
#pragma unroll 2
        for (int i = 0; i < n; ++i) {
          const uint4 r = rec[i];
          const float2 wa0 = make_float2(__uint_as_float(r.z), __uint_as_float(r.z));
          const float2 wa1 = make_float2(__uint_as_float(r.w), __uint_as_float(r.w));
#pragma unroll
          for (int j = 0; j < V; ++j) {
            uint4 q0, q1;
            if (EXPERIMENTS && (p.exp & FBEV_EXP_SHARED_GATHER_CEILING)) {
              // timing experiment: the same two 16-byte reads, from this block's shared memory (wrong values)
              const uint4* sm = reinterpret_cast<const uint4*>(smem);
              q0 = sm[(r.x + j * p.GL + lg) & 1023u];
              q1 = sm[(r.x + r.y + j * p.GL + lg) & 1023u];
            } else {
              q0 = ldg16(fl + (r.x + j * p.GL));
              q1 = ldg16(fl + (r.x + r.y + j * p.GL));
            }
            float f0[E], f1[E];
            Chunk<T>::unpack(q0, f0);
            Chunk<T>::unpack(q1, f1);
#pragma unroll
            for (int e = 0; e < E / 2; ++e)
              acc2[j * E / 2 + e] = __ffma2_rn(wa1, make_float2(f1[2 * e], f1[2 * e + 1]),
                                               __ffma2_rn(wa0, make_float2(f0[2 * e], f0[2 * e + 1]), acc2[j * E / 2 + e]));
          }
        }
        __syncwarp();
      }
      __syncwarp();

      float acc[V * E];
#pragma unroll
      for (int i = 0; i < V * E / 2; ++i) {
        acc[2 * i] = acc2[i].x;
        acc[2 * i + 1] = acc2[i].y;
      }
      if (cell_ok) {
        const int cnt = sCnt[g];
        if (p.pool == FBEV_POOL_MEAN) {
          const float c = (float)cnt;
#pragma unroll
          for (int i = 0; i < V * E; ++i) acc[i] = cnt > 0 ? __fdiv_rn(acc[i], c) : 0.0f;
        }
        const size_t cell = out_cell(p, t.b, y, x);
        if (p.out_mc != nullptr) {  // one multicast store reaches this GPU's buffer and every peer's
#pragma unroll
          for (int j = 0; j < V; ++j) store_chunk_multicast<T>(p.out_mc, p.out_f32, cell * cpt + lg + j * p.GL, acc + j * E);
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) store_chunk<T>(p.out, p.out_f32, cell * cpt + lg + j * p.GL, acc + j * E);
        }
        for (int k = 0; k < p.n_peers; ++k) {  // the same rows into the other ranks' buffers (plain peer stores)
#pragma unroll
          for (int j = 0; j < V; ++j) store_chunk<T>(p.out_peers[k], p.out_f32, cell * cpt + lg + j * p.GL, acc + j * E);
        }
        if (p.count != nullptr && lg == 0) p.count[cell] = cnt;
      }
      __syncwarp();
    }
  }  // tiles
  sched.end(p, nwarps);
}

// Any channel count and alignment: one cell per warp, lanes stride over channels
// with scalar loads.  Slow path for shapes the chunked kernel cannot take.
template <typename T>
__global__ void __launch_bounds__(kMaxWarps * 32) fwd_generic_kernel(const __grid_constant__ Dev p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const BlockHeader h = carve(smem, p.N);
  __shared__ int s_tile[2];
  float vs[3], vmin[3];
  voxel_frame(p, vs, vmin);
  const int image_h = __ldg(p.isize), image_w = __ldg(p.isize + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  unsigned char* wa = h.warp_area + (size_t)warp * warp_bytes<2>(1, p.cap);
  int* sLen = reinterpret_cast<int*>(wa);
  uint4* recs = reinterpret_cast<uint4*>(wa + 256);
  const int tile_cells = p.TX * p.TY;
  const T* fbase = reinterpret_cast<const T*>(p.feats);
  T* obase = reinterpret_cast<T*>(p.out);
  float* obase32 = reinterpret_cast<float*>(p.out);
  constexpr int KC = 4;  // channels per lane per block of 128
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
    int cnt = 0;
    for (int r0 = 0; r0 < ncand; r0 += p.cap) {  // count first (mean pooling divides every block)
      list_phase<T, false, true>(p, t, h, nvis, tc, r0, min(r0 + p.cap, ncand), vs, vmin, image_h, image_w, sLen,
                                 recs, lane);
      cnt += sLen[0];
      __syncwarp();
    }
    for (int c0 = 0; c0 < p.C; c0 += 32 * KC) {
      float acc[KC];
#pragma unroll
      for (int k = 0; k < KC; ++k) acc[k] = 0.0f;
      for (int r0 = 0; r0 < ncand; r0 += p.cap) {
        list_phase<T, false, false>(p, t, h, nvis, tc, r0, min(r0 + p.cap, ncand), vs, vmin, image_h, image_w,
                                    sLen, recs, lane);
        const int n = sLen[0];
        for (int i = 0; i < n; ++i) {
          const uint4 rw = recs[i * 2], ri = recs[i * 2 + 1];
          const float w00 = __uint_as_float(rw.x), w01 = __uint_as_float(rw.y), w10 = __uint_as_float(rw.z),
                      w11 = __uint_as_float(rw.w);
          const T* c00 = fbase + (size_t)ri.x * p.C;
          const size_t du = (size_t)ri.y * p.C, dv = (size_t)ri.z * p.C;
#pragma unroll
          for (int k = 0; k < KC; ++k) {
            const int c = c0 + k * 32 + lane;
            if (c < p.C) {
              float a = acc[k];
              a = fmaf(w00, to_float(__ldg(c00 + c)), a);
              a = fmaf(w01, to_float(__ldg(c00 + dv + c)), a);
              a = fmaf(w10, to_float(__ldg(c00 + du + c)), a);
              a = fmaf(w11, to_float(__ldg(c00 + du + dv + c)), a);
              acc[k] = a;
            }
          }
        }
        __syncwarp();
      }
#pragma unroll
      for (int k = 0; k < KC; ++k) {
        const int c = c0 + k * 32 + lane;
        if (c < p.C) {
          float v = acc[k];
          if (p.pool == FBEV_POOL_MEAN) v = cnt > 0 ? __fdiv_rn(v, (float)cnt) : 0.0f;
          if (p.out_f32) {
            obase32[cell * p.C + c] = v;
            for (int q = 0; q < p.n_peers; ++q) reinterpret_cast<float*>(p.out_peers[q])[cell * p.C + c] = v;
          } else {
            obase[cell * p.C + c] = from_float<T>(v);
            for (int q = 0; q < p.n_peers; ++q) reinterpret_cast<T*>(p.out_peers[q])[cell * p.C + c] = from_float<T>(v);
          }
        }
      }
    }
    if (p.count != nullptr && lane == 0) p.count[cell] = cnt;
  }
  }  // tiles
  loop.end(p);
}

}  // namespace fbev
