// Scan, scatter and gather kernels of the gradients' global sort by texel (entries come from emit_entries in
// the backward kernels).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fbev.h"
#include "fbev_backward.cuh"

namespace fbev {

// ---------------------------------------------------------------------------
// Gradients through a global sort by texel
// ---------------------------------------------------------------------------
// d_feats = W^T * dO with W the sparse [cells x texels] matrix of record weights.  A list-phase kernel
// (bwd_feats_kernel<EMIT> or bwd_depth_kernel<EMIT>) writes W as one entry per row record and counts the
// entries per texel (of u0); the counts become segment starts (inside ent_scatter_kernel for small feature
// maps, else tex_scan_kernel into a second array); ent_scatter_kernel moves every entry to its texel's segment;
// feats_gather_kernel walks the grouped list, gathers each entry's dO row from L2 once and accumulates it,
// in float32 registers, for the entry's two neighbouring texels -- one 16-byte reduction per chunk when the
// texel changes instead of one per record, which is some 20 times fewer reductions than the direct scatter,
// whose rate at the L2 is what bounds bwd_feats_kernel.  The parametric depth gradient (two floats per
// texel, hopelessly contended as atomics) travels with the entries and is summed the same way.

// Exclusive prefix sum of count[0, n) into start[0, n); start[n] receives the total.  Block b owns the slice
// [b * S, (b + 1) * S), S = per * 1024: it first adds up everything before its slice (all its threads, independent
// coalesced loads from L2: the counters are a few hundred KB), then scans its slice.  No block waits for another;
// the price is that the counters are read gridDim.x / 2 times over, which for the at most 128 blocks the host
// launches stays in the megabytes.  (A single block walking 67 K counters took 60 us on the training shape.)
__global__ void __launch_bounds__(1024) tex_scan_kernel(const unsigned* __restrict__ count, unsigned* __restrict__ start, unsigned n,
                                                        unsigned per) {
  grid_dependency_wait();
  __shared__ unsigned part[32];
  const unsigned tid = threadIdx.x, lane = tid & 31u, wid = tid >> 5;
  const unsigned slice0 = min(blockIdx.x * per * 1024u, n);
  unsigned sum = 0;
  if (blockIdx.x * per * 1024u <= n) {  // a multiple of 1024 counters, 16 bytes at a time (the array is 256-byte aligned)
    const uint4* c4 = reinterpret_cast<const uint4*>(count);
    for (unsigned i = tid; i < slice0 / 4u; i += 1024u) {
      const uint4 v = __ldg(c4 + i);
      sum += v.x + v.y + v.z + v.w;
    }
  } else {
    for (unsigned i = tid; i < slice0; i += 1024u) sum += __ldg(count + i);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
  if (lane == 0u) part[wid] = sum;
  __syncthreads();
  unsigned before = 0;
  for (unsigned k = 0; k < 32u; ++k) before += part[k];
  __syncthreads();
  // the slice: `per` consecutive counters per thread, shuffles inside a warp, the warp totals through shared memory
  const unsigned lo = min(slice0 + tid * per, n), hi = min(lo + per, n);
  unsigned own = 0;
  for (unsigned i = lo; i < hi; ++i) own += __ldg(count + i);
  unsigned incl = own;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const unsigned v = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= (unsigned)d) incl += v;
  }
  if (lane == 31u) part[wid] = incl;
  __syncthreads();
  unsigned warps_before = 0, all = 0;
  for (unsigned k = 0; k < 32u; ++k) {
    const unsigned wt = part[k];
    warps_before += k < wid ? wt : 0u;
    all += wt;
  }
  unsigned run = before + warps_before + incl - own;
  for (unsigned i = lo; i < hi; ++i) {
    start[i] = run;
    run += __ldg(count + i);
  }
  if (blockIdx.x == gridDim.x - 1 && tid == 0u) start[n] = before + all;
  grid_dependency_trigger();
}

constexpr unsigned kScanInBlock = 8192;  // texels up to which every scatter block scans the counts itself

// Every emitted entry moves to its place: start of its texel's segment + the position it drew there.
// SCAN: tex_count still holds counts; every block derives the starts in shared memory (dynamic,
// (texels + 1) * 4 bytes) and the total goes to total_out.  Otherwise tex_count holds the starts already.
template <bool SCAN>
__global__ void __launch_bounds__(1024) ent_scatter_kernel(const Dev p, unsigned texels, unsigned* __restrict__ total_out) {
  extern __shared__ unsigned s_start[];
  grid_dependency_wait();  // the emitting kernel (or the scan) has finished
  const unsigned* start = p.tex_count;
  if (SCAN) {
    // block-wide exclusive scan: a contiguous slice per thread, shuffles inside a warp, the warp totals through
    // shared memory (two barriers).  Every block repeats it, so blocks are large and few: the scan is paid once
    // per 1024 threads' worth of entries.
    __shared__ unsigned warp_total[32];
    const unsigned tid = threadIdx.x, lane = tid & 31u, wid = tid >> 5, nt = blockDim.x, nw = nt >> 5;
    const unsigned per = (texels + nt - 1u) / nt;
    const unsigned lo = min(tid * per, texels), hi = min(lo + per, texels);
    unsigned sum = 0;
    for (unsigned i = lo; i < hi; ++i) sum += __ldg(p.tex_count + i);
    unsigned incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const unsigned v = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= (unsigned)d) incl += v;
    }
    if (lane == 31u) warp_total[wid] = incl;
    __syncthreads();
    unsigned before = 0, all = 0;
    for (unsigned k = 0; k < nw; ++k) {
      const unsigned wt = warp_total[k];
      before += k < wid ? wt : 0u;
      all += wt;
    }
    unsigned run = before + incl - sum;
    for (unsigned i = lo; i < hi; ++i) {
      s_start[i] = run;
      run += __ldg(p.tex_count + i);
    }
    if (blockIdx.x == 0 && tid == 0u) *total_out = all;
    __syncthreads();
    start = s_start;
  }
  const unsigned n = min(*p.ent_count, p.ent_cap);
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const uint4 e = p.ent[i];
    if (e.x >= texels) continue;  // void slot
    const unsigned dst = start[e.x] + p.ent_pos[i];
    p.ent_sorted[dst] = e;
    if (p.ent_d != nullptr) p.ent_d_sorted[dst] = p.ent_d[i];
  }
  grid_dependency_trigger();  // the gather kernel's blocks may move in as this kernel's leave
}

// GF32: the upstream gradient is float32 although the features are 16-bit.
// PDEPTH: the entries also carry the parametric depth gradient (p.ent_d_sorted).
// n_entries: device word holding the number of grouped entries.
template <typename T, int V, bool GF32, bool PDEPTH>
__global__ void __launch_bounds__(128, (PDEPTH || GF32) ? 3 : 4)
    feats_gather_kernel(const __grid_constant__ Dev p, const unsigned* __restrict__ n_entries, unsigned run_len) {
  constexpr int E = Chunk<T>::E;
  constexpr int R = (GF32 && E == 8) ? 2 : 1;  // 16-byte loads per chunk of E channels
  constexpr int U = V == 4 ? 2 : 4;            // entries in flight per lane
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int g = lane / p.GL, lg = lane - g * p.GL;
  grid_dependency_wait();
  if (g >= p.CPW) {
    grid_dependency_trigger();
    return;
  }
  const unsigned n = *n_entries;
  const unsigned cpt = (unsigned)(p.GL * V);
  const unsigned groups = gridDim.x * nwarps * p.CPW;
  const uint4* gl = reinterpret_cast<const uint4*>(p.gout) + (size_t)lg * R;
  const bool feats = (p.flags & FBEV_BWD_FEATS) != 0;
  for (unsigned run = (blockIdx.x * nwarps + warp) * p.CPW + g; (unsigned long long)run * run_len < n; run += groups) {
    const unsigned i0 = run * run_len, i1 = min(i0 + run_len, n);
    // sums for texel `cur` (acc0) and its right neighbour (acc1); when the next texel is that neighbour,
    // acc1 slides into acc0
    float2 acc0[V * E / 2], acc1[V * E / 2];
    float2 d0 = make_float2(0.0f, 0.0f), d1 = make_float2(0.0f, 0.0f);  // parametric depth: d mean, d sigma
    bool any1 = false;  // acc1 / d1 received something (a texel without right neighbour never does)
#pragma unroll
    for (int k = 0; k < V * E / 2; ++k) acc0[k] = acc1[k] = make_float2(0.0f, 0.0f);
    auto flush = [&](unsigned tex, const float2* acc, float2 dd) {
      if (PDEPTH && lg == 0) {
        atomicAdd(p.gdepth + (size_t)tex * 2, dd.x);
        atomicAdd(p.gdepth + (size_t)tex * 2 + 1, dd.y);
      }
      if (!feats) return;
#pragma unroll
      for (int j = 0; j < V; ++j) {
        float* d = p.gfeat + ((size_t)tex * cpt + lg + j * p.GL) * E;
#pragma unroll
        for (int e4 = 0; e4 < E; e4 += 4)
          red_add4(d + e4, acc[(j * E + e4) / 2].x, acc[(j * E + e4) / 2].y, acc[(j * E + e4) / 2 + 1].x,
                   acc[(j * E + e4) / 2 + 1].y);
      }
    };
    // entries one step ahead, so that their latency overlaps the gathers of this step
    uint4 nx[U];
#pragma unroll
    for (int u = 0; u < U; ++u) nx[u] = __ldg(p.ent_sorted + min(i0 + u, i1 - 1));
    unsigned cur = nx[0].x;
    for (unsigned i = i0; i < i1; i += U) {
      uint4 e[U];
      uint4 q[U][V][R];
      float4 dv[U];
#pragma unroll
      for (int u = 0; u < U; ++u) e[u] = nx[u];
      if (feats) {
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int j = 0; j < V; ++j)
#pragma unroll
            for (int r = 0; r < R; ++r) q[u][j][r] = ldg16(gl + ((size_t)e[u].y * cpt + j * p.GL) * R + r);
      }
      if (PDEPTH) {
#pragma unroll
        for (int u = 0; u < U; ++u) dv[u] = __ldg(p.ent_d_sorted + min(i + u, i1 - 1));
      }
      if (i + U < i1) {
#pragma unroll
        for (int u = 0; u < U; ++u) nx[u] = __ldg(p.ent_sorted + min(i + U + u, i1 - 1));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (i + u >= i1) break;
        const unsigned t = e[u].x;
        if (t != cur) {
          flush(cur, acc0, d0);
          if (t == cur + 1u) {
#pragma unroll
            for (int k = 0; k < V * E / 2; ++k) acc0[k] = acc1[k];
            d0 = d1;
          } else {
            if (any1) flush(cur + 1u, acc1, d1);
#pragma unroll
            for (int k = 0; k < V * E / 2; ++k) acc0[k] = make_float2(0.0f, 0.0f);
            d0 = make_float2(0.0f, 0.0f);
          }
#pragma unroll
          for (int k = 0; k < V * E / 2; ++k) acc1[k] = make_float2(0.0f, 0.0f);
          d1 = make_float2(0.0f, 0.0f);
          any1 = false;
          cur = t;
        }
        const float w0 = __uint_as_float(e[u].z), w1 = __uint_as_float(e[u].w);
        any1 = any1 || w1 != 0.0f;
        if (PDEPTH) {
          d0.x += dv[u].x;
          d0.y += dv[u].y;
          d1.x += dv[u].z;
          d1.y += dv[u].w;
          any1 = any1 || dv[u].z != 0.0f || dv[u].w != 0.0f;
        }
        if (!feats) continue;
        const float2 w0v = make_float2(w0, w0), w1v = make_float2(w1, w1);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          float f[E];
          if (R == 2) {
            Chunk<float>::unpack(q[u][j][0], f);
            Chunk<float>::unpack(q[u][j][R - 1], f + 4);
          } else {
            Chunk<T>::unpack(q[u][j][0], f);
          }
#pragma unroll
          for (int k = 0; k < E / 2; ++k) {
            const float2 fv = make_float2(f[2 * k], f[2 * k + 1]);
            acc0[j * E / 2 + k] = __ffma2_rn(w0v, fv, acc0[j * E / 2 + k]);
            acc1[j * E / 2 + k] = __ffma2_rn(w1v, fv, acc1[j * E / 2 + k]);
          }
        }
      }
    }
    flush(cur, acc0, d0);
    if (any1) flush(cur + 1u, acc1, d1);
  }
  grid_dependency_trigger();
}

// The gather for the reproducible backward: the same walk over the grouped entries, but every product weight * g is
// turned into a 64-bit fixed-point integer before it is added, in registers and then (one integer atomic per channel
// when the texel changes or the run ends) in p.gfeat, which holds int64 sums.  The position an entry drew inside its
// texel's segment and the way segments split into runs change from launch to launch; integer sums do not care.
template <typename T, int V, bool GF32>
__global__ void __launch_bounds__(128, V == 4 ? 2 : 3)
    feats_gather_fixed_kernel(const __grid_constant__ Dev p, const unsigned* __restrict__ n_entries, unsigned run_len) {
  constexpr int E = Chunk<T>::E;
  constexpr int R = (GF32 && E == 8) ? 2 : 1;  // 16-byte loads per chunk of E channels
  constexpr int U = 2;                         // entries in flight per lane
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int g = lane / p.GL, lg = lane - g * p.GL;
  grid_dependency_wait();
  if (g >= p.CPW) {
    grid_dependency_trigger();
    return;
  }
  const unsigned n = *n_entries;
  const unsigned cpt = (unsigned)(p.GL * V);
  const unsigned groups = gridDim.x * nwarps * p.CPW;
  const uint4* gl = reinterpret_cast<const uint4*>(p.gout) + (size_t)lg * R;
  const float scale = p.det->scale_f;
  unsigned long long* gf = reinterpret_cast<unsigned long long*>(p.gfeat);
  for (unsigned run = (blockIdx.x * nwarps + warp) * p.CPW + g; (unsigned long long)run * run_len < n; run += groups) {
    const unsigned i0 = run * run_len, i1 = min(i0 + run_len, n);
    long long acc0[V * E], acc1[V * E];  // sums for texel `cur` and its right neighbour
    bool any1 = false;
#pragma unroll
    for (int k = 0; k < V * E; ++k) acc0[k] = acc1[k] = 0;
    auto flush = [&](unsigned tex, const long long* acc) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        unsigned long long* d = gf + ((size_t)tex * cpt + lg + j * p.GL) * E;
#pragma unroll
        for (int e = 0; e < E; ++e) atomicAdd(d + e, (unsigned long long)acc[j * E + e]);
      }
    };
    // entries one step ahead, so that their latency overlaps the gathers of this step
    uint4 nx[U];
#pragma unroll
    for (int u = 0; u < U; ++u) nx[u] = __ldg(p.ent_sorted + min(i0 + u, i1 - 1));
    unsigned cur = nx[0].x;
    for (unsigned i = i0; i < i1; i += U) {
      uint4 en[U];
      uint4 q[U][V][R];
#pragma unroll
      for (int u = 0; u < U; ++u) en[u] = nx[u];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < V; ++j)
#pragma unroll
          for (int r = 0; r < R; ++r) q[u][j][r] = ldg16(gl + ((size_t)en[u].y * cpt + j * p.GL) * R + r);
      if (i + U < i1) {
#pragma unroll
        for (int u = 0; u < U; ++u) nx[u] = __ldg(p.ent_sorted + min(i + U + u, i1 - 1));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (i + u >= i1) break;
        const unsigned t = en[u].x;
        if (t != cur) {
          flush(cur, acc0);
          if (t == cur + 1u) {
#pragma unroll
            for (int k = 0; k < V * E; ++k) acc0[k] = acc1[k];
          } else {
            if (any1) flush(cur + 1u, acc1);
#pragma unroll
            for (int k = 0; k < V * E; ++k) acc0[k] = 0;
          }
#pragma unroll
          for (int k = 0; k < V * E; ++k) acc1[k] = 0;
          any1 = false;
          cur = t;
        }
        // weight times a power of two is exact; every term rounds to an integer by itself
        const float w0 = __uint_as_float(en[u].z) * scale, w1 = __uint_as_float(en[u].w) * scale;
        any1 = any1 || w1 != 0.0f;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          float f[E];
          if (R == 2) {
            Chunk<float>::unpack(q[u][j][0], f);
            Chunk<float>::unpack(q[u][j][R - 1], f + 4);
          } else {
            Chunk<T>::unpack(q[u][j][0], f);
          }
#pragma unroll
          for (int e = 0; e < E; ++e) {
            acc0[j * E + e] += __float2ll_rn(w0 * f[e]);
            acc1[j * E + e] += __float2ll_rn(w1 * f[e]);
          }
        }
      }
    }
    flush(cur, acc0);
    if (any1) flush(cur + 1u, acc1);
  }
  grid_dependency_trigger();
}

}  // namespace fbev
