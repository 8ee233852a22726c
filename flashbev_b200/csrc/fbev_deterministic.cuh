// Bitwise reproducible backward (FBEV_BWD_DETERMINISTIC).
//
// The gradients are sums over samples that many warps produce in an order that changes from run to run; float32
// addition is not associative, so the default kernels (atomics, and a sort whose segments are filled in drawn order)
// differ between two runs in the last bits, as the reference's per-sample atomicAdd does
// (flash_bevpool_cuda.cu:667-679).  Here every contribution is turned into a 64-bit fixed-point integer and added
// with an integer atomic: integer addition is associative and commutative, so the sum does not depend on the order,
// and every contribution itself is computed by one warp in a fixed order.
//
// The fixed-point scale is a power of two chosen from the data before anything is added.  det_bounds_kernel reduces
// the inputs to four maxima (each order-independent): G = max |g|, Gn = max over cells of ||g_cell||_2, Fn = max over
// texels of ||f_texel||_2, and the largest depth weight any sample can have: max |probability| in the categorical
// mode (1 for logits), max 1 / (sigma + eps) in the parametric modes (a bilinear interpolation is a convex
// combination, so the interpolated value stays inside the corner values' range).  From these follow bounds that
// hold whatever the geometry does:
//   a contribution to d_feats is g_c * inv * (sum of at most 2 Z sample weights w_ij * weight, w_ij <= 1), doubled
//     where the two texels of a record coincide                                  =>  |.| <= 4 Z * Wmax * G
//   a contribution to d_depth is S * inv * w_ij (* d weight / d parameter), S = sum_ij w_ij <g, f_ij> a convex
//     combination of dot products, |<g, f>| <= ||g|| ||f||, `merged` of them summed before they are added (1 in
//     the kernel below, up to a warp's 32 in bwd_depth_kernel)                 =>  |.| <= merged * Gn * Fn * Dmax
//   with Dmax = 1 (categorical), 1 / (sigma + eps)_min (legacy parametric gradient) or its square (analytic one:
//   |z| exp(-z^2 / 2) < 1, |z^2 - 1| exp(-z^2 / 2) <= 1, and the Laplace counterparts are below 1 / 2).
// det_set_scales (run by the last block of det_bounds_kernel) sets scale = 2^(62 - bits - e) with 2^e above the bound
// and 2^bits above the number of contributions one element can receive (4 * rows * X * Z: every candidate of the
// texel's camera, four corners each), so no sum can leave 63 bits.  The bounds are loose by a few binary digits, the count by many; what is left
// is still finer than float32 (on the benchmark shapes a contribution keeps more than 30 digits below the largest
// one, and the sums themselves are exact).  det_finish_kernel converts the sums back.  sigma + eps <= 0 somewhere, NaN
// or infinite inputs give meaningless (but still repeatable) gradients.
//
// Two ways lead to the sums.  Large problems whose channel rows are whole 16-byte chunks, given room for the entry
// lists, run through the default backward's own kernels in their fixed-point instantiations: bwd_depth_kernel<DET>
// (list phase, entries of the feature gradient, depth contributions as integer atomics), the scatter by texel, and
// feats_gather_fixed_kernel (integer accumulators in registers, one integer atomic per channel when the texel
// changes).  The order in which entries land inside a texel's segment still varies from launch to launch; the sums
// do not.  Everything else takes bwd_det_kernel below: one cell per warp, lanes stride over the channels, any
// channel count and alignment (up to 32 cameras, fewer than 2^32 depth elements).  Per cell it builds the forward's
// merged row records and the sample list (row_list_phase), adds the records' feature contributions
//   d_feats[texel, c] += g_c * inv * weight                                     (flash_bevpool_cuda.cu:665,676-679)
// computes T = <g, texel> once per record texel and lets one lane per sample form S = sum_ij w_ij T_ij and add
// the sample's depth contributions, the arithmetic of bwd_depth_kernel.  Which way a call takes depends on its
// shape and scratch only, never on timing.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fbev.h"
#include "fbev_lists.cuh"

namespace fbev {

// The bounds of the file comment -> scale = 2^(shift - e) with 2^e above the bound; shift = 62 - bits of the
// contribution count.  depth_kind: 0 categorical probabilities, 1 logits (probabilities <= 1), 2 parametric with
// the analytic depth gradient, 3 parametric with the legacy one.  merged: how many depth contributions a kernel
// sums before it adds them.  One thread.
__device__ inline void det_set_scales(DetHeader* hdr, int shift, int Z, int depth_kind, int merged) {
  const volatile unsigned* mx = &hdr->g_max;  // the four maxima, as the other blocks' atomics left them in memory
  const double g = (double)__uint_as_float(mx[0]);
  const double gn = sqrt((double)__uint_as_float(mx[1])), fn = sqrt((double)__uint_as_float(mx[2]));
  const double d = (double)__uint_as_float(mx[3]);
  const double slack = 1.01;  // float32 rounding inside the reductions and the kernels' own products
  const double wmax = depth_kind == 1 ? 1.0 : d;
  const double dpar = depth_kind <= 1 ? 1.0 : (depth_kind == 3 ? d : d * d);
  const double bound[2] = {4.0 * (double)Z * wmax * g * slack, (double)merged * gn * fn * dpar * slack};
  float scale[2], inv[2];
  for (int k = 0; k < 2; ++k) {
    int e = 0;
    const double m = bound[k];
    if (m > 0.0 && m < 1.0e300) (void)frexp(m, &e);  // m = f * 2^e, 0.5 <= f < 1
    if (!(m < 1.0e300)) e = 1024;
    int s = shift - e;
    s = s > 100 ? 100 : (s < -100 ? -100 : s);  // both the scale and its inverse stay normal float32 numbers
    scale[k] = ldexpf(1.0f, s);
    inv[k] = ldexpf(1.0f, -s);
  }
  hdr->scale_f = scale[0];
  hdr->inv_f = inv[0];
  hdr->scale_d = scale[1];
  hdr->inv_d = inv[1];
}

// One warp per row: the cells of the upstream gradient, the texels of the features, and the depth tensor in rows of
// D values (categorical) or (mean, sigma) pairs (parametric).  A block combines its warps' maxima in shared memory
// and adds them with one atomic each (thousands of warps firing at four words would queue up at the L2); the block
// that finds all others done turns the maxima into the scales.
template <typename T>
__global__ void __launch_bounds__(256) det_bounds_kernel(DetHeader* __restrict__ hdr, const void* __restrict__ gout, int gout_f32,
                                                         size_t cells, const T* __restrict__ feats, size_t texels, int C,
                                                         const T* __restrict__ depth, int D, int categorical, float eps,
                                                         int shift, int Z, int depth_kind, int merged) {
  __shared__ float s_max[4][8];
  __shared__ bool s_last;
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  float gmax = 0.0f, gn2 = 0.0f, fn2 = 0.0f, dmax = 0.0f;
  // four rows at a time, so that their loads are in flight together (the kernel is bound by their latency)
  constexpr int R = 4;
  for (size_t row0 = warp; row0 < cells + texels; row0 += nwarps * R) {
    float m[R], q[R];
#pragma unroll
    for (int k = 0; k < R; ++k) {
      m[k] = q[k] = 0.0f;
      const size_t row = row0 + (size_t)k * nwarps;
      if (row >= cells + texels) continue;
      const bool is_g = row < cells;
      for (int c = lane; c < C; c += 32) {
        float v;
        if (is_g)
          v = gout_f32 ? __ldg(reinterpret_cast<const float*>(gout) + row * (size_t)C + c)
                       : to_float(__ldg(reinterpret_cast<const T*>(gout) + row * (size_t)C + c));
        else
          v = to_float(__ldg(feats + (row - cells) * (size_t)C + c));
        m[k] = fmaxf(m[k], fabsf(v));
        q[k] = fmaf(v, v, q[k]);
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {  // same value in every lane, every run
#pragma unroll
      for (int k = 0; k < R; ++k) q[k] += __shfl_xor_sync(0xffffffffu, q[k], off);
    }
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const size_t row = row0 + (size_t)k * nwarps;
      if (row < cells) {
        gmax = fmaxf(gmax, m[k]);
        gn2 = fmaxf(gn2, q[k]);
      } else {
        fn2 = fmaxf(fn2, q[k]);  // 0 for rows beyond the end
      }
    }
  }
  const size_t nd = categorical ? texels * (size_t)D : texels;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nd; i += (size_t)gridDim.x * blockDim.x) {
    if (categorical) {
      dmax = fmaxf(dmax, fabsf(to_float(__ldg(depth + i))));
    } else {
      const float se = to_float(__ldg(depth + i * 2 + 1)) + eps;
      dmax = fmaxf(dmax, se > 0.0f ? 1.0f / se : __int_as_float(0x7f800000));
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, off));
    gn2 = fmaxf(gn2, __shfl_xor_sync(0xffffffffu, gn2, off));
    fn2 = fmaxf(fn2, __shfl_xor_sync(0xffffffffu, fn2, off));
    dmax = fmaxf(dmax, __shfl_xor_sync(0xffffffffu, dmax, off));
  }
  if (lane == 0) {
    s_max[0][wib] = gmax;
    s_max[1][wib] = gn2;
    s_max[2][wib] = fn2;
    s_max[3][wib] = dmax;
  }
  __syncthreads();
  if (threadIdx.x < 4) {  // NaN never wins a fmaxf; zero needs no update
    float m = 0.0f;
    for (int k = 0; k < (int)(blockDim.x >> 5); ++k) m = fmaxf(m, s_max[threadIdx.x][k]);
    unsigned* word = threadIdx.x == 0 ? &hdr->g_max : threadIdx.x == 1 ? &hdr->g_norm2 : threadIdx.x == 2 ? &hdr->f_norm2 : &hdr->d_max;
    if (m > 0.0f) atomicMax(word, __float_as_uint(m));
    __threadfence();  // this block's maxima are in place before it reports itself done
  }
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&hdr->blocks_done, 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    __threadfence();
    det_set_scales(hdr, shift, Z, depth_kind, merged);
  }
}

// Dev fields as this kernel reads them: gfeat / gdepth point at int64 arrays of the tensors' shapes, det at the
// DetHeader; CPW = 1, cpt = 1 (record texel fields are plain texel indices), cap = 32.
template <typename T>
__global__ void __launch_bounds__(kMaxWarps * 32) bwd_det_kernel(const __grid_constant__ Dev p) {
  extern __shared__ __align__(16) unsigned char smem[];
  const BlockHeader h = carve(smem, p.N);
  __shared__ int s_tile[2];
  float vs[3], vmin[3];
  voxel_frame(p, vs, vmin);
  const int image_h = __ldg(p.isize), image_w = __ldg(p.isize + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  unsigned char* wa = h.warp_area + (size_t)warp * depth_warp_bytes(1, p.cap);
  int* sLen = reinterpret_cast<int*>(wa);
  int* sCnt = sLen + 32;
  int* sSmp = sCnt + 32;
  uint4* recs = reinterpret_cast<uint4*>(wa + 512);
  uint4* samp = recs + row_stride(p.cap);

  const DetHeader* hdr = p.det;
  long long* gf = reinterpret_cast<long long*>(p.gfeat);
  long long* gd = reinterpret_cast<long long*>(p.gdepth);
  const float scale_f = hdr->scale_f, scale_d = hdr->scale_d;

  const T* fbase = reinterpret_cast<const T*>(p.feats);
  const bool want_feats = (p.flags & FBEV_BWD_FEATS) != 0;
  const bool want_depth = (p.flags & FBEV_BWD_DEPTH) != 0;
  const bool legacy = (p.flags & FBEV_BWD_LEGACY_DEPTH) != 0;
  const bool cat = p.mode == FBEV_DEPTH_CATEGORICAL;
  const bool mean_pool = p.pool == FBEV_POOL_MEAN;
  const int tile_cells = p.TX * p.TY;
  const size_t C = (size_t)p.C;
  int loaded_b = -1;
  TileLoop loop;
  loop.begin(p, s_tile);
  for (int tile; (tile = loop.current(p)) >= 0; loop.advance()) {
    const Tile t = tile_of(p, tile);
    const unsigned vis = tile_visibility(p, t, h, vs, vmin, image_h, image_w, loaded_b);
    const int ncand = __popc(vis) * p.Z;
    for (int tc = warp; tc < tile_cells; tc += nwarps) {
      const int ly = tc / p.TX, lx = tc - ly * p.TX;
      const int x = t.x0 + lx, y = t.y0 + ly;
      if (!(x < t.x1 && y < t.y1)) continue;  // uniform over the warp
      const size_t cell = out_cell(p, t.b, y, x);
      float inv = 1.0f;
      if (mean_pool) {  // the count of all passes comes first
        if (lane == 0) sCnt[0] = 0;
        __syncwarp();
        for (int r0 = 0; r0 < ncand; r0 += p.cap) {
          if (lane == 0) sLen[0] = 0;
          __syncwarp();
          row_list_phase<T, false>(p, t, h, vis, 1u, tc, r0, min(r0 + p.cap, ncand), vs, vmin, image_h, image_w, sLen,
                                   sCnt, recs, lane);
        }
        const int cnt = sCnt[0];
        inv = cnt > 0 ? __fdiv_rn(1.0f, (float)cnt) : 0.0f;
        __syncwarp();
      }
      for (int r0 = 0; r0 < ncand; r0 += p.cap) {
        if (lane == 0) sLen[0] = sCnt[0] = sSmp[0] = 0;
        __syncwarp();
        row_list_phase<T, true, true>(p, t, h, vis, 1u, tc, r0, min(r0 + p.cap, ncand), vs, vmin, image_h, image_w, sLen,
                                      sCnt, recs, lane, samp, sSmp);
        const int n = sLen[0], ns = sSmp[0];
        // ---- per row record: its feature contributions, and T = <g, texel> for its two texels ----
        for (int i = 0; i < n; ++i) {
          const uint4 r = recs[i];
          const size_t tex0 = (size_t)r.x, tex1 = tex0 + r.y;  // r.y = u1 - u0 (0 in the last column)
          const float w0 = __uint_as_float(r.z) * inv, w1 = __uint_as_float(r.w) * inv;
          float t0 = 0.0f, t1 = 0.0f;
          for (int c = lane; c < p.C; c += 32) {
            const float gc = p.out_f32 ? __ldg(reinterpret_cast<const float*>(p.gout) + cell * C + c)
                                       : to_float(__ldg(reinterpret_cast<const T*>(p.gout) + cell * C + c));
            if (want_depth) {
              t0 = fmaf(gc, to_float(__ldg(fbase + tex0 * C + c)), t0);
              t1 = fmaf(gc, to_float(__ldg(fbase + tex1 * C + c)), t1);
            }
            if (want_feats) {
              det_add(gf, tex0 * C + c, gc * w0, scale_f);
              det_add(gf, tex1 * C + c, gc * w1, scale_f);
            }
          }
          if (want_depth) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
              t0 += __shfl_xor_sync(kFull, t0, off);
              t1 += __shfl_xor_sync(kFull, t1, off);
            }
            __syncwarp();
            if (lane == 0) {
              recs[i].z = __float_as_uint(t0);
              recs[i].w = __float_as_uint(t1);
            }
          }
        }
        __syncwarp();
        // ---- one lane per sample: S from four T values, then the sample's depth contributions ----
        if (want_depth) {
          for (int idx = lane; idx < ns; idx += 32) {
            const uint4* sr = samp + (size_t)idx * 3;
            const uint4 sw = sr[0], sa = sr[1], sp = sr[2];
            const float w00 = __uint_as_float(sw.x), w01 = __uint_as_float(sw.y), w10 = __uint_as_float(sw.z),
                        w11 = __uint_as_float(sw.w);
            const uint4 ra = recs[sp.x & 0xffffu], rb = recs[sp.x >> 16];
            float S = w00 * __uint_as_float(ra.z);
            S = fmaf(w10, __uint_as_float(ra.w), S);
            S = fmaf(w01, __uint_as_float(rb.z), S);
            S = fmaf(w11, __uint_as_float(rb.w), S);
            const float sd = S * inv;
            const float v00 = sd * w00, v01 = sd * w01, v10 = sd * w10, v11 = sd * w11;
            // element indices of the four corners' depth rows: (v0,u0), (v0,u1), (v1,u0), (v1,u1)
            const size_t e00 = (size_t)sa.x, e10 = e00 + sa.y, e01 = e00 + sa.z, e11 = e01 + sa.y;
            if (cat) {
              const size_t k = (size_t)sa.w;
              det_add(gd, e00 + k, v00, scale_d);
              det_add(gd, e01 + k, v01, scale_d);
              det_add(gd, e10 + k, v10, scale_d);
              det_add(gd, e11 + k, v11, scale_d);
            } else {
              const float wgt = __uint_as_float(sp.y);
              const float cm = legacy ? wgt : __uint_as_float(sp.z);
              const float cs = legacy ? wgt : __uint_as_float(sp.w);
              det_add(gd, e00, cm * v00, scale_d);
              det_add(gd, e00 + 1, cs * v00, scale_d);
              det_add(gd, e01, cm * v01, scale_d);
              det_add(gd, e01 + 1, cs * v01, scale_d);
              det_add(gd, e10, cm * v10, scale_d);
              det_add(gd, e10 + 1, cs * v10, scale_d);
              det_add(gd, e11, cm * v11, scale_d);
              det_add(gd, e11 + 1, cs * v11, scale_d);
            }
          }
        }
        __syncwarp();
      }
    }
  }  // tiles
  loop.end(p);
}

// Fixed-point sums -> gradient tensors; two arrays (either may be empty) in one launch.  which_b: the second
// array uses the depth scale.  (A sum converts to float32 with one rounding; times a power of two is exact.)
template <typename TA, typename TB>
__global__ void det_finish_kernel(const DetHeader* __restrict__ hdr, const long long* __restrict__ sa, TA* __restrict__ da,
                                  size_t na, const long long* __restrict__ sb, TB* __restrict__ db, size_t nb) {
  const float inv_f = hdr->inv_f, inv_d = hdr->inv_d;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < na + nb; i += stride) {
    if (i < na)
      da[i] = from_float<TA>(__ll2float_rn(sa[i]) * inv_f);
    else
      db[i - na] = from_float<TB>(__ll2float_rn(sb[i - na]) * inv_d);
  }
}

}  // namespace fbev
