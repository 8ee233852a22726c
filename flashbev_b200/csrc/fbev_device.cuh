// Device-side building blocks shared by the forward, backward and index kernels:
// the pinned geometry of one (cell, camera, z) candidate, the depth weight, the
// per-tile camera cull and small load/convert helpers.
//
// Arithmetic that decides an integer (texel index, depth bin, acceptance) is
// written with the round-to-nearest intrinsics (__fmul_rn, __fmaf_rn, __fdiv_rn ...),
// which the compiler neither contracts nor reorders, in the same order as the
// CPU oracle.  It follows flashbev/flashbevpool/src/flash_bevpool_cuda.cu:101-159
// (projection, rejection, texel indices, bilinear weights) and :161-186 (depth
// weight, threshold) of the reference.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fbev.h"
#include "fbev_debug.h"

namespace fbev {

constexpr unsigned kFull = 0xffffffffu;
// Dev.flags bit beside the FBEV_BWD_* ones (internal): the parametric depth sums per record texel leave the depth
// kernel as atomics although it emits entries for the feature gradient
constexpr int kBwdRecordAtomics = 16;

// Head of the scratch of the reproducible backward (fbev_deterministic.cuh; 256 bytes reserved).  The maxima are kept
// as bit patterns: non-negative floats (infinity included) order like unsigned integers, so atomicMax combines them
// in any order.
struct DetHeader {
  unsigned g_max;    // max |g|
  unsigned g_norm2;  // max over cells of sum_c g_c^2
  unsigned f_norm2;  // max over texels of sum_c f_c^2
  unsigned d_max;    // categorical: max |depth value|; parametric: max 1 / (sigma + eps), infinity when that is <= 0
  float scale_f, inv_f;   // fixed-point scale of d_feats and its inverse
  float scale_d, inv_d;   // the same for d_depth
  unsigned blocks_done;   // blocks of det_bounds_kernel that have added their maxima; the last one sets the scales
};

// One contribution to a 64-bit fixed-point sum: an integer atomic, so the sum does not depend on the order.
__device__ __forceinline__ void det_add(long long* base, size_t idx, float v, float scale) {
  atomicAdd(reinterpret_cast<unsigned long long*>(base) + idx, (unsigned long long)__float2ll_rn(v * scale));
}

// Kernel-side view of one call (passed by value as a __grid_constant__).
struct Dev {
  const void* feats;
  const void* depth;
  const float2* dstat;  // categorical depth given as logits: per texel (max, 1 / sum exp(logit - max)); else null
  const float* proj;
  const int* fsize;
  const int* isize;
  const float* roi;
  void* out;
  void* out_peers[7];  // further copies of the output to store to (other GPUs' buffers), n_peers of them
  int n_peers;
  void* out_mc;        // multicast address of the output buffer (NVSwitch replicates each store to all ranks), or null
  int* count;
  int* status;
  const void* gout;  // backward: upstream gradient
  float* gfeat;      // backward: float32 accumulation target [B,N,H,W,C]
  float* gdepth;     // backward: float32 accumulation target [B,N,H,W,D]
  int B, N, H, W, C, D, X, Y, Z, pstride, mode, pool, y0, y1;
  int out_rows, out_y0;  // rows the output / upstream gradient / count tensors hold per sample, and the first of them
  float eps, thr, d0, delta;
  float vs[3], vmin[3];
  int TX, TY, tiles_x, tiles_y;
  int GL;     // lanes that share one cell (each owns V 16-byte channel chunks)
  int cpt;    // 16-byte chunks per texel (GL * V) in the chunked kernels, 0 in the scalar ones
  int CPW;    // cells a warp works on at once = 32 / GL
  int cap;    // sample records per cell per pass
  int flags;  // FBEV_BWD_*
  int out_f32;        // output / upstream gradient are float32 although the features are 16-bit
  unsigned* sched;    // tile scheduler words {next tile, blocks done}, or null for one tile per block
  int static_units;   // forward, one sample: warps stride over (tile, group) units, no barrier, no atomic
  int exp;            // experiment bits (fbev_debug.h: fbev_set_experiment); 0 in normal use
  // gradients through a global sort by texel (null / 0 when not in use)
  unsigned* tex_count;   // [texels + 1] entries per texel (the scatter and gather kernels of large feature maps are
                         // handed tex_start in this field: start of every texel's segment, total last)
  unsigned* tex_start;   // [texels + 1] target of tex_scan_kernel, for feature maps too large to scan inside a block
  unsigned* ent_count;   // [1] entries emitted so far
  uint4* ent;            // [ent_cap] {texel of (row, u0), cell, weight of u0, weight of u1} in emission order
  unsigned* ent_pos;     // [ent_cap] position the entry drew inside its texel's segment
  uint4* ent_sorted;     // [ent_cap] the entries grouped by texel
  float4* ent_d;         // [ent_cap] parametric depth: d mean, d sigma of u0, then of u1 (else null)
  float4* ent_d_sorted;  // [ent_cap]
  unsigned ent_cap;
  // row records and sample lists a training forward leaves for the backward (null: none; fbev_lists.cuh: SavedLists)
  uint4* saved;          // [0] = {cursor, plan key, -, -}, then the directory, then the data area
  unsigned saved_dir;    // directory entries (units x passes), 16 bytes each, from saved + 1
  unsigned saved_cap;    // 16-byte units of data area that follow the directory
  unsigned saved_key;    // identifies the list layout (cells per warp, records per pass, tiling): both sides must agree
  unsigned saved_unit0;  // first unit of this launch within the saved state (backward over a slice of the batch)
  int saved_passes;      // directory entries per unit
  unsigned saved_sub_rec;  // backward over a slice of the batch: what to subtract from the saved chunk indices
  unsigned saved_sub_dep;  // ... and from the saved depth element indices (the slice's tensors start at its first sample)
  // host side only: size of the saved state, batch size it was written for, first sample of this launch in it
  unsigned long long saved_bytes;
  int saved_B, saved_b0;
  // reproducible backward: gfeat / gdepth then point at int64 fixed-point sums instead of float32 (else null)
  const DetHeader* det;
};

// Cell (b, y, x) in the output, the upstream gradient and the count tensor, which hold all Y rows of a sample or only
// the rows [y_begin, y_end) of the call (FbevProblem.compact_rows).
__device__ __forceinline__ size_t out_cell(const Dev& p, int b, int y, int x) {
  return ((size_t)b * p.out_rows + (y - p.out_y0)) * p.X + x;
}

// Programmatic dependent launch (sm_90+).  A kernel launched with the programmatic-serialization attribute may
// start while the kernel before it in the stream is still draining; grid_dependency_wait() returns once that
// kernel has completed and its writes are visible (a no-op for an ordinary launch).  grid_dependency_trigger()
// tells the scheduler that the next kernel's blocks may be brought in as resources free up.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_trigger() { asm volatile("griddepcontrol.launch_dependents;"); }

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

// Unpack one 16-byte chunk into floats: 4 (float32) or 8 (16-bit types).
template <typename T>
struct Chunk;
template <>
struct Chunk<float> {
  static constexpr int E = 4;
  static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
    f[0] = __uint_as_float(r.x);
    f[1] = __uint_as_float(r.y);
    f[2] = __uint_as_float(r.z);
    f[3] = __uint_as_float(r.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};
template <>
struct Chunk<__nv_bfloat16> {
  static constexpr int E = 8;
  static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
    // a bfloat16 is the upper half of a float32
    f[0] = __uint_as_float(r.x << 16);
    f[1] = __uint_as_float(r.x & 0xffff0000u);
    f[2] = __uint_as_float(r.y << 16);
    f[3] = __uint_as_float(r.y & 0xffff0000u);
    f[4] = __uint_as_float(r.z << 16);
    f[5] = __uint_as_float(r.z & 0xffff0000u);
    f[6] = __uint_as_float(r.w << 16);
    f[7] = __uint_as_float(r.w & 0xffff0000u);
  }
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
  }
};
template <>
struct Chunk<__half> {
  static constexpr int E = 8;
  static __device__ __forceinline__ void unpack2(uint32_t w, float* f) {
    __half2 h = *reinterpret_cast<__half2*>(&w);
    float2 v = __half22float2(h);
    f[0] = v.x;
    f[1] = v.y;
  }
  static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
    unpack2(r.x, f + 0);
    unpack2(r.y, f + 2);
    unpack2(r.z, f + 4);
    unpack2(r.w, f + 6);
  }
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
  }
};

__device__ __forceinline__ uint4 ldg16(const uint4* p) { return __ldg(p); }

// Voxel-centre coordinate  min + (i + 0.5) * size  (flash_bevpool_cuda.cu:45-46,102).
__device__ __forceinline__ float centre(int i, float vs, float vmin) {
  return __fmaf_rn(__fadd_rn(__int2float_rn(i), 0.5f), vs, vmin);
}

// One row of the 3x4 projection (flash_bevpool_cuda.cu:111-122):
// p0*x + p1*y + p2*z + p3 as fma(p2,z, fma(p1,y, p0*x)) + p3.
__device__ __forceinline__ float proj_row(const float* p, float x, float y, float z) {
  float t = __fmul_rn(p[0], x);
  t = __fmaf_rn(p[1], y, t);
  t = __fmaf_rn(p[2], z, t);
  return __fadd_rn(t, p[3]);
}

// x / d, correctly rounded.  When d is a power of two its reciprocal is exact, and x * (1 / d) rounds the same real
// number as x / d does: the same bits for one multiplication instead of a division sequence.  (Image heights of
// 256 or 512 and depth-bin widths of 0.5 or 1 are powers of two.)  d > 0, finite and normal.
__device__ __forceinline__ float div_exact(float x, float d) {
  const unsigned bits = __float_as_uint(d);
  if ((bits & 0x007fffffu) == 0u && bits >= 0x00800000u && bits <= 0x7e800000u)
    return __fmul_rn(x, __uint_as_float(0x7f000000u - bits));
  return __fdiv_rn(x, d);
}

struct Sample {
  float w00, w01, w10, w11;  // bilinear weights; first index = u offset, second = v offset (:156-159)
  float wgt;                 // depth weight
  float dmean, dsigma;       // d wgt / d mean, d wgt / d sigma (parametric modes, backward only)
  float id;                  // camera depth
  int u0, v0, u1, v1;
  int k;                     // depth bin (categorical) or -1
};

// Geometry of one candidate (flash_bevpool_cuda.cu:125-159).  False if rejected.
__device__ __forceinline__ bool geometry(const float* P, float vx, float vy, float vz, int image_h, int image_w,
                                         int fh, int fw, float eps, Sample& s) {
  const float id = proj_row(P + 8, vx, vy, vz);
  s.id = id;
  if (!(id > 0.0f)) return false;
  float iu = proj_row(P + 0, vx, vy, vz);
  float iv = proj_row(P + 4, vx, vy, vz);
  const float cd = fmaxf(id, eps);
  iu = __fdiv_rn(iu, cd);
  iv = __fdiv_rn(iv, cd);
  const float fwf = __int2float_rn(fw), fhf = __int2float_rn(fh);
  const float fu = __fmul_rn(div_exact(iu, __int2float_rn(image_w)), fwf);
  const float fv = __fmul_rn(div_exact(iv, __int2float_rn(image_h)), fhf);
  if (!(fu >= 0.0f && fu < fwf && fv >= 0.0f && fv < fhf)) return false;
  int u0 = __float2int_rd(fu);
  int v0 = __float2int_rd(fv);
  const float du = __fsub_rn(fu, __int2float_rn(u0));
  const float dv = __fsub_rn(fv, __int2float_rn(v0));
  u0 = max(0, min(u0, fw - 1));
  v0 = max(0, min(v0, fh - 1));
  s.u0 = u0;
  s.v0 = v0;
  s.u1 = min(u0 + 1, fw - 1);
  s.v1 = min(v0 + 1, fh - 1);
  const float a = __fsub_rn(1.0f, du), b = __fsub_rn(1.0f, dv);
  s.w00 = __fmul_rn(a, b);
  s.w01 = __fmul_rn(a, dv);
  s.w10 = __fmul_rn(du, b);
  s.w11 = __fmul_rn(du, dv);
  return true;
}

__device__ __forceinline__ float interp4(const Sample& s, float f00, float f01, float f10, float f11) {
  float t = __fmul_rn(s.w00, f00);
  t = __fmaf_rn(s.w01, f01, t);
  t = __fmaf_rn(s.w10, f10, t);
  t = __fmaf_rn(s.w11, f11, t);
  return t;
}

// Depth weight and acceptance of a geometrically valid sample.
//   parametric  flash_bevpool_cuda.cu:161-186
//   categorical bilinear lookup of bin floor((d - d0) / delta) with the feature weights
// `texbase`: index of texel (0, 0) of the sample's (b, camera) slice, [fh, fw, D] elements of depth from there.
// IDX: type the element indices are computed in.  size_t always works; the chunked kernels are only chosen for
// tensors of fewer than 2^32 depth elements (make_plan) and use unsigned, which spares them the 64-bit index
// arithmetic of four corners per candidate.
template <typename T, bool GRAD, typename IDX = size_t>
__device__ __forceinline__ bool depth_weight(const Dev& p, IDX texbase, int fw, Sample& s) {
  const IDX D = (IDX)p.D;
  const T* dep = reinterpret_cast<const T*>(p.depth);
  const IDX t00 = texbase + (IDX)(s.v0 * fw + s.u0), t01 = texbase + (IDX)(s.v1 * fw + s.u0);
  const IDX t10 = texbase + (IDX)(s.v0 * fw + s.u1), t11 = texbase + (IDX)(s.v1 * fw + s.u1);
  const T* p00 = dep + t00 * D;
  const T* p01 = dep + t01 * D;
  const T* p10 = dep + t10 * D;
  const T* p11 = dep + t11 * D;
  if (p.mode == FBEV_DEPTH_CATEGORICAL) {
    const float kf = div_exact(__fsub_rn(s.id, p.d0), p.delta);
    if (!(kf >= 0.0f && kf < __int2float_rn(p.D))) return false;
    const int k = __float2int_rz(kf);
    s.k = k;
    float e00 = to_float(__ldg(p00 + k)), e01 = to_float(__ldg(p01 + k)), e10 = to_float(__ldg(p10 + k)),
          e11 = to_float(__ldg(p11 + k));
    if (p.dstat != nullptr) {
      // logits: probability of bin k = exp(logit - max) / sum, with the texel's statistics from the pre-pass
      const float2* st = p.dstat;
      const float2 s00 = __ldg(st + t00), s01 = __ldg(st + t01), s10 = __ldg(st + t10), s11 = __ldg(st + t11);
      e00 = expf(e00 - s00.x) * s00.y;
      e01 = expf(e01 - s01.x) * s01.y;
      e10 = expf(e10 - s10.x) * s10.y;
      e11 = expf(e11 - s11.x) * s11.y;
    }
    s.wgt = interp4(s, e00, e01, e10, e11);
    return !(s.wgt < p.thr);
  }
  s.k = -1;
  const float mean = interp4(s, to_float(__ldg(p00)), to_float(__ldg(p01)), to_float(__ldg(p10)), to_float(__ldg(p11)));
  const float sigma = interp4(s, to_float(__ldg(p00 + 1)), to_float(__ldg(p01 + 1)), to_float(__ldg(p10 + 1)),
                              to_float(__ldg(p11 + 1)));
  const float se = __fadd_rn(sigma, p.eps);
  const float zs = __fdiv_rn(__fsub_rn(s.id, mean), se);
  if (p.mode == FBEV_DEPTH_GAUSSIAN) {
    s.wgt = __fdiv_rn(expf(__fmul_rn(__fmul_rn(-0.5f, zs), zs)), se);
    if (GRAD) {
      s.dmean = s.wgt * zs / se;
      s.dsigma = s.wgt * (zs * zs - 1.0f) / se;
    }
  } else {
    s.wgt = __fdiv_rn(__fmul_rn(0.5f, expf(-fabsf(zs))), se);
    if (GRAD) {
      const float sgn = zs > 0.0f ? 1.0f : (zs < 0.0f ? -1.0f : 0.0f);
      s.dmean = s.wgt * sgn / se;
      s.dsigma = s.wgt * (fabsf(zs) - 1.0f) / se;
    }
  }
  return !(s.wgt < p.thr);
}

// Conservative per-tile camera cull.  Returns false only when every candidate
// whose voxel centre lies in the box [bx0,bx1]x[by0,by1]x[bz0,bz1] is certain to be
// rejected by geometry() (behind the camera, outside the feature map) or, in the
// categorical mode, to fall outside the depth bins.  u, v and depth are affine in
// the voxel centre, so their extrema over the box are at its corners; the margins
// (1e-5 of the terms' magnitude, some 30x the float32 evaluation error) keep the
// decision on the safe side of every rounding in geometry().
__device__ __forceinline__ bool camera_may_see(const Dev& p, const float* P, float bx0, float bx1, float by0,
                                               float by1, float bz0, float bz1, int image_h, int image_w) {
  const float ax = fmaxf(fabsf(bx0), fabsf(bx1)), ay = fmaxf(fabsf(by0), fabsf(by1)),
              az = fmaxf(fabsf(bz0), fabsf(bz1));
  const float rel = 1e-5f;
  const float mu = rel * (fabsf(P[0]) * ax + fabsf(P[1]) * ay + fabsf(P[2]) * az + fabsf(P[3]));
  const float mv = rel * (fabsf(P[4]) * ax + fabsf(P[5]) * ay + fabsf(P[6]) * az + fabsf(P[7]));
  const float md = rel * (fabsf(P[8]) * ax + fabsf(P[9]) * ay + fabsf(P[10]) * az + fabsf(P[11]));
  const float Wf = (float)image_w * (1.0f + rel), Hf = (float)image_h * (1.0f + rel);
  const float inf = __int_as_float(0x7f800000);
  float dmax = -inf, dmin = inf, umax = -inf, umin = inf, vmax = -inf, vmin = inf, rumin = inf, rvmin = inf;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const float x = (c & 1) ? bx1 : bx0, y = (c & 2) ? by1 : by0, z = (c & 4) ? bz1 : bz0;
    const float lu = fmaf(P[2], z, fmaf(P[1], y, P[0] * x)) + P[3];
    const float lv = fmaf(P[6], z, fmaf(P[5], y, P[4] * x)) + P[7];
    const float ld = fmaf(P[10], z, fmaf(P[9], y, P[8] * x)) + P[11];
    dmax = fmaxf(dmax, ld);
    dmin = fminf(dmin, ld);
    umax = fmaxf(umax, lu);
    umin = fminf(umin, lu);
    vmax = fmaxf(vmax, lv);
    vmin = fminf(vmin, lv);
    rumin = fminf(rumin, lu - Wf * ld);
    rvmin = fminf(rvmin, lv - Hf * ld);
  }
  const float tiny = 1e-12f;
  if (dmax + md < -tiny) return false;  // behind the camera everywhere
  if (umax + mu < -tiny) return false;  // left of the image everywhere
  if (vmax + mv < -tiny) return false;  // above the image everywhere
  // right of / below the image everywhere: u >= W' * max(d, eps) with W' slightly above the width
  if (rumin - (mu + Wf * md) > tiny && umin - mu > Wf * p.eps) return false;
  if (rvmin - (mv + Hf * md) > tiny && vmin - mv > Hf * p.eps) return false;
  if (p.mode == FBEV_DEPTH_CATEGORICAL) {
    const float dfar = p.d0 + (float)p.D * p.delta;
    if (dmax + md < p.d0 - rel * fabsf(p.d0) - tiny) return false;  // nearer than the first bin
    if (dmin - md > dfar + rel * fabsf(dfar) + tiny) return false;  // beyond the last bin
  }
  return true;
}

// Voxel sizes: from the device roi_range as the reference backward kernel does
// ((max - min) / grid in float32, flash_bevpool_cuda.cu:465-470), or the host's
// values (flash_bevpool.py:62-67) when no roi pointer was given.
__device__ __forceinline__ void voxel_frame(const Dev& p, float vs[3], float vmin[3]) {
  if (p.roi != nullptr) {
    const float r0 = __ldg(p.roi + 0), r1 = __ldg(p.roi + 1), r2 = __ldg(p.roi + 2), r3 = __ldg(p.roi + 3),
                r4 = __ldg(p.roi + 4), r5 = __ldg(p.roi + 5);
    vs[0] = __fdiv_rn(__fsub_rn(r1, r0), __int2float_rn(p.X));
    vs[1] = __fdiv_rn(__fsub_rn(r3, r2), __int2float_rn(p.Y));
    vs[2] = __fdiv_rn(__fsub_rn(r5, r4), __int2float_rn(p.Z));
    vmin[0] = r0;
    vmin[1] = r2;
    vmin[2] = r4;
  } else {
    vs[0] = p.vs[0];
    vs[1] = p.vs[1];
    vs[2] = p.vs[2];
    vmin[0] = p.vmin[0];
    vmin[1] = p.vmin[1];
    vmin[2] = p.vmin[2];
  }
}

}  // namespace fbev
