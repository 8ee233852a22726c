// Index dump for bit-exact tests, projection matrices from calibration, L2 read-bandwidth probe.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fbev.h"
#include "fbev_lists.cuh"

namespace fbev {

// ---------------------------------------------------------------------------
// Integer decisions of every candidate (one thread per BEV cell)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void indices_kernel(const __grid_constant__ Dev p, int* u0, int* v0, int* kbin, unsigned char* valid) {
  const size_t cells = (size_t)p.B * p.Y * p.X;
  const size_t cell = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (cell >= cells) return;
  const int x = (int)(cell % p.X);
  const int y = (int)((cell / p.X) % p.Y);
  const int b = (int)(cell / ((size_t)p.X * p.Y));
  float vs[3], vmin[3];
  voxel_frame(p, vs, vmin);
  const int image_h = __ldg(p.isize), image_w = __ldg(p.isize + 1);
  const float vx = centre(x, vs[0], vmin[0]), vy = centre(y, vs[1], vmin[1]);
  int cnt = 0;
  for (int n = 0; n < p.N; ++n) {
    float P[12];
    for (int k = 0; k < 12; ++k) P[k] = __ldg(p.proj + ((size_t)b * p.N + n) * p.pstride + k);
    const int fh = __ldg(p.fsize + ((size_t)b * p.N + n) * 2), fw = __ldg(p.fsize + ((size_t)b * p.N + n) * 2 + 1);
    const bool fs_ok = fh > 0 && fw > 0 && (long long)fh * fw <= (long long)p.H * p.W;
    const size_t texbase = ((size_t)b * p.N + n) * (size_t)fh * fw;
    for (int z = 0; z < p.Z; ++z) {
      const size_t q = ((((size_t)b * p.N + n) * p.Y + y) * p.X + x) * p.Z + z;
      int ou = -1, ov = -1, ok = -1;
      unsigned char oval = 0;
      Sample s;
      if (fs_ok && geometry(P, vx, vy, centre(z, vs[2], vmin[2]), image_h, image_w, fh, fw, p.eps, s) &&
          depth_weight<T, false>(p, reinterpret_cast<const T*>(p.depth) + texbase * p.D, fw, s)) {
        ou = s.u0;
        ov = s.v0;
        ok = s.k;
        oval = 1;
        ++cnt;
      }
      u0[q] = ou;
      v0[q] = ov;
      kbin[q] = ok;
      valid[q] = oval;
    }
  }
  p.count[cell] = cnt;
}

// One thread per camera: P = K4 * inverse(sensor2ego), rows 0-2 (sampling_vt.py:21-33).
__global__ void projection_kernel(const float* __restrict__ s2e, const float* __restrict__ k33,
                                  const float* __restrict__ rot, const float* __restrict__ trans,
                                  float* __restrict__ out, int count) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  double m[16], inv[16];
  for (int k = 0; k < 16; ++k) m[k] = (double)s2e[(size_t)i * 16 + k];
  // adjugate / determinant
  inv[0] = m[5] * m[10] * m[15] - m[5] * m[11] * m[14] - m[9] * m[6] * m[15] + m[9] * m[7] * m[14] + m[13] * m[6] * m[11] - m[13] * m[7] * m[10];
  inv[4] = -m[4] * m[10] * m[15] + m[4] * m[11] * m[14] + m[8] * m[6] * m[15] - m[8] * m[7] * m[14] - m[12] * m[6] * m[11] + m[12] * m[7] * m[10];
  inv[8] = m[4] * m[9] * m[15] - m[4] * m[11] * m[13] - m[8] * m[5] * m[15] + m[8] * m[7] * m[13] + m[12] * m[5] * m[11] - m[12] * m[7] * m[9];
  inv[12] = -m[4] * m[9] * m[14] + m[4] * m[10] * m[13] + m[8] * m[5] * m[14] - m[8] * m[6] * m[13] - m[12] * m[5] * m[10] + m[12] * m[6] * m[9];
  inv[1] = -m[1] * m[10] * m[15] + m[1] * m[11] * m[14] + m[9] * m[2] * m[15] - m[9] * m[3] * m[14] - m[13] * m[2] * m[11] + m[13] * m[3] * m[10];
  inv[5] = m[0] * m[10] * m[15] - m[0] * m[11] * m[14] - m[8] * m[2] * m[15] + m[8] * m[3] * m[14] + m[12] * m[2] * m[11] - m[12] * m[3] * m[10];
  inv[9] = -m[0] * m[9] * m[15] + m[0] * m[11] * m[13] + m[8] * m[1] * m[15] - m[8] * m[3] * m[13] - m[12] * m[1] * m[11] + m[12] * m[3] * m[9];
  inv[13] = m[0] * m[9] * m[14] - m[0] * m[10] * m[13] - m[8] * m[1] * m[14] + m[8] * m[2] * m[13] + m[12] * m[1] * m[10] - m[12] * m[2] * m[9];
  inv[2] = m[1] * m[6] * m[15] - m[1] * m[7] * m[14] - m[5] * m[2] * m[15] + m[5] * m[3] * m[14] + m[13] * m[2] * m[7] - m[13] * m[3] * m[6];
  inv[6] = -m[0] * m[6] * m[15] + m[0] * m[7] * m[14] + m[4] * m[2] * m[15] - m[4] * m[3] * m[14] - m[12] * m[2] * m[7] + m[12] * m[3] * m[6];
  inv[10] = m[0] * m[5] * m[15] - m[0] * m[7] * m[13] - m[4] * m[1] * m[15] + m[4] * m[3] * m[13] + m[12] * m[1] * m[7] - m[12] * m[3] * m[5];
  inv[14] = -m[0] * m[5] * m[14] + m[0] * m[6] * m[13] + m[4] * m[1] * m[14] - m[4] * m[2] * m[13] - m[12] * m[1] * m[6] + m[12] * m[2] * m[5];
  inv[3] = -m[1] * m[6] * m[11] + m[1] * m[7] * m[10] + m[5] * m[2] * m[11] - m[5] * m[3] * m[10] - m[9] * m[2] * m[7] + m[9] * m[3] * m[6];
  inv[7] = m[0] * m[6] * m[11] - m[0] * m[7] * m[10] - m[4] * m[2] * m[11] + m[4] * m[3] * m[10] + m[8] * m[2] * m[7] - m[8] * m[3] * m[6];
  inv[11] = -m[0] * m[5] * m[11] + m[0] * m[7] * m[9] + m[4] * m[1] * m[11] - m[4] * m[3] * m[9] - m[8] * m[1] * m[7] + m[8] * m[3] * m[5];
  inv[15] = m[0] * m[5] * m[10] - m[0] * m[6] * m[9] - m[4] * m[1] * m[10] + m[4] * m[2] * m[9] + m[8] * m[1] * m[6] - m[8] * m[2] * m[5];
  const double det = m[0] * inv[0] + m[1] * inv[4] + m[2] * inv[8] + m[3] * inv[12];
  const double rdet = 1.0 / det;  // a singular pose gives inf / nan, as torch.inverse would complain about
  for (int k = 0; k < 16; ++k) inv[k] *= rdet;
  // K4 rows 0-2: (post_rots * camera2imgs) with post_trans added to column 2, fourth column 0
  double K[12];
  for (int r = 0; r < 3; ++r) {
    for (int c = 0; c < 3; ++c) {
      double a = 0.0;
      for (int k = 0; k < 3; ++k) a += (double)rot[(size_t)i * 9 + r * 3 + k] * (double)k33[(size_t)i * 9 + k * 3 + c];
      K[r * 4 + c] = a;
    }
    K[r * 4 + 2] += (double)trans[(size_t)i * 3 + r];
    K[r * 4 + 3] = 0.0;
  }
  for (int r = 0; r < 3; ++r)
    for (int c = 0; c < 4; ++c) {
      double a = 0.0;
      for (int k = 0; k < 4; ++k) a += K[r * 4 + k] * inv[k * 4 + c];
      out[(size_t)i * 12 + r * 4 + c] = (float)a;
    }
}

__global__ void probe_read_kernel(const uint4* __restrict__ buf, size_t n16, int repeats, unsigned* sink) {
  unsigned acc = 0;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (int r = 0; r < repeats; ++r)
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
      uint4 v;
      // volatile: every repeat re-reads memory instead of reusing registers; .cg: served by L2, not by L1
      asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(buf + i));
      acc ^= v.x ^ v.y ^ v.z ^ v.w;
    }
  if (acc == 0x9e3779b9u) *sink = acc;  // practically never true; keeps the loads alive
}

}  // namespace fbev
