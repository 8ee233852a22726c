/*
 * CPU oracle for the fused BEV pooling operator.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker the CUDA path is compared with.  Only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg may load it; the
 * product library never links or calls it.
 *
 * It restates, in plain C, the arithmetic of the reference operator
 * (yokosyun/FlashBEV):
 *   forward kernel   flashbev/flashbevpool/src/flash_bevpool_cuda.cu:31-216
 *   backward kernel  flashbev/flashbevpool/src/flash_bevpool_cuda.cu:446-681
 *   host preparation flashbev/flashbevpool/flash_bevpool.py:47-71
 * and adds the categorical depth mode (depth-bin lookup into a softmaxed
 * distribution), which the reference does not have: for that mode this file is
 * the specification, and its parity is not pinned by reference code.
 *
 * Pinning status: the parametric modes (gaussian / laplace, mean pooling) are
 * checked against outputs of the reference's own dense PyTorch path
 * (flashbev/flashbevpool/sampling_vt.py:36-123, 449-466) stored as fixtures in
 * tests/golden/, and against the reference's CUDA kernels where a built copy
 * is available.  The categorical mode is "parity unpinned".
 *
 * Operation order.  Everything that decides an integer (texel indices, depth
 * bin, validity) is evaluated in IEEE binary32 with one fixed order, written
 * with explicit fmaf() so that the CUDA kernels can reproduce it bit for bit.
 * Build with -ffp-contract=off so the compiler adds no contraction of its own.
 * Two float flavours of everything after the geometry exist: binary32 in the
 * pinned order ("f32") and binary64 ("f64", same integer decisions, wider
 * arithmetic) which bounds the rounding error of the first.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define FBEV_MODE_GAUSSIAN 0
#define FBEV_MODE_LAPLACE 1
#define FBEV_MODE_CATEGORICAL 2
#define FBEV_POOL_MEAN 0
#define FBEV_POOL_SUM 1

typedef struct {
  /* sizes */
  int B, N, H, W, C, D; /* D: last dim of the depth tensor (2 for parametric) */
  int X, Y, Z;
  int proj_stride;      /* floats per camera matrix: 12 ([3,4]) or 16 ([4,4], rows 0-2 used) */
  /* inputs (all binary32 on the host; low-precision cases pass pre-rounded values) */
  const float *feats;   /* [B,N,H,W,C] */
  const float *depth;   /* [B,N,H,W,D] */
  const float *proj;    /* [B,N,proj_stride] */
  const int32_t *feature_size; /* [B,N,2] (h, w) */
  int image_h, image_w;
  float roi[6];         /* xmin,xmax,ymin,ymax,zmin,zmax */
  float eps, threshold;
  int mode, pool;
  float d0, delta;      /* categorical: first bin edge and bin width */
  int y_begin, y_end;   /* rows computed; others are left untouched */
  int threads;          /* OpenMP threads (<=1: serial) */
} oracle_args;

typedef struct {
  int valid;            /* passed d>0 and the field-of-view test */
  int u0, v0, u1, v1;
  float du, dv;
  float id;             /* camera depth of the voxel centre */
} geom_t;

/* flash_bevpool.py:62-64 (forward) and flash_bevpool_cuda.cu:465-470 (backward):
 * voxel size = (max - min) / grid, in binary32. */
static void voxel_sizes(const oracle_args *a, float vs[3], float vmin[3]) {
  vs[0] = (a->roi[1] - a->roi[0]) / (float)a->X;
  vs[1] = (a->roi[3] - a->roi[2]) / (float)a->Y;
  vs[2] = (a->roi[5] - a->roi[4]) / (float)a->Z;
  vmin[0] = a->roi[0];
  vmin[1] = a->roi[2];
  vmin[2] = a->roi[4];
}

/* Voxel-centre coordinate, flash_bevpool_cuda.cu:45-46,102:  min + (i + 0.5f) * size. */
static inline float centre(int i, float vs, float vmin) { return fmaf((float)i + 0.5f, vs, vmin); }

/* One row of the 3x4 projection, flash_bevpool_cuda.cu:111-122:
 * p0*x + p1*y + p2*z + p3, pinned as fma(p2,z, fma(p1,y, p0*x)) + p3. */
static inline float proj_row(const float *p, float x, float y, float z) {
  float t = p[0] * x;
  t = fmaf(p[1], y, t);
  t = fmaf(p[2], z, t);
  return t + p[3];
}

/* Geometry of one (cell, camera, z) candidate: flash_bevpool_cuda.cu:125-159. */
static inline void geometry(const float *P, float vx, float vy, float vz, int image_h, int image_w,
                            int feat_h, int feat_w, float eps, geom_t *g) {
  g->valid = 0;
  float id = proj_row(P + 8, vx, vy, vz);
  g->id = id;
  if (!(id > 0.0f)) return;                       /* :125 (NaN depth is rejected too) */
  float iu = proj_row(P + 0, vx, vy, vz);
  float iv = proj_row(P + 4, vx, vy, vz);
  float cd = fmaxf(id, eps);                      /* :130 */
  iu = iu / cd;                                   /* :131 */
  iv = iv / cd;                                   /* :132 */
  float fu = iu / (float)image_w * (float)feat_w; /* :137 */
  float fv = iv / (float)image_h * (float)feat_h; /* :138 */
  /* :140.  Written so that a NaN coordinate is rejected instead of indexed. */
  if (!(fu >= 0.0f && fu < (float)feat_w && fv >= 0.0f && fv < (float)feat_h)) return;
  int u0 = (int)floorf(fu);                       /* :147 */
  int v0 = (int)floorf(fv);
  g->du = fu - (float)u0;                         /* :149 */
  g->dv = fv - (float)v0;
  if (u0 > feat_w - 1) u0 = feat_w - 1;           /* :151-154 */
  if (u0 < 0) u0 = 0;
  if (v0 > feat_h - 1) v0 = feat_h - 1;
  if (v0 < 0) v0 = 0;
  g->u0 = u0;
  g->v0 = v0;
  g->u1 = (u0 + 1 < feat_w) ? u0 + 1 : feat_w - 1;
  g->v1 = (v0 + 1 < feat_h) ? v0 + 1 : feat_h - 1;
  g->valid = 1;
}

/* Depth bin of the categorical mode: k = floor((d - d0) / delta), valid for 0 <= k < D. */
static inline int depth_bin(float id, float d0, float delta, int D) {
  float kf = (id - d0) / delta;
  if (!(kf >= 0.0f && kf < (float)D)) return -1;
  return (int)kf;
}

/* ---- binary32 flavour, pinned order ------------------------------------- */
#define REAL float
#define SUFFIX(n) n##_f32
#define R_FMA(a, b, c) fmaf((a), (b), (c))
#define R_EXP(x) expf(x)
#define R_ABS(x) fabsf(x)
#include "fbev_oracle_body.inc"
#undef REAL
#undef SUFFIX
#undef R_FMA
#undef R_EXP
#undef R_ABS

/* ---- binary64 flavour --------------------------------------------------- */
#define REAL double
#define SUFFIX(n) n##_f64
#define R_FMA(a, b, c) ((a) * (b) + (c))
#define R_EXP(x) exp(x)
#define R_ABS(x) fabs(x)
#include "fbev_oracle_body.inc"
#undef REAL
#undef SUFFIX
#undef R_FMA
#undef R_EXP
#undef R_ABS

/* Integer decisions for every candidate, [B,N,Y,X,Z] each, plus the per-cell
 * count of accepted samples [B,Y,X].  Rejected candidates hold -1 / 0.
 * `valid` is the final acceptance (geometry, depth bin, weight threshold). */
int fbev_oracle_indices(const oracle_args *a, int32_t *u0, int32_t *v0, int32_t *kbin, uint8_t *valid,
                        int32_t *count) {
  float vs[3], vmin[3];
  voxel_sizes(a, vs, vmin);
  for (int b = 0; b < a->B; ++b)
    for (int y = 0; y < a->Y; ++y)
      for (int x = 0; x < a->X; ++x) {
        float vx = centre(x, vs[0], vmin[0]);
        float vy = centre(y, vs[1], vmin[1]);
        int cnt = 0;
        for (int n = 0; n < a->N; ++n) {
          const float *P = a->proj + ((size_t)b * a->N + n) * a->proj_stride;
          int fh = a->feature_size[((size_t)b * a->N + n) * 2 + 0];
          int fw = a->feature_size[((size_t)b * a->N + n) * 2 + 1];
          const float *dep = a->depth + ((size_t)b * a->N + n) * fh * fw * a->D;
          for (int z = 0; z < a->Z; ++z) {
            size_t q = ((((size_t)b * a->N + n) * a->Y + y) * a->X + x) * a->Z + z;
            u0[q] = v0[q] = kbin[q] = -1;
            valid[q] = 0;
            geom_t g;
            geometry(P, vx, vy, centre(z, vs[2], vmin[2]), a->image_h, a->image_w, fh, fw, a->eps, &g);
            if (!g.valid) continue;
            int k = -1;
            float wgt = sample_weight_f32(a, dep, fw, &g, &k, 0, 0);
            if (k == -2) continue; /* outside the depth bins */
            if (wgt < a->threshold) continue;
            u0[q] = g.u0;
            v0[q] = g.v0;
            kbin[q] = k;
            valid[q] = 1;
            ++cnt;
          }
        }
        count[((size_t)b * a->Y + y) * a->X + x] = cnt;
      }
  return 0;
}

/* Projection matrices from calibration (create_projection_matrix, flashbev/flashbevpool/sampling_vt.py:21-33):
 * K4 = identity with K4[:3,:3] = post_rots * camera2imgs and post_trans added to column 2;
 * out = (K4 * inverse(sensor2ego))[:3, :].  Float64 throughout; the inverse by Gauss-Jordan elimination with
 * partial pivoting (torch.inverse there is an LU solve).  Returns 1 for a singular pose. */
int fbev_oracle_projection(const float* s2e, const float* k33, const float* rot, const float* trans, double* out,
                           int count) {
  for (int i = 0; i < count; ++i) {
    double a[4][8];
    for (int r = 0; r < 4; ++r)
      for (int c = 0; c < 4; ++c) {
        a[r][c] = (double)s2e[(size_t)i * 16 + r * 4 + c];
        a[r][4 + c] = r == c ? 1.0 : 0.0;
      }
    for (int col = 0; col < 4; ++col) {
      int piv = col;
      for (int r = col + 1; r < 4; ++r)
        if (fabs(a[r][col]) > fabs(a[piv][col])) piv = r;
      if (a[piv][col] == 0.0) return 1;
      if (piv != col)
        for (int c = 0; c < 8; ++c) {
          double t = a[col][c];
          a[col][c] = a[piv][c];
          a[piv][c] = t;
        }
      double inv = 1.0 / a[col][col];
      for (int c = 0; c < 8; ++c) a[col][c] *= inv;
      for (int r = 0; r < 4; ++r) {
        if (r == col) continue;
        double f = a[r][col];
        for (int c = 0; c < 8; ++c) a[r][c] -= f * a[col][c];
      }
    }
    double K[4][4] = {{0}};
    K[3][3] = 1.0;
    for (int r = 0; r < 3; ++r) {
      for (int c = 0; c < 3; ++c)
        for (int k = 0; k < 3; ++k)
          K[r][c] += (double)rot[(size_t)i * 9 + r * 3 + k] * (double)k33[(size_t)i * 9 + k * 3 + c];
      K[r][2] += (double)trans[(size_t)i * 3 + r];
    }
    for (int r = 0; r < 3; ++r)
      for (int c = 0; c < 4; ++c) {
        double acc = 0.0;
        for (int k = 0; k < 4; ++k) acc += K[r][k] * a[k][4 + c];
        out[(size_t)i * 12 + r * 4 + c] = acc;
      }
  }
  return 0;
}

int fbev_oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
