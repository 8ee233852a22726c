/*
 * fbev.h - C ABI of the B200 (sm_100a) fused BEV pooling library, libfbev.so.
 *
 * The library replaces the native half of the reference operator
 * flashbevpool.flash_bevpool (yokosyun/FlashBEV): the pybind11 module
 * flashbevpool_ext (flashbev/flashbevpool/src/flash_bevpool.cpp:79-246) and the
 * CUDA launchers and kernels behind it (src/flash_bevpool_cuda.cu).  It has no
 * torch, pybind or C++ types in its interface: plain pointers, sizes, a stream.
 *
 * Conventions
 *  - Every pointer marked "device" is device memory the caller owns; the library
 *    borrows it for the duration of the asynchronous launch and never allocates
 *    or frees device memory in these calls.
 *  - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 *  - Every function returns an FBEV_* status (0 = success) and never throws,
 *    aborts or traps.  Launch errors are collected with cudaGetLastError, without
 *    synchronising.
 *  - Layouts are the reference's (flash_bevpool.py:28-34,44): features
 *    [B,N,H,W,C] channels-last, depth [B,N,H,W,Dd], output [B,Y,X,C].
 */
#ifndef FBEV_H_
#define FBEV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FBEV_ABI_VERSION 2

/* element type of features, depth, output and gradients */
enum { FBEV_F32 = 0, FBEV_BF16 = 1, FBEV_F16 = 2 };

/* depth model.  0 and 1 are the reference's (flash_bevpool.py:35,
 * flash_bevpool_cuda.cu:178-184); 2 is the depth-bin lookup into a softmaxed
 * distribution, depth tensor [B,N,H,W,D], which the reference does not have. */
enum {
  FBEV_DEPTH_GAUSSIAN = 0,
  FBEV_DEPTH_LAPLACE = 1,
  FBEV_DEPTH_CATEGORICAL = 2,
  /* as 2, but the depth tensor holds the depth head's LOGITS: the softmax over the D bins (in a model it is a
   * pass of its own over the tensor, before the operator) is folded into the lookup, and its backward into the
   * operator's backward, which then returns the gradient with respect to the logits.  Needs depth_stats. */
  FBEV_DEPTH_CATEGORICAL_LOGITS = 3
};

/* reduction over cameras and height bins: mean over accepted samples
 * (reference, flash_bevpool_cuda.cu:212-216) or plain sum */
enum { FBEV_POOL_MEAN = 0, FBEV_POOL_SUM = 1 };

/* status codes */
enum {
  FBEV_OK = 0,
  FBEV_ERR_NULL = 1,        /* a required pointer is NULL */
  FBEV_ERR_STRUCT = 2,      /* struct_size does not match this library */
  FBEV_ERR_SHAPE = 3,       /* a size is non-positive or inconsistent */
  FBEV_ERR_DTYPE = 4,       /* unknown element type */
  FBEV_ERR_MODE = 5,        /* unknown depth model / pooling, or bad bin parameters */
  FBEV_ERR_ALIGN = 6,       /* a pointer is not aligned to its element size */
  FBEV_ERR_RANGE = 7,       /* sizes exceed what the kernels index (see fbev_strerror) */
  FBEV_ERR_SCRATCH = 8,     /* scratch buffer missing or too small */
  FBEV_ERR_LAUNCH = 9,      /* the CUDA runtime refused a launch or a memset */
  FBEV_ERR_NO_DEVICE = 10,  /* no usable sm_100 device / wrong architecture */
  FBEV_ERR_STATIC_LIMIT = 11 /* fbev_backward_static_scratch: problem larger than the built-in scratch */
};

/* bits a kernel may OR into the optional device status word */
enum {
  FBEV_DEV_BAD_FEATURE_SIZE = 1 /* a feature_size entry is <= 0 or larger than H x W; that camera was skipped */
};

/* flags of fbev_backward */
enum {
  FBEV_BWD_FEATS = 1,        /* compute grad_feats */
  FBEV_BWD_DEPTH = 2,        /* compute grad_depth */
  FBEV_BWD_LEGACY_DEPTH = 4, /* parametric modes: reproduce the reference kernel's depth gradient
                                (same value into mean and sigma, flash_bevpool_cuda.cu:665-674)
                                instead of the analytic one */
  FBEV_BWD_DETERMINISTIC = 8 /* bitwise reproducible gradients: every contribution is added as a 64-bit
                                fixed-point integer (integer addition does not depend on the order the
                                warps arrive in), at a power-of-two scale taken from bounds of the inputs.
                                Same tolerances as the default path, slower.
                                Needs N <= 32 and B*N*H*W*D < 2^32 (FBEV_ERR_RANGE otherwise) and scratch
                                for every element type: at least fbev_backward_min_scratch_bytes() with
                                this flag (256 bytes + 8 per element of both gradients, + 4 per depth
                                element for logits), better fbev_backward_scratch_bytes(), which adds the
                                entry lists that let large problems run through the sort by texel.  The
                                reference has no counterpart: its backward adds float atomics in arrival
                                order (flash_bevpool_cuda.cu:667-679). */
};

/*
 * One operator call.  Replaces the 21 positional arguments of
 * flash_bevpool_forward (flash_bevpool.cpp:79-101) and the 14 of
 * flash_bevpool_backward (:168-183); both calls share this description.
 */
typedef struct FbevProblem {
  uint32_t struct_size;        /* sizeof(FbevProblem) */
  int32_t dtype;               /* FBEV_F32 / FBEV_BF16 / FBEV_F16: features, depth and both gradients */
  int32_t out_dtype;           /* output and upstream gradient: same as dtype, or FBEV_F32 (the reference
                                  always returns float32, flash_bevpool.py:47-49,69) */
  int32_t B, N, H, W, C;       /* features [B,N,H,W,C] */
  int32_t D;                   /* last dimension of the depth tensor: 2 (mean, sigma) or the bin count */
  int32_t X, Y, Z;             /* grid_size = [X, Y, Z]; output [B,Y,X,C] */
  int32_t proj_stride;         /* floats per camera matrix: 12 ([B,N,3,4]) or 16 ([B,N,4,4], rows 0-2 used) */
  int32_t mode;                /* FBEV_DEPTH_* */
  int32_t pool;                /* FBEV_POOL_* */
  float epsilon;               /* flash_bevpool.py:23, default 1e-6 */
  float threshold;             /* depth_weight_threshold, samples with weight < threshold are dropped */
  float depth_d0, depth_delta; /* categorical: first bin edge and bin width, bin k covers [d0+k*delta, d0+(k+1)*delta) */
  int32_t y_begin, y_end;      /* BEV rows computed by this call (row sharding); 0, Y for all */
  float voxel_size[3];         /* used when roi_range is NULL: (max-min)/grid, flash_bevpool.py:62-64 */
  float voxel_min[3];          /* used when roi_range is NULL: xmin, ymin, zmin, flash_bevpool.py:65-67 */
  int32_t compact_rows;        /* 0: out, grad_out and valid_count are [B,Y,...] tensors of which this call touches
                                  rows y_begin..y_end.  Non-zero: they hold only those rows, [B, y_end - y_begin, ...]
                                  (a row shard that stays a shard: nothing to zero-fill, nothing to slice) */
  const void* image_feats;     /* device [B,N,H,W,C] */
  const void* depth;           /* device [B,N,H,W,D] */
  const float* projection;     /* device [B,N,proj_stride] float32 */
  const int32_t* feature_size; /* device [B,N,2] (h, w), as the reference reads it in-kernel (:134-135) */
  const int32_t* image_size;   /* device [2] (image_h, image_w) (:48-49) */
  const float* roi_range;      /* device [6] xmin,xmax,ymin,ymax,zmin,zmax, or NULL (then voxel_size/voxel_min) */
  int32_t* status;             /* optional device word for FBEV_DEV_* flags; NULL to ignore */
  void* workspace;             /* optional device memory, FBEV_WORKSPACE_BYTES, 16-byte aligned, zero before its
                                  first use; every call leaves it zero again.  With it the kernels balance
                                  their tiles through an atomic counter; without it (NULL) every thread block
                                  owns one fixed tile.  Calls that may overlap on the device need a workspace
                                  each. */
  void* saved_state;           /* optional device memory, 16-byte aligned, that ties a forward to its backward: a
                                  forward given it also writes the row records and sample lists it built, and a
                                  backward given the same memory (same problem otherwise) reads them instead of
                                  rebuilding them, which is most of its work.  fbev_saved_state_bytes() sizes it;
                                  with less, what does not fit is rebuilt.  NULL: nothing is saved or reused (the
                                  reference rebuilds everything in its backward, flash_bevpool_cuda.cu:477-566). */
  uint64_t saved_state_bytes;  /* size of saved_state */
  float* depth_stats;          /* FBEV_DEPTH_CATEGORICAL_LOGITS only: device scratch, 2 floats per texel
                                  (B*N*H*W*2, 8-byte aligned), caller-owned; every call fills it itself with each
                                  texel's (max logit, 1 / sum of exp(logit - max)).  NULL in the other modes. */
} FbevProblem;

#define FBEV_WORKSPACE_BYTES 16

/* Forward.  Replaces flash_bevpool_forward (flash_bevpool.cpp:79-166) ->
 * flash_bevpool() (flash_bevpool_cuda.cu:757-865).  Writes every element of
 * out[:, y_begin:y_end] (no zero fill needed); valid_count (optional, device
 * int32 [B,Y,X]) receives the number of accepted samples per cell. */
int fbev_forward(const FbevProblem* p, void* out, int32_t* valid_count, void* stream);

/* Forward whose result ends in page-locked host memory, computed in row_chunks launches (1..16) over
 * consecutive bands of rows [y_begin, y_end) so that the device-to-host copy of one band (copy engine, a side
 * stream owned by the library) runs while the next band is computed.  (No counterpart in the reference, whose
 * callers copy the whole result after the kernel.)  out_dev: device [B,Y,X,C] staging buffer; out_host:
 * page-locked host [B,Y,X,C]; both receive the rows.  The caller's stream waits for the last copy, so work
 * queued on it afterwards, or a synchronisation of it, sees the host buffer complete.  The first call on a
 * (device, stream) pair creates that pair's side stream and events under a lock; make it outside any stream
 * capture.  Calls on different streams share nothing; calls on one stream are ordered by it. */
int fbev_forward_to_host(const FbevProblem* p, void* out_dev, void* out_host, int row_chunks, void* stream);

/* Forward whose result rows also go to other GPUs.  (No counterpart in the reference, which has no
 * distributed code.)  Same as fbev_forward, and every 16-byte piece of out[:, y_begin:y_end] is stored to
 * peer_outs[0 .. n_peers) as well: device pointers of [B,Y,X,C] buffers in other GPUs' memory that this
 * device may write (peer access enabled, or a symmetric-memory mapping), n_peers <= 7, same alignment
 * modulo 16 as out.  With BEV rows split over ranks through y_begin / y_end this replaces the all-gather of
 * the output: every rank ends up with all rows once all ranks' kernels have finished, which the caller
 * establishes with its own cross-rank barrier after the launch.  Plain st.global stores; the kernel waits
 * on nothing. */
int fbev_forward_peers(const FbevProblem* p, void* out, void* const* peer_outs, int n_peers, int32_t* valid_count,
                       void* stream);

/* The same exchange with one store per chunk instead of one per peer.  (No counterpart in the reference.)
 * out: this GPU's [B,Y,X,C] buffer; out_multicast: the multicast address of that buffer, i.e. an address whose
 * stores the NVSwitch delivers to the same offset of every GPU's buffer bound to the multicast object, this GPU's
 * included (CUDA multicast objects, cuMulticastCreate / cuMulticastBindMem; torch.distributed._symmetric_memory
 * hands it out as multicast_ptr).  The kernel writes out[:, y_begin:y_end] only through out_multicast
 * (multimem.st), so each rank sends its rows over NVLink once, whatever the number of ranks.  Needs channel rows
 * that are multiples of 16 bytes and 16-byte aligned buffers (else FBEV_ERR_RANGE / FBEV_ERR_ALIGN).  As with
 * fbev_forward_peers the caller establishes completion across ranks after the launch. */
int fbev_forward_multicast(const FbevProblem* p, void* out, void* out_multicast, int32_t* valid_count, void* stream);

/* Bytes of FbevProblem.saved_state that hold the lists of this problem's forward for its backward on the
 * benchmark rigs' densities with room to spare (a directory of 16 bytes per group of cells and pass, and 24 bytes
 * per candidate (cell, camera, height bin), at most 1 GiB).  0 for an invalid problem. */
size_t fbev_saved_state_bytes(const FbevProblem* p);

/* Bytes of scratch fbev_backward works best with for this problem and flags: the float32 accumulation
 * targets of the 16-bit types (fbev_backward_min_scratch_bytes) plus, when the feature gradient is asked
 * for (or the depth gradient of a parametric mode on feature maps of fewer than 8192 texels per sample),
 * the entry lists of the sort by texel: counters (4 bytes per texel, 8 where a run of samples has more
 * than 8192 texels) and 36 bytes per entry (68 when that parametric depth gradient rides on them), one
 * entry per two candidates X*rows*N*Z of every sample (at least 4096 entries).  The lists never exceed FBEV_SORT_BUDGET_BYTES: a batch
 * that would need more is processed in runs of as many samples as fit, and a single sample that would need
 * more gets lists of that size (what does not fit is added directly, slower).  (The reference backward needs
 * no scratch at all: one atomicAdd per sample, channel and corner, flash_bevpool_cuda.cu:667-679.) */
#define FBEV_SORT_BUDGET_BYTES ((size_t)256 << 20)
size_t fbev_backward_scratch_bytes(const FbevProblem* p, int flags);

/* The least scratch fbev_backward accepts: 0 for float32 tensors (gradients accumulate in place),
 * otherwise room for float32 copies of the requested gradients; with FBEV_BWD_DETERMINISTIC the
 * fixed-point sums described at that flag, for every element type.  With less than
 * fbev_backward_scratch_bytes() the feature gradient falls back to its single-launch kernels
 * (direct float reductions), about 1.6 times slower on the benchmark shape. */
size_t fbev_backward_min_scratch_bytes(const FbevProblem* p, int flags);

/* Backward.  Replaces flash_bevpool_backward (flash_bevpool.cpp:168-241) ->
 * flash_bevpool_grad() (flash_bevpool_cuda.cu:867-938).  grad_out device
 * [B,Y,X,C]; grad_feats device [B,N,H,W,C]; grad_depth device [B,N,H,W,D]; all
 * of the problem's dtype.  The requested gradients are overwritten (the
 * library clears them itself).  scratch: device, 256-byte aligned, at least
 * fbev_backward_min_scratch_bytes() (may be NULL when that is 0), preferably
 * fbev_backward_scratch_bytes(). */
int fbev_backward(const FbevProblem* p, const void* grad_out, void* grad_feats, void* grad_depth,
                  void* scratch, size_t scratch_bytes, int flags, void* stream);

/* Backward for callers that cannot hand over scratch memory.  (No counterpart in the reference,
 * which only ever computes in float32 and so never needs a scratch buffer.)
 *
 * fbev_backward accumulates 16-bit gradients in float32 scratch the caller allocates.  Some callers
 * have no way to allocate it: a perception process that reserves its whole device-memory budget at
 * start-up and forbids cudaMalloc afterwards, or an operator hosted by a framework that owns the
 * memory pool and gives plug-ins no allocator.  This entry point takes the same arguments minus the
 * scratch and accumulates in an array that is part of the library image instead.  It allocates
 * nothing: no cudaMalloc, no cudaFree, no library routine that allocates.
 *
 * Limits and rules:
 *  - the problem's fbev_backward_min_scratch_bytes() must not exceed FBEV_STATIC_SCRATCH_BYTES, else
 *    FBEV_ERR_STATIC_LIMIT is returned and nothing is launched (float32 problems need none and
 *    always fit);
 *  - the array costs FBEV_STATIC_SCRATCH_BYTES of device memory on every GPU that loads the library,
 *    for the life of the process;
 *  - the first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current, under a lock: host threads may race to it); make that first call outside
 *    any stream capture;
 *  - all calls on a device share the one array.  Each call clears what it accumulates into, so
 *    leftovers of earlier calls do no harm, but two calls that overlap on the GPU (different
 *    streams, no ordering between them) corrupt each other's gradients: order them. */
#define FBEV_STATIC_SCRATCH_BYTES (16u << 20)
int fbev_backward_static_scratch(const FbevProblem* p, const void* grad_out, void* grad_feats, void* grad_depth,
                                 int flags, void* stream);

/* Integer decisions of every (b, n, y, x, z) candidate, for bit-exact checks:
 * texel indices after clamping (:147-154), depth bin (categorical, else -1),
 * final acceptance, each device [B,N,Y,X,Z]; count device int32 [B,Y,X].
 * Rejected candidates hold -1 / 0.  The reference keeps these values internal. */
int fbev_debug_indices(const FbevProblem* p, int32_t* u0, int32_t* v0, int32_t* kbin, uint8_t* valid,
                       int32_t* count, void* stream);

/* Drop-in for the reference launcher
 *   void flash_bevpool(int total_threads, ...)   flash_bevpool_cuda.cu:757-786
 * same arguments in the same order (float32, parametric depth, mean pooling),
 * plus the stream.  The variant flags only chose between reference kernels
 * with the same result and are ignored.  Addressing follows feature_size, as
 * in the reference. */
int fbev_flash_bevpool(int total_threads, int num_channels, int num_cameras, int batch_size,
                       int num_extrinsic_params, int num_intrinsic_params, int depth_distribution,
                       int use_shared_memory, int optimize_z_precompute, int use_warp_kernel,
                       int use_vectorized_load, float epsilon, float depth_weight_threshold,
                       const float* depth_params, const float* image_feats, const float* projection_matrices,
                       const int* feature_size, const int* image_size, int grid_x, int grid_y, int grid_z,
                       float voxel_size_x, float voxel_size_y, float voxel_size_z, float voxel_x_min,
                       float voxel_y_min, float voxel_z_min, float* out, void* stream);

/* Drop-in for the reference launcher
 *   void flash_bevpool_grad(int total_threads, ...)   flash_bevpool_cuda.cu:867-889
 * same arguments in the same order plus the tensor's H and W (the reference
 * relies on the caller having zero-filled both gradients; this call clears
 * them, which needs their size) and the stream.  Produces the reference
 * kernel's depth gradient (FBEV_BWD_LEGACY_DEPTH). */
int fbev_flash_bevpool_grad(int total_threads, int num_channels, int num_cameras, int batch_size,
                            int num_extrinsic_params, int num_intrinsic_params, int depth_distribution,
                            float epsilon, float depth_weight_threshold, const float* out_grad,
                            const float* depth_params, const float* image_feats,
                            const float* projection_matrices, const int* feature_size, const int* image_size,
                            const float* roi_range, int grid_x, int grid_y, int grid_z,
                            float* depth_params_grad, float* image_feats_grad, int feat_h, int feat_w,
                            void* stream);

/* Projection matrices from the camera calibration, one small kernel instead of the reference's chain of
 * torch ops (create_projection_matrix, flashbev/flashbevpool/sampling_vt.py:21-33):
 *   P = [post_rots * camera2imgs, post_trans added to column 2; 0 0 0 1] * inverse(sensor2ego), rows 0-2.
 * All device float32: sensor2ego [BN,4,4], camera2imgs [BN,3,3], post_rots [BN,3,3], post_trans [BN,3]
 * -> out [BN,3,4], BN = batch * cameras.  The 4x4 inverse is evaluated in float64 (cofactors). */
int fbev_projection_matrices(const float* sensor2ego, const float* camera2imgs, const float* post_rots,
                             const float* post_trans, float* out, int count, void* stream);

/* Pillar pooling over pre-sorted sample lists: drop-in for the launcher of the reference's comparison baseline
 *   void sampling_vt_pillarpool_fused(int c, int n_intervals, ...)   src/sampling_vt_cuda.cu:129-134
 * (bound by sampling_vt_pillarpool_fused_forward, src/sampling_vt.cpp:13-55), same arguments in the same order plus
 * the stream.  All device, float32 / int32: depth [B,N,h,w,2], feat [B,N,h,w,c]; per sample u, v (feature-map
 * coordinates), z (camera depth), batch_camera_indices (batch * cameras + camera), ranks_bev (flat BEV cell);
 * per interval its first sample and length.  out (flat [cells, c]) receives the mean over each interval's
 * samples; cells without an interval are not written (the caller zero-fills, sampling_vt_ops.py:24). */
int fbev_pillar_pool(int c, int n_intervals, const float* depth, const float* feat, const float* u_coords,
                     const float* v_coords, const float* z_coords, const int* batch_camera_indices, const int* ranks_bev,
                     const int* interval_starts, const int* interval_lengths, int batch_size, int num_cameras, int feat_h,
                     int feat_w, float epsilon, int depth_distribution, float* out, void* stream);

const char* fbev_strerror(int status);
int fbev_version(void);
/* SHA-256 (hex) of the sources and compiler flags this library was built from; the Python binding refuses a
 * library whose hash differs from the sources beside it.  (No counterpart in the reference.) */
const char* fbev_source_hash(void);

#ifdef __cplusplus
}
#endif
#endif /* FBEV_H_ */
