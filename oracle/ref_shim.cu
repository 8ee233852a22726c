// Exports the reference's CUDA launchers under C names so that tests and the
// benchmark can run the reference's own kernels next to the new ones on the same
// GPU.  TEST INFRASTRUCTURE ONLY.  The reference source is included from its
// checkout at build time (-I<reference>/flashbev/flashbevpool/src); nothing of it
// is stored in this repository.  Launchers: flash_bevpool_cuda.cu:757 (forward)
// and :867 (backward).  Both launch on the legacy default stream and check no
// errors; the wrappers below add the error check.
#include <cuda_runtime.h>
#include "flash_bevpool_cuda.cu"

extern "C" int flashbev_ref_forward(int total_threads, int num_channels, int num_cameras, int batch_size,
                                    int depth_distribution, int use_shared_memory, int optimize_z_precompute,
                                    float epsilon, float depth_weight_threshold, const float* depth_params,
                                    const float* image_feats, const float* projection_matrices,
                                    const int* feature_size, const int* image_size, int grid_x, int grid_y,
                                    int grid_z, float voxel_size_x, float voxel_size_y, float voxel_size_z,
                                    float voxel_x_min, float voxel_y_min, float voxel_z_min, float* out) {
  // use_warp_kernel stays false: that variant can ask for more shared memory than
  // a launch may have without an opt-in and then fails (flash_bevpool_cuda.cu:711-722).
  flash_bevpool(total_threads, num_channels, num_cameras, batch_size, 12, 12, depth_distribution,
                use_shared_memory != 0, optimize_z_precompute != 0, false, false, epsilon,
                depth_weight_threshold, depth_params, image_feats, projection_matrices, feature_size,
                image_size, grid_x, grid_y, grid_z, voxel_size_x, voxel_size_y, voxel_size_z, voxel_x_min,
                voxel_y_min, voxel_z_min, out);
  return (int)cudaGetLastError();
}

extern "C" int flashbev_ref_backward(int total_threads, int num_channels, int num_cameras, int batch_size,
                                     int depth_distribution, float epsilon, float depth_weight_threshold,
                                     const float* out_grad, const float* depth_params, const float* image_feats,
                                     const float* projection_matrices, const int* feature_size,
                                     const int* image_size, const float* roi_range, int grid_x, int grid_y,
                                     int grid_z, float* depth_params_grad, float* image_feats_grad) {
  flash_bevpool_grad(total_threads, num_channels, num_cameras, batch_size, 12, 12, depth_distribution, epsilon,
                     depth_weight_threshold, out_grad, depth_params, image_feats, projection_matrices,
                     feature_size, image_size, roi_range, grid_x, grid_y, grid_z, depth_params_grad,
                     image_feats_grad);
  return (int)cudaGetLastError();
}
