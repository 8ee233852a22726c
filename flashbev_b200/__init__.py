"""B200 (sm_100a) fused BEV pooling: the operator of yokosyun/FlashBEV's ``flashbevpool``
package on a hand-written CUDA library with a C ABI (include/fbev.h)."""
from .flash_bevpool import DepthSpec, FlashBEVPool, debug_indices, flash_bevpool, forward_with_count
from .sampling_vt import SamplingVT, create_projection_matrix

__all__ = ["FlashBEVPool", "flash_bevpool", "SamplingVT", "create_projection_matrix", "DepthSpec",
           "debug_indices", "forward_with_count"]
