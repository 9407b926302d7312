"""Host-side helpers of the contraction path (subset of the reference's tritonix/utils)."""
from tritonix_b200.utils.hilbert import (hilbert_inverse_permutation, hilbert_permutation,
                                         hilbert_rect_coords, hilbert_swizzled_coords,
                                         hilbert_tile_table)
from tritonix_b200.utils.pruners import (CoordinateMonotonicFunction, CoordinateUnimodalFunction,
                                         MonotonicCascadeTrie)
from tritonix_b200.utils.spaces import (Choice, ConfigParam, ConfigSpace, PowerOfTwo, Range,
                                        SpaceConfig)
from tritonix_b200.utils.tile_order import grouped_order, serpentine_order, tile_sequence
from tritonix_b200.utils.torch import (disable_torch_optimizations, enable_cudnn_optimizations,
                                       enable_torch_optimizations)

__all__ = ["hilbert_rect_coords", "hilbert_permutation", "hilbert_inverse_permutation",
           "hilbert_swizzled_coords", "hilbert_tile_table", "MonotonicCascadeTrie",
           "CoordinateUnimodalFunction", "CoordinateMonotonicFunction", "Choice", "Range",
           "PowerOfTwo", "SpaceConfig", "ConfigSpace", "ConfigParam", "grouped_order",
           "serpentine_order", "tile_sequence", "enable_cudnn_optimizations",
           "enable_torch_optimizations", "disable_torch_optimizations"]
