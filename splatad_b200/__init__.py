"""splatad_b200: the SplatAD render hot path (camera ``rasterization`` and lidar
``lidar_rasterization``, forward and backward) for NVIDIA B200 (sm_100a).

The public names are those the reference exports for this path (gsplat/__init__.py:4-18);
everything runs in hand-written CUDA behind the C ABI declared in ``include/splatad_b200.h``.
"""

from .ops import (
    compute_lidar_velocity,
    compute_pix_velocity,
    fully_fused_lidar_projection,
    fully_fused_projection,
    isect_lidar_tiles,
    isect_offset_encode,
    isect_tiles,
    lidar_proj,
    map_points_to_lidar_tiles,
    persp_proj,
    points_mapping_offset_encode,
    populate_image_from_points,
    quat_scale_to_covar_preci,
    rasterize_to_indices_in_range,
    rasterize_to_indices_in_range_lidar,
    rasterize_to_pixels,
    rasterize_to_points,
    spherical_harmonics,
    velocity_grads,
    world_to_cam,
)
from .densify import compute_relocation
from .rendering import lidar_rasterization, rasterization

__all__ = [
    "rasterization",
    "lidar_rasterization",
    "fully_fused_projection",
    "fully_fused_lidar_projection",
    "isect_tiles",
    "isect_lidar_tiles",
    "isect_offset_encode",
    "map_points_to_lidar_tiles",
    "points_mapping_offset_encode",
    "populate_image_from_points",
    "rasterize_to_pixels",
    "rasterize_to_points",
    "rasterize_to_indices_in_range",
    "rasterize_to_indices_in_range_lidar",
    "spherical_harmonics",
    "velocity_grads",
    "quat_scale_to_covar_preci",
    "world_to_cam",
    "persp_proj",
    "compute_pix_velocity",
    "lidar_proj",
    "compute_lidar_velocity",
    "compute_relocation",
]

__version__ = "0.1.0"
