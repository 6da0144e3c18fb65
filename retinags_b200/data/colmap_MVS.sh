#!/bin/bash
# Dense multi-view stereo with COLMAP to obtain a dense initial point cloud
# (<scene>/sparse/0/MVS_points3D.ply, used with --points3D MVS_points3D), as scripts/colmap_MVS.sh of the reference.
set -euo pipefail
SCENE=${1:?scene directory with images/ and sparse/0}
colmap image_undistorter --image_path "$SCENE/images" --input_path "$SCENE/sparse/0" --output_path "$SCENE/dense" --output_type COLMAP
colmap patch_match_stereo --workspace_path "$SCENE/dense" --workspace_format COLMAP --PatchMatchStereo.geom_consistency true
colmap stereo_fusion --workspace_path "$SCENE/dense" --workspace_format COLMAP --input_type geometric --output_path "$SCENE/sparse/0/MVS_points3D.ply"
