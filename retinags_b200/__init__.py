"""retinags_b200: model-parallel 3D Gaussian Splatting for 8xB200 (sm_100a) nodes.

Sub-packages:

* ``ops``      native kernels (ctypes binding), autograd wrappers and the pure-PyTorch oracle
* ``models``   Gaussian parameter store, PLY / optimiser-state IO, densification
* ``parallel`` spatial partition (grid + kd/BVH tree), camera/sub-model relation, scheduling,
  compositing transports (NCCL baseline, fused peer-to-peer, CPU loopback), watchdog
* ``data``     cameras, dataset readers, synthetic seeded scenes
* ``utils``    maths helpers, logging, timers, image IO
"""
__version__ = "0.1.0"


_PUBLIC = {
    "GaussianRasterizationSettings": "retinags_b200.ops.rasterize", "GaussianRasterizer": "retinags_b200.ops.rasterize",
    "RenderTask": "retinags_b200.ops.rasterize", "CompositeLoss": "retinags_b200.ops.loss",
    "GaussianStore": "retinags_b200.models.gaussians", "GaussianModel": "retinags_b200.models.gaussian_model",
    "Scene": "retinags_b200.scene", "render": "retinags_b200.gaussian_renderer", "StepEngine": "retinags_b200.engine",
    "Trainer": "retinags_b200.trainer", "BvhTree": "retinags_b200.parallel.partition", "Camera": "retinags_b200.data.cameras",
    "ViewerServer": "retinags_b200.viewer_server",
}


def __getattr__(name: str):
    """The main entry points by name (imported on first use, so that ``import retinags_b200`` stays light)."""
    if name in _PUBLIC:
        import importlib
        return getattr(importlib.import_module(_PUBLIC[name]), name)
    raise AttributeError(f"module 'retinags_b200' has no attribute {name!r}")


def __dir__():
    return sorted(list(globals()) + list(_PUBLIC))
