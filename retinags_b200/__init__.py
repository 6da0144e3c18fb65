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
