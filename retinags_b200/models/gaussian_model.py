"""Single-GPU Gaussian model with the interface of vanilla 3DGS.

The reference keeps a legacy single-GPU stack next to the model-parallel trainer: ``scene/gaussian_model.py``
(``GaussianModel``: ``create_from_pcd``, ``training_setup``, ``update_learning_rate``, ``oneupSHdegree``,
``save_ply``/``load_ply``, ``capture``/``restore``, ``reset_opacity``, ``densify_and_prune``, the ``get_*``
properties) and ``GaussianModel2`` in ``scene/gaussian_nn_module.py:296-797``.  This class offers the same calls on
top of the sub-model machinery of this package: one :class:`GaussianStore` with an unbounded box, the fused render /
loss / backward / Adam path of :class:`StepEngine`, the densification kernels.  A training loop therefore reads

    model.create_from_pcd(points, colors, extent); model.training_setup(opt)
    for it in range(...):
        model.update_learning_rate(it)
        out = model.train_step([camera])            # forward, L1 + D-SSIM, backward, Adam in one call
        model.densify_and_prune(...) / model.reset_opacity()

instead of ``loss.backward(); optimizer.step()``; code that needs autograd on its own tensors uses
``ops.rasterize.GaussianRasterizer``.
"""
from __future__ import annotations

import os

import numpy as np
import torch

from ..engine import StepEngine
from ..ops.knn import knn3_dist2
from ..utils.general import expon_lr, inverse_sigmoid
from . import densify, ply_io
from .gaussians import NAMES, GaussianStore

from ..utils.sh import C0 as SH_C0  # noqa: E402


class GaussianModel:
    def __init__(self, sh_degree: int = 3, device=None, scale_control_rate: float = 1.0, opacity_init: float = 0.1):
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        self.max_sh_degree = sh_degree
        self.scale_control_rate, self.opacity_init = scale_control_rate, opacity_init
        self.spatial_lr_scale = 1.0
        self.store = GaussianStore(4, self.device, sh_degree)
        self.opt = None
        self.lrs = (0.0,) * 6
        self.background = (0.0, 0.0, 0.0)
        self._engine: StepEngine | None = None

    # -- activated views (reference: gaussian_model.py:93-123) ------------------------------------
    @property
    def active_sh_degree(self) -> int:
        return self.store.active_sh_degree

    @active_sh_degree.setter
    def active_sh_degree(self, v: int):
        self.store.active_sh_degree = int(v)

    @property
    def get_xyz(self) -> torch.Tensor:
        return self.store.views()["xyz"]

    @property
    def get_scaling(self) -> torch.Tensor:
        return torch.exp(self.store.views()["scale"])

    @property
    def get_rotation(self) -> torch.Tensor:
        return torch.nn.functional.normalize(self.store.views()["rot"], dim=1)

    @property
    def get_opacity(self) -> torch.Tensor:
        return torch.sigmoid(self.store.views()["opacity"])

    @property
    def get_features(self) -> torch.Tensor:
        return self.store.views()["sh"].view(-1, 16, 3)

    def __len__(self) -> int:
        return self.store.count

    def oneupSHdegree(self):
        if self.store.active_sh_degree < self.max_sh_degree:
            self.store.active_sh_degree += 1

    # -- construction -------------------------------------------------------------------------------
    def _replace_store(self, g: dict):
        n = int(g["xyz"].shape[0])
        st = GaussianStore(max(n, 4), self.device, self.max_sh_degree)
        st.set_params(g)
        st.active_sh_degree = self.store.active_sh_degree
        self.store = st
        self._engine = None

    def create_from_pcd(self, points, colors, spatial_lr_scale: float = 1.0):
        """3DGS initialisation: SH DC from the colours (0..1), isotropic scale from the mean distance to the three
        nearest neighbours, identity rotation, opacity ``opacity_init``."""
        self.spatial_lr_scale = float(spatial_lr_scale)
        p = torch.as_tensor(np.asarray(points), dtype=torch.float32, device=self.device)
        c = torch.as_tensor(np.asarray(colors), dtype=torch.float32, device=self.device)
        n = p.shape[0]
        d2 = torch.clamp_min(knn3_dist2(p), 1e-7)
        sh = torch.zeros(n, 16, 3, device=self.device)
        sh[:, 0] = (c - 0.5) / SH_C0
        rot = torch.zeros(n, 4, device=self.device)
        rot[:, 0] = 1
        self.store.active_sh_degree = 0
        self._replace_store(dict(
            xyz=p, sh=sh.view(n, 48), scale=torch.log(torch.sqrt(d2) * self.scale_control_rate)[:, None].repeat(1, 3), rot=rot,
            opacity=inverse_sigmoid(self.opacity_init * torch.ones(n, 1, device=self.device))))

    # -- optimiser ------------------------------------------------------------------------------------
    def training_setup(self, opt):
        """``opt`` carries the fields of ``OptimizationParams`` (config.py)."""
        self.opt = opt
        self.update_learning_rate(0)

    def update_learning_rate(self, iteration: int) -> float:
        o = self.opt
        xyz = expon_lr(iteration, o.position_lr_init * self.spatial_lr_scale, o.position_lr_final * self.spatial_lr_scale, 0,
                       o.position_lr_delay_mult, o.position_lr_max_steps)
        self.lrs = (xyz, o.feature_lr, o.feature_lr / 20.0, o.scaling_lr, o.rotation_lr, o.opacity_lr)
        return xyz

    # -- rendering / training -----------------------------------------------------------------------------
    def engine(self) -> StepEngine:
        if self._engine is None or self._engine.stores[0] is not self.store:
            lam = self.opt.lambda_dssim if self.opt is not None else 0.2
            self._engine = StepEngine({0: self.store}, [0], self.device, None, lam, self.background)
        self._engine.background = tuple(self.background)
        return self._engine

    def render(self, camera, bg_color=None, scaling_modifier: float = 1.0) -> dict:
        """Render one camera (no gradients). Returns ``render`` (3,H,W), ``alpha`` (H,W), ``radii`` and the visibility
        filter, like the reference's ``gaussian_renderer.render``."""
        assert scaling_modifier == 1.0, "a scale modifier other than 1 is a camera field: use ops.rasterize.make_camera"
        eng = self.engine()
        out = eng.render([camera], [[0]], self.store.active_sh_degree, background=bg_color)[0]
        task = eng._task(0, 0)
        radii = task.radii(0, eng._segments(0, False))
        return dict(render=out["image"], alpha=1.0 - out["trans"], radii=radii, visibility_filter=radii > 0,
                    viewspace_points=None)

    def train_step(self, cameras: list, bg_color=None) -> dict:
        """Forward, loss, backward and one Adam update over a batch of cameras (each with its ``image``)."""
        eng = self.engine()
        res = eng.train_step(list(cameras), [[0]] * len(cameras), self.store.active_sh_degree, self.lrs, background=bg_color)
        sums = torch.stack(res.sums).sum(0).tolist()
        cl = eng._loss(0, cameras[0].height, cameras[0].width)
        info = cl.loss_from_sums([s / len(cameras) for s in sums], eng.lambda_dssim)
        eng.poll()
        return info

    # -- density control ------------------------------------------------------------------------------------
    def densify_and_prune(self, max_grad: float, min_opacity: float, extent: float, max_screen_size, **kw) -> dict:
        pd = self.opt.percent_dense if self.opt is not None else 0.01
        return densify.densify_and_prune(self.store, max_grad, min_opacity, extent, max_screen_size, pd, **kw)

    def reset_opacity(self):
        densify.reset_opacity(self.store)

    # -- files ----------------------------------------------------------------------------------------------
    def save_ply(self, path: str):
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        ply_io.save_gaussians(path, {k: v.detach().cpu() for k, v in self.store.views().items()}, self.max_sh_degree)

    def load_ply(self, path: str):
        g = ply_io.load_gaussians(path, self.max_sh_degree)
        self.store.active_sh_degree = self.max_sh_degree
        self._replace_store({k: torch.as_tensor(g[k]) for k in NAMES})

    def capture(self) -> dict:
        """Checkpoint of parameters, Adam state and density statistics (``gaussian_model.py:60-75``)."""
        st = self.store
        return dict(active_sh_degree=st.active_sh_degree, records=st.migration_records().cpu(), step=st.step,
                    max_radii=st.max_radii[:st.count].cpu(), grad_accum=st.grad_accum[:st.count].cpu(),
                    denom=st.denom[:st.count].cpu(), spatial_lr_scale=self.spatial_lr_scale)

    def restore(self, state: dict, opt=None):
        st = GaussianStore(max(int(state["records"].shape[0]), 4), self.device, self.max_sh_degree)
        st.append_migration(state["records"])
        st.step = int(state["step"])
        st.active_sh_degree = int(state["active_sh_degree"])
        n = st.count
        st.max_radii[:n] = state["max_radii"].to(self.device)
        st.grad_accum[:n] = state["grad_accum"].to(self.device)
        st.denom[:n] = state["denom"].to(self.device)
        self.spatial_lr_scale = float(state["spatial_lr_scale"])
        self.store, self._engine = st, None
        if opt is not None:
            self.training_setup(opt)
