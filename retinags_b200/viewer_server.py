"""Headless frame server for the SIBR remote viewer protocol.

The reference ships ``gaussian_renderer/network_gui.py`` (module-level socket state, never called by its trainer).
The protocol: the viewer sends a 4-byte little-endian length and a JSON message (``resolution_x/y``, ``fov_x/y``,
``z_near/z_far``, ``train``, ``shs_python``, ``rot_scale_python``, ``keep_alive``, ``scaling_modifier``, ``view_matrix``,
``view_projection_matrix`` as 16 floats each); the server answers with ``H*W*3`` bytes of RGB and a length-prefixed
ASCII string (the scene path).  This class speaks that protocol without any window or graphics API: frames are
rendered by the CUDA (or CPU) rasteriser into a device buffer and sent as bytes.
"""
from __future__ import annotations

import json
import socket

import numpy as np
import torch

from .data.cameras import Camera


class ViewerRequest:
    def __init__(self, camera: Camera | None, do_training: bool, keep_alive: bool, scaling_modifier: float):
        self.camera, self.do_training, self.keep_alive, self.scaling_modifier = camera, do_training, keep_alive, scaling_modifier


class ViewerServer:
    def __init__(self, host: str = "127.0.0.1", port: int = 6009):
        self.listener = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self.listener.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self.listener.bind((host, port))
        self.listener.listen()
        self.listener.settimeout(0)
        self.host, self.port = self.listener.getsockname()
        self.conn = None

    def try_connect(self) -> bool:
        """Non-blocking accept (call once per training iteration, as the reference's training loops do)."""
        if self.conn is not None:
            return True
        try:
            self.conn, _ = self.listener.accept()
            self.conn.settimeout(None)
            return True
        except (BlockingIOError, socket.timeout, OSError):
            return False

    def _recv_exact(self, n: int) -> bytes:
        buf = b""
        while len(buf) < n:
            chunk = self.conn.recv(n - len(buf))
            if not chunk:
                raise ConnectionError("viewer closed the connection")
            buf += chunk
        return buf

    def receive(self) -> ViewerRequest:
        n = int.from_bytes(self._recv_exact(4), "little")
        msg = json.loads(self._recv_exact(n).decode("utf-8"))
        w, h = int(msg["resolution_x"]), int(msg["resolution_y"])
        if w == 0 or h == 0:
            return ViewerRequest(None, False, bool(msg.get("keep_alive", False)), 1.0)
        # the viewer sends the transposed world-to-view matrix of an OpenGL camera: flip y and z
        wvt = np.asarray(msg["view_matrix"], dtype=np.float64).reshape(4, 4)
        wvt[:, 1] *= -1
        wvt[:, 2] *= -1
        w2c = wvt.T
        cam = Camera(uid=0, R=w2c[:3, :3].T.copy(), T=w2c[:3, 3].copy(), fovx=float(msg["fov_x"]), fovy=float(msg["fov_y"]),
                     width=w, height=h, image_name="viewer", znear=float(msg["z_near"]), zfar=float(msg["z_far"]))
        return ViewerRequest(cam, bool(msg["train"]), bool(msg["keep_alive"]), float(msg["scaling_modifier"]))

    def send(self, image: torch.Tensor | None, verify: str):
        """``image``: (3,H,W) float in [0,1] or None (no frame was requested)."""
        if image is not None:
            frame = (image.detach().clamp(0, 1) * 255).to(torch.uint8).permute(1, 2, 0).contiguous().cpu().numpy()
            self.conn.sendall(frame.tobytes())
        self.conn.sendall(len(verify).to_bytes(4, "little"))
        self.conn.sendall(verify.encode("ascii"))

    def serve_once(self, render_fn, verify: str = "") -> ViewerRequest | None:
        """Answer one pending request with ``render_fn(camera, scaling_modifier) -> (3,H,W)``; drops the connection on error."""
        if not self.try_connect():
            return None
        try:
            req = self.receive()
            self.send(render_fn(req.camera, req.scaling_modifier) if req.camera is not None else None, verify)
            return req
        except (ConnectionError, OSError, ValueError, KeyError):
            self.close_connection()
            return None

    def close_connection(self):
        if self.conn is not None:
            try:
                self.conn.close()
            finally:
                self.conn = None

    def close(self):
        self.close_connection()
        self.listener.close()
