"""Seeded synthetic inputs for the BEV pooling operator.

These stand in for nuScenes-shaped data (no dataset is available offline): a six-camera
pinhole rig, channels-last image features, and either a softmaxed depth distribution
(categorical mode) or a (mean, sigma) map derived from the same distribution
(parametric modes, the reference's own depth model, flash_bevpool.py:28).

Everything is generated on the CPU from ``torch.Generator().manual_seed(seed)`` so that
CPU checks and GPU runs see bit-identical inputs.  Tensor distributions follow the
reference's kernel-only benchmark where it has one (tools/utils/data_utils.py:144-154:
features ~ N(0,1)); image size is 16x the feature map (data_utils.py:207).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Dict, Optional, Tuple

import numpy as np
import torch

YAWS_DEG = (0.0, 60.0, -60.0, 120.0, -120.0, 180.0)


@dataclass(frozen=True)
class Workload:
    """Shapes of one benchmark / parity configuration."""
    name: str
    B: int
    N: int
    C: int
    H: int
    W: int
    D: int            # depth bins of the categorical mode
    X: int
    Y: int
    Z: int
    xy_extent: float  # BEV covers [-extent, +extent] in x and y
    z_range: Tuple[float, float] = (-5.0, 3.0)
    d0: float = 1.0
    delta: float = 0.5
    dtype: str = "bf16"
    seed: int = 0
    jitter: bool = False

    @property
    def image_size(self) -> Tuple[int, int]:
        return (16 * self.H, 16 * self.W)

    @property
    def roi(self):
        e = self.xy_extent
        return (-e, e, -e, e, self.z_range[0], self.z_range[1])

    @property
    def grid(self):
        return (self.X, self.Y, self.Z)


# The configurations the benchmark specification lists, in its order.
WORKLOADS: Dict[str, Workload] = {
    # CPU-runnable reference case
    "cfg1": Workload("cfg1", B=1, N=6, C=64, H=16, W=44, D=59, X=128, Y=128, Z=4, xy_extent=51.2,
                     d0=1.0, delta=1.0, dtype="fp32", seed=1),
    # inference sweep; Z = 8 is the headline case
    "cfg2": Workload("cfg2", B=1, N=6, C=80, H=16, W=44, D=118, X=200, Y=200, Z=8, xy_extent=50.0,
                     dtype="bf16", seed=2),
    # training
    "cfg3": Workload("cfg3", B=4, N=6, C=80, H=32, W=88, D=118, X=200, Y=200, Z=8, xy_extent=50.0,
                     dtype="fp32", seed=3, jitter=True),
    # multi-GPU batch throughput (B is the whole job; ranks take contiguous slices)
    "cfg4": Workload("cfg4", B=64, N=6, C=80, H=16, W=44, D=118, X=200, Y=200, Z=8, xy_extent=50.0,
                     dtype="bf16", seed=4, jitter=True),
    # large grid, BEV rows split across GPUs
    "cfg5": Workload("cfg5", B=1, N=6, C=256, H=32, W=88, D=118, X=512, Y=512, Z=16, xy_extent=51.2,
                     dtype="bf16", seed=5),
}


def workload(name: str, **overrides) -> Workload:
    return replace(WORKLOADS[name], **overrides)


def rig_projection(image_size: Tuple[int, int], n_cams: int = 6, jitter_seed: Optional[int] = None) -> np.ndarray:
    """[n_cams, 3, 4] float32 projection matrices of the synthetic rig.

    P = K * inverse(sensor2ego), rows 0-2: the product the reference builds in
    create_projection_matrix (sampling_vt.py:21-33) with identity post-rotation.
    Camera axes: x right, y down, z forward; the rig sits 1.5 m above the ground.
    Computed in float64, then rounded once to float32.
    """
    image_h, image_w = image_size
    f = 0.35 * image_w
    K = np.eye(4)
    K[0, 0] = K[1, 1] = f
    K[0, 2] = image_w / 2.0
    K[1, 2] = image_h / 2.0
    rng = np.random.RandomState(jitter_seed) if jitter_seed is not None else None
    out = np.zeros((n_cams, 3, 4), dtype=np.float64)
    for i in range(n_cams):
        yaw = math.radians(YAWS_DEG[i % len(YAWS_DEG)])
        t = np.array([0.8 * math.cos(yaw), 0.8 * math.sin(yaw), 1.5])
        if rng is not None:
            yaw += math.radians(rng.uniform(-2.0, 2.0))
            t = t + rng.uniform(-0.05, 0.05, size=3)
        s2e = np.eye(4)
        s2e[:3, 0] = (math.sin(yaw), -math.cos(yaw), 0.0)
        s2e[:3, 1] = (0.0, 0.0, -1.0)
        s2e[:3, 2] = (math.cos(yaw), math.sin(yaw), 0.0)
        s2e[:3, 3] = t
        out[i] = (K @ np.linalg.inv(s2e))[:3]
    return out.astype(np.float32)


def module_inputs(B: int = 2, N: int = 6, C: int = 32, H: int = 8, W: int = 22, seed: int = 5):
    """The seven-tensor input list of ``SamplingVT.forward`` (sampling_vt.py:225-239) for the synthetic rig, on the
    CPU: image features [B,N,C,H,W] ~ N(0,1), sensor2ego, ego2global, camera2imgs, post_rots, post_trans, bda, and
    the image size (16x the feature map).  Every sample's rig is jittered; post_rots / post_trans hold a small
    seeded resize-and-shift augmentation so that the matrix builder has something to fold in."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, N, C, H, W, generator=g)
    image = (16 * H, 16 * W)
    f, cx, cy = 0.35 * image[1], image[1] / 2.0, image[0] / 2.0
    K = torch.eye(3).repeat(B, N, 1, 1)
    K[..., 0, 0] = K[..., 1, 1] = f
    K[..., 0, 2], K[..., 1, 2] = cx, cy
    s2e = torch.eye(4).repeat(B, N, 1, 1)
    rng = np.random.RandomState(seed + 100)
    for b in range(B):
        for n in range(N):
            yaw = math.radians(YAWS_DEG[n % len(YAWS_DEG)] + rng.uniform(-2.0, 2.0))
            t = np.array([0.8 * math.cos(yaw), 0.8 * math.sin(yaw), 1.5]) + rng.uniform(-0.05, 0.05, size=3)
            s2e[b, n, :3, 0] = torch.tensor([math.sin(yaw), -math.cos(yaw), 0.0])
            s2e[b, n, :3, 1] = torch.tensor([0.0, 0.0, -1.0])
            s2e[b, n, :3, 2] = torch.tensor([math.cos(yaw), math.sin(yaw), 0.0])
            s2e[b, n, :3, 3] = torch.from_numpy(t).float()
    post_rots = torch.eye(3).repeat(B, N, 1, 1)
    scale = torch.from_numpy(rng.uniform(0.95, 1.05, size=(B, N))).float()
    post_rots[..., 0, 0] = scale
    post_rots[..., 1, 1] = scale
    post_trans = torch.zeros(B, N, 3)
    post_trans[..., :2] = torch.from_numpy(rng.uniform(-6.0, 6.0, size=(B, N, 2))).float()
    inputs = [x, s2e, torch.eye(4).repeat(B, N, 1, 1), K, post_rots, post_trans, torch.eye(4).repeat(B, 1, 1)]
    return inputs, image


def _torch_dtype(name: str) -> torch.dtype:
    return {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[name]


def make_inputs(w: Workload, mode: str = "categorical", batch_slice: Optional[Tuple[int, int]] = None,
                dtype: Optional[str] = None) -> Dict[str, torch.Tensor]:
    """CPU tensors of one operator call, keyed by the operator's argument names.

    mode "categorical": depth = softmax probabilities [B,N,H,W,D].
    mode "parametric":  depth = (mean, sigma) [B,N,H,W,2], moments of the same softmax,
                        sigma + 0.1 as in SamplingVT.forward_depth (sampling_vt.py:220-223).
    ``batch_slice`` = (begin, end) generates only those samples of the batch; every sample
    has its own generator seed, so a slice equals the same rows of the whole batch.
    """
    b0, b1 = batch_slice if batch_slice is not None else (0, w.B)
    td = _torch_dtype(dtype or w.dtype)
    feats, depth, proj = [], [], []
    centres = w.d0 + (torch.arange(w.D, dtype=torch.float32) + 0.5) * w.delta
    for b in range(b0, b1):
        g = torch.Generator(device="cpu").manual_seed(w.seed * 100003 + b)
        f = torch.randn(w.N, w.C, w.H, w.W, generator=g, dtype=torch.float32)
        logits = torch.randn(w.N, w.D, w.H, w.W, generator=g, dtype=torch.float32)
        prob = torch.softmax(logits, dim=1)
        feats.append(f.movedim(1, -1))
        if mode == "categorical":
            depth.append(prob.movedim(1, -1))
        else:
            c = centres.view(1, -1, 1, 1)
            mean = (prob * c).sum(1)
            sigma = ((prob * (c - mean.unsqueeze(1)) ** 2).sum(1)).sqrt() + 0.1
            depth.append(torch.stack([mean, sigma], dim=-1))
        proj.append(torch.from_numpy(
            rig_projection(w.image_size, w.N, jitter_seed=(1000 + b) if w.jitter else None)))
    B = b1 - b0
    return {
        "image_feats": torch.stack(feats).to(td).contiguous(),
        "depth_params": torch.stack(depth).to(td).contiguous(),
        "projection_matrices": torch.stack(proj).contiguous(),
        "feature_size": torch.tensor([[w.H, w.W]], dtype=torch.int32).repeat(B * w.N, 1).view(B, w.N, 2),
        "image_size": torch.tensor(list(w.image_size), dtype=torch.int32),
        "roi_range": torch.tensor(list(w.roi), dtype=torch.float32),
        "grid_size": torch.tensor([w.X, w.Y, w.Z], dtype=torch.int32),
    }


def upstream_grad(w: Workload, B: Optional[int] = None, seed_offset: int = 7) -> torch.Tensor:
    """Upstream gradient ~ N(0,1), float32, [B,Y,X,C]."""
    g = torch.Generator(device="cpu").manual_seed(w.seed * 100003 + 50000 + seed_offset)
    return torch.randn(B if B is not None else w.B, w.Y, w.X, w.C, generator=g, dtype=torch.float32)


def algorithmic_bytes(w: Workload, mode: str = "categorical", B: Optional[int] = None,
                      backward: bool = False) -> int:
    """Compulsory HBM traffic of one call: every input and output tensor moves once.

    forward : features + depth + matrices + output
    backward: upstream gradient + features + depth (re-read) + both gradients written
    """
    B = w.B if B is None else B
    s = 4 if w.dtype == "fp32" else 2
    dd = w.D if mode == "categorical" else 2
    feats = B * w.N * w.H * w.W * w.C * s
    depth = B * w.N * w.H * w.W * dd * s
    mats = B * w.N * 48
    out = B * w.Y * w.X * w.C * s
    if not backward:
        return feats + depth + mats + out
    return out + feats + depth + mats + feats + depth
