"""Generates tests/golden/*.npz from the reference's own dense PyTorch path.

Run where the reference checkout is available (see --reference); the
fixtures it writes are committed, this script is how they were made:

    python tests/golden/make_golden.py [--reference /path/to/FlashBEV]

What is recorded, per case: the inputs, the forward output of
``sampling_vt_pytorch`` fed by ``project_coords`` (flashbev/flashbevpool/sampling_vt.py:36-123,
449-466), and the gradients autograd produces through that path for a seeded upstream
gradient.  The reference package imports its compiled extensions at import time; they
are replaced by empty stand-in modules because only the pure-PyTorch functions are used.
One case takes its camera rig from the reference's calibration fixture
(inputs/calib_nuscenes.json) through the reference's ``create_projection_matrix``.
module_dense_*.npz hold a run of the reference's ``SamplingVT`` module itself (dense branch).
"""
import argparse
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from flashbev_b200 import synth  # noqa: E402


def load_reference(root):
    for n in ("flashbevpool.flashbevpool_ext", "flashbevpool.sampling_vt_ext", "flashbevpool_ext", "sampling_vt_ext"):
        sys.modules[n] = types.ModuleType(n)
    sys.path.insert(0, os.path.join(root, "flashbev"))
    import flashbevpool.sampling_vt as R
    return R


def dense_reference(R, feats, depth, proj, image_size, roi, grid, dist, threshold, grad_out):
    """feats [B,N,H,W,C], depth [B,N,H,W,2] -> out [B,Y,X,C] and autograd gradients."""
    B, N = feats.shape[:2]
    X, Y, Z = grid
    r = torch.tensor(roi, dtype=torch.float32).view(3, 2)
    vs = [(r[i, 1] - r[i, 0]) / g for i, g in enumerate(grid)]
    # SamplingVT._calculate_coords_3d (sampling_vt.py:364-378)
    axes = [torch.linspace(float(r[i, 0]), float(r[i, 1]), g + 1)[:-1] + vs[i] / 2.0 for i, g in enumerate(grid)]
    coords = torch.stack(torch.meshgrid(*axes, indexing="ij"), dim=-1)
    coords = coords.unsqueeze(0).unsqueeze(0).expand(B, N, -1, -1, -1, -1)
    uvd = R.project_coords(coords_xyz=coords, projection_matrices=proj)
    f = feats.clone().requires_grad_(True)
    d = depth.clone().requires_grad_(True)
    out = R.sampling_vt_pytorch(
        image_uvd=uvd, features_pv=f.flatten(0, 1).movedim(-1, 1), depths=d.flatten(0, 1).movedim(-1, 1),
        B=B, N=N, image_size=image_size, depth_weight_threshold=threshold, depth_distribution=dist, epsilon=1e-6)
    out = out.movedim(1, -1)  # [B,C,Y,X] -> [B,Y,X,C]
    out.backward(grad_out)
    return out.detach(), f.grad, d.grad


def synthetic_calibration(B, N, seed):
    """Seeded camera calibration with the value ranges of a surround-view rig: rigid sensor-to-ego
    poses (any yaw, small pitch/roll, metre-scale offsets), pinhole intrinsics, and the image
    augmentation's scale/flip/rotate matrix and shift."""
    g = torch.Generator().manual_seed(seed)
    u = lambda *s: torch.rand(*s, generator=g, dtype=torch.float64)  # noqa: E731
    yaw, pitch, roll = (u(B, N) * 2 - 1) * np.pi, (u(B, N) * 2 - 1) * 0.05, (u(B, N) * 2 - 1) * 0.05
    def rot(axis, a):
        c, s, o, z = torch.cos(a), torch.sin(a), torch.ones_like(a), torch.zeros_like(a)
        rows = {"z": [c, -s, z, s, c, z, z, z, o], "y": [c, z, s, z, o, z, -s, z, c], "x": [o, z, z, z, c, -s, z, s, c]}[axis]
        return torch.stack(rows, -1).view(B, N, 3, 3)
    cam = torch.tensor([[0.0, 0.0, 1.0], [-1.0, 0.0, 0.0], [0.0, -1.0, 0.0]], dtype=torch.float64)  # camera axes -> ego axes
    s2e = torch.zeros(B, N, 4, 4, dtype=torch.float64)
    s2e[..., :3, :3] = rot("z", yaw) @ rot("y", pitch) @ rot("x", roll) @ cam
    s2e[..., :3, 3] = (u(B, N, 3) * 2 - 1) * torch.tensor([1.5, 0.8, 0.3], dtype=torch.float64) + torch.tensor([0.0, 0.0, 1.5], dtype=torch.float64)
    s2e[..., 3, 3] = 1.0
    K = torch.zeros(B, N, 3, 3, dtype=torch.float64)
    K[..., 0, 0] = 1100 + 200 * u(B, N)
    K[..., 1, 1] = 1100 + 200 * u(B, N)
    K[..., 0, 2] = 800 + 30 * (u(B, N) * 2 - 1)
    K[..., 1, 2] = 450 + 30 * (u(B, N) * 2 - 1)
    K[..., 2, 2] = 1.0
    scale, ang = 0.4 + 0.1 * u(B, N), (u(B, N) * 2 - 1) * 0.1
    flip = torch.where(u(B, N) < 0.5, -1.0, 1.0).to(torch.float64)
    pr = torch.zeros(B, N, 3, 3, dtype=torch.float64)
    pr[..., 0, 0], pr[..., 0, 1] = scale * flip * torch.cos(ang), -scale * torch.sin(ang)
    pr[..., 1, 0], pr[..., 1, 1] = scale * flip * torch.sin(ang), scale * torch.cos(ang)
    pr[..., 2, 2] = 1.0
    pt = torch.zeros(B, N, 3, dtype=torch.float64)
    pt[..., :2] = (u(B, N, 2) * 2 - 1) * 60.0
    return [t.float() for t in (s2e, K, pr, pt)]


def projection_case(R):
    """Calibration -> matrices through the reference's create_projection_matrix (sampling_vt.py:21-33)."""
    s2e, K, pr, pt = synthetic_calibration(3, 6, seed=21)
    B, N = s2e.shape[:2]
    eye = torch.eye(4).expand(B, N, 4, 4)
    P = R.create_projection_matrix(s2e, eye, K, pr, pt, torch.eye(3).expand(B, 3, 3))
    path = os.path.join(HERE, "projection_synthetic.npz")
    np.savez_compressed(path, sensor2ego=s2e.numpy(), camera2imgs=K.numpy(), post_rots=pr.numpy(), post_trans=pt.numpy(),
                        proj=P.contiguous().numpy(), torch_version=np.array(torch.__version__))
    print("projection_synthetic", tuple(P.shape), os.path.getsize(path), "bytes")


MODULE_GRID = {"x": [-20.0, 20.0, 1.0], "y": [-16.0, 16.0, 1.0], "z": [-4.0, 2.0, 1.0], "depth": [1.0, 60.0, 1.0]}


def module_case(R):
    """The reference's own module, dense branch: ``SamplingVT(fuse_projection=False, use_bev_pool=False)``
    (sampling_vt.py:126-294) with the 1x1 heads initialised under seed 42 as tools/profile_differences.py:218
    does.  Recorded: the seven inputs, the state dict, the BEV output and the depth head's output."""
    inputs, image = synth.module_inputs(B=2, N=6, C=32, H=8, W=22, seed=5)
    names = ("x", "sensor2ego", "ego2global", "camera2imgs", "post_rots", "post_trans", "bda")
    for dist in ("laplace", "gaussian"):
        torch.manual_seed(42)
        m = R.SamplingVT(MODULE_GRID, image, downsample=16, in_channels=32, out_channels=16, fuse_projection=False,
                         use_bev_pool=False, depth_distribution=dist, depth_weight_threshold=0.0).eval()
        state = {k: v.detach().clone() for k, v in m.state_dict().items() if k.split(".")[0] in
                 ("context_network", "depth_network")}
        with torch.no_grad():
            bev, depths = m([t.clone() for t in inputs])
        path = os.path.join(HERE, f"module_dense_{dist}.npz")
        arrays = {f"in_{n}": t.numpy() for n, t in zip(names, inputs)}
        arrays.update({f"state_{k}": v.numpy() for k, v in state.items()})
        np.savez_compressed(path, bev=bev.numpy(), depths=depths.numpy(), image=np.array(image, np.int32),
                            torch_version=np.array(torch.__version__), **arrays)
        print(f"module_dense_{dist}", tuple(bev.shape), "nonzero cells", int((bev.abs().sum(1) > 0).sum()),
              os.path.getsize(path), "bytes")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("FBEV_REFERENCE") or os.path.join(
        os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"),
        help="root of the reference checkout (default: $FBEV_REFERENCE, else a directory 'reference' beside this repository)")
    ap.add_argument("--only-projection", action="store_true", help="write only projection_synthetic.npz")
    ap.add_argument("--only-module", action="store_true", help="write only module_dense_*.npz")
    args = ap.parse_args()
    R = load_reference(args.reference)
    torch.manual_seed(0)
    if args.only_module:
        module_case(R)
        return
    projection_case(R)
    if args.only_projection:
        return
    module_case(R)

    small = synth.Workload("golden_small", B=2, N=6, C=8, H=8, W=22, D=16, X=24, Y=20, Z=4, xy_extent=25.6,
                           d0=1.0, delta=2.0, dtype="fp32", seed=11, jitter=True)
    cases = []
    inp = synth.make_inputs(small, "parametric")
    for dist in ("laplace", "gaussian"):
        for thr in (0.0, 2e-2):
            cases.append((f"synthetic_{dist}_thr{thr:g}", inp, small, dist, thr))

    # second rig: the reference's calibration record through its own matrix builder
    with open(os.path.join(args.reference, "inputs", "calib_nuscenes.json")) as fh:
        calib = {k: torch.tensor(v, dtype=torch.float32) for k, v in json.load(fh).items()}
    nus = synth.Workload("golden_nuscenes", B=1, N=6, C=6, H=16, W=44, D=16, X=40, Y=36, Z=6, xy_extent=50.0,
                         z_range=(-4.0, 2.0), d0=1.0, delta=3.0, dtype="fp32", seed=12)
    inp_n = synth.make_inputs(nus, "parametric")
    inp_n["projection_matrices"] = R.create_projection_matrix(
        calib["sensor2ego"], calib["ego2global"], calib["camera2imgs"], calib["post_rots"], calib["post_trans"],
        calib["bda"]).contiguous()
    cases.append(("nuscenes_laplace_thr0", inp_n, nus, "laplace", 0.0))

    for name, inp, w, dist, thr in cases:
        go = synth.upstream_grad(w)
        out, dfe, dde = dense_reference(R, inp["image_feats"], inp["depth_params"], inp["projection_matrices"],
                                        w.image_size, w.roi, w.grid, dist, thr, go)
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(
            path, feats=inp["image_feats"].numpy(), depth=inp["depth_params"].numpy(),
            proj=inp["projection_matrices"].numpy(), image_size=np.array(w.image_size, np.int32),
            roi=np.array(w.roi, np.float32), grid=np.array(w.grid, np.int32), threshold=np.float32(thr),
            laplace=np.int32(dist == "laplace"), grad_out=go.numpy(), out=out.numpy(), d_feats=dfe.numpy(),
            d_depth=dde.numpy(), torch_version=np.array(torch.__version__))
        print(name, out.shape, "nonzero cells", int((out.abs().sum(-1) > 0).sum()), os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
