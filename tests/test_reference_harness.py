"""The reference's own harness code (tools/utils/*.py, tools/profile_differences.py) run unchanged against this
repository's ``flashbevpool`` package.  The harness files are not part of this repository: the tests need a
reference checkout (FBEV_REFERENCE, else a directory ``reference`` beside the repository) and are skipped without
one.  ``hydra``, ``omegaconf`` and ``matplotlib`` are replaced by the small stand-ins under tests/harness_shims
when they are not installed."""
import importlib
import inspect
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.environ.get("FBEV_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
TOOLS = os.path.join(REFERENCE, "tools")

needs_checkout = pytest.mark.skipif(not os.path.exists(os.path.join(TOOLS, "utils", "benchmark_utils.py")),
                                    reason="no reference checkout with tools/utils/benchmark_utils.py")


@pytest.fixture()
def harness():
    """Imports the reference's tools as they are, with this repository's package standing in for the reference's
    ``flashbevpool``; undone afterwards."""
    saved_path, saved_mods = list(sys.path), set(sys.modules)
    for pkg in ("hydra", "omegaconf", "matplotlib"):
        try:
            importlib.import_module(pkg)
        except ImportError:
            shim = os.path.join(ROOT, "tests", "harness_shims")
            if shim not in sys.path:
                sys.path.insert(0, shim)
    sys.path.insert(0, TOOLS)
    sys.path.insert(0, ROOT)
    mods = {name: importlib.import_module(name) for name in
            ("utils.benchmark_utils", "utils.transformer_utils", "utils.data_utils", "profile_differences")}
    import flashbevpool
    assert os.path.dirname(os.path.abspath(flashbevpool.__file__)) == os.path.join(ROOT, "flashbevpool")
    yield mods
    sys.path[:] = saved_path
    for name in set(sys.modules) - saved_mods:
        if name.split(".")[0] in ("utils", "profile_differences", "hydra", "omegaconf", "matplotlib"):
            del sys.modules[name]


@needs_checkout
def test_harness_imports_and_binds_to_this_package(harness):
    import flashbev_b200
    bu = harness["utils.benchmark_utils"]
    assert bu.flash_bevpool is flashbev_b200.flash_bevpool and bu.SamplingVT is flashbev_b200.SamplingVT
    # every keyword the kernel-only benchmark passes (tools/utils/benchmark_utils.py:27-42) is accepted
    accepted = set(inspect.signature(flashbev_b200.flash_bevpool).parameters)
    passed = {"image_feats", "depth_params", "projection_matrices", "feature_size", "image_size", "roi_range", "grid_size",
              "depth_distribution", "use_shared_memory", "optimize_z_precompute", "use_warp_kernel",
              "use_vectorized_load", "epsilon", "depth_weight_threshold"}
    assert passed <= accepted


@needs_checkout
def test_parity_harness_runs_on_the_cpu_with_the_dense_method(harness):
    """tools/profile_differences.py evaluate_methods + compare_two_methods (its :183-280, :70-127) with the
    reference's dummy input and this package's module on the CPU; the only method a CPU can run is the dense one,
    compared with itself under another name."""
    pd, du = harness["profile_differences"], harness["utils.data_utils"]
    grid = {"x": [-20.0, 20.0, 1.0], "y": [-20.0, 20.0, 1.0], "z": [-4.0, 2.0, 1.0], "depth": [1.0, 60.0, 1.0]}
    pd.set_seed(42)
    # with the reference's calibration record: its built-in dummy calibration writes into an expanded tensor and
    # raises (tools/utils/data_utils.py:100-106)
    calib = du.load_calibration_params(os.path.join(REFERENCE, "inputs", "calib_nuscenes.json"), device="cpu")
    inputs, _ = du.create_dummy_input(1, 6, 16, 16, 44, device="cpu", calib_params=calib)
    methods = [{"name": "Dense PyTorch Sampling-VT", "fuse_projection": False, "use_bev_pool": False},
               {"name": "dense again", "fuse_projection": False, "use_bev_pool": False}]
    results, baseline = pd.evaluate_methods(methods, inputs, grid, (256, 704), 16, 8, 16, device="cpu")
    assert baseline == methods[0]["name"] and results["dense again"]["metrics"]["mse"] == 0.0
    assert float(results[baseline]["output"].abs().sum()) > 0
    cmp = pd.compare_two_methods(results[baseline]["output"], results["dense again"]["output"])
    assert cmp["overall_match"]


@needs_checkout
def test_hydra_stand_in_reads_the_reference_config(harness):
    import hydra
    seen = {}

    @hydra.main(version_base=None, config_path="config", config_name="config")
    def entry(cfg):
        seen["cfg"] = cfg

    entry.__wrapped__.__module__ = "profile_differences"  # resolve the config beside the reference's script
    entry(overrides=["num_cameras=4", "grid_config.z=[-4.0, 2.0, 1.0]"])
    cfg = seen["cfg"]
    assert cfg.num_cameras == 4 and cfg.grid_config.z[2] == 1.0 and cfg.methods[1].fuse_projection is True
    assert cfg.get("seed", 0) == 42


@needs_checkout
@pytest.mark.gpu
def test_kernel_only_benchmark_of_the_reference_runs_on_this_package(harness, cuda_device):
    """benchmark_flashbevpool_kernel (tools/utils/benchmark_utils.py:12-92) on create_flashbevpool_data's tensors
    (tools/utils/data_utils.py:130-219: 4x4 matrices, sizes as device tensors), a few iterations."""
    bu, du = harness["utils.benchmark_utils"], harness["utils.data_utils"]
    calib = du.load_calibration_params(os.path.join(REFERENCE, "inputs", "calib_nuscenes.json"), device="cuda")
    sig = inspect.signature(du.create_flashbevpool_data)
    kwargs = dict(batch_size=1, num_cameras=6, in_channels=16, feature_h=16, feature_w=44, grid_x=200, grid_y=200,
                  grid_z=12, roi_range=[-50.0, 50.0, -50.0, 50.0, -4.0, 2.0], device="cuda", calib_params=calib)
    data = du.create_flashbevpool_data(**{k: v for k, v in kwargs.items() if k in sig.parameters})
    stats = bu.benchmark_flashbevpool_kernel(data, num_warmup=2, num_iterations=5)
    assert stats["latency_mean_ms"] > 0
