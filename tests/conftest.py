import pathlib
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "photon-mamba2-llm_b200"))

# Host-side deadline around every GPU test, as the reference's own GPU tests have
# (crates/pm-cuda/tests/conv1d_depthwise_bwd_gpu.rs:186-212): a kernel that stopped making progress fails the test
# instead of holding the run.  Every device-side wait is bounded too, so this only fires if that bound itself broke.
GPU_TEST_DEADLINE_S = 300


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if not config.pluginmanager.hasplugin("timeout"):
        return
    for item in items:
        if item.get_closest_marker("gpu") and not item.get_closest_marker("timeout"):
            item.add_marker(pytest.mark.timeout(GPU_TEST_DEADLINE_S))
