import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu: needs two or more CUDA devices")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        n = 0
    for item in items:
        if "gpu" in item.keywords and n == 0:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))
        if "multigpu" in item.keywords and n < 2:
            item.add_marker(pytest.mark.skip(reason="needs >= 2 CUDA devices"))


@pytest.fixture(scope="session")
def tiny_zse(tmp_path_factory):
    from zse_b200.format import synth
    path = str(tmp_path_factory.mktemp("models") / "tiny.zse")
    synth.write_random_model(path, synth.shape_config("tiny"), seed=0)
    return path


@pytest.fixture(scope="session")
def tiny_aligned_zse(tmp_path_factory):
    from zse_b200.format import synth
    path = str(tmp_path_factory.mktemp("models") / "tiny_aligned.zse")
    synth.write_random_model(path, synth.shape_config("tiny-aligned"), seed=1)
    return path


@pytest.fixture(scope="session")
def small128_zse(tmp_path_factory):
    from zse_b200.format import synth
    path = str(tmp_path_factory.mktemp("models") / "small128.zse")
    synth.write_random_model(path, synth.shape_config("small-128"), seed=2)
    return path
