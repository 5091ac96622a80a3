import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
if os.path.dirname(os.path.abspath(__file__)) not in sys.path:
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders (config.json + model.safetensors, bfloat16) for the tiny configurations,
    written once per test session into a temporary folder."""
    from tiny_configs import TINY
    from neurogrid_b200.weights import write_random_model
    out = {}
    for name, (cfg, seed) in TINY.items():
        d = tmp_path_factory.mktemp(f"model_{name}")
        write_random_model(cfg, seed, str(d))
        out[name] = str(d)
    return out


@pytest.fixture(scope="session")
def metanex_dirs(tmp_path_factory):
    """Model folders for the tiny Metanex configurations; "<name>_calm" has routers that hardly look at the
    token, for comparisons in bfloat16."""
    import metanex_models
    out = {}
    for name, (cfg, seed) in metanex_models.CONFIGS.items():
        out[name] = metanex_models.write_model(cfg, seed, str(tmp_path_factory.mktemp(f"metanex_{name}")))
        out[name + "_calm"] = metanex_models.write_model(cfg, seed, str(tmp_path_factory.mktemp(f"metanex_{name}c")),
                                                         router_gain=0.05)
    return out


@pytest.fixture(scope="session")
def rofulorn_dirs(tmp_path_factory):
    """Model folders for the tiny Rofulorn configurations."""
    import rofulorn_models
    return {name: rofulorn_models.write_model(cfg, seed, str(tmp_path_factory.mktemp(f"rofulorn_{name}")))
            for name, (cfg, seed) in rofulorn_models.CONFIGS.items()}


@pytest.fixture(scope="session")
def fuzelorn_dirs(tmp_path_factory):
    """Model folders for the tiny Fuzelorn configurations; "<name>_calm" has routers that hardly look at the token,
    for comparisons in bfloat16."""
    import fuzelorn_models
    out = {}
    for name, (cfg, seed) in fuzelorn_models.CONFIGS.items():
        out[name] = fuzelorn_models.write_model(cfg, seed, str(tmp_path_factory.mktemp(f"fuzelorn_{name}")))
        out[name + "_calm"] = fuzelorn_models.write_model(cfg, seed, str(tmp_path_factory.mktemp(f"fuzelorn_{name}c")),
                                                          router_gain=0.02)
    return out


@pytest.fixture(scope="session")
def dodilix_dirs(tmp_path_factory):
    """Model folders for the tiny Dodilix configurations; in "<name>_calm" a layer's routed experts are all alike, for
    comparisons in bfloat16 (a router's close call then changes nothing)."""
    import dodilix_models
    out = {}
    for name, (cfg, seed) in dodilix_models.CONFIGS.items():
        out[name] = dodilix_models.write_model(cfg, seed, str(tmp_path_factory.mktemp(f"dodilix_{name}")))
        out[name + "_calm"] = dodilix_models.write_model(cfg, seed, str(tmp_path_factory.mktemp(f"dodilix_{name}c")),
                                                         same_experts=True)
    return out
