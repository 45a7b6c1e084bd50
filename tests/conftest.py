import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import tiny_configs as tc  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def _folder(tmp_path_factory, name, cfgd, init, seed):
    import cbis_b200 as cb
    d = str(tmp_path_factory.mktemp(name))
    cb.write_model_folder(d, cb.config_from_dict(cfgd), seed=seed, scheme=cb.InitScheme(*init))
    return d


@pytest.fixture(scope="session")
def folder_a(tmp_path_factory):
    return _folder(tmp_path_factory, "tiny_a", tc.TINY_A, tc.INIT_A, 11)


@pytest.fixture(scope="session")
def folder_b(tmp_path_factory):
    return _folder(tmp_path_factory, "tiny_b", tc.TINY_B, tc.INIT_B, 12)


@pytest.fixture(scope="session", params=["a", "b"])
def tiny(request, folder_a, folder_b):
    """(folder, config dict, page size) of one of the two tiny configurations."""
    if request.param == "a":
        return folder_a, tc.TINY_A, tc.PAGE_A
    return folder_b, tc.TINY_B, tc.PAGE_B
