import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


try:  # property tests: the same examples on every run unless exploring is asked for (HYPOTHESIS_PROFILE=explore)
    from hypothesis import settings as _hyp_settings

    _hyp_settings.register_profile("repeatable", derandomize=True, database=None)
    _hyp_settings.register_profile("explore")
    _hyp_settings.load_profile(os.environ.get("HYPOTHESIS_PROFILE", "repeatable"))
except ImportError:
    pass


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (runs only on a GPU box)")
    config.addinivalue_line("markers", "multigpu: needs at least two GPUs on one node")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        n_gpu = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        n_gpu = 0
    for item in items:
        if "gpu" in item.keywords and n_gpu == 0:
            item.add_marker(pytest.mark.skip(reason="no GPU in this environment"))
        if "multigpu" in item.keywords and n_gpu < 2:
            item.add_marker(pytest.mark.skip(reason="needs >= 2 GPUs"))


def pytest_addoption(parser):
    pass
