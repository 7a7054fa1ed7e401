# SPDX-License-Identifier: Apache-2.0
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture()
def cpu_scheduler():
    import core_scheduler_b200 as cs

    return cs.DynamicScheduler(0, device="cpu")


@pytest.fixture()
def gpu_scheduler():
    import core_scheduler_b200 as cs

    return cs.DynamicScheduler(0, device="cuda")
