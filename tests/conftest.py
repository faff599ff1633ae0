import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200) and the compiled extension")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    from tests import helpers
    seen = helpers.BF16_VS_F32_SEEN
    if seen:
        what, worst = max(seen, key=lambda x: x[1])
        terminalreporter.write_line(
            f"bfloat16 against float32 engine: {len(seen)} comparisons, largest difference {worst:.2e} of the largest "
            f"logit ({what}); tolerance {helpers.BF16_VS_F32_TOL:.1e}")
