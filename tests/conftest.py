import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselected on CPU-only hosts")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _range_checks_stay_clean():
    """With the debug build of the kernels (WALLX_CHECKED=1) every test must leave the range-check records empty."""
    yield
    if os.environ.get("WALLX_CHECKED", "0") != "1":
        return
    import torch

    if not torch.cuda.is_available():
        return
    from wallx_b200.ops import _ext

    mod = _ext.get(required=False)
    if mod is None or not mod.checked_build():
        return
    report = mod.check_report(True)
    bad = {k: v for k, v in report.items() if v[1] != 0}
    assert not bad, f"range checks of the debug build fired (unit: [site, count, value, value]): {bad}"
