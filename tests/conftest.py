import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# the reference checkout sits beside this repository unless MGWFBP_REFERENCE_DIR says otherwise
REFERENCE_DIR = os.environ.get('MGWFBP_REFERENCE_DIR') or os.path.join(os.path.dirname(ROOT), 'reference')


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run with -m gpu on a B200)')
    config.addinivalue_line('markers', 'multigpu: needs at least two CUDA devices')


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        n_gpu = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        n_gpu = 0
    skip_gpu = pytest.mark.skip(reason='no CUDA device')
    skip_multi = pytest.mark.skip(reason='needs >= 2 CUDA devices')
    for item in items:
        if 'gpu' in item.keywords and n_gpu == 0:
            item.add_marker(skip_gpu)
        if 'multigpu' in item.keywords and n_gpu < 2:
            item.add_marker(skip_multi)


@pytest.fixture(scope='session')
def reference_dir():
    if not os.path.isdir(REFERENCE_DIR):
        pytest.skip('reference checkout not available')
    return REFERENCE_DIR
