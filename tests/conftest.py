import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, 'universal-lm-trainer_b200')
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a B200 (run with -m gpu on the GPU box)')


@pytest.fixture(scope='session')
def golden():
    here = os.path.join(ROOT, 'tests', 'golden')
    with open(os.path.join(here, 'golden.json')) as f:
        meta = json.load(f)
    arrays = dict(np.load(os.path.join(here, 'golden.npz')))
    return meta, arrays
