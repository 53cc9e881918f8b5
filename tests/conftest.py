"""Shared pytest configuration: the ``gpu`` marker and import paths."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, 'deepgemm-ascend_b200')
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (B200, sm_100a)')


@pytest.fixture(scope='session')
def golden():
    import torch
    return torch.load(os.path.join(ROOT, 'tests', 'golden', 'reference_vectors.pt'), weights_only=False)
