import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


class SynthGraph:
    """A seeded synthetic graph made by the oracle's generators (CPU)."""

    def __init__(self, xadj, adjncy, adjwgt):
        self.xadj, self.adjncy, self.adjwgt = xadj, adjncy, adjwgt
        self.V, self.E = len(xadj) - 1, len(adjncy)


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def rmat16(oracle):
    """benchmark configuration 1: R-MAT scale 16, edge factor 16, weights in [1,10)."""
    x, a = oracle.gen_rmat(16, 16 << 16, 0.57, 0.19, 0.19, False, seed=1)
    return SynthGraph(x, a, oracle.gen_weights(len(a), 7))


@pytest.fixture(scope="session")
def rmat12(oracle):
    x, a = oracle.gen_rmat(12, 16 << 12, 0.57, 0.19, 0.19, False, seed=3)
    return SynthGraph(x, a, oracle.gen_weights(len(a), 9))


@pytest.fixture(scope="session")
def plaw(oracle):
    """Small undirected power-law graph with sorted adjacency (node2vec needs both)."""
    x, a = oracle.gen_powerlaw(20000, 300000, 2.1, 4.0, 3000, seed=5)
    return SynthGraph(x, a, oracle.gen_weights(len(a), 11))


@pytest.fixture(scope="session")
def ctx():
    from skywalker_b200.api import Context
    c = Context(0)
    yield c
    c.close()
