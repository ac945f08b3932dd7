import importlib.util
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load_package():
    """The package directory is `legion-ibp_b200`; it is imported under the name legion_ibp_b200."""
    if "legion_ibp_b200" in sys.modules:
        return sys.modules["legion_ibp_b200"]
    pkg_dir = os.path.join(ROOT, "legion-ibp_b200")
    spec = importlib.util.spec_from_file_location("legion_ibp_b200", os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["legion_ibp_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


_load_package()
sys.path.insert(0, os.path.join(ROOT, "oracle"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    # the allocation-free entry point is checked last
    items.sort(key=lambda it: 1 if "test_zz_" in it.nodeid else 0)


def small_graph(n_nodes=3000, n_pairs=40000, seed=0):
    """Seeded R-MAT CSR as numpy arrays (int64 indptr, int32 indices)."""
    import torch
    from legion_ibp_b200 import synth
    ip, ix = synth.rmat_csr(n_nodes, n_pairs, seed=seed)
    return ip.numpy().astype(np.int64), ix.numpy().astype(np.int32)


@pytest.fixture(scope="session")
def graph_small():
    return small_graph()


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle
    oracle.build()
    return oracle
