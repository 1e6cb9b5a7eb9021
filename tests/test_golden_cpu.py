"""The committed golden vectors and the CPU oracle must agree (guards against drift of either)."""
import importlib.util
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def test_oracle_reproduces_committed_golden_vectors():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    fresh = module.build()
    stored = np.load(os.path.join(HERE, "golden", "nvfp4_golden.npz"))
    assert set(fresh) == set(stored.files)
    for key, value in fresh.items():
        assert np.array_equal(np.asarray(value), stored[key]), key
