import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def load_package():
    """Imports the package whose directory name has a dot (llm.cu_b200) under the name llm_cu_b200."""
    if "llm_cu_b200" in sys.modules:
        return sys.modules["llm_cu_b200"]
    pkg_dir = os.path.join(ROOT, "llm.cu_b200")
    if not os.path.exists(os.path.join(pkg_dir, "libllm_b200.so")):
        spec_b = importlib.util.spec_from_file_location("llm_cu_b200_build", os.path.join(pkg_dir, "build.py"))
        mod_b = importlib.util.module_from_spec(spec_b)
        spec_b.loader.exec_module(mod_b)
        mod_b.build()
    spec = importlib.util.spec_from_file_location("llm_cu_b200", os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["llm_cu_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle_lib
    oracle_lib.lib()
    return oracle_lib


@pytest.fixture(scope="session")
def tiny_weights(pkg, oracle):
    return oracle.Weights(pkg.CONFIGS["tiny"], seed=0)


@pytest.fixture(scope="session")
def weights_8b_l2(pkg, oracle):
    """LLaMA3-8B layer shape, two layers, 1024 embedding rows: the shape pinned against the reference."""
    return oracle.Weights(pkg.CONFIGS["llama3_8b_l2"], seed=0, keep_file=False)
