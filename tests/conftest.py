import importlib.util
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_DIR = os.path.join(ROOT, "project-axiom-ai-llm_b200")
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def load_package():
    """Imports the package directory (its name is not a Python identifier)."""
    name = "project_axiom_ai_llm_b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(
        name, os.path.join(PKG_DIR, "__init__.py"), submodule_search_locations=[PKG_DIR])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) device")


@pytest.fixture(scope="session")
def axm():
    return load_package()


@pytest.fixture(scope="session")
def workloads():
    load_package()
    import importlib
    return importlib.import_module("project_axiom_ai_llm_b200.workloads")


@pytest.fixture(scope="session")
def oracle():
    import oracle_binding
    return oracle_binding.load()


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    return torch.device("cuda:0")
