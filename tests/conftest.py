import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import insignia_b200._lib as L

    L.lib()  # fail loudly if the extension is missing
    return torch.device("cuda:0")


@pytest.fixture(scope="session")
def workdir(tmp_path_factory):
    """Scratch directory for synthetic checkpoints; RAM-backed when there is room."""
    import shutil

    base = None
    try:
        if shutil.disk_usage("/dev/shm").free > (12 << 30):
            base = "/dev/shm"
    except OSError:
        pass
    if base:
        import tempfile

        d = tempfile.mkdtemp(prefix="insg_", dir=base)
        yield d
        shutil.rmtree(d, ignore_errors=True)
    else:
        yield str(tmp_path_factory.mktemp("insg"))


GOLDEN_CFG = dict(layers=(0, 1, 2, 3), vocab_rows=64, mtp=False, lm_head=True, seed=7, norms="random")


@pytest.fixture(scope="session")
def golden_ckpt(workdir):
    """The 4-layer synthetic checkpoint the golden vectors were made from: (safetensors path, index path)."""
    from insignia_b200 import synth

    st, idx = os.path.join(workdir, "golden4.safetensors"), os.path.join(workdir, "golden4.idx")
    synth.write_checkpoint(synth.SynthConfig(**GOLDEN_CFG), st, idx)
    return st, idx
