import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as orc
    orc.build()
    return orc


# every GPU test runs against each kernel configuration: the default dispatch, the large-batch
# kernels (wide and narrow kernel instances chosen by the batch, or forced), the shared-memory cluster kernel
# with its automatic and forced sizes, and the single-CTA kernel
VARIANTS = {"auto": (0, 0), "batch": (2, 0), "batch_w256": (4, 0), "batch_w1024": (5, 0), "batch_n128": (6, 0), "batch_n256": (7, 0),
            "cluster1": (3, 1), "cluster2": (3, 2), "cluster4": (3, 4),
            "cluster8": (3, 8), "single_cta": (1, 0)}


@pytest.fixture(scope="session")
def _sampler_session():
    from gorch_b200 import build, sampling
    build.build()
    s = sampling.CudaSampler(0)
    yield s
    s.release()


@pytest.fixture(params=list(VARIANTS))
def sampler(request, _sampler_session):
    variant, csize = VARIANTS[request.param]
    _sampler_session.set_kernel_variant(variant, csize)
    yield _sampler_session
    _sampler_session.set_kernel_variant(0, 0)
