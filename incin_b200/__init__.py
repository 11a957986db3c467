"""incin_b200 — a Blackwell-native (sm_100a) deep-learning framework with the capabilities of incin.

PyTorch is the tensor/autograd substrate; every hot op on CUDA is a hand-written
sm_100a kernel in ``libincin_sm100.so`` (tcgen05/TMEM GEMM fed by TMA, norms,
cross-entropy, optimisers, fused collectives over NVLink peer memory); the CPU
backend (PyTorch CPU + the C++ oracle in ``libincin_host.so``) is the default
backend and the correctness reference.
"""
__version__ = "0.1.0"

from . import _native  # noqa: F401


def build(force: bool = False):
    """Compile the native libraries in-tree (nvcc for sm_100a, g++ for the host runtime)."""
    from . import _build
    return _build.build_all(force)
