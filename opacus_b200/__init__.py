"""opacus_b200: differentially private training of PyTorch models, built for
NVIDIA B200 (sm_100a).  Public surface of the reference library
(``opacus/__init__.py:16-28``) plus the native kernels and parallel engines."""
from . import utils
from .grad_sample import GradSampleModule, GradSampleModuleFastGradientClipping
from .privacy_engine import PrivacyEngine
from .version import __version__

__all__ = [
    "PrivacyEngine",
    "GradSampleModule",
    "GradSampleModuleFastGradientClipping",
    "utils",
    "__version__",
]
