from .adaptive_clipping_utils import (
    DPLossFastGradientAdaptiveClipping,
    DPTensorFastGradientAdaptiveClipping,
    PrivacyEngineAdaptiveClipping,
)

__all__ = [
    "DPTensorFastGradientAdaptiveClipping",
    "DPLossFastGradientAdaptiveClipping",
    "PrivacyEngineAdaptiveClipping",
]
