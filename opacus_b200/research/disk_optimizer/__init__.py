"""DiSK: Kalman-filtered DP optimizers (``research/disk_optimizer`` of the reference)."""
from .kf_optimizer import (
    KF_AdaClipDPOptimizer,
    KF_DistributedDPOptimizer,
    KF_DistributedDPOptimizerFastGradientClipping,
    KF_DistributedPerLayerOptimizer,
    KF_DPOptimizer,
    KF_DPOptimizerFastGradientClipping,
    KF_DPPerLayerOptimizer,
    KF_SimpleDistributedPerLayerOptimizer,
    KalmanFilterMixin,
    get_optimizer_class,
)
from .kf_privacy_engine import KF_PrivacyEngine

__all__ = [
    "KF_AdaClipDPOptimizer", "KF_DistributedDPOptimizer", "KF_DistributedDPOptimizerFastGradientClipping",
    "KF_DistributedPerLayerOptimizer", "KF_DPOptimizer", "KF_DPOptimizerFastGradientClipping",
    "KF_DPPerLayerOptimizer", "KF_SimpleDistributedPerLayerOptimizer", "KalmanFilterMixin", "KF_PrivacyEngine",
    "get_optimizer_class",
]
