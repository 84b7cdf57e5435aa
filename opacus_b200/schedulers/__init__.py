from .grad_clip_scheduler import ExponentialGradClip, LambdaGradClip, StepGradClip, _GradClipScheduler
from .noise_scheduler import ExponentialNoise, LambdaNoise, StepNoise, _NoiseScheduler

__all__ = [
    "ExponentialGradClip", "LambdaGradClip", "StepGradClip", "_GradClipScheduler",
    "ExponentialNoise", "LambdaNoise", "StepNoise", "_NoiseScheduler",
]
