"""Reference model definitions used by the benchmarks and tests.  All of them
are DP-compatible as written: no BatchNorm, no buffers on trainable modules."""
from .cnn import SmallCNN
from .llama import Llama, LlamaConfig, llama_1b_config, llama_8b_config
from .resnet_gn import resnet18_gn

__all__ = ["Llama", "LlamaConfig", "llama_1b_config", "llama_8b_config", "SmallCNN", "resnet18_gn"]
