"""Multi-GPU engines: symmetric memory over NVLink, fused data-parallel and
sharded steps, tensor-parallel layers."""
