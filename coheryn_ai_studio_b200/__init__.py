"""A single-GPU inference engine for NVIDIA B200 (sm_100a): paged cache, one step
function for mixed prefill/decode batches, continuous batching, hand-written CUDA."""

__version__ = "0.1.0"
