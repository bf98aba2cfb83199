"""quicknn_b200: a small, whole, single-GPU generation library for NVIDIA B200 (sm_100a).

Everything between a request's tokens and its next token: typed configuration and
registry, safetensors weights, layers assembled from parts, a paged cache with a
slot per sequence, one step function, a generation loop, sampling, and the
hand-written CUDA kernels they run on.
"""
__version__ = "0.1.0"
