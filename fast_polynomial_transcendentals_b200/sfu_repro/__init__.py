"""Configuration and patching layer of the reference (`sfu_repro`), bound to this package's kernels.

Importing it loads nothing heavy: CUDA, the kernel library and the attention backend are reached only by the
function that needs them.
"""
__all__ = ["activations", "fa4", "rope"]
