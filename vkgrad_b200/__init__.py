"""vkgrad_b200: the training-step hot path of BrettKnox/vkgrad on NVIDIA B200.

Modules mirror the reference's: `vk` (runtime), `kernels`, `tkernels`,
`autograd`, `transformer`, `dataparallel`.  Everything computes on the GPU
through libvkgrad_b200.so (C ABI in include/vkgrad_b200.h); there is no CPU
fallback, and importing a module never builds or JIT-compiles anything.
"""

__version__ = "0.1.0"
