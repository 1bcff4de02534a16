"""Version and capability table of the package.

Parity: the reference exposes ``__version__`` and a ``COMPATIBILITY_MATRIX``
dict with a feature list (mccl/version.py:1-17); the keys are kept, the values
describe the Blackwell build.
"""
__version__ = "0.4.0"
__protocol_version__ = 1

COMPATIBILITY_MATRIX = {
    "os": ["Linux x86_64", "Linux aarch64"],
    "python": ["3.10", "3.11", "3.12", "3.13"],
    "pytorch": ["2.6+ (built against 2.11, CUDA 12.8/12.9)"],
    "hardware": "NVIDIA B200 (sm_100a), 1-8 GPUs of one NVSwitch domain; CPU tensors on any host",
    "interconnect": "NVLink 5 / NVSwitch for CUDA tensors (peer-mapped memory, NVLS multimem); TCP for CPU tensors",
    "features": [
        "distributed_memory_manager",
        "one_sided_put_get_atomics",
        "cuda_kernel_dispatch",
        "data_parallel_sharding",
        "tensor_parallel_sharding",
        "pipeline_parallel_sharding",
        "fused_bf16_wire_allreduce",
        "nvls_allreduce",
        "coherence_protocol",
        "cluster_manager_scheduler",
    ],
}
