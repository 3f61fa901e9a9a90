"""B200-native Mamba-2 SSD forward behind the WorkloadSuite ``mamba`` workload contract.

``ssd_forward``       functional SSD core on CUDA tensors (sm_100a kernels through a C ABI)
``ssd_forward_host``  the same for CPU tensors, pipelined over PCIe
``mamba_model``       drop-in ``Model`` / ``get_init_inputs`` / ``get_inputs`` module
``sharded``           head-sharded and sequence-sharded multi-GPU forwards
"""
from .ssd import (HostRunner, SsdError, device_status, fold_states, kernel_name, plan, ssd_forward,  # noqa: F401
                  ssd_forward_host)

__all__ = ["ssd_forward", "ssd_forward_host", "HostRunner", "fold_states", "kernel_name", "plan", "device_status", "SsdError"]
