"""B200-native Mamba-2 SSD forward behind the WorkloadSuite ``mamba`` workload contract.

``ssd_forward``       functional SSD core on CUDA tensors (sm_100a kernels through a C ABI)
``ssd_forward_host``  the same for CPU tensors, pipelined over PCIe
``ssd_step``          one token of the recurrence with the state carried in place (decode-style use)
``conv1d_silu``       causal depthwise conv + SiLU producing the core's X (``model_ref.py:83-86``)
``dt_prologue``       softplus(dt + bias) and A_dt = -exp(A_log) dt in one pass (``model_ref.py:94, 102-103``)
``mamba_model``       drop-in ``Model`` / ``get_init_inputs`` / ``get_inputs`` module
``sharded``           head-sharded and sequence-sharded multi-GPU forwards
"""
from .ssd import (HostRunner, SsdError, conv1d_silu, device_status, dt_prologue, fold_states, kernel_name, plan,  # noqa: F401
                  ssd_forward, ssd_forward_host, ssd_step)

__all__ = ["ssd_forward", "ssd_forward_host", "ssd_step", "conv1d_silu", "dt_prologue", "HostRunner", "fold_states", "kernel_name", "plan", "device_status", "SsdError"]
