"""Communication layer: torch.distributed (NCCL / gloo) for bootstrap, control plane and the
``nccl_baseline`` mode; symmetric-memory + in-kernel NVLink paths for the ``fused`` mode."""
