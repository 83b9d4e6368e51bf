"""Operators: one module per fused op. CUDA tensors run the sm_100a kernels of
``lib/libneox_b200.so``; CPU tensors run the plain-PyTorch statement of the same math."""
