"""Operators: hand-written sm_100a kernels on CUDA tensors, plain PyTorch maths on CPU tensors."""
