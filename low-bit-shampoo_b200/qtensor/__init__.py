"""Blockwise low-bit tensors for Shampoo preconditioner state on NVIDIA B200."""
