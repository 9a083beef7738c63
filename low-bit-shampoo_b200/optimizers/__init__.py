"""Shampoo optimizers with low-bit preconditioner state for NVIDIA B200."""
