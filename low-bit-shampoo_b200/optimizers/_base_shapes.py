"""Shape arithmetic of the blocking rule (no tensors): which blocks and which preconditioner
orders a parameter shape produces (reference: optimizers/shampoo2.py:43-65, :115-121)."""
import itertools
import math


def matrix_shape(shape):
    """(rows, cols) the optimizer reshapes a parameter to, or None when it has fewer than two
    non-unit dimensions (no preconditioner)."""
    dims = [d for d in shape if d != 1]
    if len(dims) < 2:
        return None
    return dims[0], math.prod(dims[1:])


def cut(d, block):
    if block > 0 and d > block:
        full, rest = divmod(d, block)
        return [block] * full + ([rest] if rest else [])
    return [d]


def block_shapes(shape, prec_maxorder):
    ms = matrix_shape(tuple(shape))
    if ms is None:
        return []
    return list(itertools.product(cut(ms[0], prec_maxorder), cut(ms[1], prec_maxorder)))
