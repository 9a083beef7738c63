"""4-bit Shampoo with eigen-factor statistics (drop-in for the reference's optimizers/shampoo2.py).

Public names and constructor arguments are the reference's (ShampooSGD :278-296,
ShampooAdamW :370-388, Preconditioner :102-107, BlockPartitioner :35-99, CODE :32); the
work of a step is executed batched per preconditioner order by optimizers/_engine.py.
"""
from optimizers._base import (CODE, BlockPartitioner, Preconditioner as _Preconditioner, ShampooAdamWBase,
                              ShampooSGDBase)


class Preconditioner(_Preconditioner):
    """Statistics in eigen-factor form (QTensorSVDFast), preconditioners as QTensorDiagReal."""
    flavour = "s2"


class ShampooSGD(ShampooSGDBase):
    """SGD with momentum on Shampoo-preconditioned, norm-grafted gradients.

    Args (beyond torch.optim.SGD's): start_prec_step, stat_compute_steps (T1),
    prec_compute_steps (T2), stat_decay (beta), matrix_eps (epsilon), prec_maxorder,
    prec_bits, min_lowbit_size, quan_blocksize, rect_t1, rect_t2,
    inv_root_mode (0: eigen-factor inverse root, 1: Schur-Newton iteration).
    """
    preconditioner_cls = Preconditioner

    def __init__(self, params, lr=0.1, momentum=0.9, weight_decay=0.0, nesterov=False,
                 start_prec_step=1, stat_compute_steps=100, prec_compute_steps=500,
                 stat_decay=0.95, matrix_eps=1e-6, prec_maxorder=1200,
                 prec_bits=32, min_lowbit_size=4096, quan_blocksize=64,
                 rect_t1=1, rect_t2=4, inv_root_mode=0, process_group=None):
        super().__init__(params, lr=lr, momentum=momentum, weight_decay=weight_decay, nesterov=nesterov,
                         start_prec_step=start_prec_step, stat_compute_steps=stat_compute_steps,
                         prec_compute_steps=prec_compute_steps, stat_decay=stat_decay, matrix_eps=matrix_eps,
                         prec_maxorder=prec_maxorder, prec_bits=prec_bits, min_lowbit_size=min_lowbit_size,
                         quan_blocksize=quan_blocksize, rect_t1=rect_t1, rect_t2=rect_t2, inv_root_mode=inv_root_mode,
                         process_group=process_group)


class ShampooAdamW(ShampooAdamWBase):
    """AdamW moments on Shampoo-preconditioned, norm-grafted gradients (same extra arguments
    as ShampooSGD)."""
    preconditioner_cls = Preconditioner

    def __init__(self, params, lr=0.001, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 start_prec_step=1, stat_compute_steps=100, prec_compute_steps=500,
                 stat_decay=0.95, matrix_eps=1e-6, prec_maxorder=1200,
                 prec_bits=32, min_lowbit_size=4096, quan_blocksize=64,
                 rect_t1=1, rect_t2=4, inv_root_mode=0, process_group=None, cuda_graph=False):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                         start_prec_step=start_prec_step, stat_compute_steps=stat_compute_steps,
                         prec_compute_steps=prec_compute_steps, stat_decay=stat_decay, matrix_eps=matrix_eps,
                         prec_maxorder=prec_maxorder, prec_bits=prec_bits, min_lowbit_size=min_lowbit_size,
                         quan_blocksize=quan_blocksize, rect_t1=rect_t1, rect_t2=rect_t2, inv_root_mode=inv_root_mode,
                         process_group=process_group, cuda_graph=cuda_graph)
