"""Naive 4-bit Shampoo: the dense statistic L itself is stored quantized (drop-in for the
reference's optimizers/shampoo1.py; ShampooSGD :247-262, ShampooAdamW :334-350,
Preconditioner :102-146).  The inverse root is always the Schur-Newton iteration."""
from optimizers._base import (CODE, BlockPartitioner, Preconditioner as _Preconditioner, ShampooAdamWBase,
                              ShampooSGDBase)


class Preconditioner(_Preconditioner):
    """Statistics and preconditioners both as QTensorDiagReal."""
    flavour = "s1"


class ShampooSGD(ShampooSGDBase):
    """SGD with momentum on Shampoo-preconditioned gradients, dense quantized statistics."""
    preconditioner_cls = Preconditioner

    def __init__(self, params, lr=0.1, momentum=0.9, weight_decay=0.0, nesterov=False,
                 start_prec_step=1, stat_compute_steps=100, prec_compute_steps=500,
                 stat_decay=0.95, matrix_eps=1e-6, prec_maxorder=1200,
                 prec_bits=32, min_lowbit_size=4096, quan_blocksize=64, process_group=None):
        super().__init__(params, lr=lr, momentum=momentum, weight_decay=weight_decay, nesterov=nesterov,
                         start_prec_step=start_prec_step, stat_compute_steps=stat_compute_steps,
                         prec_compute_steps=prec_compute_steps, stat_decay=stat_decay, matrix_eps=matrix_eps,
                         prec_maxorder=prec_maxorder, prec_bits=prec_bits, min_lowbit_size=min_lowbit_size,
                         quan_blocksize=quan_blocksize, process_group=process_group)


class ShampooAdamW(ShampooAdamWBase):
    """AdamW moments on Shampoo-preconditioned gradients, dense quantized statistics."""
    preconditioner_cls = Preconditioner

    def __init__(self, params, lr=0.001, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 start_prec_step=1, stat_compute_steps=100, prec_compute_steps=500,
                 stat_decay=0.95, matrix_eps=1e-6, prec_maxorder=1200,
                 prec_bits=32, min_lowbit_size=4096, quan_blocksize=64, process_group=None):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                         start_prec_step=start_prec_step, stat_compute_steps=stat_compute_steps,
                         prec_compute_steps=prec_compute_steps, stat_decay=stat_decay, matrix_eps=matrix_eps,
                         prec_maxorder=prec_maxorder, prec_bits=prec_bits, min_lowbit_size=min_lowbit_size,
                         quan_blocksize=quan_blocksize, process_group=process_group)
