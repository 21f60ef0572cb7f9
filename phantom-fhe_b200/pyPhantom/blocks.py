"""Small host compositions over the evaluator that the reference binds next to it
(python/src/binding.cu:522-531, 589-593; src/linear.cu, src/ps.cu): slot-block sums, replication and
polynomial evaluation. They are calls into the same C ABI as everything else."""
import math

import numpy as np

from . import add, rotate
from . import boot, bootmath


def inner_sum(context, galois_key_, ct, block_size):
    """src/linear.cu: slot i gets the sum of slots i .. i + block_size - 1 (log2(block_size) rotations by 1, 2, 4, ...)"""
    if block_size == 0 or block_size & (block_size - 1):
        raise ValueError("inner_sum: block_size must be a power of 2")
    acc, stride = ct, 1
    while stride < block_size:
        acc = add(context, acc, rotate(context, acc, stride, galois_key_))
        stride <<= 1
    return acc


def replicate(context, galois_key_, ct, period, num_slots):
    """src/linear.cu: a vector living in the first `period` slots copied over all num_slots (rotations by -period, -2 period, ...)"""
    if period == 0 or period & (period - 1):
        raise ValueError("replicate: period must be a power of 2")
    if num_slots == 0 or num_slots & (num_slots - 1):
        raise ValueError("replicate: num_slots must be a power of 2")
    if period > num_slots:
        raise ValueError("replicate: period exceeds num_slots")
    acc, stride = ct, period
    while stride < num_slots:
        acc = add(context, acc, rotate(context, acc, -stride, galois_key_))
        stride <<= 1
    return acc


def eval_polynomial(context, encoder, relin_key_, ct, coeffs):
    """sum_k coeffs[k] x^k on every slot (src/ps.cu:131-200). The reference runs Paterson-Stockmeyer in the monomial
    basis with a chain of dependent powers; here the polynomial is rewritten in the Chebyshev basis (an exact change of
    basis) and evaluated by the bootstrapping pipeline's evaluator, whose powers have logarithmic depth and whose
    scales are tracked instead of snapped. The result is handed back at the chain index the reference ends on
    (input + m + l - 2 with m = ceil(sqrt(d + 1)), l = ceil((d + 1) / m)) and at the input's scale."""
    c = np.asarray(coeffs, dtype=np.float64).ravel()
    if c.size < 2:
        raise ValueError("eval_polynomial: degree must be >= 1")
    d = c.size - 1
    m = math.ceil(math.sqrt(d + 1))
    n_chunks = (d + 1 + m - 1) // m
    ref_out_chain = ct.chain_index() + m + n_chunks - 2
    cheb = np.polynomial.chebyshev.poly2cheb(c)
    ops = boot.CtOps(context, relin_key_)
    babies = 1 << max(1, math.ceil(math.log2(math.sqrt(d + 1))))
    ev = bootmath.ChebyshevEvaluator(ops, ct, babies)
    out = ev.evaluate(cheb, ct.scale())
    if out.chain_index() > ref_out_chain:
        raise ValueError("eval_polynomial: not enough levels left")
    out = ops.drop(out, context.limbs_at(ref_out_chain))
    out.set_scale(ct.scale())
    return out
