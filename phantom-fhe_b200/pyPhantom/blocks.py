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


def schedule_chain_index(ct, degree):
    """where the reference's Paterson-Stockmeyer schedule ends for this degree (src/ps.cu:131-200):
    input + m + l - 2 with m = ceil(sqrt(d + 1)), l = ceil((d + 1) / m)"""
    m = math.ceil(math.sqrt(degree + 1))
    return ct.chain_index() + m + (degree + m) // m - 2


def eval_chebyshev_series(context, relin_key_, ct, cheb, out_chain_index):
    """sum_k cheb[k] T_k(x) on every slot by the bootstrapping pipeline's evaluator (powers of logarithmic depth, scales
    tracked instead of snapped); the result is dropped to out_chain_index and carries the input's scale"""
    cheb = np.asarray(cheb, dtype=np.float64).ravel()
    d = cheb.size - 1
    ops = boot.CtOps(context, relin_key_)
    babies = 1 << max(1, math.ceil(math.log2(math.sqrt(d + 1))))
    ev = bootmath.ChebyshevEvaluator(ops, ct, babies, tight=True)
    out = ev.evaluate(cheb, ct.scale())
    if out.chain_index() > out_chain_index:
        raise ValueError("eval_polynomial: not enough levels left")
    out = ops.drop(out, context.limbs_at(out_chain_index))
    out.set_scale(ct.scale())
    return out


def eval_polynomial(context, encoder, relin_key_, ct, coeffs):
    """sum_k coeffs[k] x^k on every slot (src/ps.cu:131-200). The reference runs Paterson-Stockmeyer in the monomial
    basis with a chain of dependent powers; here the polynomial is rewritten in the Chebyshev basis (an exact change of
    basis) and evaluated by eval_chebyshev_series. The result is handed back at the chain index the reference ends on
    and at the input's scale."""
    c = np.asarray(coeffs, dtype=np.float64).ravel()
    if c.size < 2:
        raise ValueError("eval_polynomial: degree must be >= 1")
    cheb = np.polynomial.chebyshev.poly2cheb(c)
    if cheb.size < c.size:
        cheb = np.concatenate([cheb, np.zeros(c.size - cheb.size)])
    return eval_chebyshev_series(context, relin_key_, ct, cheb, schedule_chain_index(ct, c.size - 1))
