"""CPU restatement (numpy, fp32 arithmetic) of the reference's gated activations and RMSNorm.  TEST INFRASTRUCTURE ONLY: the
product never imports this module.

Follows primus_turbo/triton/activation/swiglu_kernel.py:40-60 (forward) and :95-125 (backward), geglu_kernel.py with
triton/utils/gelu.py (erf form), and triton/normalization/rmsnorm_kernel.py:55-80 (forward), :120-170 (backward).
Parity note: the reference tests these operators against torch (F.silu / F.gelu / F.rms_norm) within 1e-2 for 16-bit
types; the kernels under test use hardware exp / division approximations, so this oracle is compared within a few ulp of
the output type, not bit for bit.
"""
import math

import numpy as np

F32 = np.float32
_erf = np.vectorize(math.erf, otypes=[np.float64])


def _act(a, act):
    a = a.astype(np.float64)
    if act == "silu":
        return a / (1.0 + np.exp(-a))
    return 0.5 * a * (1.0 + _erf(a / math.sqrt(2.0)))


def _act_grad(a, act):
    a = a.astype(np.float64)
    if act == "silu":
        s = 1.0 / (1.0 + np.exp(-a))
        return s * (1.0 + a * (1.0 - s))
    return 0.5 * (1.0 + _erf(a / math.sqrt(2.0))) + a * np.exp(-0.5 * a * a) / math.sqrt(2.0 * math.pi)


def glu_fwd(x, probs, act, row_mask=None):
    """x [rows, 2H] (fp32 view of the input), probs [rows] -> act(a) * b * p, rows masked out are zero."""
    H = x.shape[1] // 2
    a, b = x[:, :H], x[:, H:]
    out = _act(a, act) * b.astype(np.float64) * probs.astype(np.float64)[:, None]
    if row_mask is not None:
        out[row_mask == 0] = 0
    return out


def glu_bwd(g, x, probs, act, row_mask=None):
    """(grad_x [rows, 2H], grad_probs [rows]) for the upstream gradient g [rows, H]."""
    H = x.shape[1] // 2
    a, b = x[:, :H], x[:, H:].astype(np.float64)
    g = g.astype(np.float64)
    p = probs.astype(np.float64)[:, None]
    act_a = _act(a, act)
    gx = np.concatenate([g * p * b * _act_grad(a, act), g * p * act_a], axis=1)
    gp = (g * act_a * b).sum(axis=1)
    if row_mask is not None:
        gx[row_mask == 0] = 0
        gp[row_mask == 0] = 0
    return gx, gp


def rmsnorm_fwd(x, gamma, eps, zero_centered=False):
    """(y, rstd); x [rows, H]."""
    x = x.astype(np.float64)
    rstd = 1.0 / np.sqrt((x * x).mean(axis=1) + eps)
    g = gamma.astype(np.float64) + (1.0 if zero_centered else 0.0)
    return x * rstd[:, None] * g[None, :], rstd


def rmsnorm_bwd(dy, x, gamma, eps, zero_centered=False, dxpr=None):
    """(dx, dgamma)."""
    x, dy = x.astype(np.float64), dy.astype(np.float64)
    rstd = 1.0 / np.sqrt((x * x).mean(axis=1) + eps)
    g = gamma.astype(np.float64) + (1.0 if zero_centered else 0.0)
    x_hat = x * rstd[:, None]
    m = (dy * g[None, :] * x_hat).mean(axis=1)
    dx = (dy * g[None, :] - x_hat * m[:, None]) * rstd[:, None]
    if dxpr is not None:
        dx = dx + dxpr.astype(np.float64)
    return dx, (dy * x_hat).sum(axis=0)
