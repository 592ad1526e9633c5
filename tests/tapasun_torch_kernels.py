"""Plain torch statements of the kernels that Tapasun's parts call beyond those of ``torch_kernels``,
``makilorn_torch_kernels``, ``karesun_torch_kernels`` and ``mapalorn_torch_kernels``, with the signatures of
``kairyu_b200.kernels``, for CPU runs of the cache manager, the step function, the scheduler and the command line
(32-bit only).  ``install`` puts them all in place of the kernels for one test.  They are test code: the package has no
implementation but its kernels."""

from __future__ import annotations

import torch

import mapalorn_torch_kernels
from makilorn_torch_kernels import _convolve, _recurrence
from mapalorn_torch_kernels import _place, _turn


def sandwich_norm(residual, pending, weight, eps, out, *, rows=None):
    picked = rows.long() if rows is not None else slice(None)
    total = residual[picked]
    if pending is not None:
        y = pending.values[picked].float()
        total = total + y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + pending.eps) * pending.weight.float()
        if rows is None:
            residual.copy_(total)
    if out is not None:
        normed = total * torch.rsqrt(total.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
        out[: normed.shape[0]].copy_(normed.to(out.dtype))


def rotate_heads(x, *, heads, head_dim, cos, sin, positions, interleaved=False, inverse=False, flag=None):
    for t in range(x.shape[0]):
        position = int(positions[t])
        for h in range(heads):
            head = x[t, h * head_dim : (h + 1) * head_dim].float()
            x[t, h * head_dim : (h + 1) * head_dim] = _turn(head, cos[position], -sin[position] if inverse else sin[position], interleaved).to(x.dtype)


def scaled_sum(a, scale_a, b, scale_b, out):
    out.copy_((scale_a * a.float() + scale_b * b.float()).to(out.dtype))


def ssm_prepare(packed, dt_raw, taps, conv_bias, conv_state, *, row_ids, qo_indptr, state_slots, a_log, dt_bias, groups, state, heads, vdim,
                x, b, c, dt, decay, flag=None):
    inner, gn = heads * vdim, groups * state
    tokens = packed.shape[0]
    act = _convolve(lambda t0, t1: packed[t0:t1, : inner + 2 * gn].float(), taps, conv_state, qo_indptr, state_slots, tokens, conv_bias)
    x.view(tokens, inner).copy_(act[:, :inner])
    b.view(tokens, gn).copy_(act[:, inner : inner + gn])
    c.view(tokens, gn).copy_(act[:, inner + gn :])
    dt.copy_(torch.nn.functional.softplus(dt_raw + dt_bias))
    decay.copy_(torch.exp(-torch.exp(a_log) * dt))


def ssm_recurrence(c, b, x, dt, decay, states, out, *, qo_indptr, state_slots, groups, state, heads, vdim):
    _recurrence(c, b, x, dt, decay, states, out, qo_indptr, state_slots, groups, state, heads, vdim, False, False)


def ssm_gated_norm(y, x, skip, z, weight, eps, out, *, heads, vdim, norm_groups):
    tokens, inner = out.shape
    value = (y.view(tokens, heads, vdim) + skip[None, :, None] * x.view(tokens, heads, vdim)).reshape(tokens, inner)
    zf = z.float()
    value = (value * zf * torch.sigmoid(zf)).view(tokens, norm_groups, inner // norm_groups)
    normed = value * torch.rsqrt(value.pow(2).mean(-1, keepdim=True) + eps)
    out.copy_((normed.reshape(tokens, inner) * weight).to(out.dtype))


_NAMES = [
    "sandwich_norm", "rotate_heads", "scaled_sum", "ssm_prepare", "ssm_recurrence", "ssm_gated_norm",
]


def install(monkeypatch) -> None:
    import kairyu_b200.kernels as kernels

    mapalorn_torch_kernels.install(monkeypatch)
    for name in _NAMES:
        monkeypatch.setattr(kernels, name, globals()[name])
