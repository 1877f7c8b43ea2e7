"""Shared helpers of the parity tests: seeded inputs with the distributions of the benchmark
configurations, comparison against the fp64 oracle, and tolerances.

Tolerances (max|x-y|/max|x| and RMS(x-y)/RMS(x), both must hold):
  fp32 operators (RWKV-4, depthwise_conv1d)          1e-5
  bf16 operators (RWKV-5/5a/6/6-state/7)             2e-2
  fp32 instances of the multi-head operators          1e-4 (fp32 accumulation over T steps)
"""
import math

import numpy as np
import torch

from oracle import wkv_oracle as O

TOL_FP32_STRICT = 1e-5
TOL_FP32 = 1e-4
TOL_BF16 = 2e-2


def tol_for(dtype):
    return TOL_BF16 if dtype == torch.bfloat16 else TOL_FP32


def assert_close(got, want, tol, what):
    """`want` is the fp64 oracle value."""
    got = got.detach().double().cpu().reshape(want.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    m, e = O.max_err(want, got), O.err_ratio(want, got)
    assert m <= tol and e <= tol, f"{what}: max err {m:.3e}, rms err {e:.3e} > {tol:g}"
    return m, e


def rounded(x, dtype):
    """x rounded to `dtype`, as (device-dtype tensor, fp64 copy of the rounded values)."""
    xd = x.to(dtype)
    return xd, xd.double()


def gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def randn(g, *shape):
    return torch.randn(*shape, generator=g, dtype=torch.float32)


def rand(g, *shape, lo=0.0, hi=1.0):
    return torch.rand(*shape, generator=g, dtype=torch.float32) * (hi - lo) + lo


def v7_inputs(B, T, H, N, seed=42):
    """Config-5 distributions: w_raw ~ N(0,1); r,k,v ~ 0.5 N(0,1); kk = normalised N(0,1) per head;
    a = -kk, b = kk*sigmoid(N(0,1)); s0 ~ 0.1 N(0,1); dy ~ N(0,1); dsT ~ N(0,1)."""
    g = gen(seed)
    C = H * N
    r, k, v = (0.5 * randn(g, B, T, C) for _ in range(3))
    w = randn(g, B, T, C)
    kk = torch.nn.functional.normalize(randn(g, B, T, H, N), dim=-1).view(B, T, C)
    a = -kk
    b = kk * torch.sigmoid(randn(g, B, T, C))
    s0 = 0.1 * randn(g, B, H, N, N)
    dy = randn(g, B, T, C)
    dsT = randn(g, B, H, N, N)
    return dict(r=r, w=w, k=k, v=v, a=a, b=b, s0=s0, dy=dy, dsT=dsT)


def v7_oracle(inp64, H, use_s0=True, use_dsT=True):
    """fp64 oracle outputs and gradients for RWKV-7 on already-rounded fp64 inputs."""
    leaves = {n: inp64[n].clone().requires_grad_(True) for n in ("r", "w", "k", "v", "a", "b")}
    s0 = inp64["s0"].clone().requires_grad_(True) if use_s0 else None
    y, sT = O.wkv7(leaves["r"], leaves["w"], leaves["k"], leaves["v"], leaves["a"], leaves["b"], H, s0=s0)
    if use_dsT:
        torch.autograd.backward([y, sT], [inp64["dy"], inp64["dsT"]])
    else:
        y.backward(inp64["dy"])
    out = dict(y=y.detach(), sT=sT.detach())
    for n, x in leaves.items():
        out["d" + n] = x.grad
    if use_s0:
        out["ds0"] = s0.grad
    return out


def units(x, picks, H):
    """Select (batch, head) units from a (B,T,H*N) tensor -> (len(picks), T, N) (one head each)."""
    B, T, C = x.shape
    N = C // H
    x4 = x.view(B, T, H, N)
    return torch.stack([x4[b, :, h, :] for b, h in picks], 0).contiguous()


def state_units(s, picks):
    """Select units from a (B,H,N,N) state -> (len(picks), 1, N, N)."""
    return torch.stack([s[b, h] for b, h in picks], 0).unsqueeze(1).contiguous()
