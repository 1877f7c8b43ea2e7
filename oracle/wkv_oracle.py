"""CPU oracle for the WKV / depthwise_conv1d operators.

TEST INFRASTRUCTURE ONLY.  This module restates, in plain PyTorch on the CPU, the
formula path of every operator of BlinkDL/RWKV-CUDA that the CUDA library implements.
It is the checker that the parity tests, the smoke test and the benchmark's CPU-baseline
leg compare against (or time); the product path never imports it.

Every function is vectorised over batch and head, loops over time only, and is evaluated in
the dtype of its inputs (fp64 for parity, fp32 when timed as the CPU baseline).  Gradients
come from autograd through the forward, exactly as every reference harness obtains them.

Parity pin: each restatement is checked against the reference's own formula functions,
lifted from the reference checkout and evaluated in fp64 on seeded inputs; the resulting
input/output vectors are committed under tests/golden/ and re-checked by the CPU test
tier (tests/test_oracle_golden.py).

Reference formulas followed (paths inside the reference project):
  wkv4            wkv/run.py:46-78              RUN_FORMULA_VERY_SLOW / RUN_PYTORCH
  timex           depthwise_conv1d/run.py:45-60 RUN_FORMULA_VERY_SLOW / RUN_PYTORCH
  wkv5            wkv5/run.py:47-87             RUN_FORMULA_1 / RUN_FORMULA_1A
  wkv5a           wkv5a/run.py:164-190,260-289  PYTHON_1 / PYTHON_2
  wkv6            wkv6/run.py:183-218           RUN_TORCH
  wkv6state       wkv6_state/run.py:137-165     RUN_TORCH (initial state term tt=-1)
  rwkv7 (3 forms) rwkv7_fast_fused/rwkv7_cuda_benchmark.py:46-69,
                  rwkv7_cuda_benchmark_state.py:46-68,
                  rwkv7_cuda_benchmark_state_passing.py:46-68
"""
from __future__ import annotations

import math
import torch
import torch.nn.functional as F

W_SCALE = -math.exp(-0.5)  # rwkv7_fast_fused/cuda/rwkv7_statepassing_clampw.cu:16


# --------------------------------------------------------------------------------------
# RWKV-4
# --------------------------------------------------------------------------------------
def wkv4(time_decay, u, k, v):
    """RWKV-4 WKV.  time_decay,u: (C); k,v: (B,T,C).  w = -exp(time_decay) (wkv/run.py:47,95).

    y_t = (sum_{s<t} e^{(t-1-s)w+k_s} v_s + e^{u+k_t} v_t) / (sum_{s<t} e^{(t-1-s)w+k_s} + e^{u+k_t})
    evaluated with a running log-scale so that it never overflows (the reference formula
    overflows for large k; its CUDA kernel does not, wkv/cuda/wkv_cuda_v2.cu:21-37).
    """
    B, T, C = k.shape
    w = -torch.exp(time_decay)
    p = torch.zeros(B, C, dtype=k.dtype)
    q = torch.zeros(B, C, dtype=k.dtype)
    o = torch.full((B, C), -1e38, dtype=k.dtype)
    ys = []
    for t in range(T):
        kt, vt = k[:, t], v[:, t]
        no = torch.maximum(o, (u + kt).detach()).detach()
        A = torch.exp(o - no)
        Bc = torch.exp(u + kt - no)
        ys.append((A * p + Bc * vt) / (A * q + Bc))
        no = torch.maximum((w + o).detach(), kt.detach()).detach()
        A = torch.exp(w + o - no)
        Bc = torch.exp(kt - no)
        p = A * p + Bc * vt
        q = A * q + Bc
        o = no
    return torch.stack(ys, dim=1)


def wkv4_bruteforce(time_decay, u, k, v):
    """O(T^2) literal form of wkv/run.py:46-63 (small shapes only)."""
    B, T, C = k.shape
    w = -torch.exp(time_decay)
    out = torch.empty(B, T, C, dtype=k.dtype)
    for t in range(T):
        num = torch.exp(u + k[:, t]) * v[:, t]
        den = torch.exp(u + k[:, t])
        for s in range(t):
            e = torch.exp(k[:, s] + w * (t - s - 1))
            num = num + e * v[:, s]
            den = den + e
        out[:, t] = num / den
    return out


# --------------------------------------------------------------------------------------
# depthwise_conv1d ("TimeX")
# --------------------------------------------------------------------------------------
def timex(w, k, eps=0.0):
    """out[b,c,t] = eps + sum_{u<=t} w[c,(T-1)-(t-u)] k[b,c,u]  (depthwise_conv1d/run.py:41-55)."""
    B, C, T = k.shape
    idx_t = torch.arange(T).view(T, 1)
    idx_u = torch.arange(T).view(1, T)
    tap = (T - 1) - (idx_t - idx_u)                      # (t,u)
    mask = (idx_u <= idx_t).to(k.dtype)
    toe = w[:, tap.clamp(0, T - 1)] * mask               # (C,t,u)
    return torch.einsum("ctu,bcu->bct", toe, k) + eps


def timex_conv(w, k, eps=0.0):
    """Same operator via a grouped convolution (depthwise_conv1d/run.py:58-60); large shapes."""
    B, C, T = k.shape
    return F.conv1d(F.pad(k, (T - 1, 0)), w.unsqueeze(1), groups=C) + eps


# --------------------------------------------------------------------------------------
# RWKV-5 / 5a  (static decay)
# --------------------------------------------------------------------------------------
def wkv5(r, k, v, w_raw, u, H):
    """RWKV-5.  r,k,v: (B,T,C); w_raw,u: (H,N) or (C).  decay = exp(-exp(w_raw)).

    y_t[i] = sum_j r_t[j] (u[j] k_t[j] v_t[i] + S[j,i]);  S[j,i] <- decay[j] S[j,i] + k_t[j] v_t[i]
    (wkv5/run.py:66-87 with w already exponentiated by the autograd wrapper, :483-484).
    """
    B, T, C = r.shape
    N = C // H
    r4, k4, v4 = (x.view(B, T, H, N) for x in (r, k, v))
    decay = torch.exp(-torch.exp(w_raw.reshape(H, N)))
    uu = u.reshape(H, N)
    S = torch.zeros(B, H, N, N, dtype=r.dtype)           # [key j, value i]
    ys = []
    for t in range(T):
        kv = k4[:, t, :, :, None] * v4[:, t, :, None, :]
        ys.append(torch.einsum("bhj,bhji->bhi", r4[:, t], uu[None, :, :, None] * kv + S))
        S = decay[None, :, :, None] * S + kv
    return torch.stack(ys, dim=1).reshape(B, T, C)


def wkv5_bruteforce(r, k, v, w_raw, u, H):
    """O(T^2) literal form of wkv5/run.py:47-64 (small shapes only)."""
    B, T, C = r.shape
    N = C // H
    r4, k4, v4 = (x.view(B, T, H, N) for x in (r, k, v))
    decay = torch.exp(-torch.exp(w_raw.reshape(H, N)))
    uu = u.reshape(H, N)
    out = torch.zeros(B, T, H, N, dtype=r.dtype)
    for t in range(T):
        for tt in range(t + 1):
            ww = uu if tt == t else decay ** (t - tt - 1)
            out[:, t] += torch.einsum("bhj,bhi->bhi", r4[:, t] * ww * k4[:, tt], v4[:, tt])
    return out.reshape(B, T, C)


def wkv5a(r, k, v, w1_raw, u1, w2_raw, u2, H):
    """RWKV-5a: decay w1[j]*w2[i], bonus u1[j]+u2[i]  (wkv5a/run.py:164-190, :260-289)."""
    B, T, C = r.shape
    N = C // H
    r4, k4, v4 = (x.view(B, T, H, N) for x in (r, k, v))
    d1 = torch.exp(-torch.exp(w1_raw.reshape(H, N)))
    d2 = torch.exp(-torch.exp(w2_raw.reshape(H, N)))
    decay = d1[:, :, None] * d2[:, None, :]               # [h, j, i]
    bonus = u1.reshape(H, N)[:, :, None] + u2.reshape(H, N)[:, None, :]
    S = torch.zeros(B, H, N, N, dtype=r.dtype)
    ys = []
    for t in range(T):
        kv = k4[:, t, :, :, None] * v4[:, t, :, None, :]
        ys.append(torch.einsum("bhj,bhji->bhi", r4[:, t], bonus[None] * kv + S))
        S = decay[None] * S + kv
    return torch.stack(ys, dim=1).reshape(B, T, C)


# --------------------------------------------------------------------------------------
# RWKV-6 (per-token decay), optional initial / final state
# --------------------------------------------------------------------------------------
def wkv6(r, k, v, w_raw, u, H, s0=None, return_state=False):
    """RWKV-6.  w_raw: (B,T,C) raw decay, decay_t = exp(-exp(w_raw_t))  (wkv6/run.py:183-218).

    s0: optional initial state (B,H,N,N) indexed [value i, key j]; it enters token 0
    undecayed (the tt=-1 term of wkv6_state/run.py:137-165).  With return_state the final
    state is returned in the same layout (the reference operator has no such output; the
    extended entry points of the CUDA library do).
    """
    B, T, C = r.shape
    N = C // H
    r4, k4, v4, w4 = (x.view(B, T, H, N) for x in (r, k, v, w_raw))
    decay = torch.exp(-torch.exp(w4))
    uu = u.reshape(H, N)
    S = torch.zeros(B, H, N, N, dtype=r.dtype) if s0 is None else s0.transpose(-1, -2)  # [j,i]
    ys = []
    for t in range(T):
        kv = k4[:, t, :, :, None] * v4[:, t, :, None, :]
        ys.append(torch.einsum("bhj,bhji->bhi", r4[:, t], uu[None, :, :, None] * kv + S))
        S = decay[:, t, :, :, None] * S + kv
    y = torch.stack(ys, dim=1).reshape(B, T, C)
    if return_state:
        return y, S.transpose(-1, -2)
    return y


def wkv6_bruteforce(r, k, v, w_raw, u, H, s0=None):
    """O(T^2) literal form of wkv6_state/run.py:137-165 (small shapes only)."""
    B, T, C = r.shape
    N = C // H
    r4, k4, v4, w4 = (x.view(B, T, H, N) for x in (r, k, v, w_raw))
    decay = torch.exp(-torch.exp(w4))
    uu = u.reshape(H, N)
    out = torch.zeros(B, T, H, N, dtype=r.dtype)
    for t in range(T):
        for tt in range(-1, t + 1):
            if tt == t:
                ww = uu[None].expand(B, H, N)
            else:
                ww = torch.ones(B, H, N, dtype=r.dtype)
                for zz in range(tt + 1, t):
                    ww = ww * decay[:, zz]
            if tt == -1:
                if s0 is not None:
                    out[:, t] += torch.einsum("bhj,bhij->bhi", r4[:, t] * ww, s0)
            else:
                out[:, t] += torch.einsum("bhj,bhi->bhi", r4[:, t] * ww * k4[:, tt], v4[:, tt])
    return out.reshape(B, T, C)


# --------------------------------------------------------------------------------------
# RWKV-7 (generalised delta rule, soft-clamped decay)
# --------------------------------------------------------------------------------------
def wkv7(r, w_raw, k, v, a, b, H, s0=None):
    """RWKV-7 "clampw".  All of r,w_raw,k,v,a,b are (B,T,C); s0 (B,H,N,N) [value i, key j].

    decay_t = exp(-exp(-softplus(-w_raw) - 0.5)) = exp(-e^{-0.5} sigmoid(w_raw))
    S <- S diag(decay_t) + (S a_t) b_t^T + v_t k_t^T ;  y_t = S r_t
    (rwkv7_fast_fused/rwkv7_cuda_benchmark_state_passing.py:46-68).  Returns (y, S_T).
    """
    B, T, C = r.shape
    N = C // H
    r4, k4, v4, a4, b4 = (x.view(B, T, H, N) for x in (r, k, v, a, b))
    wl = -F.softplus(-w_raw) - 0.5
    decay = torch.exp(-torch.exp(wl.view(B, T, H, N)))
    S = torch.zeros(B, H, N, N, dtype=r.dtype) if s0 is None else s0
    ys = []
    for t in range(T):
        sa = torch.einsum("bhik,bhk->bhi", S, a4[:, t])
        S = (S * decay[:, t, :, None, :]
             + sa[..., None] * b4[:, t, :, None, :]
             + v4[:, t, :, :, None] * k4[:, t, :, None, :])
        ys.append(torch.einsum("bhj,bhij->bhi", r4[:, t], S))
    return torch.stack(ys, dim=1).reshape(B, T, C), S


# --------------------------------------------------------------------------------------
# helpers shared by tests and the benchmark
# --------------------------------------------------------------------------------------
def err_ratio(x, y):
    """RMS(x-y)/RMS(x), the reference's error metric (wkv/run.py:26-29)."""
    x = x.detach().double().flatten()
    y = y.detach().double().flatten()
    base = x.square().mean().sqrt().item()
    return (x - y).square().mean().sqrt().item() / (base if base > 0 else 1.0)


def max_err(x, y):
    """max|x-y| / max|x|: 'max relative error' normalised by the tensor's largest magnitude."""
    x = x.detach().double().flatten()
    y = y.detach().double().flatten()
    base = x.abs().max().item()
    return (x - y).abs().max().item() / (base if base > 0 else 1.0)


def strange_loss(y):
    """((y*y) - tanh(y)).sum(), the loss every harness uses to get a non-trivial dL/dy
    (wkv/run.py:199)."""
    return ((y * y) - torch.tanh(y)).sum()
