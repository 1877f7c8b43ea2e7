"""Generate the golden vectors under tests/golden/ from the reference's own formula functions.

The reference ships no stored vectors; its harnesses pin results only by agreement between
independent formula implementations on seeded inputs.  This script lifts those formula
functions straight out of a reference checkout (by AST, nothing is copied into this
repository), evaluates them on the CPU in fp64 on seeded inputs at the harnesses' own tiny
shapes, takes gradients by autograd through them exactly as the harnesses do, and stores
inputs, outputs and gradients as small .npz files.  tests/test_oracle_golden.py then holds
the oracle to these vectors.

Run (only where a reference checkout exists):
    python tests/golden/make_golden.py /path/to/RWKV-CUDA
"""
import ast
import math
import os
import sys

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


class _Cuda2Cpu(ast.NodeTransformer):
    def visit_Constant(self, node):
        if node.value == "cuda":
            return ast.copy_location(ast.Constant("cpu"), node)
        return node


def lift(path, name, env, owner=None):
    """Return function `name` (optionally a method of class `owner`) compiled from `path`."""
    tree = ast.parse(open(path).read())
    body = tree.body
    if owner is not None:
        body = next(n for n in body if isinstance(n, ast.ClassDef) and n.name == owner).body
    fn = next(n for n in body if isinstance(n, ast.FunctionDef) and n.name == name)
    fn.decorator_list = []
    mod = ast.fix_missing_locations(ast.Module(body=[_Cuda2Cpu().visit(fn)], type_ignores=[]))
    ns = dict(torch=torch, nn=nn, F=F, exp=math.exp, np=np, DEVICE="cpu")
    ns.update(env)
    exec(compile(mod, path, "exec"), ns)
    return ns[name]


def strange_loss(y):
    return ((y * y) - torch.tanh(y)).sum()


def leaf(*shape, lo=-1.0, hi=1.0):
    return torch.empty(*shape, dtype=torch.float64).uniform_(lo, hi).requires_grad_(True)


def save(name, **arrays):
    out = {k: (v.detach().numpy() if torch.is_tensor(v) else np.asarray(v)) for k, v in arrays.items()}
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print("wrote", name, {k: tuple(v.shape) for k, v in out.items()})


def grads(loss, *leaves):
    for x in leaves:
        x.grad = None
    loss.backward()
    return [x.grad.clone() for x in leaves]


def main(ref):
    torch.set_default_dtype(torch.float64)

    # ---- RWKV-4: wkv/run.py  (CHECK_PYTORCH shape B3 T11 C5) -------------------------
    torch.manual_seed(42)
    B, T, C = 3, 11, 5
    p = os.path.join(ref, "wkv/run.py")
    slow = lift(p, "RUN_FORMULA_VERY_SLOW", {})
    conv = lift(p, "RUN_PYTORCH", {})
    w, u, k, v = leaf(C), leaf(C), leaf(B, T, C), leaf(B, T, C)
    y_slow = slow(B, T, C, w.detach(), u.detach(), k.detach(), v.detach())
    curve = torch.tensor([-(T - 2 - i) for i in range(T - 1)]).unsqueeze(0)
    y = conv(B, T, C, w, u, k, v, curve)
    assert torch.allclose(y_slow, y, atol=1e-12), "reference formulas disagree (wkv4)"
    gw, gu, gk, gv = grads(strange_loss(y), w, u, k, v)
    save("wkv4", w=w, u=u, k=k, v=v, y=y, gw=gw, gu=gu, gk=gk, gv=gv)

    # ---- depthwise_conv1d: depthwise_conv1d/run.py (B3 C5 T11, eps 0.1) --------------
    torch.manual_seed(42)
    B, C, T, eps = 3, 5, 11, 0.1
    p = os.path.join(ref, "depthwise_conv1d/run.py")
    slow = lift(p, "RUN_FORMULA_VERY_SLOW", {})
    conv = lift(p, "RUN_PYTORCH", {})
    w = torch.rand(C, T).requires_grad_(True)
    k = torch.rand(B, C, T).requires_grad_(True)
    y_slow = slow(w.detach(), k.detach(), B, C, T, eps)
    y = conv(w, k, B, C, T, eps)
    assert torch.allclose(y_slow, y, atol=1e-12), "reference formulas disagree (timex)"
    gw, gk = grads(strange_loss(y), w, k)
    save("timex", w=w, k=k, eps=eps, y=y, gw=gw, gk=gk)

    # ---- RWKV-5: wkv5/run.py (job 'backward': B3 T5 C8 N4) ---------------------------
    torch.manual_seed(42)
    B, T, C, N = 3, 5, 8, 4
    H = C // N
    p = os.path.join(ref, "wkv5/run.py")
    f1 = lift(p, "RUN_FORMULA_1", {})
    f1a = lift(p, "RUN_FORMULA_1A", {})
    bw1 = lift(p, "RUN_BACKWARD_1", {})
    r, k, v, w, u = leaf(B, T, C), leaf(B, T, C), leaf(B, T, C), leaf(C), leaf(C)
    y = f1(B, T, C, H, r, k, v, torch.exp(-torch.exp(w)), u)
    y1a = f1a(B, T, C, H, r.detach(), k.detach(), v.detach(), torch.exp(-torch.exp(w.detach())), u.detach())
    assert torch.allclose(y, y1a, atol=1e-12), "reference formulas disagree (wkv5)"
    yy = y.detach().clone().requires_grad_(True)
    strange_loss(yy).backward()
    gy = yy.grad.clone()
    gr, gk, gv, gw, gu = grads(strange_loss(y), r, k, v, w, u)
    hr, hk, hv, hw, hu = bw1(B, T, C, H, gy, r.detach(), k.detach(), v.detach(), w.detach(), u.detach())
    for a_, b_ in ((gr, hr), (gk, hk), (gv, hv), (gw, hw.flatten()), (gu, hu.flatten())):
        assert torch.allclose(a_, b_.reshape(a_.shape), atol=1e-10), "reference hand backward disagrees (wkv5)"
    save("wkv5", H=H, r=r, k=k, v=v, w=w, u=u, y=y, gy=gy, gr=gr, gk=gk, gv=gv, gw=gw, gu=gu)

    # ---- RWKV-5a: wkv5a/run.py (job 1: B3 T5 C8 N4) ----------------------------------
    torch.manual_seed(42)
    B, T, C, N = 3, 5, 8, 4
    H = C // N
    p = os.path.join(ref, "wkv5a/run.py")
    env = dict(B=B, T=T, C=C, H=H, N=N)
    p1 = lift(p, "PYTHON_1", env)
    p2 = lift(p, "PYTHON_2", env)
    r, k, v = leaf(B, T, C), leaf(B, T, C), leaf(B, T, C)
    w1, u1, w2, u2 = leaf(H, N), leaf(H, N), leaf(H, N), leaf(H, N)
    y = p1(r, k, v, w1, u1, w2, u2)
    y2 = p2(*[x.detach() for x in (r, k, v, w1, u1, w2, u2)])
    assert torch.allclose(y, y2, atol=1e-12), "reference formulas disagree (wkv5a)"
    yy = y.detach().clone().requires_grad_(True)
    strange_loss(yy).backward()
    gy = yy.grad.clone()
    g = grads(strange_loss(y), r, k, v, w1, u1, w2, u2)
    save("wkv5a", H=H, r=r, k=k, v=v, w1=w1, u1=u1, w2=w2, u2=u2, y=y, gy=gy,
         gr=g[0], gk=g[1], gv=g[2], gw1=g[3], gu1=g[4], gw2=g[5], gu2=g[6])

    # ---- RWKV-6: wkv6/run.py (CHECK_REF shape B2 T7 C8 N4) ---------------------------
    torch.manual_seed(42)
    B, T, C, N = 2, 7, 8, 4
    H = C // N
    p = os.path.join(ref, "wkv6/run.py")
    fwd = lift(p, "forward", {}, owner="RUN_TORCH")
    bwd = lift(p, "TORCH_BACKWARD", {})
    r, k, v, u = leaf(B, T, C), leaf(B, T, C), leaf(B, T, C), leaf(H, N)
    w = leaf(B, T, C, lo=-3.0, hi=1.0)
    y = fwd(None, B, T, C, H, r, k, v, w, u)
    yy = y.detach().clone().requires_grad_(True)
    strange_loss(yy).backward()
    gy = yy.grad.clone()
    gr, gk, gv, gw, gu = grads(strange_loss(y), r, k, v, w, u)
    hr, hk, hv, hw, hu = bwd(B, T, C, H, gy, r.detach(), k.detach(), v.detach(), w.detach(), u.detach())
    for a_, b_ in ((gr, hr), (gk, hk), (gv, hv), (gw, hw), (gu, hu)):
        assert torch.allclose(a_, b_.reshape(a_.shape), atol=1e-10), "reference hand backward disagrees (wkv6)"
    save("wkv6", H=H, r=r, k=k, v=v, w=w, u=u, y=y, gy=gy, gr=gr, gk=gk, gv=gv, gw=gw, gu=gu)

    # ---- RWKV-6 with state: wkv6_state/run.py (B3 T7 C8 N4) --------------------------
    torch.manual_seed(42)
    B, T, C, N = 3, 7, 8, 4
    H = C // N
    p = os.path.join(ref, "wkv6_state/run.py")
    fwd = lift(p, "forward", {}, owner="RUN_TORCH")
    r, k, v, u = leaf(B, T, C), leaf(B, T, C), leaf(B, T, C), leaf(H, N)
    w = leaf(B, T, C, lo=-3.0, hi=1.0)
    s = leaf(B, H, N, N)
    y = fwd(None, B, T, C, H, r, k, v, w, u, s)
    yy = y.detach().clone().requires_grad_(True)
    strange_loss(yy).backward()
    gy = yy.grad.clone()
    gr, gk, gv, gw, gu, gs = grads(strange_loss(y), r, k, v, w, u, s)
    save("wkv6state", H=H, r=r, k=k, v=v, w=w, u=u, s=s, y=y, gy=gy,
         gr=gr, gk=gk, gv=gv, gw=gw, gu=gu, gs=gs)

    # ---- RWKV-7, three variants (B2 T64 C32 N16, harness input distributions) --------
    B, T, C, N = 2, 64, 32, 16
    H = C // N
    env = dict(B=B, T=T, C=C, H=H, N=N)
    d = os.path.join(ref, "rwkv7_fast_fused")

    def v7_inputs():
        torch.manual_seed(42)
        r = (torch.empty(B, T, C).uniform_(-1, 1) * 3).requires_grad_(True)
        w = torch.empty(B, T, C).uniform_(-6, 0).requires_grad_(True)
        k = (torch.empty(B, T, C).uniform_(-1, 1) * 3).requires_grad_(True)
        v = (torch.empty(B, T, C).uniform_(-1, 1) * 3).requires_grad_(True)
        a = F.normalize(torch.empty(B, T, C).uniform_(-1, 1) * 2, dim=-1, p=2.0).requires_grad_(True)
        b = F.normalize(torch.empty(B, T, C).uniform_(-1, 1) * 2, dim=-1, p=2.0).requires_grad_(True)
        s = (torch.empty(B, H, N, N).uniform_(-1, 1) * 10).requires_grad_(True)
        return s, r, w, k, v, a, b

    s, r, w, k, v, a, b = v7_inputs()
    f = lift(os.path.join(d, "rwkv7_cuda_benchmark.py"), "RWKV7_CLAMPW_REF", env)
    y = f(r, w, k, v, a, b)
    yy = y.detach().clone().requires_grad_(True)
    strange_loss(yy).backward()
    g = grads(strange_loss(y), r, w, k, v, a, b)
    save("wkv7_clampw", H=H, r=r, w=w, k=k, v=v, a=a, b=b, y=y, dy=yy.grad,
         dr=g[0], dw=g[1], dk=g[2], dv=g[3], da=g[4], db=g[5])

    s, r, w, k, v, a, b = v7_inputs()
    f = lift(os.path.join(d, "rwkv7_cuda_benchmark_state.py"), "RWKV7_STATE_CLAMPW_REF", env)
    y = f(s, r, w, k, v, a, b)
    yy = y.detach().clone().requires_grad_(True)
    strange_loss(yy).backward()
    g = grads(strange_loss(y), s, r, w, k, v, a, b)
    save("wkv7_state_clampw", H=H, s0=s, r=r, w=w, k=k, v=v, a=a, b=b, y=y, dy=yy.grad,
         ds0=g[0], dr=g[1], dw=g[2], dk=g[3], dv=g[4], da=g[5], db=g[6])

    s, r, w, k, v, a, b = v7_inputs()
    f = lift(os.path.join(d, "rwkv7_cuda_benchmark_state_passing.py"), "RWKV7_STATE_PASSING_CLAMPW_REF", env)
    y, sT = f(s, r, w, k, v, a, b)
    yy = y.detach().clone().requires_grad_(True)
    ss = sT.detach().clone().requires_grad_(True)
    # the harness's loss with a state term so that dsT != 0 (rwkv7_cuda_benchmark_state_passing.py:150-151)
    (strange_loss(yy) + 16 * (ss * ss + torch.tanh(ss)).sum()).backward()
    loss = strange_loss(y) + 16 * (sT * sT + torch.tanh(sT)).sum()
    g = grads(loss, s, r, w, k, v, a, b)
    save("wkv7_statepassing_clampw", H=H, s0=s, r=r, w=w, k=k, v=v, a=a, b=b, y=y, sT=sT,
         dy=yy.grad, dsT=ss.grad, ds0=g[0], dr=g[1], dw=g[2], dk=g[3], dv=g[4], da=g[5], db=g[6])


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("RWKV_CUDA_REF")
    if not ref:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/RWKV-CUDA   (or RWKV_CUDA_REF=...)")
    main(ref)
