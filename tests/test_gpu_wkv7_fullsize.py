"""RWKV-7 tensor-core kernels at the size that is benchmarked (B16 T4096 H64: 1024 thread blocks, several
waves, three / two blocks per SM sharing tensor memory), and state passing over many segments.

The fp64 oracle is run on a few (batch, head) units only: units are independent, so a unit of the full
launch must equal the oracle on that unit's inputs."""
import pytest
import torch

from oracle import wkv_oracle as O
from tests import helpers as Hh
from tests import ref_kernel

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16
NAMES = ("r", "w", "k", "v", "a", "b", "dy")


def _device_inputs(B, T, H, N, seed):
    """Benchmark distributions, drawn on the device (the full batch on the CPU would take minutes)."""
    g = torch.Generator(device=DEV)
    g.manual_seed(seed)
    mk = lambda sc=1.0: torch.randn(B, T, H, N, generator=g, device=DEV) * sc
    r, k, v, w = mk(0.5), mk(0.5), mk(0.5), mk()
    kk = torch.nn.functional.normalize(mk(), dim=-1)
    a, b, dy = -kk, kk * torch.sigmoid(mk()), mk()
    d = {n: x.to(BF) for n, x in zip(NAMES, (r, w, k, v, a, b, dy))}
    d["s0"] = 0.1 * torch.randn(B, H, N, N, generator=g, device=DEV)
    d["dsT"] = torch.randn(B, H, N, N, generator=g, device=DEV)
    return d


def _run(R, d, fwd=None, bwd=None):
    fwd, bwd = fwd or R.ops.wkv7_forward, bwd or R.ops.wkv7_backward
    B, T, H, N = d["r"].shape
    y = torch.empty(B, T, H, N, dtype=BF, device=DEV)
    sT, ds0 = torch.empty_like(d["s0"]), torch.empty_like(d["s0"])
    s = torch.empty(B, H, T // 16, N, N, device=DEV)
    sa = torch.empty(B, T, H, N, device=DEV)
    fwd(d["s0"], d["r"], d["w"], d["k"], d["v"], d["a"], d["b"], y, sT, s, sa)
    g = [torch.empty_like(y) for _ in range(6)]
    bwd(d["r"], d["w"], d["k"], d["v"], d["a"], d["b"], d["dy"], d["dsT"], s, sa, ds0, *g)
    torch.cuda.synchronize()
    return dict(y=y, sT=sT, ds0=ds0, **dict(zip(("dr", "dw", "dk", "dv", "da", "db"), g)))


def _oracle_unit(d, b, h):
    """fp64 oracle on unit (b, h) of device inputs d: dict of (1,T,N) / (1,1,N,N) tensors."""
    inp64 = {n: d[n][b : b + 1, :, h].double().cpu().contiguous() for n in NAMES}
    inp64["s0"] = d["s0"][b : b + 1, h : h + 1].double().cpu()
    inp64["dsT"] = d["dsT"][b : b + 1, h : h + 1].double().cpu()
    return Hh.v7_oracle(inp64, 1)


def test_benchmark_size_units_against_oracle():
    import rwkv_cuda_b200 as R
    from rwkv_cuda_b200 import _lib
    B, T, H, N = 16, 4096, 64, 64
    d = _device_inputs(B, T, H, N, seed=42)
    out = _run(R, d)
    assert _lib.lib().rwkvb200_device_status() == 0
    for t in out.values():
        assert torch.isfinite(t).all()
    rep = []
    for b, h in [(0, 0), (6, 21), (15, 63)]:   # first, one in a middle wave, last
        want = _oracle_unit(d, b, h)
        for n in ("y", "dr", "dw", "dk", "dv", "da", "db"):
            m, e = Hh.assert_close(out[n][b, :, h], want[n].view(T, N), Hh.TOL_BF16, f"{n} of unit ({b},{h})")
            rep.append(f"({b},{h}) {n}: rms {e:.2e}")
        for n in ("sT", "ds0"):
            m, e = Hh.assert_close(out[n][b, h], want[n].view(N, N), Hh.TOL_BF16, f"{n} of unit ({b},{h})")
            rep.append(f"({b},{h}) {n}: rms {e:.2e}")
    print("\n".join(rep))


@pytest.mark.parametrize("nseg,Tseg", [(16, 256)])
def test_state_passing_over_many_segments(nseg, Tseg):
    """A sequence processed segment by segment (sT -> s0 forwards, ds0 -> dsT backwards) against ONE fp64
    pass over the whole sequence: the error of the carried state must not grow beyond the tolerance, and
    the drift per segment is printed next to the reference kernel's where that one is built."""
    import rwkv_cuda_b200 as R
    B, H, N = 1, 2, 64
    T = nseg * Tseg
    d = _device_inputs(B, T, H, N, seed=7)
    want = {}
    for h in range(H):
        w = _oracle_unit(d, 0, h)
        for n, x in w.items():
            want.setdefault(n, []).append(x)
    want_sT = torch.stack([x.view(N, N) for x in want["sT"]])
    want_ds0 = torch.stack([x.view(N, N) for x in want["ds0"]])
    # fp64 states at the segment boundaries, for the drift report
    bounds = []
    for h in range(H):
        xs = [d[n][0:1, :, h].double().cpu() for n in ("r", "w", "k", "v", "a", "b")]
        st = d["s0"][0:1, h : h + 1].double().cpu()
        per = []
        for sg in range(nseg):
            sl = slice(sg * Tseg, (sg + 1) * Tseg)
            _, st = O.wkv7(*[x[:, sl] for x in xs], 1, s0=st)
            per.append(st.view(N, N))
        bounds.append(per)

    def chain(fwd, bwd):
        seg = lambda x, sg: x[:, sg * Tseg : (sg + 1) * Tseg].contiguous()
        states, saved = [d["s0"]], []
        ys = []
        for sg in range(nseg):
            y = torch.empty(B, Tseg, H, N, dtype=BF, device=DEV)
            sT = torch.empty_like(d["s0"])
            s = torch.empty(B, H, Tseg // 16, N, N, device=DEV)
            sa = torch.empty(B, Tseg, H, N, device=DEV)
            fwd(states[-1], *(seg(d[n], sg) for n in ("r", "w", "k", "v", "a", "b")), y, sT, s, sa)
            states.append(sT)
            saved.append((s, sa))
            ys.append(y)
        dstate = d["dsT"]
        grads = [None] * nseg
        for sg in reversed(range(nseg)):
            ds0 = torch.empty_like(d["s0"])
            g = [torch.empty(B, Tseg, H, N, dtype=BF, device=DEV) for _ in range(6)]
            bwd(*(seg(d[n], sg) for n in ("r", "w", "k", "v", "a", "b")), seg(d["dy"], sg), dstate, *saved[sg], ds0, *g)
            dstate = ds0
            grads[sg] = g
        torch.cuda.synchronize()
        out = {"y": torch.cat(ys, 1), "sT": states[-1], "ds0": dstate, "states": states[1:]}
        for i, n in enumerate(("dr", "dw", "dk", "dv", "da", "db")):
            out[n] = torch.cat([g[i] for g in grads], 1)
        return out

    ours = chain(R.ops.wkv7_forward, R.ops.wkv7_backward)
    ref = chain(ref_kernel.forward, ref_kernel.backward) if ref_kernel.available() else None
    drift = []
    for sg in range(nseg):
        w64 = torch.stack([bounds[h][sg] for h in range(H)])
        line = f"after segment {sg + 1:2d}: state rms error ours {O.err_ratio(w64, ours['states'][sg][0].double().cpu()):.2e}"
        if ref is not None:
            line += f"   reference kernel {O.err_ratio(w64, ref['states'][sg][0].double().cpu()):.2e}"
        drift.append(line)
    print("\n".join(drift))
    Hh.assert_close(ours["sT"][0], want_sT, Hh.TOL_BF16, "final state")
    Hh.assert_close(ours["ds0"][0], want_ds0, Hh.TOL_BF16, "gradient of the initial state")
    # the state error stays at the single-segment level (about 2e-4): no growth with the number of segments
    assert O.err_ratio(want_sT, ours["sT"][0].double().cpu()) < 1e-3
    for n in ("y", "dr", "dw", "dk", "dv", "da", "db"):
        w64 = torch.stack([x.view(T, N) for x in want[n]], 1)   # (T, H, N)
        Hh.assert_close(ours[n][0], w64, Hh.TOL_BF16, n)


def test_batch_shards_equal_the_whole_batch():
    """Sharding by batch (what every rank of a multi-GPU run does) does not change a single bit: the rows
    computed from a slice of the batch equal those rows of the whole-batch run.  With two devices the
    second shard runs on the second device."""
    import rwkv_cuda_b200 as R
    B, T, H, N = 4, 128, 8, 64
    d = _device_inputs(B, T, H, N, seed=3)
    whole = _run(R, d)
    ndev = torch.cuda.device_count()
    for shard, lo in enumerate((0, 2)):
        dev = torch.device("cuda", shard % ndev)
        with torch.cuda.device(dev):
            part = {n: x[lo : lo + 2].to(dev).contiguous() for n, x in d.items()}
            B2 = 2
            y = torch.empty(B2, T, H, N, dtype=BF, device=dev)
            sT, ds0 = torch.empty_like(part["s0"]), torch.empty_like(part["s0"])
            s = torch.empty(B2, H, T // 16, N, N, device=dev)
            sa = torch.empty(B2, T, H, N, device=dev)
            R.ops.wkv7_forward(part["s0"], *(part[n] for n in ("r", "w", "k", "v", "a", "b")), y, sT, s, sa)
            g = [torch.empty_like(y) for _ in range(6)]
            R.ops.wkv7_backward(*(part[n] for n in ("r", "w", "k", "v", "a", "b")), part["dy"], part["dsT"], s, sa, ds0, *g)
            torch.cuda.synchronize(dev)
            got = dict(y=y, sT=sT, ds0=ds0, **dict(zip(("dr", "dw", "dk", "dv", "da", "db"), g)))
        for n, x in got.items():
            assert torch.equal(x.cpu(), whole[n][lo : lo + 2].cpu()), n
