"""Host-buffer front end of the RWKV-7 state-passing operator.

`Wkv7HostPipeline.forward_backward(...)` takes every operand in pinned HOST memory and leaves
every result in pinned host memory.  The batch is cut into slices that stream through the GPU
on three CUDA streams (host->device copies, kernels, device->host copies), so the two copy
directions of the PCIe link and the kernels overlap; device memory holds three slices at a time,
whatever the batch size.  Units (batch, head) are independent, so slicing does not change results.
"""
import contextlib
import os

import torch

from . import ops


def gpu_numa_node(device):
    """NUMA node of the host that the GPU hangs off (from sysfs, by the GPU's PCI address), or None when
    the platform does not say (one node, a container without sysfs, no NVML)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        idx = torch.device(device).index or 0
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ent = vis.split(",")[idx].strip()
            h = pynvml.nvmlDeviceGetHandleByUUID(ent) if ent.startswith("GPU-") else pynvml.nvmlDeviceGetHandleByIndex(int(ent))
        else:
            h = pynvml.nvmlDeviceGetHandleByIndex(idx)
        bus = pynvml.nvmlDeviceGetPciInfo(h).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        bus = bus.lower()
        if len(bus.split(":")[0]) == 8:          # NVML prints an 8-digit domain, sysfs uses 4
            bus = bus[4:]
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read())
        return node if node >= 0 else None
    except Exception:
        return None


@contextlib.contextmanager
def host_memory_near(device):
    """Runs the body with the calling thread bound to the CPUs of the GPU's NUMA node, so that pinned host
    buffers allocated inside come from memory next to the GPU's PCIe root (with several GPUs per host, buffers
    that all sit on one node send the other socket's traffic across the inter-socket link).  Yields the node,
    or None when nothing was bound; the previous affinity is restored afterwards."""
    node, old = gpu_numa_node(device), None
    try:
        if node is not None:
            cpus = set()
            for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
            old = os.sched_getaffinity(0)
            if cpus & old:
                os.sched_setaffinity(0, cpus & old)
            else:
                node, old = None, None
    except Exception:
        node, old = None, None
    try:
        yield node
    finally:
        if old is not None:
            os.sched_setaffinity(0, old)


class Wkv7HostPipeline:
    IN = ("r", "w", "k", "v", "a", "b", "dy")
    OUT = ("y", "dr", "dw", "dk", "dv", "da", "db")

    def __init__(self, T, H, N, device, slice_batch=1, depth=3, dtype=torch.bfloat16, chunk_len=16):
        self.T, self.H, self.N, self.sb, self.depth = T, H, N, slice_batch, depth
        self.dev = torch.device(device)
        self.h2d, self.comp, self.d2h = (torch.cuda.Stream(self.dev) for _ in range(3))
        big = lambda: torch.empty(slice_batch, T, H, N, dtype=dtype, device=self.dev)
        st = lambda: torch.empty(slice_batch, H, N, N, dtype=torch.float32, device=self.dev)
        self.sets = []
        for _ in range(depth):
            d = {n: big() for n in self.IN + self.OUT}
            d.update(s0=st(), dsT=st(), sT=st(), ds0=st())
            d["s"] = torch.empty(slice_batch, H, T // chunk_len, N, N, dtype=torch.float32, device=self.dev)
            d["sa"] = torch.empty(slice_batch, T, H, N, dtype=torch.float32, device=self.dev)
            d["free"] = None   # event: the device->host copies that last used this set
            self.sets.append(d)

    def forward_backward(self, host_in, host_out):
        """host_in: r,w,k,v,a,b,dy (B,T,H,N) and s0,dsT (B,H,N,N); host_out: y,dr,dw,dk,dv,da,db and sT,ds0.
        All pinned CPU tensors.  Returns after everything has been enqueued; call `synchronize()`
        (or wait on the returned event) before reading host_out."""
        B = host_in["r"].shape[0]
        cur = torch.cuda.current_stream(self.dev)
        for st in (self.h2d, self.comp, self.d2h):
            st.wait_stream(cur)
        n = 0
        for lo in range(0, B, self.sb):
            hi = min(lo + self.sb, B)
            m = hi - lo
            d = self.sets[n % self.depth]
            n += 1
            with torch.cuda.stream(self.h2d):
                if d["free"] is not None:
                    self.h2d.wait_event(d["free"])
                for name in self.IN + ("s0", "dsT"):
                    d[name][:m].copy_(host_in[name][lo:hi], non_blocking=True)
                ev_in = self.h2d.record_event()
            with torch.cuda.stream(self.comp):
                self.comp.wait_event(ev_in)
                v = {k_: t[:m] for k_, t in d.items() if isinstance(t, torch.Tensor)}
                ops.wkv7_forward(v["s0"], v["r"], v["w"], v["k"], v["v"], v["a"], v["b"], v["y"], v["sT"], v["s"], v["sa"])
                ops.wkv7_backward(v["r"], v["w"], v["k"], v["v"], v["a"], v["b"], v["dy"], v["dsT"], v["s"], v["sa"],
                                  v["ds0"], v["dr"], v["dw"], v["dk"], v["dv"], v["da"], v["db"])
                ev_done = self.comp.record_event()
            with torch.cuda.stream(self.d2h):
                self.d2h.wait_event(ev_done)
                for name in self.OUT + ("sT", "ds0"):
                    host_out[name][lo:hi].copy_(d[name][:m], non_blocking=True)
                d["free"] = self.d2h.record_event()
        done = self.d2h.record_event()
        cur.wait_event(done)
        return done

    def synchronize(self):
        """Waits for the last forward_backward and checks the device status word: a bounded wait that
        ran out inside a kernel leaves invalid results, which must not pass silently."""
        self.d2h.synchronize()
        from . import _lib
        st = _lib.lib().rwkvb200_device_status()
        if st != 0:
            raise _lib.RwkvB200Error(f"device status {st}: a bounded wait ran out inside a tensor-core kernel; results are invalid "
                                     "(rwkvb200_device_status_clear resets the word)")
