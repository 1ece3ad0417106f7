"""Host-buffer front end: run an element-wise operator over pinned host arrays in chunks, overlapping the
host-to-device copy, the kernel and the device-to-host copy of neighbouring chunks on three streams.

This is the call a user with data in host memory makes; the PCIe link is full duplex, so with the two copy
directions on separate streams the cost per element approaches max(H2D, D2H) instead of their sum.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


def bind_host_thread_to_device_node(device_index: int) -> str | None:
    """Restrict the calling thread to the CPUs of the NUMA node the GPU hangs off, so that the pinned buffers it
    allocates next land in memory local to that GPU's PCIe root (first touch).  With one process per GPU on a two-socket
    host this keeps half of the copies off the socket interconnect.  Returns a short description, or None when the
    topology cannot be read or the node's CPUs are not available to this process (then nothing is changed)."""
    import os
    try:
        props = torch.cuda.get_device_properties(device_index)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as fh:
            node = int(fh.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as fh:
            cpus: set[int] = set()
            for part in fh.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return f"numa node {node}, {len(allowed)} cpus"
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None


class HostPipeline:
    """Double-buffered chunk pipeline for operators of the form outs = fn(*ins) on flat tensors.

    ``in_specs`` / ``out_specs``: (dtype, elements per work item) for every input / output array; an array
    holds ``items * per_item`` elements and a chunk covers ``chunk_items`` items of every array.
    """

    def __init__(self, device: torch.device, in_specs: Sequence[tuple[torch.dtype, int]],
                 out_specs: Sequence[tuple[torch.dtype, int]], chunk_items: int, depth: int = 3):
        self.device = device
        self.chunk_items = int(chunk_items)
        self.depth = depth
        self.in_specs, self.out_specs = list(in_specs), list(out_specs)
        self.h2d, self.d2h = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self.compute = torch.cuda.Stream(device)
        self.slots = []
        for _ in range(depth):
            ins = [torch.empty(self.chunk_items * per, dtype=dt, device=device) for dt, per in self.in_specs]
            outs = [torch.empty(self.chunk_items * per, dtype=dt, device=device) for dt, per in self.out_specs]
            self.slots.append((ins, outs, torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()))

    def run(self, fn: Callable[[list[torch.Tensor], list[torch.Tensor], int], None],
            host_ins: Sequence[torch.Tensor], host_outs: Sequence[torch.Tensor], items: int) -> int:
        """fn(device_ins, device_outs, n_items) must enqueue on the current stream.  Returns kernel launches."""
        launches = 0
        n_chunks = (items + self.chunk_items - 1) // self.chunk_items
        for c in range(n_chunks):
            ins, outs, copied_in, computed, copied_out = self.slots[c % self.depth]
            lo = c * self.chunk_items
            n = min(self.chunk_items, items - lo)
            with torch.cuda.stream(self.h2d):
                self.h2d.wait_event(computed)      # previous use of this slot's inputs has been consumed
                for dev, host, (_, per) in zip(ins, host_ins, self.in_specs):
                    dev[: n * per].copy_(host[lo * per:(lo + n) * per], non_blocking=True)
                copied_in.record(self.h2d)
            with torch.cuda.stream(self.compute):
                self.compute.wait_event(copied_in)
                self.compute.wait_event(copied_out)  # previous result of this slot has left the device
                fn([t[: n * per] for t, (_, per) in zip(ins, self.in_specs)],
                   [t[: n * per] for t, (_, per) in zip(outs, self.out_specs)], n)
                launches += 1
                computed.record(self.compute)
            with torch.cuda.stream(self.d2h):
                self.d2h.wait_event(computed)
                for dev, host, (_, per) in zip(outs, host_outs, self.out_specs):
                    host[lo * per:(lo + n) * per].copy_(dev[: n * per], non_blocking=True)
                copied_out.record(self.d2h)
        return launches

    def synchronize(self) -> None:
        self.h2d.synchronize()
        self.compute.synchronize()
        self.d2h.synchronize()
