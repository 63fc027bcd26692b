"""Backward pass over HOST (pinned) buffers, pipelined by (batch x KV-head) groups.

The groups of a GQA problem are independent (see :mod:`.sharding`), so the tensors are cut into chunks of
groups and three CUDA streams overlap the host->device copy of chunk i+1, the ``gqa_bwd`` call on chunk i
(through the C ABI, on its own stream) and the device->host copy of chunk i-1.  Staging buffers on the
device are allocated once per :class:`HostBackward` and double-buffered.

This is the path ``bench.py`` times as ``e2e``; with PCIe as the bottleneck the copies dominate
(270 MB per headline-shape step), so hiding the compute behind them is what matters.
"""
from __future__ import annotations

import math

import torch

from . import ops, sharding


class HostBackward:
    def __init__(self, B, Hq, Hkv, S, D, causal=False, scale=None, chunks=8, device=None, n_slots=2):
        self.shape = (B, Hq, Hkv, S, D)
        self.causal = bool(causal)
        self.scale = 1.0 / math.sqrt(D) if scale is None else float(scale)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        n_groups = B * Hkv
        n_chunks = max(1, min(int(chunks), n_groups))
        self.ranges = [sharding.group_range(c, n_chunks, n_groups) for c in range(n_chunks)]
        self.chunks = len(self.ranges)
        g_max = max(e - b for b, e in self.ranges)
        G = Hq // Hkv
        dev, bf, f32 = self.device, torch.bfloat16, torch.float32
        mk = lambda *s, dt=bf: torch.empty(s, dtype=dt, device=dev)
        # staging slots (two by default): inputs, outputs and a workspace each
        self.slots = [dict(q=mk(g_max, G, S, D), k=mk(g_max, 1, S, D), v=mk(g_max, 1, S, D), o=mk(g_max, G, S, D),
                           do=mk(g_max, G, S, D), lse=mk(g_max, G, S, dt=f32), dq=mk(g_max, G, S, D),
                           dk=mk(g_max, 1, S, D), dv=mk(g_max, 1, S, D),
                           ws=torch.empty(ops.bwd_workspace_bytes(g_max, G, 1, S, D, causal), dtype=torch.uint8,
                                          device=dev)) for _ in range(max(2, int(n_slots)))]
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
        self.h2d_bytes = (3 * B * Hq * S * D + 2 * B * Hkv * S * D) * 2 + B * Hq * S * 4
        self.d2h_bytes = (B * Hq * S * D + 2 * B * Hkv * S * D) * 2

    def __call__(self, q, k, v, o, do, lse, dq, dk, dv):
        """All arguments are pinned host tensors in the reference layout; dq/dk/dv are filled in.
        Returns after the last device->host copy has been enqueued; call ``synchronize()`` to wait."""
        B, Hq, Hkv, S, D = self.shape
        hin = [sharding.as_groups(t, Hkv) for t in (q, k, v, o, do, lse)]
        hout = [sharding.as_groups(t, Hkv) for t in (dq, dk, dv)]
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        copied = [torch.cuda.Event() for _ in self.ranges]
        computed = [torch.cuda.Event() for _ in self.ranges]
        drained = [torch.cuda.Event() for _ in self.ranges]
        for c, (b, e) in enumerate(self.ranges):
            ns = len(self.slots)
            slot, n = self.slots[c % ns], e - b
            with torch.cuda.stream(self.s_in):
                if c >= ns:
                    self.s_in.wait_event(computed[c - ns])   # the slot's inputs were consumed
                for name, h in zip(("q", "k", "v", "o", "do", "lse"), hin):
                    slot[name][:n].copy_(h[b:e], non_blocking=True)
                copied[c].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(copied[c])
                if c >= ns:
                    self.s_run.wait_event(drained[c - ns])   # the slot's outputs were copied out
                ops.gqa_backward(slot["q"][:n], slot["k"][:n], slot["v"][:n], slot["o"][:n], slot["do"][:n],
                                 slot["lse"][:n], causal=self.causal, scale=self.scale, workspace=slot["ws"],
                                 dq=slot["dq"][:n], dk=slot["dk"][:n], dv=slot["dv"][:n], stream=self.s_run)
                computed[c].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(computed[c])
                for name, h in zip(("dq", "dk", "dv"), hout):
                    h[b:e].copy_(slot[name][:n], non_blocking=True)
                drained[c].record(self.s_out)
        cur.wait_stream(self.s_out)

    def synchronize(self):
        """Wait for the last device->host copy, then raise if a bounded device-side wait gave up in any chunk."""
        self.s_out.synchronize()
        for slot in self.slots:
            ops.check_status(slot["ws"], stream=self.s_run)
