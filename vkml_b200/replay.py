"""Replays recorded backend traffic through the C ABI.

A *program* is the exact sequence of calls vkML's framework makes on a device
while it runs a model: allocations, uploads, `compute()` spans with their node
descriptors, batched device copies, downloads.  Programs are recorded once from
the real framework (by a `vkml::Backend` that logs instead of computing) and
stored with buffer references made relative -- ``["pro", j]`` is the j-th
allocation of the prologue, ``[d, j]`` the j-th allocation of the step ``d``
steps back (0 = this one) -- so the steady-state step is one template that can
be replayed any number of times, the way vkML plans to re-submit a cached
command buffer for an unchanged step (docs/ARCHITECTURE.md:565-569 there).

Replaying needs only this package and the CUDA library: every event becomes one
call on `vkml_b200.Backend`.
"""
from __future__ import annotations

import gzip
import json
from typing import Callable, Optional

import numpy as np

from .backend import COMPUTE_GRAD_SYNC, Backend, Storage
from .graph import DType, NodeDesc, TensorDesc, pack_nodes


def load_program(path: str) -> dict:
    opener = gzip.open if path.endswith(".gz") else open
    with opener(path, "rt") as f:
        return json.load(f)


class Replayer:
    """Executes a program's prologue once and its step templates on demand.

    `feed(tag, nbytes)` supplies the bytes of each upload: it is called with the
    upload's position (``("pro", i)`` or ``("step", i)``, i counting uploads inside the
    prologue / the current step) and must return a C-contiguous array of `nbytes`
    bytes, or None to leave the buffer as it is (timing runs).
    """

    def __init__(self, backend: Backend, program: dict, feed: Optional[Callable] = None,
                 grad_sync: bool = False):
        self.b = backend
        self.p = program
        self.feed = feed
        self.grad_sync = grad_sync
        self.pro: list = []          # prologue allocations
        self.history: list = []      # per-step allocation lists, newest last
        self.steps_run = 0
        self.downloads: list = []    # (step, array) for every d2h event
        self._packed_cache: dict = {}
        self._run_events(self.p["prologue"], self.pro, ("pro",))

    # -- buffer references ------------------------------------------------------
    def _resolve(self, ref, current: list) -> Storage:
        if ref is None:
            return None
        where, j = ref
        if where == "pro":
            return self.pro[j]
        if where == 0:
            return current[j]
        return self._back(where)[j]

    def _back(self, steps_back: int) -> list:
        """Allocation list of the step `steps_back` before the one running (which is history[-1])."""
        return self.history[len(self.history) - 1 - steps_back]

    def _tensor(self, t: dict, current: list) -> TensorDesc:
        st = self._resolve(t["buf"], current)
        addr = (st.data + t["off"]) if st is not None and st.data else 0
        return TensorDesc(addr, tuple(t["dims"]), tuple(t["strides"]), DType(t["dtype"]))

    # -- execution ----------------------------------------------------------------
    def _run_events(self, events: list, current: list, tag: tuple) -> None:
        b = self.b
        uploads = 0
        for ev in events:
            kind = ev["ev"]
            if kind == "alloc":
                current.append(b.allocate(ev["bytes"]))
            elif kind == "free":
                # the Storage object is dropped when its allocation list goes out of
                # scope; an explicit early release keeps peak memory at the recorded level
                where, j = ev["buf"]
                lst = self.pro if where == "pro" else (current if where == 0 else self._back(where))
                lst[j] = None
            elif kind == "h2d":
                data = self.feed(tag + (uploads,), ev["bytes"]) if self.feed else None
                uploads += 1
                if data is not None:
                    st = self._resolve(ev["buf"], current)
                    b.copy_from_host(st, ev["off"], np.ascontiguousarray(data).view(np.uint8).reshape(-1),
                                     ev["bytes"])
            elif kind == "compute":
                nodes = [NodeDesc(n["op"], self._tensor(n["out"], current),
                                  [self._tensor(s, current) for s in n["src"]], bytes.fromhex(n["params"]))
                         for n in ev["nodes"]]
                flags = COMPUTE_GRAD_SYNC if (self.grad_sync and ev.get("grad_sync")) else 0
                b.compute_packed(pack_nodes(nodes), len(nodes), flags)
            elif kind == "d2d":
                b.copy_device_to_device([(self._resolve(d, current), doff, self._resolve(s, current), soff, n)
                                         for d, doff, s, soff, n in ev["copies"]])
            elif kind == "d2h":
                out = np.empty(ev["bytes"], dtype=np.uint8)
                b.copy_to_host(out, self._resolve(ev["buf"], current), ev["off"], ev["bytes"])
                self.downloads.append((self.steps_run, out))
            elif kind == "sync":
                b.synchronize()

    def step(self) -> None:
        """Run the next training step: the recorded first steps in order, then the
        steady-state template for every step after them."""
        templates = self.p["steps"]
        template = templates[min(self.steps_run, len(templates) - 1)]
        current: list = []
        self.history.append(current)
        self._run_events(template, current, ("step",))
        # allocations older than the program ever reaches back can go
        keep = self.p.get("lookback", 1) + 1
        if len(self.history) > keep:
            del self.history[: len(self.history) - keep]
        self.steps_run += 1
