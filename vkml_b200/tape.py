"""Native replay of a recorded program: the step tape.

`replay.Replayer` turns every recorded event into one Python call on the backend, which
costs a scripting language's overhead per node.  A `Tape` encodes the same program once
into flat 64-bit words (format: vkml_b200/csrc/tape.cu) and lets the library issue the
calls itself, so a replayed step costs on the host what the same calls cost from vkML's
C++ executor.  Same events, same order, same bytes: tests/test_training_gpu.py checks the
two replays against each other.
"""
from __future__ import annotations

import ctypes as C
import struct
from typing import Optional, Sequence

import numpy as np

from . import _abi
from .backend import COMPUTE_GRAD_SYNC, Backend

_EV = {"alloc": 1, "free": 2, "h2d": 3, "compute": 4, "d2d": 5, "d2h": 6, "sync": 7}


def _ref(ref) -> tuple:
    if ref is None:
        return (-2, 0)
    where, j = ref
    return (-1 if where == "pro" else int(where), int(j))


def _tensor(t: dict) -> list:
    dims = list(t["dims"])
    strides = list(t["strides"])
    nd = len(dims)
    assert nd <= 4 and len(strides) == nd
    return [*_ref(t["buf"]), int(t["off"]), int(t["dtype"]), nd, *(dims + [0] * (4 - nd)),
            *(strides + [0] * (4 - nd))]


def encode(events: list) -> tuple:
    """One template's events as int64 words; also the number of uploads and the byte
    sizes of its downloads, in order."""
    words: list = []
    uploads = 0
    downloads: list = []
    for ev in events:
        kind = ev["ev"]
        words.append(_EV[kind])
        if kind == "alloc":
            words.append(int(ev["bytes"]))
        elif kind == "free":
            words.extend(_ref(ev["buf"]))
        elif kind == "h2d":
            words.extend([*_ref(ev["buf"]), int(ev["off"]), int(ev["bytes"]), uploads])
            uploads += 1
        elif kind == "compute":
            words.extend([len(ev["nodes"]), 1 if ev.get("grad_sync") else 0])
            for n in ev["nodes"]:
                params = bytes.fromhex(n["params"]).ljust(64, b"\0")
                assert len(params) == 64
                words.extend([int(n["op"]), len(n["src"]), *struct.unpack("<8q", params)])
                words.extend(_tensor(n["out"]))
                for s in n["src"]:
                    words.extend(_tensor(s))
        elif kind == "d2d":
            words.append(len(ev["copies"]))
            for d, doff, s, soff, n in ev["copies"]:
                words.extend([*_ref(d), int(doff), *_ref(s), int(soff), int(n)])
        elif kind == "d2h":
            words.extend([*_ref(ev["buf"]), int(ev["off"]), int(ev["bytes"]), len(downloads)])
            downloads.append(int(ev["bytes"]))
    return np.asarray(words, dtype=np.int64), uploads, downloads


class Tape:
    """A program on the library's native replayer.

    `run_prologue(uploads)` once, then `step(uploads)` per training step; `uploads` are host
    addresses (ints, e.g. of pinned buffers) or arrays, one per upload of the template, None to
    skip one.  Downloads land in `self.downloads[i]` (numpy uint8 arrays, reused every step).
    """

    def __init__(self, backend: Backend, program: dict, grad_sync: bool = False):
        self.b = backend
        self._lib = backend._lib
        self.grad_flags = COMPUTE_GRAD_SYNC if grad_sync else 0
        handle = C.c_void_p()
        backend._check(self._lib.b200_tape_create(backend._ctx, int(program.get("lookback", 1)), C.byref(handle)),
                       "tape_create")
        self._tape = handle
        self._templates = []
        self._keep = []
        for events, is_pro in [(program["prologue"], 1)] + [(s, 0) for s in program["steps"]]:
            words, n_up, down = encode(events)
            idx = C.c_int()
            backend._check(self._lib.b200_tape_add_template(
                self._tape, words.ctypes.data_as(C.POINTER(C.c_int64)), words.size, is_pro, C.byref(idx)),
                "tape_add_template")
            bufs = [np.zeros(n, dtype=np.uint8) for n in down]
            ptrs = (C.c_void_p * max(1, len(bufs)))(*[b.ctypes.data for b in bufs])
            self._templates.append((idx.value, n_up, bufs, ptrs))
        self.n_step_templates = len(program["steps"])
        self.steps_run = 0
        self.downloads: list = []

    def _run(self, t: int, uploads: Optional[Sequence]) -> None:
        idx, n_up, bufs, down_ptrs = self._templates[t]
        ups = list(uploads) if uploads is not None else []
        ups += [None] * (n_up - len(ups))
        keep = []
        addrs = []
        for u in ups[:n_up]:
            if u is None:
                addrs.append(None)
            elif isinstance(u, int):
                addrs.append(u)
            else:
                a = np.ascontiguousarray(u)
                keep.append(a)
                addrs.append(a.ctypes.data)
        up_ptrs = (C.c_void_p * max(1, n_up))(*addrs)
        self.b._check(self._lib.b200_tape_run(self._tape, idx, up_ptrs, n_up, down_ptrs, len(bufs), self.grad_flags),
                      "tape_run")
        self.downloads = bufs

    def upload_ptrs(self, t: int, uploads: Sequence):
        """Pre-built pointer array for `step_fast`: addresses only (ints or None)."""
        _, n_up, _, _ = self._templates[t]
        return (C.c_void_p * max(1, n_up))(*list(uploads)[:n_up])

    def run_prologue(self, uploads: Optional[Sequence] = None) -> None:
        self._run(0, uploads)

    def template_for_step(self, step: int) -> int:
        return 1 + min(step, self.n_step_templates - 1)

    def step(self, uploads: Optional[Sequence] = None) -> None:
        self._run(self.template_for_step(self.steps_run), uploads)
        self.steps_run += 1

    def step_fast(self, up_ptrs) -> None:
        """A steady-state step with a pointer array from `upload_ptrs`: one foreign call."""
        idx, n_up, bufs, down_ptrs = self._templates[self.n_step_templates]
        rc = self._lib.b200_tape_run(self._tape, idx, up_ptrs, n_up, down_ptrs, len(bufs), self.grad_flags)
        if rc != 0:
            self.b._check(rc, "tape_run")
        self.downloads = bufs
        self.steps_run += 1

    def enable_graphs(self, on: bool = True) -> None:
        """Replay steady-state steps as captured CUDA graphs (see b200_tape_enable_graphs)."""
        self.b._check(self._lib.b200_tape_enable_graphs(self._tape, 1 if on else 0), "tape_enable_graphs")

    def stats(self) -> dict:
        steps, launches, captures = C.c_uint64(), C.c_uint64(), C.c_uint64()
        self.b._check(self._lib.b200_tape_stats(self._tape, C.byref(steps), C.byref(launches), C.byref(captures)),
                      "tape_stats")
        return {"steps": steps.value, "graph_launches": launches.value, "graph_captures": captures.value}

    def close(self) -> None:
        if self._tape:
            self._lib.b200_tape_destroy(self._tape)
            self._tape = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
