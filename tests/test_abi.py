"""The C-ABI library loads without a GPU, exports every symbol the header
declares, answers `supports()` honestly, and refuses to run without a device
(there is no CPU fallback)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import vkml_b200
from vkml_b200 import _abi, graph
from vkml_b200.graph import DType, NodeDesc, Op, TensorDesc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "vkml_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _abi.load()
    names = declared_functions()
    assert len(names) >= 25
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in vkml_b200.h but not exported"
    # and the Python binding table covers the same set
    assert sorted(_abi.SYMBOLS) == names


def test_struct_layouts_match_the_header():
    assert C.sizeof(_abi.Tensor) == 8 + 32 + 32 + 4 + 4
    assert C.sizeof(_abi.Node) == 8 + 80 + 4 * 80 + 64
    assert C.sizeof(_abi.Copy) == 24
    assert _abi.load().b200_abi_version() == 1


def test_op_numbering_matches_vkml():
    # spot values of vkml::OpKind (include/vkml/graph/op.h:30-139)
    assert Op.INPUT == 0 and Op.FULL == 2 and Op.CONTIGUOUS == 11 and Op.SCALED_ADD == 17
    assert Op.NEG == 28 and Op.CLAMP == 46 and Op.SUM == 47 and Op.MATMUL == 54
    assert Op.LOG_SOFTMAX == 56 and Op.SLICE_BACKWARD == 63 and Op.TRIL == 66 and graph.OP_COUNT == 67
    assert [int(d) for d in DType] == [0, 1, 2, 3, 4]


def _node(op, out_dt, src_dts, shape=(4, 4), params=b""):
    srcs = [TensorDesc.contiguous(0x1000, shape, dt) for dt in src_dts]
    return NodeDesc(int(op), TensorDesc.contiguous(0x2000, shape, out_dt), srcs, params)


def test_supports_is_honest():
    lib = _abi.load()

    def sup(node):
        c = node.to_c()
        return bool(lib.b200_supports(C.byref(c)))

    assert sup(_node(Op.ADD, DType.F32, [DType.F32, DType.F32]))
    assert sup(_node(Op.RESHAPE, DType.F32, [DType.F32]))            # views and leaves always
    assert sup(_node(Op.INPUT, DType.F16, []))
    # F16 is a storage dtype: floating operands and result of one dtype (vulkan_backend.cpp:1055-1184)
    assert sup(_node(Op.ADD, DType.F16, [DType.F16, DType.F16]))
    assert not sup(_node(Op.ADD, DType.F16, [DType.F16, DType.F32]))
    assert not sup(_node(Op.ADD, DType.F32, [DType.F16, DType.F16]))
    assert sup(_node(Op.LESS, DType.BOOL, [DType.F16, DType.F16]))
    assert sup(_node(Op.ARGMAX, DType.I64, [DType.F16]))
    assert sup(_node(Op.SOFTMAX, DType.F16, [DType.F16]))
    assert sup(_node(Op.MATMUL, DType.F16, [DType.F16, DType.F16], shape=(1, 1, 4, 4)))
    assert sup(_node(Op.PROD, DType.F16, [DType.F16]))
    assert not sup(_node(Op.RAND, DType.F16, []))
    assert sup(_node(Op.PROD, DType.F32, [DType.F32]))                # in index order, as on the CPU
    assert sup(_node(Op.EQUAL, DType.BOOL, [DType.F32, DType.F32]))
    assert not sup(_node(Op.EQUAL, DType.F32, [DType.F32, DType.F32]))
    assert sup(_node(Op.ARGMAX, DType.I64, [DType.F32]))
    assert not sup(_node(Op.ARGMAX, DType.F32, [DType.F32]))
    assert sup(_node(Op.CAST, DType.I64, [DType.BOOL]))
    assert not sup(_node(Op.CAST, DType.F16, [DType.I64]))
    assert sup(_node(Op.MATMUL, DType.F32, [DType.F32, DType.F32], shape=(1, 1, 4, 4)))
    assert not sup(_node(Op.MATMUL, DType.F32, [DType.F32, DType.F32], shape=(4, 4)))  # rank-4 only
    # a strided OUTPUT is never legal: computed nodes are dense (src/dispatch/executor.cpp:40-45)
    n = _node(Op.RELU, DType.F32, [DType.F32])
    n.out = TensorDesc(0x2000, (4, 4), (4, 16), DType.F32)
    assert not sup(n)
    bad = _node(Op.ADD, DType.F32, [DType.F32, DType.F32])
    bad.op = 999
    assert not sup(bad)


def test_status_names():
    lib = _abi.load()
    assert lib.b200_status_name(0) == b"ok"
    assert lib.b200_status_name(4) == b"index error"
    assert lib.b200_status_name(7) == b"out of memory"


def test_null_arguments_are_rejected_not_dereferenced():
    lib = _abi.load()
    assert lib.b200_device_count(None) == 8
    assert lib.b200_create(0, None) == 8
    assert lib.b200_get_caps(None, None) == 8
    assert lib.b200_compute(None, None, 0, 0) == 8
    assert lib.b200_synchronize(None) == 8
    assert lib.b200_last_error(None) == b""
    lib.b200_destroy(None)


def test_no_device_means_an_error_not_a_fallback():
    lib = _abi.load()
    n = C.c_int(-1)
    rc = lib.b200_device_count(C.byref(n))
    if rc == 0 and n.value > 0:
        pytest.skip("a CUDA device is present")
    with pytest.raises(vkml_b200.DeviceError):
        vkml_b200.Backend(0)


def test_param_packing_matches_the_cxx_structs():
    assert graph.reduce_params([1], 2, True) == b"\x02\x00\x00\x00\x01"
    assert len(graph.slice_params(1, 2, 10, 2)) == 32
    assert graph.slice_params(1, 2, 10, 2)[8:16] == (2).to_bytes(8, "little")
    assert len(graph.unfold_params((3, 3), (1, 1), (1, 1), (1, 1), (8, 8))) == 40
    assert graph.clamp_params(None, 1.0)[8:10] == b"\x00\x01"
    assert np.frombuffer(graph.scaled_add_params(0.9, -0.1), dtype=np.float32).tolist() == [
        np.float32(0.9), np.float32(-0.1)]


def test_tape_encoding_round_trips():
    """vkml_b200.tape.encode against an independent decoder of the documented word format:
    every recorded program decodes back to its own events."""
    import glob
    import os
    import struct
    from vkml_b200.replay import load_program
    from vkml_b200.tape import encode

    def ref(w, i):
        where, j = int(w[i]), int(w[i + 1])
        return (None if where == -2 else ["pro" if where == -1 else where, j]), i + 2

    def tensor(w, i):
        buf, i = ref(w, i)
        off, dtype, nd = int(w[i]), int(w[i + 1]), int(w[i + 2])
        dims = [int(v) for v in w[i + 3:i + 3 + nd]]
        strides = [int(v) for v in w[i + 7:i + 7 + nd]]
        return {"buf": buf, "off": off, "dtype": dtype, "dims": dims, "strides": strides}, i + 11

    def decode(w):
        out, i = [], 0
        while i < len(w):
            ev = int(w[i]); i += 1
            if ev == 1:
                out.append({"ev": "alloc", "bytes": int(w[i])}); i += 1
            elif ev == 2:
                buf, i = ref(w, i); out.append({"ev": "free", "buf": buf})
            elif ev in (3, 6):
                buf, i = ref(w, i)
                out.append({"ev": "h2d" if ev == 3 else "d2h", "buf": buf, "off": int(w[i]), "bytes": int(w[i + 1])})
                i += 3
            elif ev == 4:
                n, gs = int(w[i]), int(w[i + 1]); i += 2
                nodes = []
                for _ in range(n):
                    op, n_src = int(w[i]), int(w[i + 1])
                    params = struct.pack("<8q", *[int(v) for v in w[i + 2:i + 10]])
                    i += 10
                    o, i = tensor(w, i)
                    srcs = []
                    for _ in range(n_src):
                        t, i = tensor(w, i); srcs.append(t)
                    nodes.append({"op": op, "params": params, "out": o, "src": srcs})
                out.append({"ev": "compute", "grad_sync": bool(gs), "nodes": nodes})
            elif ev == 5:
                n = int(w[i]); i += 1
                copies = []
                for _ in range(n):
                    d, i = ref(w, i); doff = int(w[i]); i += 1
                    s, i = ref(w, i); soff, nb = int(w[i]), int(w[i + 1]); i += 2
                    copies.append([d, doff, s, soff, nb])
                out.append({"ev": "d2d", "copies": copies})
            elif ev == 7:
                out.append({"ev": "sync"})
            else:
                raise AssertionError(ev)
        return out

    here = os.path.dirname(os.path.abspath(__file__))
    paths = sorted(glob.glob(os.path.join(here, "golden", "programs", "*.json.gz")))
    assert paths
    for path in paths:
        program = load_program(path)
        for events in [program["prologue"]] + program["steps"]:
            words, n_up, downs = encode(events)
            got = decode(words)
            assert len(got) == len(events)
            assert n_up == sum(e["ev"] == "h2d" for e in events)
            assert downs == [e["bytes"] for e in events if e["ev"] == "d2h"]
            for g, e in zip(got, events):
                assert g["ev"] == e["ev"]
                if e["ev"] == "compute":
                    assert g["grad_sync"] == bool(e.get("grad_sync")) and len(g["nodes"]) == len(e["nodes"])
                    for gn, en in zip(g["nodes"], e["nodes"]):
                        assert gn["op"] == en["op"] and gn["out"] == {k: en["out"][k] for k in gn["out"]}
                        assert gn["params"] == bytes.fromhex(en["params"]).ljust(64, b"\0")
                        assert gn["src"] == [{k: s[k] for k in ("buf", "off", "dtype", "dims", "strides")}
                                             for s in en["src"]]
                elif e["ev"] == "d2d":
                    assert g["copies"] == [list(c) for c in e["copies"]]
                else:
                    for k in ("bytes", "buf", "off"):
                        if k in e:
                            assert g[k] == e[k], (k, g, e)
