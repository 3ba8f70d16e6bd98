"""Regenerates tests/golden/reference_outputs.npz.

Runs the `quick` subset of the seeded cases in tests/cases.py, and the F16 storage cases, through the
reference CPU backend compiled from its own sources (oracle/_ref/libvkml_ref.so,
built by `make -C oracle ref` where the reference tree is present) and stores
the OUTPUT bytes.  Inputs are not stored: they are regenerated from the same
seeds.  Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import cases  # noqa: E402
from helpers import RefImpl  # noqa: E402

LIMIT_BYTES = 6_000  # per output, keeps the fixture small


def main():
    ref = RefImpl()
    names, arrays = [], {}
    seen = set()
    import itertools
    for case in itertools.chain(cases.all_cases(quick=True), cases.f16_cases()):
        if case.name in seen:
            continue
        seen.add(case.name)
        rc, out = ref.run_status(case.op, case.srcs, case.out_shape, case.out_dtype, case.params)
        if rc != 0 or out.nbytes > LIMIT_BYTES:
            continue
        # keep a spread: every op family, not every layout (all of the F16 storage cases)
        family = case.name.split("/")[0]
        if family != "f16" and len([n for n in names if n.split("/")[0] == family]) >= 6:
            continue
        arrays[f"out_{len(names)}"] = out
        names.append(case.name)
    arrays["__index__"] = np.array(json.dumps(names))
    np.savez_compressed(os.path.join(HERE, "reference_outputs.npz"), **arrays)
    print(f"wrote {len(names)} reference outputs")


if __name__ == "__main__":
    main()
