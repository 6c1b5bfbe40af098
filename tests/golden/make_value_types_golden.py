#!/usr/bin/env python
"""Generate ``value_types_reference.npz``: the fp8 value types' constructors and
conversion operators, and the bf16 <-> integer conversions that have a host path,
computed by the reference's own vendored headers (``oracle/_ref``, built by
``oracle/Makefile`` from a numba-cuda source tree)::

    python tests/golden/make_value_types_golden.py [output.npz]

Inputs come from ``tests/value_type_inputs.py``; only outputs are stored.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import oracle  # noqa: E402
from value_type_inputs import INT_NAMES, bf16_patterns, integers  # noqa: E402

FORMATS = {"e4m3": oracle.E4M3, "e5m2": oracle.E5M2, "e8m0": oracle.E8M0}
TARGETS = {"f16": oracle.F16, "bf16": oracle.BF16, "f32": oracle.F32, "f64": oracle.F64, "bool": oracle.BOOL}
INTS = {name: getattr(oracle, "I" + name[3:] if name.startswith("int") else "U" + name[4:]) for name in INT_NAMES}


def main(out_path):
    if not oracle.have_ref_headers():
        raise SystemExit("build oracle/_ref first: make -C oracle ref REFERENCE_ROOT=<numba-cuda tree>")
    out = {}
    codes = np.arange(256, dtype=np.uint8)
    halves = np.arange(65536, dtype=np.uint16).view(np.float16)
    for fname, fmt in FORMATS.items():
        for tname, dst in {**TARGETS, **INTS}.items():
            got = oracle.ref_value_to(codes, fmt, dst)
            out[f"{fname}_to_{tname}"] = got.view(np.uint16) if dst == oracle.F16 else got
        for iname, src in INTS.items():
            out[f"{fname}_from_{iname}"] = oracle.ref_value_from(integers(iname), src, fmt)
        out[f"{fname}_from_f16"] = oracle.ref_value_from(halves, oracle.F16, fmt)
    for fname in ("e4m3", "e5m2"):
        for sat in (0, 1):
            out[f"{fname}_from_f16_sat{sat}"] = oracle.ref_f16_to_fp8(halves, FORMATS[fname], sat)
    pats = bf16_patterns()
    for iname, code in INTS.items():
        out[f"bf16_to_{iname}_rz"] = oracle.ref_bf16_to_int_rz(pats, code)
        if iname not in ("int8", "uint8"):
            out[f"bf16_rn_from_{iname}"] = oracle.ref_int_to_bf16_rn(integers(iname), code)
    np.savez_compressed(out_path, **out)
    print(out_path, os.path.getsize(out_path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "value_types_reference.npz"))
