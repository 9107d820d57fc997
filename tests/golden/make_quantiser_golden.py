"""Generates tests/golden/quantiser_c11.npz from the reference's own numpy restatement of
the quantiser (kiln: scripts/c11_marlin_audit.py:208-241, `marlin_dequant_groupwise`).

Run in a container that has the kiln tree mounted:
    python tests/golden/make_quantiser_golden.py <path of the kiln tree>     (or KILN_REF in the environment)
The fixture holds the seed-derived input and that function's outputs; the test suite never
needs the kiln tree.
"""
import importlib.util
import os
import sys

import numpy as np


def main(ref_root: str) -> None:
    path = os.path.join(ref_root, "scripts", "c11_marlin_audit.py")
    spec = importlib.util.spec_from_file_location("c11_marlin_audit", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["c11_marlin_audit"] = mod
    spec.loader.exec_module(mod)
    rng = np.random.default_rng(20240611)
    k, n = 128, 256
    w = (rng.standard_normal((k, n)) * 0.05).astype(np.float32)
    w[:, 7] = 0.0  # an all-zero column exercises the max_abs == 0 guard
    w[5, :] *= 40.0  # outliers exercise the clamp
    w_dq, scales = mod.marlin_dequant_groupwise(w, 128)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quantiser_c11.npz")
    np.savez_compressed(out, w=w, w_dq=w_dq.astype(np.float32), scales=scales.astype(np.float32))
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["KILN_REF"])
