"""Freezes SHA-256 digests of the oracle packer's output for seeded inputs into
tests/golden/pack_hashes.json.  These are regression pins made by this repository's own
oracle (both restatements must agree before a digest is written); the kiln tree holds no
golden vectors for the packed format.

    python tests/golden/make_pack_hashes.py
"""
import hashlib
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import oracle  # noqa: E402
from oracle import C  # noqa: E402

CASES = [  # (k, n, groupsize, seed)
    (128, 256, 128, 1), (128, 256, -1, 2), (256, 512, 128, 3), (256, 256, -1, 4),
    (2560, 512, 128, 5), (2560, 4096, 128, 6), (4096, 2560, 128, 7), (9216, 2560, 128, 8),
    (2560, 9216, 128, 1234),
]


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def synth_weight(k, n, seed):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((k, n)) * 0.05).astype(np.float32)


def main():
    out = {}
    for k, n, gs, seed in CASES:
        w = synth_weight(k, n, seed)
        p, s, d, q = C.quantize_and_pack(w, gs)
        p2, s2, d2, q2 = oracle.np_quantize_and_pack(w, gs)
        assert (p == p2).all() and (s.view(np.uint16) == s2.view(np.uint16)).all() and (d == d2).all()
        assert (C.unpack_fragment(p, k, n) == q).all()
        out[f"{k}x{n}_g{gs}_s{seed}"] = {
            "packed": digest(p), "scales": digest(s.view(np.uint16)), "dequant": digest(d), "q": digest(q),
        }
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "pack_hashes.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print("wrote", path)


if __name__ == "__main__":
    main()
