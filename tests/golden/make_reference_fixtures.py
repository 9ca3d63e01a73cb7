#!/usr/bin/env python3
"""Golden whole-model outputs produced by the REFERENCE's own CPU code.

Runs the unmodified reference CPU sources (compiled in place into oracle/_ref by
oracle/Makefile) on seeded synthetic models and stores their outputs as small .npz
fixtures next to this script. The reference tree exists only in the build container, so
the fixtures are committed; the GPU parity tests compare against them wherever they run.

Each fixture holds the inputs (ids, mask, segment ids), a checksum of the seeded weights
(so that a change of the weight generator is noticed) and the float32 outputs.

Usage: python tests/golden/make_reference_fixtures.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from cubert_b200 import synthetic  # noqa: E402
from oracle import bindings  # noqa: E402

# name -> (config, weight seed, batch, seq, lengths, segments)
CASES = {
    "tiny": ("tiny", 7, 5, 16, (3, 16), "half"),
    "tiny_mean": ("tiny_mean", 8, 3, 48, "full", "random"),
    "small": ("small", 9, 4, 32, (8, 32), "half"),
}


def weight_checksum(var):
    return float(sum(np.sum(v.astype(np.float64) * (1.0 + (i % 7))) for i, (k, v) in enumerate(sorted(var.items()))))


def main():
    bindings.build(ref=True)
    ref = bindings.Reference()
    for name, (cfg_name, seed, batch, seq, lengths, segments) in CASES.items():
        cfg = synthetic.config(cfg_name)
        var = synthetic.random_weights(cfg, seed)
        ids, mask, seg, _ = synthetic.random_inputs(cfg, batch, seq, seed, lengths=lengths, segments=segments)
        out = ref.bert_forward(var, synthetic.model_geometry(cfg, seq), ids, mask, seg)
        path = os.path.join(HERE, "reference_forward_%s.npz" % name)
        np.savez_compressed(path, ids=ids, mask=mask, seg=seg, weight_checksum=weight_checksum(var), **out)
        print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
