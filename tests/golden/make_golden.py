"""Regenerates the committed golden vectors in this folder.

Two independent pins for the CPU oracle:

* ``kquant_decode.npz`` -- Q4_K / Q6_K super-blocks together with their decode
  by gguf-py's numpy implementation (``gguf.quants.dequantize``), which is
  independent of both the oracle and the CUDA kernels.  Half of the blocks come
  from the oracle's encoder on seeded N(0, 0.02) data, half are random bytes
  (every bit pattern of the packed fields is a valid block) with finite f16
  scales.
* ``routing_kat.json`` -- the routing known-answer cases of the reference's
  unit tests (src/moe.rs:405-484 of the reference): hand-built logits, biases,
  expected expert ids and expected weights (computed here in float64 from the
  closed form, as those tests do).

Run from the repository root:  python tests/golden/make_golden.py
Needs the ``gguf`` Python package; the tests themselves only read the files.
"""
import json
import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from oracle import oracle as orc  # noqa: E402


def kquant_vectors():
    import gguf
    from gguf import quants

    rng = np.random.default_rng(20240611)
    out = {}
    for name, dt, qt in (("q4k", orc.Q4_K, gguf.GGMLQuantizationType.Q4_K),
                         ("q6k", orc.Q6_K, gguf.GGMLQuantizationType.Q6_K)):
        ts = orc.TYPE_SIZE[dt]
        enc = orc.quantize(dt, (rng.standard_normal(6 * 256) * 0.02).astype(np.float32)).reshape(6, ts)
        rnd = rng.integers(0, 256, size=(6, ts), dtype=np.uint8)
        scales = rng.uniform(1e-4, 2e-2, size=(6, 2)).astype(np.float16).view(np.uint8).reshape(6, 4)
        if dt == orc.Q4_K:
            rnd[:, 0:4] = scales
        else:
            rnd[:, 208:210] = scales[:, 0:2]
        blocks = np.concatenate([enc, rnd], axis=0)
        deq = quants.dequantize(blocks.reshape(-1), qt).astype(np.float32).reshape(12, 256)
        out[name + "_blocks"] = blocks
        out[name + "_decoded"] = deq
    np.savez_compressed(os.path.join(HERE, "kquant_decode.npz"), **out)


def routing_kats():
    sig = lambda v: 1.0 / (1.0 + math.exp(-v))
    row = [2.0, -2.0, 0.0, 1.0, -1.0, 3.0, 0.5, -0.5]
    floor = 6.103515625e-5

    def norm(ids, logits, scale=2.5):
        p = [sig(logits[i]) for i in ids]
        s = max(sum(p), floor)
        return [v / s * scale for v in p]

    cases = [
        dict(name="positive_bias_displaces", logits=row, bias=[0, 0, 0, 0, 0, 0, 0.2, 0], top_k=3,
             scale=2.5, norm=True, ids=[5, 0, 6], weights=norm([5, 0, 6], row), atol=1e-5, rtol=0.0),
        dict(name="negative_bias_excludes", logits=row, bias=[0, 0, 0, 0, 0, -1.0, 0, 0], top_k=3,
             scale=2.5, norm=True, ids=[0, 3, 6], weights=norm([0, 3, 6], row), atol=1e-5, rtol=0.0),
        dict(name="ties_pick_lowest_indices", logits=[0.0] * 8, bias=[0.0] * 8, top_k=3,
             scale=2.5, norm=True, ids=[0, 1, 2], weights=norm([0, 1, 2], [0.0] * 8), atol=1e-5, rtol=0.0),
        dict(name="clamps_tiny_denominator", logits=[-30.0] * 8, bias=[0.0] * 8, top_k=3,
             scale=2.5, norm=True, ids=[0, 1, 2], weights=norm([0, 1, 2], [-30.0] * 8), atol=0.0, rtol=1e-3),
    ]
    with open(os.path.join(HERE, "routing_kat.json"), "w") as f:
        json.dump(cases, f, indent=1)


if __name__ == "__main__":
    kquant_vectors()
    routing_kats()
    print("wrote", sorted(os.listdir(HERE)))
