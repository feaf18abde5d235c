"""Regenerates tests/golden/sdpa_bundles.npz from the reference checkout.

Usage: python tests/golden/make_golden.py /path/to/tract

The reference ships six input/expected-output bundles for `tract_transformers_sdpa`
under harness/nnef-test-cases/sdpa/<case>/io.npz (checked by its CI with
`--assert-output-bundle`).  This script copies the arrays of each bundle into one
npz next to this file, together with the op attributes written in each case's
graph.nnef (restated in CASES below; the graph files are text and were read, not
executed).  The one constant tensor a graph embeds (simple-mask-f32/v0.dat, an
NNEF tensor file: 128-byte header then f32 data, shape [2, 1]) is decoded here.
"""
import json
import os
import sys

import numpy as np

# case -> attributes of the tract_transformers_sdpa call in graph.nnef
CASES = {
    # q = k = v = input_0, rank 3 [B, S, D]
    "simple-causal-f32": dict(qkv=["input_0"] * 3, dtype="f32", causal=True, scale=None),
    "simple-non-causal-f32": dict(qkv=["input_0"] * 3, dtype="f32", causal=False, scale=None),
    "simple-scale-f32": dict(qkv=["input_0"] * 3, dtype="f32", causal=False, scale=1.3),
    # input cast to f16, sdpa in f16 with f32 accumulation, cast back to f32; rank 4
    "simple-f16": dict(qkv=["input_0"] * 3, dtype="f16", causal=False, scale=None),
    # three inputs + constant mask v0 [2, 1] unsqueezed to [1, 2, 1]
    "simple-mask-f32": dict(qkv=["input_0", "input_1", "input_2"], dtype="f32", causal=False, scale=None,
                            mask_file="v0.dat", mask_shape=[1, 2, 1]),
    # one-layer Llama (hidden 8, 4 q heads, 2 kv heads) run with unfold-kv-cache: inputs are
    # token ids and the past K/V [1, 2, 10, 2]; outputs 1 and 2 are the caches after the step.
    # Only the cache-append part is usable without the model weights: out[:, :, :10] == past.
    "simple-grouped-query-att-f32": dict(kv_io=True),
}


def main(ref):
    base = os.path.join(ref, "harness", "nnef-test-cases", "sdpa")
    out, meta = {}, {}
    for case, attrs in CASES.items():
        z = np.load(os.path.join(base, case, "io.npz"))
        for k in z.files:
            out[f"{case}/{k}"] = z[k]
        attrs = dict(attrs)
        if "mask_file" in attrs:
            raw = np.fromfile(os.path.join(base, case, attrs.pop("mask_file")), dtype=np.uint8)
            out[f"{case}/mask"] = raw[128:].view(np.float32).reshape(attrs.pop("mask_shape"))
        meta[case] = attrs
    out["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "sdpa_bundles.npz"), **out)
    print("wrote", len(out) - 1, "arrays for", len(meta), "cases")


if __name__ == "__main__":
    main(sys.argv[1])
