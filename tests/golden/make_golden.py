#!/usr/bin/env python
"""Writes the golden fixtures of tests/golden/ from the reference checkout. Run in the build
container, where the reference is mounted; the fixtures (not the reference) travel with the repo.

  python tests/golden/make_golden.py /path/to/reference

1. gguf_golden_blocks.json: the real Q4_K / Q5_K / Q6_K block of each format that the reference's
   own known-answer test decodes (Tests/SploshOracleTests/GgufGoldenBlocks.swift, checked by
   Tests/SploshOracleTests/GgufTests.swift:237), bytes and expected float32 values, read from that
   file as data.
2. gguf_check_vectors.npz: blocks of seeded random bytes with sane fp16 scale fields, decoded by the
   reference's runnable numpy decoder tools/gguf_check.py (`decode`), imported from the checkout.
"""
import importlib.util
import json
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def golden_blocks(reference):
    text = open(os.path.join(reference, "Tests/SploshOracleTests/GgufGoldenBlocks.swift")).read()
    out = {}
    for name, kind in (("q4K", "Q4_K"), ("q5K", "Q5_K"), ("q6K", "Q6_K")):
        body = text[text.index(f"static let {name} = GgufGoldenBlock("):]
        body = body[:body.index("\n        ])") + 10]
        raw = body[body.index("bytes: [") + 8:body.index("],\n        values:")]
        vals = body[body.index("values: [") + 9:]
        vals = vals[:vals.rindex("]")]
        out[kind] = {"bytes": [int(x, 16) for x in re.findall(r"0x[0-9a-fA-F]{2}", raw)],
                     "values": [float(x) for x in re.findall(r"-?\d+\.?\d*(?:e-?\d+)?", vals)]}
    return out


def check_vectors(reference):
    spec = importlib.util.spec_from_file_location("gguf_check", os.path.join(reference, "tools/gguf_check.py"))
    mod = importlib.util.module_from_spec(spec); spec.loader.exec_module(mod)
    rng = np.random.default_rng(0x5EED)
    out = {}
    for kind, size, fields in (("Q4_K", 144, [(0, 2e-4), (2, 1.5e-3)]), ("Q5_K", 176, [(0, 1e-4), (2, 1.5e-3)]), ("Q6_K", 210, [(208, 5e-5)])):
        raw = rng.integers(0, 256, (24, size), dtype=np.uint8)
        for block in range(raw.shape[0]):
            for offset, magnitude in fields:       # the scale fields as the reference's kernel tests set them
                value = magnitude * (0.75 + 0.5 * rng.random()) * (-1 if block % 4 == 3 else 1)
                raw[block, offset:offset + 2] = np.frombuffer(np.float16(value).tobytes(), np.uint8)
        out[kind + "_raw"] = raw
        out[kind + "_values"] = mod.decode(kind, raw).astype(np.float32)
    return out


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of the reference checkout>")
    reference = sys.argv[1]
    with open(os.path.join(HERE, "gguf_golden_blocks.json"), "w") as f:
        json.dump(golden_blocks(reference), f)
    np.savez_compressed(os.path.join(HERE, "gguf_check_vectors.npz"), **check_vectors(reference))
    print("wrote fixtures")
