"""A safetensors file the way the format is laid out (an 8-byte little-endian header length, a JSON object of
{dtype, shape, data_offsets} per tensor, the data), for the drafter's loader tests."""
import json
import struct

import numpy as np


def write(path, tensors, dtype="BF16", metadata=None, drop=(), lie=None):
    """tensors: name -> uint16 array of bf16 bits. `drop`: names left out; `lie`: name -> dtype string written instead."""
    header, blobs, at = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, bits in tensors.items():
        if name in drop:
            continue
        raw = np.ascontiguousarray(bits, np.uint16).tobytes()
        header[name] = {"dtype": (lie or {}).get(name, dtype), "shape": list(np.shape(bits)), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw); at += len(raw)
    text = json.dumps(header).encode()
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text))); f.write(text)
        for raw in blobs:
            f.write(raw)
