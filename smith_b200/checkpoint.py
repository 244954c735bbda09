"""Packed weights on disk -- the role src/checkpoint.js plays for f32 parameters in the reference.

The reference saves a model as ``path.json`` (a manifest with one entry per
parameter: shape, size, offset) plus ``path.bin`` (all parameters in one flat
array), src/checkpoint.js:10-62.  The same two files here hold the PACKED
weights: quantizing a 70B-shaped stack takes 52 GB of device packing per run,
loading the packed bytes does not.  Block layouts are the ones the matmul
kernels read (24-byte Q4 blocks, 34-byte Q8 blocks, block (g, col) at
(g * N + col) * block_bytes), so a loaded record goes straight to
matmulQ4 / matmulQ8.
"""
import json

import numpy as np

from . import device
from .ops.quantize import GROUP_BYTES, Q8_BLOCK_BYTES, Quantized

FORMAT = "smith-b200-packed-v1"


def _block_bytes(kind):
    if kind == "q4":
        return GROUP_BYTES
    if kind == "q8":
        return Q8_BLOCK_BYTES
    raise ValueError(f"saveQuantized: kind must be 'q4' or 'q8', got {kind!r}")


def saveQuantized(records, path):
    """``records``: {name: (kind, record)} with record = the {buffer, K, N, groups, totalBytes} of
    quantizeQ4 / quantizeQ8.  Writes ``path.json`` and ``path.bin``."""
    entries, offset = [], 0
    with open(path + ".bin", "wb") as f:
        for name, (kind, rec) in records.items():
            bb = _block_bytes(kind)
            total = int(rec["totalBytes"])
            if total != int(rec["groups"]) * int(rec["N"]) * bb:
                raise ValueError(f"saveQuantized: {name}: totalBytes does not match groups * N * {bb}")
            device.synchronize()
            f.write(device.download(rec["buffer"], total, np.uint8).tobytes())
            entries.append({"name": name, "kind": kind, "K": int(rec["K"]), "N": int(rec["N"]),
                            "groups": int(rec["groups"]), "totalBytes": total, "offset": offset})
            offset += total
    with open(path + ".json", "w") as f:
        json.dump({"format": FORMAT, "totalBytes": offset, "weights": entries}, f, indent=2)


def loadQuantized(path):
    """{name: (kind, record)} with the packed bytes back in device memory."""
    with open(path + ".json") as f:
        manifest = json.load(f)
    if manifest.get("format") != FORMAT:
        raise ValueError(f"loadQuantized: {path}.json is not a {FORMAT} manifest")
    blob = np.memmap(path + ".bin", dtype=np.uint8, mode="r")
    if blob.size != manifest["totalBytes"]:
        raise ValueError(f"loadQuantized: {path}.bin holds {blob.size} bytes, the manifest says {manifest['totalBytes']}")
    out = {}
    for e in manifest["weights"]:
        bb = _block_bytes(e["kind"])
        if e["totalBytes"] != e["groups"] * e["N"] * bb or e["offset"] + e["totalBytes"] > blob.size:
            raise ValueError(f"loadQuantized: entry {e['name']} is inconsistent")
        buf = device.alloc(e["totalBytes"], device.PRIVATE)
        device.upload(buf, np.ascontiguousarray(blob[e["offset"]:e["offset"] + e["totalBytes"]]))
        out[e["name"]] = (e["kind"], Quantized(buffer=buf, K=e["K"], N=e["N"], groups=e["groups"],
                                               totalBytes=e["totalBytes"]))
    return out
