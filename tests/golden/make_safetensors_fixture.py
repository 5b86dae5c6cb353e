"""Builds tests/golden/xyz2_crop.safetensors and tests/golden/safetensors_reference.json from the reference's own
safetensors fixture (zyx/tests/xyz2.safetensors, read by its test `matmul_disk`, zyx/tests/05_misc.rs:638-660, which
asserts z == x.matmul(y) on the loaded I64 tensors).

  python tests/golden/make_safetensors_fixture.py /path/to/zyx

The crop keeps the reference's bytes and layout: rows 0..15 of x, columns 0..15 of y and the matching 16 x 16 corner of
z (so z_crop == x_crop . y_crop still holds), written with the header exactly as Module::save formats it
(zyx/src/module.rs:36-63).  The JSON records the reference file's header verbatim and a SHA-256 per tensor."""
import hashlib
import json
import struct
import sys

import numpy as np


def main(root):
    raw = open(root + "/zyx/tests/xyz2.safetensors", "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    header = raw[8:8 + n].decode()
    meta = json.loads(header)
    data = raw[8 + n:]
    t = {k: np.frombuffer(data[v["data_offsets"][0]:v["data_offsets"][1]], "<i8").reshape(v["shape"]) for k, v in meta.items()}
    crop = {"x": t["x"][:16, :], "y": t["y"][:, :16], "z": t["z"][:16, :16]}
    assert np.array_equal(crop["x"] @ crop["y"], crop["z"])
    out_header, begin = "{", 0
    for k, a in crop.items():
        size = a.size * 8
        out_header += '"%s":{"dtype":"I64","shape":[%s],"data_offsets":[%d,%d]},' % (k, ",".join(str(d) for d in a.shape), begin, begin + size)
        begin += size
    out_header = out_header[:-1] + "}"
    with open("tests/golden/xyz2_crop.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(out_header)))
        f.write(out_header.encode())
        for a in crop.values():
            f.write(np.ascontiguousarray(a).astype("<i8").tobytes())
    ref = {"source": "zyx/tests/xyz2.safetensors", "header": header, "file_bytes": len(raw),
           "sha256": {k: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest() for k, a in t.items()},
           "crop_sha256": {k: hashlib.sha256(np.ascontiguousarray(a).astype("<i8").tobytes()).hexdigest() for k, a in crop.items()},
           "z_first_row": t["z"][0, :8].tolist()}
    json.dump(ref, open("tests/golden/safetensors_reference.json", "w"), indent=1)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_safetensors_fixture.py /path/to/zyx-checkout")
    main(sys.argv[1])
