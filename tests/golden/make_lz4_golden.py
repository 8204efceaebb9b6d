"""Golden vector for the LZ4 block-stream container: the one matrix file the
BIDMach checkout holds that BIDMat itself wrote through lz4-java,
scripts/networks/modelmat_test.fmat.lz4.  Writes

  lz4block_tail.bin    its last data block and the end mark, byte for byte (8.4 KB)
  lz4block_meta.json   the header fields of every block, the matrix header ints and
                       the XXH32 (seed 0) of the whole decompressed payload

Run from the repository root, giving the path of the BIDMach checkout (or set
BIDMACH_REFERENCE, as oracle/build.py reads it):
    python tests/golden/make_lz4_golden.py <BIDMach checkout>
"""
import json
import os
import struct
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from bidmach_b200 import matio  # noqa: E402


def main(ref_root):
    src = os.path.join(ref_root, "scripts", "networks", "modelmat_test.fmat.lz4")
    data = open(src, "rb").read()
    blocks, at = [], 0
    while at < len(data):
        assert data[at: at + 8] == b"LZ4Block"
        token, clen, olen, check = struct.unpack_from("<BiiI", data, at + 8)
        blocks.append({"offset": at, "token": token, "compressed": clen, "original": olen, "checksum": check})
        at += 21 + clen
    assert at == len(data) and blocks[-1]["original"] == 0
    payload = matio.lz4_stream_decompress(data)
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "lz4block_tail.bin"), "wb") as f:
        f.write(data[blocks[-2]["offset"]:])
    meta = {"source": "scripts/networks/modelmat_test.fmat.lz4", "file_bytes": len(data),
            "payload_bytes": len(payload), "payload_xxh32_seed0": matio.xxh32(payload, 0),
            "matrix_header_ints": list(struct.unpack_from("<6i", payload, 0)), "blocks": blocks}
    with open(os.path.join(here, "lz4block_meta.json"), "w") as f:
        json.dump(meta, f, indent=1)
    print(meta)


if __name__ == "__main__":
    from oracle.build import REF_ROOT  # noqa: E402  (BIDMACH_REFERENCE or its default)
    main(sys.argv[1] if len(sys.argv) > 1 else REF_ROOT)
