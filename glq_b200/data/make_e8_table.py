"""Write ``e8_shell_packed.npy`` from the reference's bundled codebook file.

    python glq_b200/data/make_e8_table.py <path-to-reference>/glq/e8_codebook.pt

The E8 shell codebook (65,536 lattice points, shells 0-5 complete plus 8,655 points of
shell 6) is defined by the reference's file: the order of equal-norm rows comes from an
unstable sort and cannot be regenerated from the mathematics alone.  Each row is stored
as one uint32 with nibble i = 2*coord_i + 6 (glq/codebook.py:102-115), 256 KiB in all.
Users who hold the reference's fp16 table pass that to the ops instead; this file only
serves callers (tests, the benchmark) that run where the reference is not installed.
"""
import os
import sys

import numpy as np
import torch

if __name__ == "__main__":
    d = torch.load(sys.argv[1], map_location="cpu", weights_only=True)
    tab = d["codebook"].numpy().astype(np.float64)
    codes = np.rint(tab * 2).astype(np.int64) + 6
    assert codes.min() >= 0 and codes.max() <= 12 and tab.shape == (65536, 8)
    packed = np.zeros(65536, dtype=np.uint32)
    for i in range(8):
        packed |= codes[:, i].astype(np.uint32) << np.uint32(4 * i)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "e8_shell_packed.npy")
    np.save(out, packed)
    print("wrote", out, packed.nbytes, "bytes")
