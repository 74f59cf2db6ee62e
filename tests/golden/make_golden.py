"""Writes the golden fixtures (``<case>.npz``) next to this file.

Run from the repository root: ``python tests/golden/make_golden.py``.  Each file
holds the CPU oracle's output and natural-log LSE for the case (float16 output to
keep the files small where the case is 16-bit, float32 otherwise) and float64
checksums of the regenerated inputs.
"""

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

import cases  # noqa: E402


def main():
    for name, c in cases.CASES.items():
        inp = cases.make_inputs(name)
        out, lse = cases.oracle_outputs(name, inp)
        sums = cases.input_checksums(inp)
        store = out.numpy() if c["dtype"] == "f32" else out.numpy().astype(np.float16)
        np.savez_compressed(
            os.path.join(HERE, f"{name}.npz"), out=store, lse=lse.numpy(),
            checksum_keys=np.array(sorted(sums)), checksum_vals=np.array([sums[k] for k in sorted(sums)]))
        print(name, store.shape, os.path.getsize(os.path.join(HERE, f"{name}.npz")))


if __name__ == "__main__":
    main()
