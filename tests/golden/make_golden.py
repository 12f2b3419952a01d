"""Extracts the reference's golden console outputs for the row operations into
tests/golden/primitives_golden.npz.

Run in a container that has the reference checkout:

    python tests/golden/make_golden.py <reference checkout>

Sources (all under test_text_outputs/primitives/, printed by the tests in
ml/primitives.spi:851-989 with seed 12344321): test2/{a,b} print the first 1024
elements of input, softmax, masked softmax (legal iff j < 4), the j < 11 masked
softmax (file "output_softmax'.txt", written last by ml/primitives.spi:985-986),
L2 row normalisation and argmax; test3/{a,b} print (input, identity) pairs and
the masked regret matching (legal iff j < 3) of the same rows.  Values carry 6
decimals, so comparisons against them use an absolute tolerance of 2e-6.
"""
import os
import re
import sys

import numpy as np

NUM = re.compile(r"-?\d+\.\d+(?:[eE][-+]?\d+)?|-?\d+")


def read_rows(path, pair=False):
    """Parses '[[a; b; ...]; [c; d; ...]]' (or '[a; b; ...]') into a 2-D (1-D) array."""
    text = open(path).read().strip()
    rows = []
    for chunk in re.findall(r"\[([^\[\]]*)\]", text):
        vals = [float(v) for v in NUM.findall(chunk)]
        if pair:
            vals = vals[0::2]
        rows.append(vals)
    width = max(len(r) for r in rows)
    rows = [r for r in rows if len(r) == width]   # the printer may truncate the last row
    arr = np.array(rows, dtype=np.float64)
    return arr[0] if text.count("[") == 1 else arr


def main(ref_root):
    base = os.path.join(ref_root, "test_text_outputs", "primitives")
    out = {}
    for sub in ("a", "b"):
        d = os.path.join(base, "test2", sub)
        out["t2%s_input" % sub] = read_rows(os.path.join(d, "input.txt")).astype(np.float32)
        out["t2%s_softmax" % sub] = read_rows(os.path.join(d, "output_softmax.txt")).astype(np.float32)
        out["t2%s_masked_softmax4" % sub] = read_rows(os.path.join(d, "output_masked_softmax.txt")).astype(np.float32)
        out["t2%s_masked_softmax11" % sub] = read_rows(os.path.join(d, "output_softmax'.txt")).astype(np.float32)
        out["t2%s_ln_l2" % sub] = read_rows(os.path.join(d, "output_ln.txt")).astype(np.float32)
        out["t2%s_argmax" % sub] = read_rows(os.path.join(d, "output_argmax.txt")).astype(np.int32)
        d = os.path.join(base, "test3", sub)
        out["t3%s_input" % sub] = read_rows(os.path.join(d, "zip_input_output_identity_map.txt"), pair=True).astype(np.float32)
        out["t3%s_masked_regret3" % sub] = read_rows(os.path.join(d, "output_op_map.txt")).astype(np.float32)
    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "primitives_golden.npz"), **out)
    for k, v in sorted(out.items()):
        print(k, v.shape, v.dtype)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <reference checkout>")
    main(sys.argv[1])
