"""Regenerates the committed fixtures in this folder.

Run in a checkout that has the reference mounted:  python tests/golden/make_fixtures.py /path/to/bullet
  batch_head.bf   first 1024 of the 16273 32-byte ChessBoard records of examples/tests/batch.bf
                  (real positions; the only data file the reference ships)
`reference_kats.json` is transcribed by hand from the unit tests cited inside it.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))

if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_fixtures.py /path/to/bullet")
    ref = sys.argv[1]
    with open(os.path.join(ref, "examples", "tests", "batch.bf"), "rb") as f:
        data = f.read()
    assert len(data) == 16273 * 32
    with open(os.path.join(HERE, "batch_head.bf"), "wb") as f:
        f.write(data[: 1024 * 32])
