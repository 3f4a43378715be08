"""Writes tests/golden/graph_v2.kgph.hex: the bytes of the reference's frozen KGPH v2 golden blob
(kurumi_core/tests/fixtures/graph_v2.kgph, 175 bytes, pinned by kurumi_core/src/graph/serialize/tests.rs:188-221:
Const [[1,2,3],[4,5,6]] + Const 2.0 x 6 -> Add -> Sum(axis 1) = [12, 21]).

Run in a checkout that has the reference tree: python tests/golden/make_graph_blob_fixture.py <reference root>
"""
import os
import sys


def main():
    ref = sys.argv[1]
    blob = open(os.path.join(ref, "kurumi_core", "tests", "fixtures", "graph_v2.kgph"), "rb").read()
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "graph_v2.kgph.hex")
    with open(out, "w") as f:
        f.write(blob.hex() + "\n")
    print(f"{out}: {len(blob)} bytes")


if __name__ == "__main__":
    main()
