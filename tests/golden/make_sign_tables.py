"""Writes tests/golden/reference_sign_tables.json from the reference's product tables.

    python tests/golden/make_sign_tables.py /path/to/reference

Reads src/algebras.cc of the reference checkout and stores, per algebra, its SIGNTABLE as a flat list of
(left, right, sign) triples in the file's own order (rows of D entries per output component) and its
BACKPROP_ORDER. The JSON is what the tests read; the reference checkout is needed only to regenerate it.
"""
import json
import os
import re
import sys


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_sign_tables.py /path/to/reference")
    ref = sys.argv[1]
    text = open(os.path.join(ref, "src", "algebras.cc")).read()
    out = {"_comment": "Product tables of the reference (src/algebras.cc:5-145), transcribed as data by make_sign_tables.py: "
                       "entries are [left component (input), right component (filter), sign], D per output component."}
    for name in ("REAL", "COMPLEX", "QUATERNION", "GA_300"):
        table = re.search(r"CliffordProductSpec<Algebra::%s>::SIGNTABLE\[\]\s*=\s*\{(.*?)\};" % name, text, re.S).group(1)
        entries = [[int(l), int(r), 1 if s == "true" else -1]
                   for l, r, s in re.findall(r"\{\s*(\d+)\s*,\s*(\d+)\s*,\s*(true|false)\s*\}", table)]
        order = re.search(r"CliffordProductSpec<Algebra::%s>::BACKPROP_ORDER\[\]\s*=\s*\{(.*?)\};" % name, text, re.S).group(1)
        out[name] = {"entries": entries, "backprop_order": [int(v) for v in re.findall(r"\d+", order)]}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_sign_tables.json")
    with open(path, "w") as f:
        json.dump(out, f, separators=(",", ":"))
        f.write("\n")
    print(path, {k: len(v["entries"]) for k, v in out.items() if k != "_comment"})


if __name__ == "__main__":
    main()
