"""Generates tests/golden/input_topology.json: what the REFERENCE's own Topology reader (src/topology.cpp compiled in place,
oracle/_ref/libdsmd_ref_topology.so) parses from the topology / parameter files that tests/input_cases.py writes.
Run from the repository root where the reference tree is present:

    make -C oracle && python tests/golden/make_input_golden.py
"""
import json
import os
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import input_cases  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for name, case in input_cases.topology_cases(tmp).items():
            parsed = input_cases.reference_topology(case["topology_file"], case.get("parameter_file"))
            if parsed is None:
                raise SystemExit(f"the reference's reader refused case {name}")
            out[name] = parsed
            print(name, {k: (len(v) if isinstance(v, list) else v) for k, v in parsed.items()})
    with open(os.path.join(HERE, "input_topology.json"), "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
        f.write("\n")


if __name__ == "__main__":
    main()
