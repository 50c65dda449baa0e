#!/usr/bin/env python
"""Renders the state machines of this library as Graphviz.

Every per-operation state machine (the pipe's read and write operations, channel operations) is written
as a list of `attemptTransition(op, FROM, TO, condition, actions)` edges, so the graph can be read
straight off the source. The reference ships a clang-LibTooling program for the same purpose
(tensorpipe/misc/dump_state_machine.cc:52-138); a regular expression is enough for this code base.

    python misc/dump_state_machine.py src/core/pipe.cc | dot -Tsvg > pipe.svg
"""
import re
import sys

EDGE = re.compile(r"attemptTransition\(\s*\w+\s*,\s*([\w:]+)\s*,\s*([\w:]+)\s*,\s*(.*?)(?:,\s*\[|\);)", re.S)


def main(paths):
    print("digraph state_machines {\n  rankdir=LR;\n  node [shape=box, fontname=Helvetica];")
    for path in paths:
        text = open(path).read()
        # one cluster per advance function
        for fn in re.finditer(r"void\s+(\w+)::(advance\w+)\(.*?\)\s*\{(.*?)\n\}", text, re.S):
            cls, name, body = fn.groups()
            edges = EDGE.findall(body)
            if not edges:
                continue
            print(f'  subgraph "cluster_{cls}_{name}" {{\n    label="{cls}::{name}";')
            for src, dst, cond in edges:
                cond = " ".join(cond.split())
                cond = cond[:70] + ("..." if len(cond) > 70 else "")
                s, d = src.split("::")[-1], dst.split("::")[-1]
                print(f'    "{name}.{s}" -> "{name}.{d}" [label="{cond.replace(chr(34), chr(39))}", fontsize=9];')
                print(f'    "{name}.{s}" [label="{s}"]; "{name}.{d}" [label="{d}"];')
            print("  }")
    print("}")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    main(sys.argv[1:])
