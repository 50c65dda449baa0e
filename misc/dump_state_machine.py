#!/usr/bin/env python
"""Renders the stage machines of this library as Graphviz.

A pipe is set up through a sequence of phases (`PipeCore::Phase`) and every incoming message moves
through a sequence of stages (`Inbound::Stage`); both only ever move forward, except into `kFailed`,
which any phase can reach. The code says so in the plainest way: an enumeration, and assignments
`phase_ = Phase::kX` / `stage = Inbound::kX` in the functions that make the step. This script reads
the enumerations from the header and the assignments from the sources and draws, for every
assignment, an edge into the assigned state from the state declared before it, labelled with the
function that makes the step. The reference ships a clang-LibTooling program for the same purpose
(tensorpipe/misc/dump_state_machine.cc:52-138); regular expressions are enough for this code base.

    python misc/dump_state_machine.py src/core/core.h src/core/pipe_setup.cc src/core/pipe_traffic.cc | dot -Tsvg > pipe.svg
"""
import re
import sys

ENUM = re.compile(r"enum\s+(?:class\s+)?(\w+)\s*(?::\s*\w+\s*)?\{([^}]*)\}", re.S)
FUNCTION = re.compile(r"^[\w:<>&\*\s]+?\b(\w+)::(\w+)\([^;{]*\)\s*(?:const\s*)?\{", re.M)
ASSIGN = re.compile(r"\b(\w+)\s*=\s*(?:\w+::)*(\w+)::(k\w+)\s*;")


def main(paths):
    texts = {p: open(p).read() for p in paths}
    enums = {}
    for text in texts.values():
        for name, body in ENUM.findall(text):
            members = [m.split("=")[0].strip() for m in re.sub(r"//.*", "", body).split(",")]
            members = [m for m in members if re.fullmatch(r"k\w+", m)]
            if len(members) >= 3:
                enums[name] = members
    edges = {}  # enum -> set of (from, to, function)
    for text in texts.values():
        starts = [(m.start(), f"{m.group(1)}::{m.group(2)}") for m in FUNCTION.finditer(text)]
        for m in ASSIGN.finditer(text):
            _, enum, value = m.groups()
            # `Inbound::kOffered` names the struct the enumeration lives in; match by member.
            owner = next((e for e, members in enums.items() if value in members and (e == enum or enum not in enums)), None)
            if owner is None:
                continue
            fn = "?"
            for pos, name in starts:
                if pos < m.start():
                    fn = name
            if fn == "?":
                continue  # a member initialiser, not a step
            members = enums[owner]
            i = members.index(value)
            src = "any" if value == "kFailed" or i == 0 else members[i - 1]
            edges.setdefault(owner, set()).add((src, value, fn))
    print("digraph stage_machines {\n  rankdir=LR;\n  node [shape=box, fontname=Helvetica];")
    for owner, es in sorted(edges.items()):
        print(f'  subgraph "cluster_{owner}" {{\n    label="{owner}";')
        for member in enums[owner]:
            print(f'    "{owner}.{member}" [label="{member}"];')
        if any(src == "any" for src, _, _ in es):
            print(f'    "{owner}.any" [label="(any)", shape=plaintext];')
        for src, dst, fn in sorted(es):
            print(f'    "{owner}.{src}" -> "{owner}.{dst}" [label="{fn}", fontsize=9];')
        print("  }")
    print("}")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    main(sys.argv[1:])
