"""Writes tests/golden/ref_op_schemas.json: the operator schemas that the
reference's own ``TORCH_LIBRARY(npc, m)`` block (src/pybind.cc:18-48) registers,
as PyTorch infers them from the C++ signatures.

Needs no GPU: it loads oracle/_ref/libnpc_ref.so (the reference compiled by
``python oracle/build_ref.py``) in a fresh process, in which apt_b200 must not
be imported (both register the ``npc`` namespace), and asks the dispatcher for
each schema string.

    python tests/golden/make_ref_schemas.py
"""
import json
import os
import re

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    torch.classes.load_library(os.path.join(ROOT, "oracle", "_ref", "libnpc_ref.so"))
    names = set()
    for s in torch._C._jit_get_all_schemas():
        if s.name.startswith("npc::"):
            names.add(s.name[5:])
    out = {}
    for name in sorted(names):
        text = str(torch._C._get_schema("npc::" + name, ""))
        out[name] = re.sub(r"^npc::", "", text)
    path = os.path.join(ROOT, "tests", "golden", "ref_op_schemas.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
        f.write("\n")
    print(f"{len(out)} schemas -> {path}")


if __name__ == "__main__":
    main()
