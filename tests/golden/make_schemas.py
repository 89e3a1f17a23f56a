"""Extracts the operator schema strings that the reference registers for this path
(cust_op/framework/torch_plugin/torch_library/2.6.0/split_embedding_codegen_forward_unweighted/*.cpp, every
`m.def("...")`) and writes them, normalised by torch's schema parser, to op_schemas.txt.  Run in a container that
has the reference tree:  python tests/golden/make_schemas.py"""
import glob
import os
import re

import torch

_REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF = os.environ.get("RECSDK_REFERENCE_ROOT") or os.path.join(os.path.dirname(_REPO), "reference")
SRC = os.path.join(REF, "cust_op", "framework", "torch_plugin", "torch_library", "2.6.0",
                   "split_embedding_codegen_forward_unweighted")
OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "op_schemas.txt")

lines = []
for f in sorted(glob.glob(os.path.join(SRC, "*.cpp"))):
    s = open(f).read()
    for m in re.finditer(r"m\.def\((.*?)\);", s, re.S):
        txt = re.sub(r"\s+", " ", "".join(re.findall(r'"(.*?)"', m.group(1))))
        lines.append(str(torch._C.parse_schema(txt)))
open(OUT, "w").write("\n".join(sorted(lines)) + "\n")
print(len(lines), "schemas ->", OUT)
