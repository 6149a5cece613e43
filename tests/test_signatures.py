"""The ctypes argument types declared in pagedserve_b200/kernels/ops.py against the C sources."""

import glob
import os
import re

from pagedserve_b200.kernels.ops import _SIGNATURES

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "pagedserve_b200", "csrc")


def test_declared_argument_types_match_the_entry_points():
    source = "".join(open(path).read() for path in glob.glob(os.path.join(CSRC, "*.cu")))
    letters = {"c_void_p": "P", "c_int": "I", "c_float": "F", "c_longlong": "L", "c_long": "L"}
    for functions in _SIGNATURES.values():
        for name, argtypes in functions.items():
            match = re.search(r"PS_EXPORT int " + name + r"\((.*?)\)\s*\{", source, re.S)
            assert match, f"{name} is not exported by any source file"
            kinds = []
            for parameter in (part.strip() for part in match.group(1).split(",")):
                if "*" in parameter:
                    kinds.append("P")
                elif parameter.startswith("float"):
                    kinds.append("F")
                elif parameter.startswith("long long"):
                    kinds.append("L")
                else:
                    kinds.append("I")
            assert "".join(kinds) == "".join(letters[a.__name__] for a in argtypes), name
