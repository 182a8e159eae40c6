"""Writes tests/golden/reference_signatures.json: names and defaults of the parameters of the reference's public
Python entry points for the hot path, read from the reference's source files with `ast` (nothing is imported):

    python tests/golden/make_reference_signatures.py <reference checkout> [output.json]

tests/test_host_api.py compares the signatures of this package with the file."""

import ast
import json
import os
import sys

ENTRY_POINTS = {
    "flashomni/attention.py": {"BatchFlashOmniFAWithRaggedKVWrapper": [
        "__init__", "plan", "run", "forward", "forward_return_lse", "reset_workspace_buffer", "end_forward"]},
    "flashomni/gemm.py": {None: ["flashomni_gemm", "flashomni_gemm_reduction"]},
    "flashomni/quantization.py": {None: ["packbits", "segment_packbits"]},
}


def describe(fn: ast.FunctionDef):
    a = fn.args
    names = [x.arg for x in a.posonlyargs + a.args]
    defaults = [None] * (len(names) - len(a.defaults)) + [ast.unparse(d) for d in a.defaults]
    return {"positional": [[n, d] for n, d in zip(names, defaults)],
            "keyword_only": [[x.arg, None if d is None else ast.unparse(d)] for x, d in zip(a.kwonlyargs, a.kw_defaults)]}


def main(ref_root, out_path):
    out = {}
    for rel, groups in ENTRY_POINTS.items():
        tree = ast.parse(open(os.path.join(ref_root, rel)).read())
        for cls, names in groups.items():
            body = tree.body
            if cls is not None:
                body = next(n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == cls).body
            for n in body:
                if isinstance(n, ast.FunctionDef) and n.name in names:
                    out[(cls + "." if cls else "") + n.name] = dict(describe(n), source=f"{rel}:{n.lineno}")
    with open(out_path, "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
        f.write("\n")
    print(f"{len(out)} entry points -> {out_path}")


if __name__ == "__main__":
    here = os.path.dirname(os.path.abspath(__file__))
    main(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else os.path.join(here, "reference_signatures.json"))
