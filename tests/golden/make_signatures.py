"""Writes tests/golden/op_signatures.json: parameter names and defaults of the reference's public op functions and
layer constructors / forwards, read from the reference's source text with ``ast`` (nothing is imported or run).

    python tests/golden/make_signatures.py /path/to/NeuralAttentionSearchLinear
"""
import ast
import json
import os
import sys

TARGETS = {
    "src/nats/ops/mixed_ops/mixed_attn_gdn.py": ["nats_mixed_attn_gdn", "nats_mixed_attn_gdn_chunk_inference",
                                                 "nats_mixed_attn_gdn_recurrent"],
    "src/nats/ops/mixed_ops/mixed_attn_mamba.py": ["nats_mixed_attn_mamba", "nats_mixed_attn_mamba_chunk_inference",
                                                   "nats_mixed_attn_mamba_recurrent"],
    "src/nats/layers/natsl_attn_gdn.py": ["NeuralAttentionSearchLinearAttnGDN.__init__",
                                          "NeuralAttentionSearchLinearAttnGDN.forward"],
    "src/nats/layers/natsl_attn_mamba2.py": ["NeuralAttentionSearchLinearAttnMamba.__init__",
                                             "NeuralAttentionSearchLinearAttnMamba.forward"],
}


def signature(fn: ast.FunctionDef):
    a = fn.args
    pos = a.posonlyargs + a.args
    defaults = [None] * (len(pos) - len(a.defaults)) + list(a.defaults)
    out = []
    for arg, d in zip(pos, defaults):
        out.append([arg.arg, "<required>" if d is None else ast.unparse(d)])
    for arg, d in zip(a.kwonlyargs, a.kw_defaults):
        out.append([arg.arg, "<required>" if d is None else ast.unparse(d)])
    if a.kwarg is not None:
        out.append(["**" + a.kwarg.arg, "<var>"])
    return out


def main(root):
    res = {}
    for rel, names in TARGETS.items():
        tree = ast.parse(open(os.path.join(root, rel)).read())
        for name in names:
            cls, _, fn = name.rpartition(".")
            body = tree.body
            if cls:
                body = next(n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == cls).body
            node = next(n for n in body if isinstance(n, ast.FunctionDef) and n.name == fn)
            res[name] = {"file": rel, "line": node.lineno, "params": signature(node)}
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "op_signatures.json")
    json.dump(res, open(out, "w"), indent=1)
    print("wrote", out)


if __name__ == "__main__":
    main(sys.argv[1])
