"""The op functions and layer classes keep the reference's parameter names, order and defaults.  The expected
signatures are read from the reference's source text by ``tests/golden/make_signatures.py`` and stored in
``tests/golden/op_signatures.json``."""
import ast
import inspect
import json
import os

import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "op_signatures.json")
REQUIRED = ["nats_mixed_attn_gdn", "nats_mixed_attn_gdn_chunk_inference", "nats_mixed_attn_mamba",
            "nats_mixed_attn_mamba_chunk_inference", "NeuralAttentionSearchLinearAttnGDN.__init__",
            "NeuralAttentionSearchLinearAttnGDN.forward", "NeuralAttentionSearchLinearAttnMamba.__init__",
            "NeuralAttentionSearchLinearAttnMamba.forward"]


def _lookup(name):
    import neuralattentionsearchlinear_b200 as nat
    obj = nat
    for part in name.split("."):
        obj = getattr(obj, part, None)
        if obj is None:
            return None
    return obj


def _norm(text):
    """Compare defaults as Python values where they are literals (2 == 2.0 stays distinct from '2')."""
    try:
        return ast.literal_eval(text)
    except (ValueError, SyntaxError):
        return text


@pytest.mark.parametrize("name", sorted(json.load(open(GOLDEN))))
def test_signature_matches_reference(name):
    want = json.load(open(GOLDEN))[name]["params"]
    fn = _lookup(name)
    if fn is None:
        assert name not in REQUIRED, f"{name} is missing from the package"
        pytest.skip(f"{name} is not built")
    got = []
    for p in inspect.signature(fn).parameters.values():
        if p.kind is p.VAR_KEYWORD:
            got.append(["**" + p.name, "<var>"])
        else:
            got.append([p.name, "<required>" if p.default is p.empty else p.default])
    assert [g[0] for g in got] == [w[0] for w in want], "parameter names / order differ from the reference"
    for (n, g), (_, w) in zip(got, want):
        if w in ("<required>", "<var>"):
            assert g == w, f"{name}: {n} must have no default"
        else:
            assert g == _norm(w), f"{name}: default of {n} is {g!r}, the reference has {w}"
