"""Every command-line flag and every ``Namespace`` default of the reference exists here with the same default."""
import os
import re

import pytest

# the reference sources: the in-tree install used by the benchmark's reference arm, or a checkout named by DICEE_SRC
_HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("DICEE_SRC") or os.path.join(os.path.dirname(_HERE), "baseline", "_ref", "dicee")


def _reference_flags():
    text = open(os.path.join(REF, "scripts", "run.py")).read()
    return sorted(set(re.findall(r"add_argument\(\s*[\"'](--[A-Za-z0-9_]+)[\"']", text)))


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference sources are not on this machine")
def test_all_reference_flags_are_accepted():
    from dice_embeddings_b200.cli import get_default_arguments
    ours = get_default_arguments([])
    missing = [f for f in _reference_flags() if not hasattr(ours, f[2:])]
    assert not missing, missing


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference sources are not on this machine")
def test_namespace_defaults_match_the_reference():
    import ast
    from dice_embeddings_b200 import Namespace
    tree = ast.parse(open(os.path.join(REF, "config.py")).read())
    ref = {}
    for node in ast.walk(tree):
        if isinstance(node, (ast.Assign, ast.AnnAssign)):
            tgt = node.targets[0] if isinstance(node, ast.Assign) else node.target
            if isinstance(tgt, ast.Attribute) and isinstance(tgt.value, ast.Name) and tgt.value.id == "self" \
                    and node.value is not None:
                try:
                    ref[tgt.attr] = ast.literal_eval(node.value)
                except Exception:
                    pass
    ours = Namespace()
    assert len(ref) > 40
    diff = {k: (v, getattr(ours, k, "<missing>")) for k, v in ref.items()
            if getattr(ours, k, "<missing>") != v and not (v in ({}, []) and getattr(ours, k, None) in (None, {}, []))}
    assert not diff, diff


def test_cli_defaults_of_the_additions():
    from dice_embeddings_b200.cli import get_default_arguments
    a = get_default_arguments([])
    assert a.kernel_backend == "auto" and a.comm == "p2p" and a.block_size == 8
    b = get_default_arguments(["--trainer", "Sharded", "--model", "ComplEx", "--scoring_technique", "NegSample"])
    assert b.trainer == "Sharded" and b.scoring_technique == "NegSample"
