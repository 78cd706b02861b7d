"""Acceptance: the reference project's own hot-path test files, run unmodified against this
repository's modules by import aliasing (``tests/ref_alias_plugin.py``).

The files are the copies ``oracle/make_ref.py`` places under ``oracle/_ref`` (git-ignored; made from a
reference checkout where one is present, and shipped with the working tree).  When neither the copies
nor a checkout exist the tests skip.

  * CPU: ``tests/test_voting.py`` in full, and the tokenisation / position / dihedral / colour
    classes of ``tests/test_data.py`` (its dataset, batching and training-integration classes test the
    training data pipeline, which is outside the inference path: they are deselected);
  * GPU: ``tests/test_inference.py`` in full with ``src.inference`` aliased to the drop-in, and the
    full-model and generation classes of ``tests/test_transformer.py`` with the model factories
    returning the B200-backed wrapper (``test_backward_pass`` needs autograd, which the inference
    engine does not provide: deselected).
"""
import os
import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "oracle" / "_ref"


@pytest.fixture(scope="module")
def ref_tests():
    from oracle import make_ref
    if not make_ref.available() and not make_ref.make():
        pytest.skip("no reference checkout and no oracle/_ref copy: run `python oracle/make_ref.py <path>`")
    return REF / "tests"


def _run(files, env_extra, extra_args=()):
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([str(ROOT / "tests"), str(ROOT), env.get("PYTHONPATH", "")])
    env["PYTHONDONTWRITEBYTECODE"] = "1"
    env.update(env_extra)
    cmd = [sys.executable, "-m", "pytest", "-q", "-p", "ref_alias_plugin", "-p", "no:cacheprovider",
           "--import-mode=importlib", "--rootdir", str(REF), "-c", os.devnull, *extra_args, *map(str, files)]
    res = subprocess.run(cmd, capture_output=True, text=True, cwd=str(REF), env=env, timeout=1500)
    tail = (res.stdout + res.stderr)[-3000:]
    m = re.search(r"(\d+) passed", res.stdout)
    return res.returncode, int(m.group(1)) if m else 0, tail


def test_reference_voting_tests_pass_unmodified(ref_tests):
    rc, passed, tail = _run([ref_tests / "test_voting.py"], {"ARCB_REF_ALIAS": "host"})
    print(f"reference tests/test_voting.py against mdlarc_scale_b200.voting: {passed} passed")
    assert rc == 0 and passed >= 30, tail


def test_reference_data_codec_tests_pass_unmodified(ref_tests):
    rc, passed, tail = _run([ref_tests / "test_data.py"], {"ARCB_REF_ALIAS": "host"},
                            ["-k", "TestTokenization or TestPositions or TestDihedralTransforms or TestColorAugmentation"])
    print(f"reference tests/test_data.py (codec classes) against mdlarc_scale_b200.data: {passed} passed")
    assert rc == 0 and passed >= 25, tail


@pytest.mark.gpu
def test_reference_inference_tests_pass_unmodified_on_the_gpu(ref_tests):
    rc, passed, tail = _run([ref_tests / "test_inference.py"], {"ARCB_REF_ALIAS": "gpu"})
    print(f"reference tests/test_inference.py against mdlarc_scale_b200.inference: {passed} passed")
    assert rc == 0 and passed >= 14, tail


@pytest.mark.gpu
def test_reference_full_model_tests_pass_on_the_wrapped_model(ref_tests):
    rc, passed, tail = _run([ref_tests / "test_transformer.py"], {"ARCB_REF_ALIAS": "gpu", "ARCB_REF_WRAP_MODEL": "1"},
                            ["-k", "(TestTinyTransformer or TestGeneration) and not test_backward_pass"])
    print(f"reference tests/test_transformer.py (full-model classes) on B200TinyTransformer: {passed} passed")
    assert rc == 0 and passed >= 7, tail
