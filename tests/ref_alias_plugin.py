"""pytest plugin that lets the reference project's own test files run UNMODIFIED against this
repository's drop-in modules.  Loaded (``-p ref_alias_plugin``) only by the child pytest process
that ``tests/test_reference_suite.py`` starts; it installs a package called ``src`` whose
sub-modules are:

  src.voting       mdlarc_scale_b200.voting
  src.data         mdlarc_scale_b200.data, falling back to the reference's own module for the names
                   the hot path does not cover (the training dataset / sampler / collate classes)
  src.transformer  the reference's module (the weight contract is a reference TinyTransformer); with
                   ARCB_REF_ALIAS=gpu its create_*_model factories return the model wrapped in
                   B200TinyTransformer, so that calling the model runs the B200 engine
  src.inference    with ARCB_REF_ALIAS=gpu: mdlarc_scale_b200.inference; otherwise the reference's

The reference files come from ``oracle/_ref`` (see ``oracle/make_ref.py``).
"""
import os
import sys
import types
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


class _Fallback(types.ModuleType):
    """Attribute lookup in ``first``, then in ``second``."""

    def __init__(self, name, first, second):
        super().__init__(name)
        self.__dict__["_first"] = first
        self.__dict__["_second"] = second

    def __getattr__(self, item):
        try:
            return getattr(self.__dict__["_first"], item)
        except AttributeError:
            return getattr(self.__dict__["_second"], item)


def _install():
    from oracle import make_ref
    from mdlarc_scale_b200 import data as my_data
    from mdlarc_scale_b200 import voting as my_voting
    gpu = os.environ.get("ARCB_REF_ALIAS", "host") == "gpu"
    ref = make_ref.load_reference_modules("arcref")
    pkg = types.ModuleType("src")
    pkg.__path__ = []
    mods = {"src": pkg, "src.voting": my_voting, "src.data": _Fallback("src.data", my_data, ref["data"])}
    if gpu:
        from mdlarc_scale_b200 import inference as my_inference
        from mdlarc_scale_b200.transformer import B200TinyTransformer
        tr = _Fallback("src.transformer", types.SimpleNamespace(
            create_tiny_model=lambda *a, **k: B200TinyTransformer(ref["transformer"].create_tiny_model(*a, **k)),
            create_small_model=lambda *a, **k: B200TinyTransformer(ref["transformer"].create_small_model(*a, **k)),
        ), ref["transformer"]) if os.environ.get("ARCB_REF_WRAP_MODEL") == "1" else ref["transformer"]
        mods["src.transformer"] = tr
        mods["src.inference"] = my_inference
    else:
        mods["src.transformer"] = ref["transformer"]
        mods["src.inference"] = ref["inference"]
    for name, mod in mods.items():
        sys.modules[name] = mod
        if "." in name:
            setattr(pkg, name.split(".", 1)[1], mod)


_install()
