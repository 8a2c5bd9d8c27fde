"""Imports the mirrored reference package (``oracle/_ref``, made by ``oracle/build_ref.py``).  TEST INFRASTRUCTURE ONLY:
tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may call it; the product package never
does.  Nothing of the reference is modified on disk; what newer library releases need is patched at import time:

* ``LEAN_USE_JIT=0``: TorchScript rejects the ``torch.dtype`` annotation of lean_transformer/rotary.py:48;
* ``LeanGPTConfig.__hash__`` / ``LeanAlbertConfig.__hash__``: transformers >= 5 re-wraps config subclasses as
  dataclasses, which drops the ``__hash__`` (lean_transformer/config.py:143-144) that the ``lru_cache``d factory
  methods of the config need;
* ``all_tied_weights_keys = {}`` on the model classes: they call ``init_weights()`` rather than ``post_init()``
  (lean_transformer/models/gpt.py:202).
"""
import os
import sys
import warnings
from pathlib import Path
from types import SimpleNamespace
from typing import Optional

REF_DIR = Path(__file__).resolve().parent / "_ref"
_cached = None


def available() -> bool:
    return (REF_DIR / "lean_transformer" / "ffn.py").is_file()


def import_reference() -> Optional[SimpleNamespace]:
    """The reference's modules as a namespace (ffn, linear, native_backend, layout, utils, transformer, attn, gpt,
    config, package), or None when ``oracle/_ref`` has not been built."""
    global _cached
    if _cached is not None:
        return _cached
    if not available():
        return None
    os.environ.setdefault("LEAN_USE_JIT", "0")
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        import lean_transformer as package
        from lean_transformer import attn, config, ffn, transformer, utils
        from lean_transformer.blocksparse import layout, linear, native_backend
        from lean_transformer.models import albert, gpt
    base_hash = config.LeanTransformerConfig.__hash__
    for cls in (gpt.LeanGPTConfig, albert.LeanAlbertConfig):
        cls.__hash__ = base_hash
    for name in ("LeanGPTModel", "LeanGPTForPreTraining", "LeanAlbertModel", "LeanAlbertForPreTraining"):
        for module in (gpt, albert):
            cls = getattr(module, name, None)
            if cls is not None:
                cls.all_tied_weights_keys = {}
    _cached = SimpleNamespace(package=package, ffn=ffn, linear=linear, native_backend=native_backend, layout=layout,
                              utils=utils, transformer=transformer, attn=attn, gpt=gpt, albert=albert, config=config)
    return _cached
