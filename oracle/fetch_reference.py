"""Places an unmodified copy of the reference's Python package where the benchmark's reference arm looks for it.

    python oracle/fetch_reference.py [--reference <path to the reference project root>]

TEST / BENCHMARK INFRASTRUCTURE, not part of the product: nothing under ``neuralattentionsearch_b200`` imports it.

The reference is pure Python and its ``setup.py`` cannot be installed (its ``install_requires`` list lacks commas, so
metadata generation fails), therefore this copies ``src/nats`` as it is into ``baseline/_ref/nats`` -- a folder that is
git-ignored (no reference source enters the history) but travels with the working tree to the machine the benchmark
runs on.  ``bench.py --impl reference`` imports it from there, with stub modules for the files the reference imports
but does not ship (see ``load_reference`` below), and times the reference's own eager attention path on the host cores.
"""
from __future__ import annotations

import argparse
import os
import shutil
import sys
import types

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TARGET = os.path.join(ROOT, 'baseline', '_ref')


def default_reference_root() -> str:
    """The reference checkout: ``$NATS_REFERENCE_ROOT``, else a folder ``reference`` next to this repository."""
    return os.environ.get('NATS_REFERENCE_ROOT') or os.path.join(os.path.dirname(ROOT), 'reference')


def fetch(reference_root: str) -> str | None:
    src = os.path.join(reference_root, 'src', 'nats')
    if not os.path.isdir(src):
        return None
    dst = os.path.join(TARGET, 'nats')
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.makedirs(TARGET, exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns('__pycache__', '*.pyc'))
    return dst


def available() -> bool:
    return os.path.isfile(os.path.join(TARGET, 'nats', 'components', 'cache', 'dyn_cache.py'))


def load_reference():
    """Imports the reference's cache container and chunk attention layer from ``baseline/_ref``.  Four modules the
    reference imports but does not ship are stubbed (they are only used in training or on a GPU), the device-capability
    query it makes at import time is answered without a GPU, and its ``torch.compile`` decorators run eagerly."""
    import torch

    def stub(name, **attrs):
        m = types.ModuleType(name)
        m.__path__ = []
        for key, val in attrs.items():
            setattr(m, key, val)
        sys.modules[name] = m
    stub('nats.components.cache.triton')
    stub('nats.components.cache.triton.update_one_step', post_update_one_step=None)
    stub('nats.models.transformer.triton.flashattention_mask_on_chip', nats_attention=None)
    stub('nats.models.transformer.triton.nats_chunk_attention', nats_chunk_attention=None)
    torch.cuda.get_device_capability = lambda *a, **k: (10, 0)
    torch.cuda.empty_cache = lambda *a, **k: None
    import torch._dynamo as dynamo
    dynamo.config.disable = True
    if TARGET not in sys.path:
        sys.path.insert(0, TARGET)
    from nats.components.cache.dyn_cache import NAtSCache
    from nats.models.transformer.attention.nats_chunk_attention import LlamaNAtSChunkAttentionLayer
    return NAtSCache, LlamaNAtSChunkAttentionLayer


if __name__ == '__main__':
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', default=default_reference_root())
    where = fetch(ap.parse_args().reference)
    print(where or 'reference project not found: nothing copied')
