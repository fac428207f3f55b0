"""Locates the native extension `deep_ep._C`.

The extension is built in-tree (`python setup.py build_ext --inplace`). If it is missing this module
builds it once, unless `EP_NO_AUTO_BUILD=1`. Nothing here falls back to Python: a GPU box without
the extension fails at import.
"""
import importlib
import os
import subprocess
import sys

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _import():
    return importlib.import_module('deep_ep._C')


try:
    _C = _import()
except ImportError as first_error:  # pragma: no cover - exercised only on a fresh checkout
    if os.environ.get('EP_NO_AUTO_BUILD', '0') == '1' or not os.path.exists(os.path.join(_ROOT, 'setup.py')):
        raise
    print(f'[deep_ep] native extension missing ({first_error}); building in-tree ...', file=sys.stderr, flush=True)
    subprocess.check_call([sys.executable, 'setup.py', 'build_ext', '--inplace'], cwd=_ROOT,
                          stdout=subprocess.DEVNULL)
    importlib.invalidate_caches()
    _C = _import()
