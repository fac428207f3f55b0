#!/bin/sh
# In-place development build: compiles csrc/ for sm_100a and drops deep_ep/_C*.so next to the Python sources.
set -e
cd "$(dirname "$0")"
python setup.py build_ext --inplace
python csrc/generate_pyi.py
