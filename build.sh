#!/bin/sh
# Builds a wheel (dist/deep_ep-*.whl) that contains the extension, the Python package and the kernel headers
# the run-time compiler needs (deep_ep/include).
set -e
cd "$(dirname "$0")"
python setup.py bdist_wheel
