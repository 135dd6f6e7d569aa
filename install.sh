#!/usr/bin/env bash
# Builds the native libraries in-tree and installs the package in development mode.
#   ./install.sh            build (needs nvcc with sm_100a support for the kernel library; g++ for the host libraries)
#                           and `pip install -e .`
#   ./install.sh --no-pip   build only; use the checkout through PYTHONPATH
set -euo pipefail
cd "$(dirname "$0")"
python -m rustral_b200._build
python -m rustral_b200.utils.check_env || true
if [ "${1:-}" != "--no-pip" ]; then
  python -m pip install --no-build-isolation --no-deps -e .
fi
echo "done: python -c 'import rustral_b200; print(rustral_b200.__file__)'"
