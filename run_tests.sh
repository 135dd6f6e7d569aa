#!/usr/bin/env bash
# Test runner: `./run_tests.sh` (CPU suite), `./run_tests.sh gpu` (on a B200), `./run_tests.sh all`.
# Builds the in-tree libraries first when nvcc is available and one of them is missing.
set -euo pipefail
cd "$(dirname "$0")"
what="${1:-cpu}"
if ! python -m rustral_b200.utils.check_env >/dev/null 2>&1; then
  if command -v nvcc >/dev/null 2>&1 || [ -x /usr/local/cuda/bin/nvcc ]; then
    echo "--- building the in-tree libraries ---"
    python -m rustral_b200._build
  fi
fi
python -m rustral_b200.utils.check_env || true
failed=0
run() {
  echo ""
  echo "--- $1 ---"
  shift
  if "$@"; then echo "PASS"; else echo "FAIL"; failed=1; fi
}
case "$what" in
  cpu) run "CPU suite (oracle, framework, gloo multi-rank)" python -m pytest tests -q -m "not gpu" ;;
  gpu) run "GPU suite" python -m pytest tests -q -m gpu ;;
  all) run "CPU suite" python -m pytest tests -q -m "not gpu"
       run "GPU suite" python -m pytest tests -q -m gpu ;;
  *) echo "usage: $0 [cpu|gpu|all]" >&2; exit 2 ;;
esac
exit $failed
