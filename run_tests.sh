#!/usr/bin/env bash
# Test runner: `./run_tests.sh` (CPU suite), `./run_tests.sh gpu` (on a B200), `./run_tests.sh all`,
# `./run_tests.sh perf` (throughput floors on a B200; also added to gpu / all by RUSTRAL_RUN_GPU_PERF=1),
# `./run_tests.sh examples` (every example with its wall time; also added to all by RUSTRAL_RUN_EXAMPLE_PERF=1).
# RUSTRAL_REQUIRE_GPU=1 makes a missing GPU an error instead of a skip.
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
perf() { run "performance floors (B200)" python -m pytest tests -q -m perf; }
examples() { run "examples with wall times" python -m pytest tests/test_examples.py tests/test_examples_gallery.py -q --durations=0; }
case "$what" in
  cpu) run "CPU suite (oracle, framework, gloo multi-rank)" python -m pytest tests -q -m "not gpu" ;;
  gpu) run "GPU suite" python -m pytest tests -q -m gpu
       if [ "${RUSTRAL_RUN_GPU_PERF:-0}" = "1" ]; then perf; fi ;;
  perf) perf ;;
  examples) examples ;;
  all) run "CPU suite" python -m pytest tests -q -m "not gpu"
       run "GPU suite" python -m pytest tests -q -m gpu
       if [ "${RUSTRAL_RUN_GPU_PERF:-0}" = "1" ]; then perf; fi
       if [ "${RUSTRAL_RUN_EXAMPLE_PERF:-0}" = "1" ]; then examples; fi ;;
  *) echo "usage: $0 [cpu|gpu|perf|examples|all]" >&2; exit 2 ;;
esac
exit $failed
