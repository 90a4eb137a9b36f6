#!/usr/bin/env bash
# Test tiers of this repository (counterpart of the reference's scripts/run_ci_tests.sh and ci/gpu_tests.py).
#
#   ci/run_tests.sh cpu     everything that needs no GPU: semantics, parity against the reference package when it
#                           is installed under baseline/_ref, gloo multi-process paths, migration CLI, helpers
#   ci/run_tests.sh gpu     kernels against fp32 PyTorch definitions on one B200, one pytest process per file so a
#                           failure in one file cannot hide the others (the reference rents one machine per file)
#   ci/run_tests.sh multi   the 2-GPU data-parallel and FSDP tests
#   ci/run_tests.sh build   cross-compile every CUDA source for sm_100a (works without a GPU)
set -euo pipefail
cd "$(dirname "$0")/.."

export PYTHONWARNINGS="${PYTHONWARNINGS:+$PYTHONWARNINGS,}ignore:CUDA initialization:UserWarning,ignore:Can't initialize NVML:UserWarning"
FLAGS=(--maxfail=1 --disable-warnings -q --color=no -p no:cacheprovider)

case "${1:-cpu}" in
  build)
    python -c 'import __graft_entry__ as g; g.build()'
    ;;
  cpu)
    CUDA_VISIBLE_DEVICES="" python -m pytest "${FLAGS[@]}" tests -m "not gpu"
    ;;
  gpu)
    status=0
    for f in tests/test_*gpu*.py tests/test_zz_no_alloc.py; do
      case "$f" in *ddp*|*fsdp*) continue ;; esac
      echo "::group::$f"
      python -m pytest "${FLAGS[@]}" "$f" -m gpu --timeout 600 || status=1
      echo "::endgroup::"
    done
    exit $status
    ;;
  multi)
    python -m pytest "${FLAGS[@]}" tests/test_ddp_gpu.py -m gpu --timeout 900
    ;;
  *)
    echo "usage: $0 {cpu|gpu|multi|build}" >&2
    exit 2
    ;;
esac
