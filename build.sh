#!/bin/bash
# Build and test driver (the role of the reference's build.sh: --pkg, -u/--ut, -s/--st, --asan).
#
#   ./build.sh                 build hccl_b200/lib/libhccl_b200.so (nvcc, sm_100a only; g++ for host code)
#   ./build.sh --force         rebuild every object
#   ./build.sh --asan          also build the AddressSanitizer variant of the host code
#   ./build.sh -u | --ut       build, then the unit tier: step tables, config, selector, verifier self-tests, Python layers
#   ./build.sh -s | --st       build, then the host-engine tier: every algorithm on simulated ranks with trace verification
#   ./build.sh --gpu           build, then the device tier (needs a B200)
#   ./build.sh --cov           coverage build of the host code, the unit and host-engine tiers against it, line coverage per file
#   ./build.sh --pkg           build, then pack library + headers + Python package + examples into dist/hccl_b200-<version>.tar.gz
set -euo pipefail
cd "$(dirname "$0")"
PY=${PYTHON:-python}
force=""; asan=0; ut=0; st=0; gpu=0; pkg=0; cov=0
for a in "$@"; do
  case "$a" in
    --force) force="--force" ;;
    --asan) asan=1 ;;
    -u|--ut) ut=1 ;;
    -s|--st) st=1 ;;
    --gpu) gpu=1 ;;
    --pkg) pkg=1 ;;
    --cov) cov=1 ;;
    -h|--help) sed -n 2,13p "$0"; exit 0 ;;
    *) echo "unknown option $a" >&2; exit 2 ;;
  esac
done
$PY hccl_b200/build.py $force
if [ $asan -eq 1 ]; then $PY hccl_b200/build.py --asan; fi
if [ $ut -eq 1 ]; then
  $PY -m pytest -q -m "not gpu" tests/test_unit_tables_config_selector.py tests/test_verifier_selftests.py tests/test_cpu_python_layers.py \
      tests/test_graph_mode_api.py tests/test_examples_build.py tests/test_tuner_workflow.py tests/test_kernel_harness_cpu.py
fi
if [ $st -eq 1 ]; then
  $PY -m pytest -q -m "not gpu" tests/test_host_engine.py tests/test_host_executors.py tests/test_host_retry.py
  if [ $asan -eq 1 ]; then $PY -m pytest -q tests/test_asan_host_engine.py; fi
fi
if [ $cov -eq 1 ]; then
  covlib=$($PY hccl_b200/build.py --cov | tail -1)
  rm -f build/obj_cov/*.gcda
  HCCL_B200_LIB=$covlib $PY -m pytest -q -m "not gpu" tests/test_unit_tables_config_selector.py tests/test_verifier_selftests.py \
      tests/test_graph_mode_api.py tests/test_host_engine.py tests/test_host_executors.py tests/test_host_retry.py tests/test_rank_table.py \
      tests/test_offline_bindings.py tests/test_context_parallel.py tests/test_data_parallel.py
  $PY hccl_b200/build.py --cov-report
fi
if [ $gpu -eq 1 ]; then $PY -m pytest -q -m gpu tests; fi
if [ $pkg -eq 1 ]; then
  version=$($PY -c "import ctypes, pathlib; l = ctypes.CDLL(str(pathlib.Path('hccl_b200/lib/libhccl_b200.so').resolve())); l.HcclGetVersion.restype = ctypes.c_char_p; print(l.HcclGetVersion().decode().split()[-1])")
  stage=$(mktemp -d)
  root="$stage/hccl_b200-$version"
  mkdir -p "$root/lib" "$root/include" "$root/python" dist
  cp hccl_b200/lib/libhccl_b200.so "$root/lib/"
  cp -r csrc/include/hccl "$root/include/"
  tar -C . --exclude='__pycache__' --exclude='*.so' -cf - hccl_b200 | tar -C "$root/python" -xf -
  mkdir -p "$root/python/hccl_b200/lib" && cp hccl_b200/lib/libhccl_b200.so "$root/python/hccl_b200/lib/"
  cp -r examples docs README.md "$root/"
  tar -C "$stage" -czf "dist/hccl_b200-$version.tar.gz" "hccl_b200-$version"
  rm -rf "$stage"
  echo "dist/hccl_b200-$version.tar.gz"
fi
