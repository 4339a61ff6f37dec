#!/usr/bin/env bash
# Checks to run before a commit (counterpart of the reference's scripts/pre_commit.sh):
# format check, import order, the kernel library build and the CPU test suite.
#
#   ./pre_commit.sh            all checks
#   ./pre_commit.sh --no-tests skip pytest
#   ./pre_commit.sh --fix      let ruff rewrite formatting and import order first
set -uo pipefail

cd "$(dirname "$0")"
[ -d khaosz_b200 ] && [ -d tests ] || { echo "pre_commit.sh: run from the repository root" >&2; exit 1; }

run_tests=1
fix=0
for arg in "$@"; do
    case "$arg" in
        --no-tests) run_tests=0 ;;
        --fix) fix=1 ;;
        *) echo "pre_commit.sh: unknown flag $arg" >&2; exit 1 ;;
    esac
done

failed=()
step() {            # step NAME CMD...
    local name="$1"; shift
    echo "== $name"
    "$@" || failed+=("$name")
}

if command -v ruff >/dev/null 2>&1; then
    if [ "$fix" = 1 ]; then
        ruff format khaosz_b200 tests bench.py __graft_entry__.py
        ruff check --select I --fix khaosz_b200 tests bench.py __graft_entry__.py
    fi
    step "format (ruff format --check)" ruff format --check khaosz_b200 tests bench.py __graft_entry__.py
    step "import order (ruff check --select I)" ruff check --select I khaosz_b200 tests bench.py __graft_entry__.py
else
    echo "== ruff not installed: format and import checks skipped"
fi
step "python sources compile" python -m compileall -q khaosz_b200 tests bench.py __graft_entry__.py
if command -v nvcc >/dev/null 2>&1; then
    step "kernel library builds for sm_100a" python -c "import __graft_entry__ as g; g.build()"
else
    echo "== nvcc not found: kernel build skipped"
fi
if [ "$run_tests" = 1 ]; then
    step "CPU tests" python -m pytest tests/ -x -q -m "not gpu"
fi

if [ ${#failed[@]} -gt 0 ]; then
    printf 'FAILED: %s\n' "${failed[@]}" >&2
    exit 1
fi
echo "all checks passed"
