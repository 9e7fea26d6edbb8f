#!/usr/bin/env bash
# TEST INFRASTRUCTURE.  Builds the CPU restatement (oracle/ft_oracle.cpp) into oracle/libft_oracle.so.
# IEEE arithmetic is kept as written: no fast-math, no FMA contraction.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
g++ -O2 -std=c++17 -fPIC -shared -fopenmp -ffp-contract=off -Wall -Wno-unused-function \
    "$HERE/ft_oracle.cpp" -o "$HERE/libft_oracle.so"
echo "built $HERE/libft_oracle.so"
