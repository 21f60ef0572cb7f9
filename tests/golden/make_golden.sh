#!/bin/bash
# Regenerates the golden records in this directory by running the UNMODIFIED reference library on a
# GPU through oracle/_ref/ref_harness (built by `make -C oracle ref` where the reference checkout is
# present). Each record holds per-limb content hashes of every stage of the key-switching path on
# synthetic limbs that the CPU oracle can regenerate from the seed.
#   usage: tests/golden/make_golden.sh [OUT_DIR]     (default: this directory)
set -euo pipefail
HERE="$(cd "$(dirname "$0")" && pwd)"
ROOT="$(cd "$HERE/../.." && pwd)"
OUT="${1:-$HERE}"
H="$ROOT/oracle/_ref/ref_harness"
mkdir -p "$OUT"
B40x23=$(printf '40,%.0s' $(seq 23))
# small cases: every stage, ragged last digits, alpha = 1, 2, 3
"$H" --logn 12 --bits 50,36,36,36,36,36,50,50 --special 2 --level 6 --seed 7 --steps 1,2,-1 --out "$OUT/n12_l6_a2.json"
"$H" --logn 12 --bits 50,36,36,36,36,36,50,50 --special 2 --level 5 --seed 8 --steps 3,0 --out "$OUT/n12_l5_a2.json"
"$H" --logn 13 --bits 60,40,40,40,40,40,40,60,60,60 --special 3 --level 7 --seed 9 --steps 1,-2 --out "$OUT/n13_l7_a3.json"
"$H" --logn 13 --bits 60,40,40,40,40,40,40,60,60,60 --special 3 --level 4 --seed 10 --steps 5 --out "$OUT/n13_l4_a3.json"
# BSGS matrix-vector driver (chained baby rotations, fused MAC, Horner over giants, one rescale)
"$H" --logn 12 --bits 50,36,36,36,36,36,50,50 --special 2 --level 6 --seed 12 --steps 1,2,4 --bsgs 4,2 --out "$OUT/n12_bsgs_m4g2.json"
"$H" --logn 13 --bits 60,40,40,40,40,40,40,60,60,60 --special 3 --level 5 --seed 13 --steps 1,2 --bsgs 2,3 --out "$OUT/n13_bsgs_m2g3.json"
# the NTT configuration: N = 2^14, 8 limbs of 50 bits, seed 0 (alpha = 1 exercises the single-P path)
"$H" --logn 14 --bits 50,50,50,50,50,50,50,50 --special 1 --level 7 --seed 0 --steps 1 --out "$OUT/n14_ntt8x50.json"
"$H" --logn 15 --bits 58,45,45,45,45,45,45,45,45,58,58 --special 2 --level 9 --seed 11 --steps 1,64 --out "$OUT/n15_l9_a2.json"
# the key-switching configuration: N = 2^16, 24 Q limbs (60 + 23 x 40 bits), 8 special 60-bit primes, dnum 3
"$H" --logn 16 --bits 60,${B40x23}60,60,60,60,60,60,60,60 --special 8 --level 24 --seed 2 --steps 1,2,-1 --time 40 --out "$OUT/n16_l24_a8.json"
"$H" --logn 16 --bits 60,${B40x23}60,60,60,60,60,60,60,60 --special 8 --level 16 --seed 3 --steps 1,64 --time 40 --out "$OUT/n16_l16_a8.json"
"$H" --logn 16 --bits 60,${B40x23}60,60,60,60,60,60,60,60 --special 8 --level 5 --seed 4 --steps 7 --time 40 --out "$OUT/n16_l5_a8.json"
