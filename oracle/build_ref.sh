#!/usr/bin/env bash
# Compiles the reference's own CUDA implementation of the quantized-matmul path -- its sources,
# where they lie in the read-only reference tree -- for sm_100a into oracle/_ref/libascendcl_ref.so.
# Used (a) on a B200 to produce the golden fixtures under tests/golden/ and (b) as the
# "reference CUDA backend on the same GPU" baseline.  Test infrastructure only; no reference source
# is copied into this repository, and oracle/_ref/ is git-ignored.
#
# The reference's vendor headers (acl/acl.h, aclnn/acl_meta.h, hccl/hccl_types.h) are not shipped
# with it; this repository's self-declared subset under include/ stands in for them.
set -euo pipefail
REF=${REFERENCE_ROOT:?set REFERENCE_ROOT to the reference source tree}
HERE=$(cd "$(dirname "$0")" && pwd)
OUT=$HERE/_ref
[ -d "$REF/cuda/src" ] || { echo "reference tree not found at $REF"; exit 1; }
mkdir -p "$OUT/obj"
FLAGS="-gencode arch=compute_100a,code=sm_100a -std=c++17 -O2 -Xcompiler -fPIC -I$REF/include -I$HERE/../include -I$REF/cuda/src"
for f in ops/matmul.cu ops/cast.cu meta.cu; do
  o=$OUT/obj/$(basename "$f" .cu).o
  if [ ! -f "$o" ] || [ "$REF/cuda/src/$f" -nt "$o" ]; then
    nvcc $FLAGS -c "$REF/cuda/src/$f" -o "$o"
  fi
done
gcc -O2 -fPIC -c "$HERE/ref_stubs.c" -o "$OUT/obj/ref_stubs.o"
nvcc -gencode arch=compute_100a,code=sm_100a -shared -cudart static -o "$OUT/libascendcl_ref.so" \
  "$OUT/obj/matmul.o" "$OUT/obj/cast.o" "$OUT/obj/meta.o" "$OUT/obj/ref_stubs.o" -lcublasLt -lcublas
echo "built $OUT/libascendcl_ref.so"
