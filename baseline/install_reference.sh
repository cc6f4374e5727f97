#!/bin/bash
# Put the reference's GDPA package where its own absolute imports (ads_mkl.ops.oss.gdpa...) resolve:
#   baseline/_ref/ads_mkl/ops/oss/gdpa  <-  <reference root>/gdpa
# baseline/_ref is git-ignored; it travels to the GPU box with the working tree.  The reference has no
# setup.py / pyproject for its root, so there is nothing for pip to install: its kernels are Python DSL
# sources that compile themselves at the first call.
#   usage: baseline/install_reference.sh /path/to/ads_model_kernel_library
set -e
ref=${1:?usage: install_reference.sh /path/to/ads_model_kernel_library}
here=$(cd "$(dirname "$0")" && pwd)
dst=$here/_ref/ads_mkl/ops/oss
mkdir -p "$dst"
rm -rf "$dst/gdpa"
cp -r "$ref/gdpa" "$dst/gdpa"
rm -rf "$dst/gdpa/assets"
echo "installed $(find "$dst/gdpa" -name '*.py' | wc -l) python files under $dst/gdpa"
