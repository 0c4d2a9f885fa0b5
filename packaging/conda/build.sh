#!/bin/bash
# Build the conda package: FAIRRING_VERSION=x.y.z packaging/conda/build.sh
set -euo pipefail
cd "$(dirname "$0")"
conda build . --no-anaconda-upload
