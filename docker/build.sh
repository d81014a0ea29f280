#!/bin/bash
# Builds the serving image from the repository root:  docker/build.sh [tag]
set -euo pipefail
cd "$(dirname "$0")/.."
docker build -f docker/Dockerfile -t "${1:-lightllm_b200:latest}" .
