#!/bin/bash
# Container entrypoint: optional S3-backed model cache sync down before launch and up on SIGTERM, then the launcher.
# (Same contract as the reference's container-entrypoint.sh / sync.sh: HF_CACHE_BUCKET names the bucket.)
set -u
sync_down() { [ -n "${HF_CACHE_BUCKET:-}" ] && command -v aws >/dev/null && aws s3 sync "s3://${HF_CACHE_BUCKET}" "${HUGGINGFACE_HUB_CACHE:-/data}" --only-show-errors || true; }
sync_up() { [ -n "${HF_CACHE_BUCKET:-}" ] && command -v aws >/dev/null && aws s3 sync "${HUGGINGFACE_HUB_CACHE:-/data}" "s3://${HF_CACHE_BUCKET}" --only-show-errors || true; }
sync_down
lorax-launcher "$@" &
child=$!
trap 'kill -TERM "$child" 2>/dev/null; wait "$child"; sync_up; exit 0' TERM INT
wait "$child"
code=$?
sync_up
exit $code
