#!/bin/bash
# SageMaker: map the platform's environment onto launcher settings (HF_MODEL_ID -> MODEL_ID, SM_NUM_GPUS -> NUM_SHARD,
# port 8080, /invocations and /ping are served by the router).
if [[ -z "${HF_MODEL_ID:-}" ]]; then echo "HF_MODEL_ID must be set"; exit 1; fi
export MODEL_ID="${HF_MODEL_ID}"
[[ -n "${HF_MODEL_REVISION:-}" ]] && export REVISION="${HF_MODEL_REVISION}"
[[ -n "${SM_NUM_GPUS:-}" ]] && export NUM_SHARD="${SM_NUM_GPUS}"
[[ -n "${HF_MODEL_QUANTIZE:-}" ]] && export QUANTIZE="${HF_MODEL_QUANTIZE}"
exec lorax-launcher --port 8080
