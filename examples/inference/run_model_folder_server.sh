#!/bin/bash
# Serve a model folder (config.json naming a registered architecture, e.g. Zikunex, + model.safetensors) with the dynamic engine:
# paged latents for the latent-attention layers, one state row per request for the recurrent layers, continuous batching.
#   MODEL_DIR=/path/to/folder examples/inference/run_model_folder_server.sh                       # REST on $PORT
#   MODEL_DIR=... examples/inference/run_model_folder_server.sh --prompts "5 9 23" --num-tokens-to-generate 16
ROOT="$(cd "$(dirname "$0")/../.." && pwd)"
python "$ROOT/tools/run_text_generation_server.py" --model-dir "${MODEL_DIR:?set MODEL_DIR}" --dtype ${DTYPE:-bfloat16} \
  --port ${PORT:-5000} --inference-max-requests ${MAX_REQUESTS:-16} --cache-tokens ${CACHE_TOKENS:-65536} "$@"
