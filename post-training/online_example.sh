#!/usr/bin/env bash
# Online REINFORCE-style post-training on one 8-GPU node: two sampling servers (4 GPUs each, any server with an
# OpenAI-compatible /v1/completions route, here vLLM), the online data server that scores their samples, and the
# trainer, which pulls batches from the data server (configs/post-training/llama3-8b-reinforce.yml) and pushes
# refreshed weights to the samplers through the weight server (gpt_neox_b200/models/weight_server.py).
# Reference flow: post-training/online_example.sh, post-training/online_training.md.
set -euo pipefail
MODEL=${MODEL:-meta-llama/Meta-Llama-3-8B-Instruct}

CUDA_VISIBLE_DEVICES=0,1,2,3 python -m vllm.entrypoints.openai.api_server --model "$MODEL" --dtype auto \
    --tensor-parallel-size 4 --enforce-eager --gpu-memory-utilization 0.2 --port 8000 --max-model-len 1024 &
CUDA_VISIBLE_DEVICES=4,5,6,7 python -m vllm.entrypoints.openai.api_server --model "$MODEL" --dtype auto \
    --tensor-parallel-size 4 --enforce-eager --gpu-memory-utilization 0.2 --port 8001 --max-model-len 1024 &

python post-training/online_data_server.py --dp-size 2 --batch-per-rank 64 --num-completions 4 \
    --tokenizer "$MODEL" --model "$MODEL" --endpoint 'http://localhost:{port}/v1/completions' \
    --endpoint-base-port 8000 --stop '<|eot_id|>' --eos-text '<|eot_id|>' \
    --prompts "${PROMPTS:-data/prompts.jsonl}" --reward-pipeline lvwerra/distilbert-imdb --reward-label POSITIVE &

python deepy.py train.py configs/post-training/llama3-8b-reinforce.yml
