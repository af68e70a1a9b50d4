#!/usr/bin/env bash
# Serve one model instance on the GPUs of this box with the standalone engine.
#
#   MODEL=/data/models/Llama-3-8B TP=1 PORT=8000 ./examples/serve-single-instance.sh
#   source examples/models/deepseek_v3.sh && ./examples/serve-single-instance.sh
#
# One process per GPU: for TP > 1 the server is started under torch.distributed.run, every
# rank runs the same scheduler (SPMD) and rank 0 answers HTTP.
set -euo pipefail

MODEL=${MODEL:-llama-3-8b}                 # preset name or HF checkpoint directory
TP=${TP:-1}
DP=${DP:-1}
PORT=${PORT:-8000}
MAX_NUM_SEQS=${MAX_NUM_SEQS:-128}
MAX_MODEL_LEN=${MAX_MODEL_LEN:-8192}
MAX_BATCHED_TOKENS=${MAX_BATCHED_TOKENS:-8192}
BLOCK_SIZE=${BLOCK_SIZE:-16}
GPU_MEM_UTIL=${GPU_MEM_UTIL:-0.9}
ENABLE_EP=${ENABLE_EP:-0}                  # expert parallelism for MoE models
ENABLE_MTP=${ENABLE_MTP:-0}                # speculative decoding with the model's MTP head
GRAPH_SIZES=${GRAPH_SIZES:-}               # e.g. "1,2,4,8,16,32,64,128" (default: automatic gears)
EXTRA_ARGS=${EXTRA_ARGS:-}

export OMNI_B200_TRACE=${OMNI_B200_TRACE:-0}
export NCCL_DEBUG=${NCCL_DEBUG:-WARN}

args=(--model "$MODEL" --port "$PORT" --tensor-parallel-size "$TP" --data-parallel-size "$DP"
      --max-num-seqs "$MAX_NUM_SEQS" --max-model-len "$MAX_MODEL_LEN"
      --max-num-batched-tokens "$MAX_BATCHED_TOKENS" --block-size "$BLOCK_SIZE"
      --gpu-memory-utilization "$GPU_MEM_UTIL" --enable-kv-rmsnorm-rope-cache)

if [[ -n "$GRAPH_SIZES" ]]; then
  args+=(--compilation-config "{\"cudagraph_mode\":\"FULL_DECODE_ONLY\",\"cudagraph_capture_sizes\":[${GRAPH_SIZES}]}")
fi
[[ "$ENABLE_EP" == "1" ]] && args+=(--enable-expert-parallel)
[[ "$ENABLE_MTP" == "1" ]] && args+=(--speculative-config '{"num_speculative_tokens":1,"method":"deepseek_mtp"}')
[[ -n "${REASONING_PARSER:-}" ]] && args+=(--reasoning-parser "$REASONING_PARSER")
[[ -n "${TOOL_CALL_PARSER:-}" ]] && args+=(--tool-call-parser "$TOOL_CALL_PARSER")

if [[ "$TP" -gt 1 || "$DP" -gt 1 ]]; then
  exec python -m torch.distributed.run --nnodes=1 --nproc-per-node $((TP * DP)) \
       --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29500}" \
       -m omni_npu_b200.serving.api_server "${args[@]}" $EXTRA_ARGS
fi
exec python -m omni_npu_b200.serving.api_server "${args[@]}" $EXTRA_ARGS
