#!/usr/bin/env bash
# Prefill / decode disaggregation on one 8-GPU box: a prefill instance on the first GPUs, a
# decode instance on the rest.  The decode instance pulls the KV blocks of a request from
# the prefill instance over NVLink (CUDA IPC mapping + one copy kernel per pull); control
# messages (pull acknowledgements, heartbeats) go over ZMQ on 127.0.0.1.
#
#   MODEL=/data/models/DeepSeek-V3 PREFILL_GPUS=0,1,2,3 DECODE_GPUS=4,5,6,7 ./examples/serve-pd-disaggregate.sh
#
# A client sends a request to the prefill endpoint with max_tokens=1, takes the
# kv_transfer_params of the answer and passes them to the decode endpoint.
set -euo pipefail

MODEL=${MODEL:-llama-3-8b}
PREFILL_GPUS=${PREFILL_GPUS:-0,1,2,3}
DECODE_GPUS=${DECODE_GPUS:-4,5,6,7}
PREFILL_PORT=${PREFILL_PORT:-8100}
DECODE_PORT=${DECODE_PORT:-8200}
KV_PORT=${KV_PORT:-30000}
MAX_MODEL_LEN=${MAX_MODEL_LEN:-8192}
count() { awk -F, '{print NF}' <<<"$1"; }
PREFILL_TP=$(count "$PREFILL_GPUS")
DECODE_TP=$(count "$DECODE_GPUS")

export PREFILL_POD_NUM=1 DECODE_POD_NUM=1

kv_cfg() {  # role rank
  printf '{"kv_connector":"LLMDataDistConnector","kv_role":"%s","kv_rank":%d,"kv_parallel_size":2,"kv_port":%d,"kv_connector_extra_config":{"kv_producer_dp_size":1}}' "$1" "$2" "$KV_PORT"
}

launch() {  # role gpus tp port kv_role kv_rank master_port
  ROLE=$1 CUDA_VISIBLE_DEVICES=$2 python -m torch.distributed.run --nnodes=1 --nproc-per-node "$3" \
      --master-addr 127.0.0.1 --master-port "$7" -m omni_npu_b200.serving.api_server \
      --model "$MODEL" --port "$4" --tensor-parallel-size "$3" --max-model-len "$MAX_MODEL_LEN" \
      --kv-transfer-config "$(kv_cfg "$5" "$6")" --enable-kv-rmsnorm-rope-cache ${EXTRA_ARGS:-} &
}

# prefill: large token budget, no decode graphs needed
EXTRA_ARGS="--max-num-batched-tokens 16384 --max-num-seqs 32 --enforce-eager" \
  launch prefill "$PREFILL_GPUS" "$PREFILL_TP" "$PREFILL_PORT" kv_producer 0 29601
# decode: many sequences, one CUDA graph per batch size
EXTRA_ARGS="--max-num-batched-tokens 2048 --max-num-seqs 128" \
  launch decode "$DECODE_GPUS" "$DECODE_TP" "$DECODE_PORT" kv_consumer 1 29602

trap 'kill $(jobs -p) 2>/dev/null || true' EXIT
wait
