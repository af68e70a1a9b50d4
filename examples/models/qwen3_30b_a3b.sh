# Qwen3-30B-A3B (MoE) with the token-sharded residual stream inside the TP group.
export MODEL=${MODEL:-/data/models/Qwen3-30B-A3B} TP=4 ENABLE_EP=1
export MAX_NUM_SEQS=256 MAX_MODEL_LEN=32768 BLOCK_SIZE=16
export EXTRA_ARGS='--additional-config {"sequence_parallel_residual":true}'
