# DeepSeek-V3.2 (sparse attention via the lightning indexer); chunked prefill is not combined
# with sparse attention, so prompts are prefilled whole.
export MODEL=${MODEL:-/data/models/DeepSeek-V3.2} TP=8 ENABLE_EP=1 ENABLE_MTP=1
export MAX_NUM_SEQS=64 MAX_MODEL_LEN=65536 MAX_BATCHED_TOKENS=65536 BLOCK_SIZE=64
export EXTRA_ARGS="--no-enable-chunked-prefill"
