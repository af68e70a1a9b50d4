# openPangu Ultra MoE with its reasoning / tool-call parsers.
export MODEL=${MODEL:-/data/models/openPangu-Ultra-MoE} TP=8 ENABLE_EP=1 ENABLE_MTP=1
export REASONING_PARSER=pangu TOOL_CALL_PARSER=pangu MAX_NUM_SEQS=64 MAX_MODEL_LEN=32768 BLOCK_SIZE=64
