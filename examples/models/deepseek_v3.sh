# DeepSeek-V3 / R1 (fp8 checkpoint) on one 8 x B200 box: TP 8 attention, experts over all 8 GPUs,
# MTP speculative decoding, decode graphs for every batch size up to 128.
export MODEL=${MODEL:-/data/models/DeepSeek-V3} TP=8 ENABLE_EP=1 ENABLE_MTP=1
export MAX_NUM_SEQS=128 MAX_MODEL_LEN=32768 MAX_BATCHED_TOKENS=8192 BLOCK_SIZE=64 GPU_MEM_UTIL=0.92
