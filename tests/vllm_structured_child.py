"""Child process of the structured-output test: a vLLM ``LLM`` on this package's CPU platform with a
toy word-level tokenizer, one request constrained to a choice of two words, one free.  Prints one
JSON line."""
import json, os, sys, tempfile
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
os.environ["OMNI_B200_PLUGIN"] = "cpu"
os.environ["VLLM_ENABLE_V1_MULTIPROCESSING"] = "0"
os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")
os.environ.setdefault("VLLM_HOST_IP", "127.0.0.1")
from omni_npu_b200.plugin import write_entry_point_metadata
meta = tempfile.mkdtemp(prefix="omni_b200_meta_")
write_entry_point_metadata(meta)
sys.path.insert(0, meta)
os.environ["PYTHONPATH"] = os.pathsep.join([ROOT, meta, os.environ.get("PYTHONPATH", "")])
from tokenizers import Tokenizer, models, pre_tokenizers
from transformers import PreTrainedTokenizerFast
vocab = {"<unk>": 0, "<s>": 1, "</s>": 2}
for w in ["yes", "no", "maybe", "the", "a", "cat", "dog", "is", "red", "blue"] + [f"w{i}" for i in range(1024 - 13)]:
    vocab[w] = len(vocab)
tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
tok.pre_tokenizer = pre_tokenizers.Whitespace()
d = tempfile.mkdtemp(prefix="omni_b200_model_")
PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", bos_token="<s>", eos_token="</s>").save_pretrained(d)
cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 256, "intermediate_size": 512,
       "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 1024,
       "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 2048, "hidden_act": "silu",
       "tie_word_embeddings": False, "torch_dtype": "float32", "bos_token_id": 1, "eos_token_id": 2}
json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
from vllm import LLM, SamplingParams
from vllm.sampling_params import StructuredOutputsParams
llm = LLM(model=d, load_format="dummy", dtype="float32", max_model_len=256, max_num_seqs=4, max_num_batched_tokens=64,
          block_size=16, enforce_eager=True, seed=0, enable_prefix_caching=False, gpu_memory_utilization=0.3)
outs = llm.generate(["the cat is", "a dog is"],
                    [SamplingParams(max_tokens=4, temperature=0.0, structured_outputs=StructuredOutputsParams(choice=["red", "blue"])),
                     SamplingParams(max_tokens=4, temperature=0.0)], use_tqdm=False)
worker = llm.llm_engine.engine_core.engine_core.model_executor.driver_worker.worker
print("RESULT", json.dumps({"texts": [o.outputs[0].text for o in outs], "ids": [list(o.outputs[0].token_ids) for o in outs],
                            "steps": dict(worker.steps)}))
