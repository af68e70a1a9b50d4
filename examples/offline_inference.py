"""Offline generation with the standalone engine (token ids in, token ids out).

    python examples/offline_inference.py --model llama-3-8b --max-tokens 32
"""
import argparse

from omni_npu_b200 import LLM, SamplingParams

ap = argparse.ArgumentParser()
ap.add_argument("--model", default="tiny-llama")
ap.add_argument("--max-tokens", type=int, default=16)
ap.add_argument("--device", default="auto")
args = ap.parse_args()

llm = LLM(model=args.model, device=args.device, load_format="dummy")
outs = llm.generate([[1, 2, 3, 4, 5], [9, 8, 7]], SamplingParams(max_tokens=args.max_tokens, ignore_eos=True))
for o in outs:
    print(o.request_id, o.output_token_ids, f"ttft={o.ttft:.4f}s" if o.ttft else "")
