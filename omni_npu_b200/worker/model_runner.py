"""Standalone model runner: owns the model, the paged KV cache, the persistent
input batch and the CUDA-graph cache, and turns a scheduler output into
sampled token ids.

It is self-contained (it does not derive from vLLM's GPU model runner, which
the reference does: omni_npu/worker/npu_model_runner.py:68).  Responsibilities
matching the reference's runner: ``load_model`` (+ graph wrapping, :237-272),
``get_kv_cache_spec`` / ``initialize_kv_cache`` (:125-187), ``capture_model``
(:274-281), ``execute_model`` / ``sample_tokens`` (:283-297) and
``_dummy_run`` (:306-583).

Decode steps replay a CUDA graph that contains the whole step: embedding,
all layers (attention reads lengths and block tables from device buffers),
LM head and sampling.  Prefill steps run eagerly.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..attention.gqa import GQABackend
from ..attention.metadata import AttentionMetadata, set_forward_context
from ..compilation.cuda_graph import CUDAGraphRunner
from ..config import EngineConfig
from ..engine.scheduler import SchedulerOutput
from ..logger import logger
from ..models.registry import resolve_model_cls
from ..models.utils import iter_safetensors, random_init_
from ..parallel import state as pstate
from ..sample.rejection_sampler import RejectionSampler, SpecDecodeMetadata
from ..sample.sampler import Sampler
from .input_batch import InputBatch, StepLayout


@dataclass
class KVCacheSpec:
    kind: str                  # "gqa" | "mla" | "dsa"
    num_layers: int
    block_size: int
    bytes_per_block: int       # all layers of this rank
    shapes: Dict[str, Tuple[int, ...]]


class ModelRunner:
    def __init__(self, config: EngineConfig, device: torch.device) -> None:
        self.config = config
        self.device = device
        self.model_config = config.model
        self.model: Optional[torch.nn.Module] = None
        self.kv_caches: List = []
        self.num_blocks = 0
        sc = config.scheduler
        dcp = config.parallel.decode_context_parallel_size
        self.input_batch = InputBatch(sc.max_num_seqs, sc.max_model_len, config.cache.block_size,
                                      sc.max_num_batched_tokens, device, cp_world=dcp,
                                      cp_rank=pstate.get_tp_group().rank_in_group if dcp > 1 else 0)
        self.input_batch.base_seed = int(config.seed or 0)
        self.sampler = Sampler(config, device)
        self.rejection_sampler = RejectionSampler(self.sampler)
        self.graphs: Dict[int, CUDAGraphRunner] = {}
        self.capture_sizes: List[int] = []
        pin = device.type == "cuda"
        self.sampled_host = torch.zeros(max(sc.max_num_seqs, 1), dtype=torch.int32, pin_memory=pin)
        # with a draft head: the sampled token and its k drafts per sequence
        self.mtp_k = max(1, int(config.speculative.num_speculative_tokens or 1))
        self.sampled_host2 = torch.zeros(max(sc.max_num_seqs, 1), 1 + self.mtp_k, dtype=torch.int32, pin_memory=pin)
        # Penalties and the thinking-token budget work on each request's token history, which lives
        # on the host: a step that needs them runs eagerly with ``_logits_fn`` set (never from a
        # graph, never launched ahead of the previous step's tokens).
        self._logits_fn = None
        from ..sample.logits_processors import ThinkingTokenBudgetLogitsProcessor
        from ..serving.reasoning_config import ReasoningConfig
        rc = ReasoningConfig.from_cli(config.additional_config.get("reasoning_config"))
        self.thinking_processor = ThinkingTokenBudgetLogitsProcessor(rc, sc.max_num_seqs, device)
        self.mtp = None                       # the model's multi-token-prediction head, if it drafts
        self.last_drafts: List[List[int]] = []
        self.extra_logits_fn = None
        self.structured = None      # sample/structured.py manager, once a tokenizer is known
        self.last_logprobs: Dict[int, Tuple[float, List[Tuple[int, float]]]] = {}   # of the last step, by index in its seqs
        self._lp_capture = None
        # log-probabilities of prompt tokens: the plan of the step in flight, what it captured on the
        # device, and the result by index in the step's seqs: (position of the first entry, entries)
        self._plp_plan = None
        self._plp_capture = None
        self.last_prompt_logprobs: Dict[int, Tuple[int, list]] = {}
        self.step_counter = torch.zeros(1, dtype=torch.int64, device=device)
        self.d2h_bytes_last = 0
        self.kv_connector = None
        pp = pstate.get_pp_group()
        self.pp_group = pp if pp.world_size > 1 else None     # set: this rank runs one pipeline stage
        pcp = pstate.get_pcp_group()
        self.pcp_group = pcp if pcp.world_size > 1 else None  # set: prefill steps are split over these ranks
        # decode steps of such a deployment: every rank decodes every sequence (default), or each
        # sequence is decoded by one rank of the group (additional_config["pcp_decode_split"])
        self.pcp_decode_split = bool((config.additional_config or {}).get("pcp_decode_split", False))
        self._pcp_owner = {}
        self.pcp_decode_rows = 0
        self.timings: Dict[str, float] = {}
        # optional device-side timing of every step (CUDA events around the kernels)
        self.enable_step_events = False
        self._step_events: List[Tuple[torch.cuda.Event, torch.cuda.Event, str]] = []
        self.step_ms_by_kind: Dict[str, float] = {}      # device time per kind of step, filled by drain_step_events
        self.step_count_by_kind: Dict[str, int] = {}

    # ------------------------------------------------------------------ model
    def load_model(self) -> None:
        cfg = self.config
        t0 = time.time()
        cls = resolve_model_cls(cfg.model.architecture)
        prev = torch.get_default_dtype()
        torch.set_default_dtype(cfg.model.dtype)
        try:
            self.model = cls(cfg, device=self.device)
        finally:
            torch.set_default_dtype(prev)
        if self.pp_group is not None and not callable(getattr(self.model, "make_empty_intermediate_tensors", None)):
            raise ValueError(f"{type(self.model).__name__} does not implement pipeline stages "
                             "(pipeline_parallel_size > 1 needs make_empty_intermediate_tensors)")
        if cfg.model_path and cfg.load_format != "dummy":
            loaded = self.model.load_weights(iter_safetensors(cfg.model_path))
            logger.info("loaded %d tensors from %s", len(loaded), cfg.model_path)
        else:
            random_init_(self.model, seed=cfg.seed, by_name=True if self.pp_group is not None else None)
        for m in self.model.modules():
            hook = getattr(m, "process_weights_after_loading", None)
            if callable(hook):
                hook()
        post = getattr(self.model, "post_load", None)
        if callable(post):
            post()
        self.model.eval()
        if cfg.speculative.method in ("mtp", "deepseek_mtp") and cfg.speculative.num_speculative_tokens > 0:
            self.mtp = getattr(self.model, "mtp", None)
            if self.mtp is None:
                raise ValueError(f"{type(self.model).__name__} has no multi-token-prediction head")
        tp = pstate.get_tp_group()
        ep = pstate.get_ep_group()
        tp.comm.prepare_communication_buffer_for_model(self.model)
        if ep is not tp:
            ep.comm.prepare_communication_buffer_for_model(self.model)
        self.timings["load_model_s"] = time.time() - t0

    def get_model(self) -> torch.nn.Module:
        return self.model

    # --------------------------------------------------------------- KV cache
    def get_kv_cache_spec(self) -> KVCacheSpec:
        mc = self.model_config
        bs = self.config.cache.block_size
        tp = pstate.tp_world_size()
        spec_fn = getattr(self.model, "get_kv_cache_spec", None)
        if callable(spec_fn):
            return spec_fn(bs)
        hk = max(1, mc.num_kv_heads // tp)
        per_layer = GQABackend.bytes_per_block(bs, hk, mc.head_dim, mc.dtype)
        k_shape, v_shape = GQABackend.get_kv_cache_shape(1, bs, hk, mc.head_dim)
        n_layers = getattr(self.model, "num_kv_layers", mc.num_layers)
        return KVCacheSpec("gqa", n_layers, bs, per_layer * n_layers,
                           {"k": k_shape[1:], "v": v_shape[1:]})

    @torch.inference_mode()
    def profile_run(self) -> int:
        """One eager prefill-shaped forward with the largest token count to find
        the activation peak.  Returns peak bytes allocated during the run."""
        if self.device.type != "cuda":
            return 0
        torch.cuda.synchronize(self.device)
        torch.cuda.reset_peak_memory_stats(self.device)
        before = torch.cuda.memory_allocated(self.device)
        sc = self.config.scheduler
        self._init_kv_cache_tensors(num_blocks=max(8, sc.max_num_batched_tokens // self.config.cache.block_size + 8))
        self._dummy_run(num_tokens=sc.max_num_batched_tokens, prefill=True)
        torch.cuda.synchronize(self.device)
        peak = torch.cuda.max_memory_allocated(self.device) - before
        self.kv_caches = []
        torch.cuda.empty_cache()
        return peak

    def determine_num_blocks(self) -> int:
        cc = self.config.cache
        if cc.num_gpu_blocks:
            return cc.num_gpu_blocks
        spec = self.get_kv_cache_spec()
        if self.device.type != "cuda":
            return max(64, 4 * self.config.scheduler.max_num_seqs)
        peak = self.profile_run()
        free, total = torch.cuda.mem_get_info(self.device)
        budget = int(total * cc.gpu_memory_utilization) - (total - free) - peak
        n = budget // spec.bytes_per_block
        sc = self.config.scheduler
        # never take more than every sequence at full length could use
        cap = sc.max_num_seqs * ((sc.max_model_len + cc.block_size - 1) // cc.block_size) + 64
        n = int(min(n, cap))
        if n < 16:
            raise RuntimeError(f"not enough memory for the KV cache (budget {budget} bytes)")
        logger.info("KV cache: %d blocks of %d tokens (%.2f GiB), activation peak %.2f GiB", n,
                    cc.block_size, n * spec.bytes_per_block / 2**30, peak / 2**30)
        return n

    def _init_kv_cache_tensors(self, num_blocks: int) -> None:
        alloc = getattr(self.model, "allocate_kv_cache", None)
        if callable(alloc):
            self.kv_caches = alloc(num_blocks, self.config.cache.block_size, self.device)
        else:
            mc = self.model_config
            hk = max(1, mc.num_kv_heads // pstate.tp_world_size())
            self.kv_caches = [GQABackend.allocate_kv_cache(num_blocks, self.config.cache.block_size,
                                                           hk, mc.head_dim, mc.dtype, self.device)
                              for _ in range(getattr(self.model, "num_kv_layers", mc.num_layers))]
        self.num_blocks = num_blocks

    def initialize_kv_cache(self, num_blocks: int) -> None:
        self._init_kv_cache_tensors(num_blocks)
        if self.kv_connector is not None:
            self.kv_connector.register_kv_caches(self.kv_caches)

    # ------------------------------------------------------------- execution
    def _metadata(self, lay: StepLayout, views, is_prefill: bool, num_seqs: int, num_tokens: int,
                  max_q_len: int, max_seq_len: int, q_len: int, actual_tokens: int,
                  actual_seqs: int) -> AttentionMetadata:
        return AttentionMetadata(is_prefill=is_prefill, num_seqs=num_seqs, num_tokens=num_tokens,
                                 max_q_len=max_q_len, max_seq_len=max_seq_len, q_len=q_len,
                                 positions=views["pos"], slot_mapping=views["slot"],
                                 block_tables=views["bt"], seq_lens=views["seq_lens"],
                                 cu_q=views["cu_q"], num_actual_tokens=actual_tokens,
                                 num_actual_seqs=actual_seqs)

    def _forward_and_sample(self, views, md: AttentionMetadata, num_samples: int) -> torch.Tensor:
        """Model forward + LM head + sampling for the staged step (device side only).
        Returns the sampled tokens [num_samples]; with an MTP head int32 [num_samples, 1 + k]:
        the sampled token and the k drafts for the tokens after it."""
        if self.pp_group is not None:
            return self._forward_and_sample_pipeline(views, md, num_samples)
        with set_forward_context(md, self.kv_caches, self.config):
            hidden_all = self.model(views["ids"], views["pos"])
            idx = views["logits_idx"][:num_samples].long() if md.is_prefill else None
            hidden = hidden_all.index_select(0, idx) if idx is not None else hidden_all[:num_samples]
            logits = self.model.compute_logits(hidden)
            if self._plp_plan:
                self._capture_prompt_logprobs(hidden_all)
            if self._logits_fn is not None:
                logits = self._logits_fn(logits)
            # (no step offset: the staged seed of a row already carries the index of the token it samples)
            sampled = self.sampler(logits, views["temp"][:num_samples], views["top_k"][:num_samples],
                                   views["top_p"][:num_samples], views["seeds"][:num_samples], None)
            if self.mtp is None:
                return sampled
            # successor of every fed token: known for prompt tokens, the fresh sample otherwise
            tok = sampled.to(torch.int32)
            if idx is not None:
                nxt = views["next_ids"].clone()
                cur = nxt.index_select(0, idx)
                nxt.index_copy_(0, idx, torch.where(cur < 0, tok, cur))
            else:
                nxt = views["next_ids"].clone()
                nxt[:num_samples] = tok
                nxt.clamp_(min=0)
            h = self.model.mtp_forward(nxt, views["pos"], hidden_all)
            h = h.index_select(0, idx) if idx is not None else h[:num_samples]
            draft = ops.argmax(self.model.mtp_logits(h)).to(torch.int32)
            drafts = [draft]
            if self.mtp_k > 1:
                pos = views["pos"]
                last = pos.index_select(0, idx) if idx is not None else pos[:num_samples]
                drafts += self._mtp_chain(h, draft, last, views["bt"][:num_samples], md)
        return torch.stack([tok] + drafts, dim=1)

    def _decode_split_pcp(self, out: SchedulerOutput, ib, n: int) -> List[int]:
        """A decode step of a prefill-context-parallel deployment with every sequence decoded by ONE
        rank of the group.  After its prompt (whose keys every rank holds) a sequence gets an owner,
        the least loaded rank at that moment (all ranks run the same scheduler on the same inputs, so
        they agree without talking); only the owner attends to and stores the sequence's new keys.
        Each rank runs one forward pass per step, a dummy batch when it owns nothing, so that
        expert-parallel exchanges stay in step; the sampled tokens are gathered over the group."""
        if self._logits_fn is not None:
            raise NotImplementedError("prefill context parallelism: logits processors are not supported")
        g = self.pcp_group
        P, r = g.world_size, g.rank_in_group
        rids = [s.request.request_id for s in out.seqs]
        load = [0] * P
        for rid in rids:
            if rid in self._pcp_owner:
                load[self._pcp_owner[rid]] += 1
        for rid in rids:
            if rid not in self._pcp_owner:
                j = load.index(min(load))
                self._pcp_owner[rid] = j
                load[j] += 1
        self._pcp_owner = {rid: self._pcp_owner[rid] for rid in rids}        # finished requests drop out
        lists = [[i for i, rid in enumerate(rids) if self._pcp_owner[rid] == j] for j in range(P)]
        mine, cap = lists[r], max(load)
        ev = self._event_start()
        buf = torch.full((cap,), -1, dtype=torch.int32, device=self.device)
        if mine:
            m = len(mine)
            reqs = [out.seqs[i].request for i in mine]
            padded = self._pad_decode_size(m) if self.graphs else None
            S = padded or m
            lay = ib.layout_for(S, S)
            ib.stage_decode(lay, reqs)
            ib.upload(lay)
            if padded is not None:
                sampled = self.graphs[padded].replay()
            else:
                views = ib.views(lay, ib.dev)
                md = self._metadata(lay, views, False, S, S, 1, self.config.scheduler.max_model_len, 1, m, m)
                sampled = self._forward_and_sample(views, md, S)
            buf[:m] = sampled[:m].to(torch.int32)
            self.pcp_decode_rows += m
        else:
            self._dummy_run(1, prefill=False)
        got = g.all_gather(buf, dim=0).view(P, cap)
        self.step_counter += 1
        self._event_stop(ev, out.kind)
        host = got.cpu() if self.device.type != "cuda" else self._to_host(got)
        self.d2h_bytes_last = P * cap * 4
        rows = host.tolist()
        tokens = [0] * n
        for j in range(P):
            for k, i in enumerate(lists[j]):
                tokens[i] = int(rows[j][k])
        return tokens

    def _forward_and_sample_pcp(self, views, seqs, T: int, max_seq: int) -> torch.Tensor:
        """A prefill step split over the ranks of the prefill-context-parallel group.  The step is
        staged in full on every rank (all ranks run the same scheduler); this rank runs the model on
        tokens [lo, hi) of the flat batch.  Each attention layer gathers the step's keys and values
        from all ranks, writes ALL of them into the local cache and attends with its own query rows
        (``attention/gqa.py``), so afterwards every rank holds the whole KV cache.  A sequence's
        next token is sampled by the rank that owns its last row and shared with a max-reduction.
        (vLLM's prefill context parallelism, which the reference's model patches assume around
        their MoE block: omni_npu/vllm_patches/patches/models/pangu72b-vl/patch_fusedmoe.py:148-159.)"""
        if self._logits_fn is not None or self.mtp is not None:
            raise NotImplementedError("prefill context parallelism: logits processors and draft heads are not supported")
        if getattr(self, "_pcp_checked", None) is None:
            # every module that writes this step's keys into the cache must gather the other shards'
            lacking = sorted({type(m).__name__ for m in self.model.modules()
                              if hasattr(m, "layer_idx") and "Attention" in type(m).__name__
                              and not getattr(m, "supports_prefill_context_parallel", False)})
            if lacking:
                raise NotImplementedError(f"prefill context parallelism is not supported by {', '.join(lacking)}")
            self._pcp_checked = True
        g = self.pcp_group
        P, r = g.world_size, g.rank_in_group
        dev = self.device
        self.pcp_steps = getattr(self, "pcp_steps", 0) + 1
        bounds = [j * T // P for j in range(P + 1)]           # every rank gets at least one token
        lo, hi = bounds[r], bounds[r + 1]
        sizes = [bounds[j + 1] - bounds[j] for j in range(P)]
        pad = max(sizes)
        # rows of the gathered [P * pad] tensor that hold real tokens, in flat-batch order
        gather_idx = torch.tensor([j * pad + i for j in range(P) for i in range(sizes[j])], dtype=torch.long,
                                  device=dev)
        own_seq, own_q, own_len, cu = [], [], [], [0]
        owner_of_last, off = [], 0
        for i, s in enumerate(seqs):
            cs, ce = off, off + s.num_new_tokens
            a, b = max(cs, lo), min(ce, hi)
            if b > a:
                own_seq.append(i)
                own_q.append(b - a)
                own_len.append(s.start + (b - cs))            # keys up to this rank's last row of the sequence
                cu.append(cu[-1] + (b - a))
            owner_of_last.append(lo <= ce - 1 < hi)
            off = ce
        idx_seq = torch.tensor(own_seq, dtype=torch.long, device=dev)
        md = AttentionMetadata(
            is_prefill=True, num_seqs=len(own_seq), num_tokens=hi - lo, max_q_len=max(own_q),
            max_seq_len=max_seq, q_len=0, positions=views["pos"][lo:hi], slot_mapping=views["slot"][lo:hi],
            block_tables=views["bt"].index_select(0, idx_seq).contiguous(),
            seq_lens=torch.tensor(own_len, dtype=torch.int32, device=dev),
            cu_q=torch.tensor(cu, dtype=torch.int32, device=dev), num_actual_tokens=hi - lo,
            num_actual_seqs=len(own_seq))
        md.extra["seq_lens_host"] = own_len
        md.extra["pcp"] = {"group": g, "pad": pad, "gather_idx": gather_idx, "positions_all": views["pos"][:T],
                           "slot_all": views["slot"][:T]}
        n = len(seqs)
        tokens = torch.full((n,), -1, dtype=torch.int32, device=dev)
        with set_forward_context(md, self.kv_caches, self.config):
            hidden = self.model(views["ids"][lo:hi], views["pos"][lo:hi])
            mine = [i for i in range(n) if owner_of_last[i] and seqs[i].samples]
            if mine:
                sel = torch.tensor(mine, dtype=torch.long, device=dev)
                rows = (views["logits_idx"][:n].long().index_select(0, sel) - lo)
                logits = self.model.compute_logits(hidden.index_select(0, rows))
                seeds = views["seeds"][:n].index_select(0, sel)
                got = self.sampler(logits, views["temp"][:n].index_select(0, sel),
                                   views["top_k"][:n].index_select(0, sel), views["top_p"][:n].index_select(0, sel),
                                   seeds, None)
                tokens.index_copy_(0, sel, got.to(torch.int32))
        # a token id is >= 0 and exactly one rank holds it: the maximum over the group is the token
        import torch.distributed as dist
        dist.all_reduce(tokens, op=dist.ReduceOp.MAX, group=g.device_group)
        return tokens.clamp_(min=0)

    def _mtp_chain(self, h: torch.Tensor, draft: torch.Tensor, last_pos: torch.Tensor, bt: torch.Tensor,
                   md: AttentionMetadata) -> List[torch.Tensor]:
        """Draft tokens 2..k of a draft head that is run as a chain: step j feeds the token drafted
        by step j - 1 and that step's hidden state at position ``last_pos + j`` (a one-token decode
        step of the head's own cache layer; the scheduler keeps these slots allocated).  Everything
        is computed on the device, so the chain is part of a captured decode step.  Same flow as the
        draft loop of the reference's proposer (omni_npu/vllm_patches/patches/common/patch_eagle.py:417-560)."""
        n = h.shape[0]
        bs = self.config.cache.block_size
        cu = torch.arange(n + 1, dtype=torch.int32, device=h.device)
        out = []
        for j in range(1, self.mtp_k):
            pos = (last_pos + j).to(torch.int32)
            blk_idx = (pos // bs).clamp(max=bt.shape[1] - 1).long().unsqueeze(1)
            slot = (bt.gather(1, blk_idx).squeeze(1) * bs + pos % bs).to(torch.int32)
            md_j = AttentionMetadata(is_prefill=False, num_seqs=n, num_tokens=n, max_q_len=1,
                                     max_seq_len=md.max_seq_len + j, q_len=1, positions=pos, slot_mapping=slot,
                                     block_tables=bt, seq_lens=pos + 1, cu_q=cu, num_actual_tokens=n,
                                     num_actual_seqs=n)
            with set_forward_context(md_j, self.kv_caches, self.config):
                h = self.model.mtp_forward(draft.clamp_min(0), pos, h, spec_step=j)
                draft = ops.argmax(self.model.mtp_logits(h)).to(torch.int32)
            out.append(draft)
        return out

    def _forward_and_sample_pipeline(self, views, md: AttentionMetadata, num_samples: int) -> torch.Tensor:
        """One step of this rank's pipeline stage.  Activations travel stage to stage with
        point-to-point sends inside the pipeline group; the last stage computes logits and
        samples, then broadcasts the tokens so that every rank's scheduler (all ranks run the
        same deterministic scheduler) books the same result.
        (reference: intermediate-tensor buffers in omni_npu/worker/npu_model_runner.py:494-508,
        ``send``/``recv`` in omni_npu/distributed/communicator.py:247-257)"""
        pp = self.pp_group
        T = views["ids"].shape[0]
        it = None
        if not pp.is_first_rank:
            it = self.model.make_empty_intermediate_tensors(T, self.model_config.dtype, self.device)
            for _, t in sorted(it.items()):
                pp.comm.recv(t.shape, t.dtype, src=pp.rank_in_group - 1, out=t)
        with set_forward_context(md, self.kv_caches, self.config):
            out = self.model(views["ids"], views["pos"], intermediate_tensors=it)
            if pp.is_last_rank:
                idx = views["logits_idx"][:num_samples].long() if md.is_prefill else None
                hidden = out.index_select(0, idx) if idx is not None else out[:num_samples]
                logits = self.model.compute_logits(hidden)
                if self._logits_fn is not None:
                    logits = self._logits_fn(logits)
                sampled = self.sampler(logits, views["temp"][:num_samples], views["top_k"][:num_samples],
                                       views["top_p"][:num_samples], views["seeds"][:num_samples],
                                       None).to(torch.int64)
            else:
                for _, t in sorted(out.items()):
                    pp.comm.send(t.contiguous(), dst=pp.rank_in_group + 1)
                sampled = torch.empty(num_samples, dtype=torch.int64, device=self.device)
        return pp.comm.broadcast(sampled, src=pp.world_size - 1)

    def _forward_and_verify(self, views, md: AttentionMetadata, seqs) -> torch.Tensor:
        """Verification step of speculative decoding: logits at every fed position, target
        tokens sampled there, drafts accepted while they agree.  Returns int32
        [n, max_k + 2 (+k)]: the settled tokens (-1 padded), their count and, with an MTP
        head, the k drafts for the next step."""
        n = len(seqs)
        with set_forward_context(md, self.kv_caches, self.config):
            hidden = self.model(views["ids"], views["pos"])
            logits = self.model.compute_logits(hidden)
            smd = SpecDecodeMetadata.make([s.spec_token_ids for s in seqs], self.device)
            toks, counts = self.rejection_sampler(smd, None, logits, views["temp"][:n], views["top_k"][:n],
                                                  views["top_p"][:n], views["seeds"][:n],
                                                  self.step_counter)
            cols = [toks, counts.unsqueeze(1)]
            if self.mtp is not None:
                # fed token j of sequence i is followed by verified token (i, j); the draft for
                # the next step comes from the last verified position
                nxt = toks.reshape(-1).index_select(0, views["next_ids"].long()).clamp_min(0)
                h = self.model.mtp_forward(nxt, views["pos"], hidden)
                rows = (views["cu_q"][:n] + counts - 1).long()
                h_last = h.index_select(0, rows)
                draft = ops.argmax(self.model.mtp_logits(h_last)).to(torch.int32)
                cols.append(draft.unsqueeze(1))
                if self.mtp_k > 1:
                    last = views["pos"].index_select(0, rows)
                    cols += [d.unsqueeze(1) for d in self._mtp_chain(h_last, draft, last, views["bt"][:n], md)]
        return torch.cat(cols, dim=1)

    @staticmethod
    def needs_host_logits(req) -> bool:
        """Whether sampling for this request needs its token history (penalties, thinking budget)."""
        sp = req.sampling_params
        return (sp.has_penalties or sp.thinking_token_budget is not None or bool(sp.logprobs)
                or sp.structured is not None or bool(sp.logit_bias) or sp.min_p > 0
                or bool(sp.allowed_token_ids) or bool(sp.bad_words_token_ids)
                or (sp.min_tokens > 0 and len(req.output_token_ids) < sp.min_tokens))

    def enable_structured_outputs(self, tokenizer) -> None:
        """Structured outputs need the tokenizer's vocabulary (token id -> text)."""
        from ..sample.structured import StructuredOutputManager
        self.structured = StructuredOutputManager(tokenizer, self.config.model.vocab_size)

    def _penalty_cache(self, vocab: int):
        """The device-resident penalty state (created on first use: most workloads never ask)."""
        pc = getattr(self, "_pen_cache", None)
        if pc is None or pc.vocab_size != vocab:
            from ..sample.sampler_cache import PenaltyCache
            pc = PenaltyCache(max(8, 2 * self.config.scheduler.max_num_seqs), vocab, self.device)
            self._pen_cache = pc
        return pc

    def _make_logits_fn(self, seqs):
        """Logits adjustment for one step, or None when no scheduled sequence asks for any.
        Row i of the logits belongs to ``seqs[i]``.  Penalties: occurrence counts of the generated
        tokens and a mask of the prompt's tokens are built on the device from the token lists
        (only for the rows that ask), then ``apply_penalties``
        (reference: omni_npu/sample/sampler.py:115-158).  Thinking budget: the per-request state
        machine forces the end-of-thinking marker once the budget is spent."""
        from ..sample.sampler import apply_penalties
        use_pen = self.config.use_penalty
        pen_rows = [i for i, s in enumerate(seqs)
                    if s.samples and use_pen and s.request.sampling_params.has_penalties]
        tp = self.thinking_processor
        think_rows = [i for i, s in enumerate(seqs) if s.samples and tp.enabled
                      and s.request.sampling_params.thinking_token_budget is not None]
        # log-probabilities: of the model's own distribution (before penalties, temperature and
        # truncation), for the sampled token and the most likely tokens
        lp_rows = [i for i, s in enumerate(seqs) if s.samples and s.request.sampling_params.logprobs]
        self._lp_capture = None
        # a logits adjustment supplied for this one step by whoever drives the runner (the vLLM
        # worker's grammar bitmask): applied last, to the rows of ``seqs`` in order
        extra = getattr(self, "extra_logits_fn", None)
        # structured outputs: the request's grammar says which tokens may come next
        so = self.structured
        so_rows = [i for i, s in enumerate(seqs) if s.samples and s.request.sampling_params.structured is not None]
        if so_rows and so is None:
            raise RuntimeError("a request asks for structured output but the engine has no tokenizer "
                               "(LLM.enable_structured_outputs)")
        # logit bias, and end tokens held back until min_tokens outputs exist
        bias_rows = [i for i, s in enumerate(seqs) if s.samples and s.request.sampling_params.logit_bias]
        min_rows = [i for i, s in enumerate(seqs) if s.samples and s.request.sampling_params.min_tokens > 0
                    and len(s.request.output_token_ids) < s.request.sampling_params.min_tokens]
        allow_rows = [i for i, s in enumerate(seqs) if s.samples and s.request.sampling_params.allowed_token_ids]
        bad_rows = [i for i, s in enumerate(seqs) if s.samples and s.request.sampling_params.bad_words_token_ids]
        minp_rows = [i for i, s in enumerate(seqs) if s.samples and s.request.sampling_params.min_p > 0]
        if not pen_rows and not think_rows and not lp_rows and not so_rows and not bias_rows and not min_rows \
                and not allow_rows and not minp_rows and not bad_rows and extra is None:
            return None
        for i in think_rows:
            r = seqs[i].request
            if r.request_id not in tp.state:
                tp.add_request(r.request_id, r.prompt_token_ids, r.sampling_params.thinking_token_budget)
        dev = self.device

        def fn(logits: torch.Tensor) -> torch.Tensor:
            logits = logits.float()
            V = logits.shape[-1]
            if lp_rows:
                self._lp_capture = (lp_rows, torch.log_softmax(
                    logits.index_select(0, torch.tensor(lp_rows, device=dev)), dim=-1))
            if pen_rows:
                # per-request prompt mask and occurrence counts live on the device from admission
                # to completion; a step adds only the tokens generated since the last one
                pc = self._penalty_cache(V)
                rids = []
                for i in pen_rows:
                    r = seqs[i].request
                    if not pc.has(r.request_id):
                        pc.add_request(r.request_id, r.prompt_token_ids)
                    pc.sync_from_history(r.request_id, r.output_token_ids)
                    rids.append(r.request_id)
                sps = [seqs[i].request.sampling_params for i in pen_rows]
                idx = torch.tensor(pen_rows, device=dev)
                sub = pc.apply(
                    logits.index_select(0, idx), pc.slot_index(rids),
                    torch.tensor([sp.presence_penalty for sp in sps], dtype=torch.float32, device=dev),
                    torch.tensor([sp.frequency_penalty for sp in sps], dtype=torch.float32, device=dev),
                    torch.tensor([sp.repetition_penalty for sp in sps], dtype=torch.float32, device=dev))
                logits = logits.index_copy(0, idx, sub)
            if think_rows:
                idx = torch.tensor(think_rows, device=dev)
                sub = tp.apply(logits.index_select(0, idx).clone(),
                               [seqs[i].request.request_id for i in think_rows],
                               [seqs[i].request.output_token_ids for i in think_rows])
                logits = logits.index_copy(0, idx, sub)
            for i in bias_rows:
                lb = seqs[i].request.sampling_params.logit_bias
                ids = torch.tensor([int(t) for t in lb if 0 <= int(t) < V], dtype=torch.long, device=dev)
                vals = torch.tensor([float(v) for t, v in lb.items() if 0 <= int(t) < V], dtype=torch.float32, device=dev)
                logits[i, ids] += vals
            for i in min_rows:
                r = seqs[i].request
                ends = set(r.sampling_params.stop_token_ids or ())
                if r.eos_token_id is not None and not r.sampling_params.ignore_eos:
                    ends.add(r.eos_token_id)
                ends = [t for t in ends if 0 <= t < V]
                if ends:
                    logits[i, torch.tensor(ends, dtype=torch.long, device=dev)] = float("-inf")
            for i in allow_rows:
                ok = torch.tensor([int(t) for t in seqs[i].request.sampling_params.allowed_token_ids if 0 <= int(t) < V],
                                  dtype=torch.long, device=dev)
                keep = torch.zeros(V, dtype=torch.bool, device=dev)
                keep[ok] = True
                logits[i] = logits[i].masked_fill(~keep, float("-inf"))
            for i in bad_rows:
                out_ids = list(seqs[i].request.output_token_ids)
                banned = [int(w[-1]) for w in seqs[i].request.sampling_params.bad_words_token_ids
                          if len(w) and 0 <= int(w[-1]) < V
                          and (len(w) == 1 or (len(out_ids) >= len(w) - 1
                                               and out_ids[len(out_ids) - len(w) + 1:] == [int(t) for t in w[:-1]]))]
                if banned:
                    logits[i, torch.tensor(banned, dtype=torch.long, device=dev)] = float("-inf")
            for i in minp_rows:
                sp = seqs[i].request.sampling_params
                p = torch.softmax(logits[i] / max(float(sp.temperature), 1e-5), dim=-1)
                logits[i] = logits[i].masked_fill(p < sp.min_p * p.max(), float("-inf"))
            if so_rows:
                rids = []
                for i in so_rows:
                    r = seqs[i].request
                    if not so.has(r.request_id):
                        so.add_request(r.request_id, r.sampling_params.structured)
                    rids.append(r.request_id)
                idx = torch.tensor(so_rows, device=dev)
                sub = so.apply(logits.index_select(0, idx), rids, [seqs[i].request.output_token_ids for i in so_rows])
                logits = logits.index_copy(0, idx, sub)
            if extra is not None:
                logits = extra(logits)
            return logits
        return fn

    def _plan_prompt_logprobs(self, out: SchedulerOutput):
        """Rows of a prefill step whose next prompt token is known and asked about:
        [(index in seqs, first row, rows, position of the first predicted token, k)].  A step's rows
        are its sequences' new tokens in order; row j of a sequence fed from ``start`` predicts the
        prompt token at ``start + j + 1``."""
        plan, row = [], 0
        for i, q in enumerate(out.seqs):
            k = q.request.sampling_params.prompt_logprobs
            if k is not None:
                rows = min(q.num_new_tokens, q.request.num_prompt_tokens - 1 - q.start)
                if rows > 0:
                    plan.append((i, row, rows, q.start + 1, int(k)))
            row += q.num_new_tokens
        return plan or None

    def _capture_prompt_logprobs(self, hidden_all: torch.Tensor) -> None:
        """Log-probabilities of the planned prompt tokens and their most likely alternatives, kept on
        the device until the step's tokens are read (LM head on at most 1024 rows at a time)."""
        cap = []
        for i, row, rows, first, k, targets in self._plp_plan:
            lps, tops = [], []
            for a in range(0, rows, 1024):
                b = min(rows, a + 1024)
                lsm = torch.log_softmax(self.model.compute_logits(hidden_all[row + a: row + b]).float(), dim=-1)
                lps.append(lsm.gather(1, targets[a:b].unsqueeze(1)).squeeze(1))
                if k > 0:
                    tops.append(lsm.topk(k, dim=-1))
            cap.append((i, first, torch.cat(lps), torch.cat([t.values for t in tops]) if tops else None,
                        torch.cat([t.indices for t in tops]) if tops else None))
        self._plp_capture = cap

    def _collect_prompt_logprobs(self) -> Dict[int, Tuple[int, list]]:
        cap, self._plp_capture = self._plp_capture, None
        res = {}
        for i, first, lp, vals, ids in cap or ():
            lp = lp.tolist()
            vals = vals.tolist() if vals is not None else [[]] * len(lp)
            ids = ids.tolist() if ids is not None else [[]] * len(lp)
            res[i] = (first, [(lp[j], list(zip(ids[j], vals[j]))) for j in range(len(lp))])
        return res

    def _collect_logprobs(self, seqs, tokens) -> Dict[int, Tuple[float, List[Tuple[int, float]]]]:
        """Log-probabilities of this step's sampled tokens for the sequences that asked:
        {index in seqs: (log-probability of the token, [(token id, log-probability)] of the top k,
        rank of the token among all tokens)}."""
        cap, self._lp_capture = getattr(self, "_lp_capture", None), None
        if cap is None:
            return {}
        rows, logp = cap
        ks = [min(20, int(seqs[i].request.sampling_params.logprobs)) for i in rows]
        top_v, top_i = logp.topk(max(ks), dim=-1)
        tok = torch.tensor([int(tokens[i]) for i in rows], device=logp.device).unsqueeze(1)
        picked = logp.gather(1, tok).squeeze(1)
        rank = ((logp > picked.unsqueeze(1)).sum(dim=1) + 1).cpu().tolist()      # 1 = the most likely token
        top_v, top_i, picked = top_v.cpu().tolist(), top_i.cpu().tolist(), picked.cpu().tolist()
        return {i: (picked[j], list(zip(top_i[j][: ks[j]], top_v[j][: ks[j]])), rank[j]) for j, i in enumerate(rows)}

    def _pad_decode_size(self, n: int) -> Optional[int]:
        for s in self.capture_sizes:
            if s >= n:
                return s
        return None

    @torch.inference_mode()
    def execute_model(self, out: SchedulerOutput) -> List[int]:
        """Run one scheduled step; returns one sampled token per scheduled sequence
        (meaningless for sequences whose chunk does not end their prompt)."""
        ib = self.input_batch
        for rid in out.finished_req_ids:
            ib.remove_request(rid)
            self.thinking_processor.remove_request(rid)
            if getattr(self, "_pen_cache", None) is not None:
                self._pen_cache.remove_request(rid)
            if self.structured is not None:
                self.structured.remove_request(rid)
        for rid in out.preempted:
            ib.remove_request(rid)
        if self.kv_connector is not None and out.kv_connector_metadata is not None:
            self.kv_connector.start_load_kv(out.kv_connector_metadata)
        if out.kind == "idle" or not out.seqs:
            return []
        n = len(out.seqs)
        ev = None
        self.last_logprobs = {}
        self._logits_fn = self._make_logits_fn(out.seqs) if out.kind != "spec_decode" else None
        self.last_prompt_logprobs = {}
        if out.kind == "prefill" and any(q.request.sampling_params.prompt_logprobs is not None for q in out.seqs):
            plan = self._plan_prompt_logprobs(out) or []
            self._plp_plan = [p + (torch.tensor(out.seqs[p[0]].request.prompt_token_ids[p[3]: p[3] + p[2]],
                                                dtype=torch.long, device=self.device),) for p in plan]
        try:
            tokens = self._execute_scheduled(out, ib, n, ev)
            self.last_prompt_logprobs = self._collect_prompt_logprobs()
            return tokens
        finally:
            self._logits_fn = None
            self._plp_plan = self._plp_capture = None

    def _execute_scheduled(self, out: SchedulerOutput, ib, n: int, ev) -> List[int]:
        if out.kind == "spec_decode":
            T = out.num_tokens
            lay = ib.layout_for(T, n)
            _, max_q = ib.stage_spec_decode(lay, out.seqs)
            ib.upload(lay)
            ev = self._event_start()
            views = ib.views(lay, ib.dev)
            max_seq = max(s.start + s.num_new_tokens for s in out.seqs)
            md = self._metadata(lay, views, True, n, T, max_q, max_seq, 0, T, n)
            packed = self._forward_and_verify(views, md, out.seqs)
            self.step_counter += max_q
            self._event_stop(ev, "spec_decode")
            host = packed.cpu() if self.device.type != "cuda" else self._to_host(packed)
            self.d2h_bytes_last = packed.numel() * 4
            rows = host.tolist()
            if self.mtp is not None:
                k = self.mtp_k
                self.last_drafts = [r[-k:] for r in rows]
                return [r[: r[-k - 1]] for r in rows]
            return [r[: r[-1]] for r in rows]
        if out.kind == "decode" and self.pcp_group is not None and self.pcp_decode_split:
            return self._decode_split_pcp(out, ib, n)
        if out.kind == "decode":
            reqs = [s.request for s in out.seqs]
            padded = self._pad_decode_size(n) if self.graphs and self._logits_fn is None else None
            S = padded or n
            lay = ib.layout_for(S, S)
            ib.stage_decode(lay, reqs)
            ib.upload(lay)
            ev = self._event_start()
            if padded is not None:
                sampled = self.graphs[padded].replay()
            else:
                views = ib.views(lay, ib.dev)
                md = self._metadata(lay, views, False, S, S, 1, self.config.scheduler.max_model_len,
                                    1, n, n)
                sampled = self._forward_and_sample(views, md, S)
        else:
            T = out.num_tokens
            lay = ib.layout_for(T, n)
            _, max_q = ib.stage_prefill(lay, out.seqs)
            ib.upload(lay)
            ev = self._event_start()
            views = ib.views(lay, ib.dev)
            max_seq = max(s.start + s.num_new_tokens for s in out.seqs)
            md = self._metadata(lay, views, True, n, T, max_q, max_seq, 0, T, n)
            md.extra["seq_lens_host"] = [s.start + s.num_new_tokens for s in out.seqs]
            if self.pcp_group is not None and T >= 2 * self.pcp_group.world_size:
                sampled = self._forward_and_sample_pcp(views, out.seqs, T, max_seq)
                self.step_counter += 1
                self._event_stop(ev, out.kind)
                host = self.sampled_host[:n]
                host.copy_(sampled[:n], non_blocking=True)
                if self.device.type == "cuda":
                    torch.cuda.current_stream(self.device).synchronize()
                self.d2h_bytes_last = n * 4
                return host.tolist()
            nd = getattr(out, "num_decode_seqs", 0)
            if nd:
                # mixed batch: the first nd sequences are decoding (one row each); attention layers
                # that know about it run them through the decode kernel and the rest as a prefill
                # whose query offsets start at zero
                md.extra["num_decode_seqs"] = nd
                md.extra["cu_q_prefill"] = views["cu_q"][nd: n + 1] - nd
                md.extra["max_q_len_prefill"] = max(s.num_new_tokens for s in out.seqs[nd:])
                # the two halves as metadata of their own, for attention layers that hand them to
                # their decode and prefill paths unchanged (latent attention)
                import dataclasses
                lens = md.extra["seq_lens_host"]
                md.extra["md_decode"] = dataclasses.replace(
                    md, is_prefill=False, num_seqs=nd, num_tokens=nd, max_q_len=1, q_len=1,
                    positions=views["pos"][:nd], slot_mapping=views["slot"][:nd], block_tables=views["bt"][:nd],
                    seq_lens=views["seq_lens"][:nd], cu_q=views["cu_q"][: nd + 1], num_actual_tokens=nd,
                    num_actual_seqs=nd, extra={"seq_lens_host": lens[:nd]})
                md.extra["md_prefill"] = dataclasses.replace(
                    md, num_seqs=n - nd, num_tokens=T - nd, max_q_len=md.extra["max_q_len_prefill"],
                    positions=views["pos"][nd:T], slot_mapping=views["slot"][nd:T], block_tables=views["bt"][nd:n],
                    seq_lens=views["seq_lens"][nd:n], cu_q=md.extra["cu_q_prefill"], num_actual_tokens=T - nd,
                    num_actual_seqs=n - nd, extra={"seq_lens_host": lens[nd:]})
            sampled = self._forward_and_sample(views, md, n)
        self.step_counter += 1
        self._event_stop(ev, out.kind)
        # D2H of the step's result (pinned), then the host learns the tokens
        if self.mtp is not None:
            host = self.sampled_host2[:n]
            host.copy_(sampled[:n], non_blocking=True)
            if self.device.type == "cuda":
                torch.cuda.current_stream(self.device).synchronize()
            self.d2h_bytes_last = n * 4 * (1 + self.mtp_k)
            pairs = host.tolist()
            tokens = [p[0] for p in pairs]
            self.last_drafts = [p[1:] if s.samples else [] for p, s in zip(pairs, out.seqs)]
        else:
            host = self.sampled_host[:n]
            host.copy_(sampled[:n], non_blocking=True)
            if self.device.type == "cuda":
                torch.cuda.current_stream(self.device).synchronize()
            self.d2h_bytes_last = n * 4
            tokens = host.tolist()
        self.last_logprobs = self._collect_logprobs(out.seqs, tokens)
        if self.kv_connector is not None:
            self.kv_connector.wait_for_save()
        return tokens

    # ------------------------------------------- decode steps launched ahead of their results
    @torch.inference_mode()
    def launch_decode(self, out: SchedulerOutput, prev: Optional[dict] = None) -> dict:
        """Enqueue a plain decode step and return without waiting for it.  Requests whose newest
        token is still a placeholder (their previous step, ``prev``, has not been read back yet) get
        it on the device from that step's output.  ``collect_decode`` returns the tokens."""
        ib = self.input_batch
        for rid in out.finished_req_ids:
            ib.remove_request(rid)
            if getattr(self, "_pen_cache", None) is not None:
                self._pen_cache.remove_request(rid)
        for rid in out.preempted:
            ib.remove_request(rid)
        n = len(out.seqs)
        reqs = [s.request for s in out.seqs]
        padded = self._pad_decode_size(n) if self.graphs else None
        S = padded or n
        cuda = self.device.type == "cuda"
        lay = ib.layout_for(S, S)
        ib.stage_decode(lay, reqs)        # waits until the last H2D copy has read the staging buffer
        ib.upload(lay)
        views = ib.views(lay, ib.dev)
        if prev is not None:
            where = {id(r): i for i, r in enumerate(prev["reqs"])}
            fb = [where.get(id(r), -1) if (r.output_token_ids and r.output_token_ids[-1] < 0) else -1 for r in reqs]
            if any(i >= 0 for i in fb):
                fb_host = torch.tensor(fb, dtype=torch.int64, pin_memory=cuda)
                fb_dev = fb_host.to(self.device, non_blocking=True)
                src = prev["sampled"].reshape(-1).to(torch.int32)
                ids = views["ids"][:n]
                ids.copy_(torch.where(fb_dev >= 0, src.index_select(0, fb_dev.clamp_min(0)), ids))
        ev = self._event_start()
        if padded is not None:
            sampled = self.graphs[padded].replay()
        else:
            md = self._metadata(lay, views, False, S, S, 1, self.config.scheduler.max_model_len, 1, n, n)
            sampled = self._forward_and_sample(views, md, S)
        self.step_counter += 1
        self._event_stop(ev, "decode")
        parity = getattr(self, "_launch_parity", 0)
        self._launch_parity = parity ^ 1
        if not hasattr(self, "_sampled_hosts"):
            self._sampled_hosts = [torch.zeros_like(self.sampled_host, pin_memory=cuda) for _ in range(2)]
        host = self._sampled_hosts[parity][:n]
        host.copy_(sampled[:n], non_blocking=True)
        done = None
        if cuda:
            done = torch.cuda.Event()
            done.record()
        self.d2h_bytes_last = n * 4
        return {"reqs": reqs, "sampled": sampled, "host": host, "event": done, "n": n}

    def collect_decode(self, handle: dict) -> List[int]:
        if handle["event"] is not None:
            handle["event"].synchronize()
        return handle["host"].tolist()

    def _to_host(self, t: torch.Tensor) -> torch.Tensor:
        """Device -> pinned host copy of a small result, synchronised."""
        host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        host.copy_(t, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return host

    def _event_start(self):
        if not self.enable_step_events or self.device.type != "cuda":
            return None
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        return (e0, e1)

    def _event_stop(self, ev, kind: str = "prefill") -> None:
        if ev is not None:
            ev[1].record()
            self._step_events.append((ev[0], ev[1], kind))

    def drain_step_events(self) -> float:
        """Sum (ms) of the device time of the steps recorded since the last call."""
        if not self._step_events:
            return 0.0
        torch.cuda.synchronize(self.device)
        total = 0.0
        for a, b, kind in self._step_events:
            ms = a.elapsed_time(b)
            total += ms
            self.step_ms_by_kind[kind] = self.step_ms_by_kind.get(kind, 0.0) + ms
            self.step_count_by_kind[kind] = self.step_count_by_kind.get(kind, 0) + 1
        self._step_events = []
        return total

    # ------------------------------------------------------------ dummy / graphs
    @torch.inference_mode()
    def _dummy_run(self, num_tokens: int, prefill: bool = False) -> None:
        """Forward over synthetic inputs that touch only KV block 0."""
        ib = self.input_batch
        bs = self.config.cache.block_size
        if prefill:
            T = num_tokens
            max_len = min(self.config.scheduler.max_model_len - 1, T,
                          (self.num_blocks - 1) * bs if self.num_blocks else T)
            n_seq = max(1, (T + max_len - 1) // max_len)
            n_seq = min(n_seq, self.config.scheduler.max_num_seqs)
            per = T // n_seq
            T = per * n_seq
            lay = ib.layout_for(T, n_seq)
            ib.wait_upload()
            h = ib.host_np
            h[lay.ids: lay.ids + T] = 0
            pos = np.tile(np.arange(per, dtype=np.int32), n_seq)
            h[lay.pos: lay.pos + T] = pos
            h[lay.slot: lay.slot + T] = -1
            h[lay.next_ids: lay.next_ids + T] = 0
            h[lay.seq_lens: lay.seq_lens + n_seq] = per
            h[lay.cu_q: lay.cu_q + n_seq + 1] = np.arange(n_seq + 1, dtype=np.int32) * per
            h[lay.logits_idx: lay.logits_idx + n_seq] = np.arange(1, n_seq + 1, dtype=np.int32) * per - 1
            h[lay.temp: lay.temp + n_seq] = 0
            h[lay.top_k: lay.top_k + n_seq] = 0
            h[lay.top_p: lay.top_p + n_seq] = np.float32(1.0).view(np.int32)
            bt = h[lay.bt: lay.bt + n_seq * lay.max_blocks].reshape(n_seq, lay.max_blocks)
            nb = (per + bs * ib.cp_world - 1) // (bs * ib.cp_world)
            bt[:, :nb] = np.arange(nb, dtype=np.int32) % max(1, self.num_blocks)
            ib.upload(lay)
            views = ib.views(lay, ib.dev)
            md = self._metadata(lay, views, True, n_seq, T, per, per, 0, T, n_seq)
            md.extra["seq_lens_host"] = [per] * n_seq
            self._forward_and_sample(views, md, n_seq)
        else:
            S = num_tokens
            lay = ib.layout_for(S, S)
            ib.stage_decode(lay, [])
            ib.upload(lay)
            views = ib.views(lay, ib.dev)
            md = self._metadata(lay, views, False, S, S, 1, self.config.scheduler.max_model_len, 1, 0, 0)
            self._forward_and_sample(views, md, S)

    def execute_dummy_batch(self) -> None:
        """Keeps collectives in lock-step on data-parallel ranks with no work."""
        self._dummy_run(1, prefill=False)

    @torch.inference_mode()
    def capture_model(self) -> None:
        """Capture one full-step decode graph per batch size."""
        cc = self.config.compilation
        if self.device.type != "cuda" or cc.cudagraph_mode == "NONE":
            return
        if self.pp_group is not None:
            logger.info("pipeline parallelism: decode steps run eagerly (stage-to-stage sends are not captured)")
            return
        t0 = time.time()
        self.capture_sizes = cc.capture_sizes(self.config.scheduler.max_num_seqs)
        ib = self.input_batch
        pool = None
        for S in sorted(self.capture_sizes, reverse=True):
            lay = ib.layout_for(S, S)
            ib.stage_decode(lay, [])
            ib.upload(lay)
            views = ib.views(lay, ib.dev)
            md = self._metadata(lay, views, False, S, S, 1, self.config.scheduler.max_model_len, 1, 0, 0)
            runner = CUDAGraphRunner(lambda v=views, m=md, s=S: self._forward_and_sample(v, m, s),
                                     self.device, pool)
            runner.capture(warmup=2)
            pool = runner.pool
            self.graphs[S] = runner
        torch.cuda.synchronize(self.device)
        self.timings["capture_s"] = time.time() - t0
        logger.info("captured %d decode graphs in %.1f s", len(self.graphs), time.time() - t0)
