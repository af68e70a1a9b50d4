"""Worker entry for multi-process tests (CPU/gloo and multi-GPU/NCCL).

    python tests/dist_worker.py <task> <rank> <world> <port> <workdir> [device]

Each task writes ``<workdir>/result_<rank>.json``.
"""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch  # noqa: E402


def setup(rank, world, port, device_kind, nccl_nvls="0"):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE=nccl_nvls)
    from omni_npu_b200.parallel import state
    if device_kind == "cuda":
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
    else:
        dev = torch.device("cpu")
    state.init_distributed(dev, timeout_s=120)
    return dev, state


def task_comm(rank, world, port, workdir, device_kind):
    """Communicator semantics against closed-form expectations."""
    dev, state = setup(rank, world, port, device_kind)
    state.init_model_parallel(tp=world, device=dev)
    g = state.get_tp_group()
    res = {}
    x = torch.full((4, 6), float(rank + 1), device=dev)
    res["all_reduce"] = g.all_reduce(x.clone()).flatten()[0].item()
    ag = g.all_gather(torch.full((2, 3), float(rank), device=dev), dim=0)
    res["all_gather0"] = ag[:, 0].tolist()
    ag1 = g.all_gather(torch.full((2, 3), float(rank), device=dev), dim=-1)
    res["all_gather_last_shape"] = list(ag1.shape)
    res["all_gather_last_row"] = ag1[0].tolist()
    rs = g.reduce_scatter(torch.arange(world * 2, dtype=torch.float32, device=dev).view(world * 2, 1).repeat(1, 2), dim=0)
    res["reduce_scatter"] = rs[:, 0].tolist()
    sizes = [r + 1 for r in range(world)]
    agv = g.all_gatherv(torch.full((rank + 1, 2), float(rank), device=dev), dim=0, sizes=sizes)
    res["all_gatherv"] = agv[:, 0].tolist()
    rsv = g.reduce_scatterv(torch.ones(sum(sizes), 2, device=dev), dim=0, sizes=sizes)
    res["reduce_scatterv_shape"] = list(rsv.shape)
    res["reduce_scatterv_val"] = rsv[0, 0].item()
    a2a = g.comm.all_to_all(torch.arange(world * 2, dtype=torch.float32, device=dev).view(world * 2, 1) + 100 * rank,
                            scatter_dim=0, gather_dim=0)
    res["all_to_all"] = a2a[:, 0].tolist()
    gat = g.comm.gather(torch.full((1, 2), float(rank), device=dev), dst=0, dim=0)
    res["gather"] = gat[:, 0].tolist() if gat is not None else None
    if world == 2:
        res["swap"] = g.swap(torch.full((3,), float(rank + 10), device=dev)).tolist()
    if world >= 2:
        if rank == 0:
            g.send(torch.tensor([7.0, 8.0], device=dev), dst=1)
        elif rank == 1:
            res["recv"] = g.recv((2,), torch.float32, src=0).tolist()
    # asynchronous forms: result + a handle to wait on before the result is used
    y, h = g.all_reduce_async(torch.full((4, 6), float(rank + 1), device=dev))
    z, h2 = g.all_gather_async(torch.full((2, 3), float(rank), device=dev), dim=0)
    w, h3 = g.reduce_scatter_async(torch.arange(world * 2, dtype=torch.float32, device=dev).view(world * 2, 1).repeat(1, 2), dim=0)
    for hh in (h, h2, h3):
        hh.wait()
    res["async"] = [y.flatten()[0].item(), z[:, 0].tolist(), w[:, 0].tolist()]
    res["bcast_obj"] = g.broadcast_object({"k": rank} if rank == 0 else None, src=0)
    lg = state.register_layer_group("self_attn.o_proj", world)
    res["layer_group"] = [lg.world_size, lg.rank_in_group]
    g.barrier()
    json.dump(res, open(os.path.join(workdir, f"result_{rank}.json"), "w"))
    state.destroy_distributed()


def task_tp_engine(rank, world, port, workdir, device_kind):
    """Tiny Llama with tensor parallelism; rank 0 writes the generated tokens."""
    dev, state = setup(rank, world, port, device_kind)
    from omni_npu_b200 import SamplingParams
    from omni_npu_b200.engine.llm import LLM
    model_dir = os.path.join(workdir, "model")
    prompts = json.load(open(os.path.join(workdir, "prompts.json")))
    kw = dict(device=device_kind, tensor_parallel_size=world, max_num_seqs=4, max_num_batched_tokens=64,
              max_model_len=256, block_size=16, num_gpu_blocks=64)
    if device_kind == "cpu":
        kw["dtype"] = "float32"
    if os.path.exists(os.path.join(workdir, "sequence_parallel")):
        kw["sequence_parallel_residual"] = True
    if os.path.exists(os.path.join(workdir, "additional_config.json")):
        kw["additional_config"] = json.load(open(os.path.join(workdir, "additional_config.json")))
    if os.path.exists(os.path.join(workdir, "pipeline_parallel")):
        pp = int(open(os.path.join(workdir, "pipeline_parallel")).read())
        kw.update(pipeline_parallel_size=pp, tensor_parallel_size=world // pp)
    if os.path.exists(os.path.join(workdir, "prefill_context_parallel")):
        pcp = int(open(os.path.join(workdir, "prefill_context_parallel")).read() or world)
        kw.update(prefill_context_parallel_size=pcp, tensor_parallel_size=world // pcp)
        if os.path.exists(os.path.join(workdir, "pcp_decode_split")):
            kw["additional_config"] = dict(kw.get("additional_config") or {}, pcp_decode_split=True)
    if os.path.exists(os.path.join(workdir, "long_prompts")):
        kw.update(max_num_batched_tokens=256, max_model_len=512)
        from omni_npu_b200.models.llama import LlamaModel
        LlamaModel.auto_sequence_parallel = True
    llm = LLM(model=model_dir, **kw)
    # logits of the step that ends each prompt (captured through the runner's logits hook), for a
    # tolerance comparison against another deployment of the same weights
    first_logits = []
    runner = llm.engine.worker.model_runner
    real_hook = runner._make_logits_fn
    if os.path.exists(os.path.join(workdir, "capture_logits")):
        def hook(seqs):
            def fn(logits):
                rows = [i for i, q in enumerate(seqs) if q.samples and not q.request.output_token_ids]
                for i in rows:
                    first_logits.append((seqs[i].request.request_id, logits[i].float().cpu().tolist()))
                return logits
            return fn
        runner._make_logits_fn = hook
    outs = llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    runner._make_logits_fn = real_hook
    kinds = sorted({type(m).__name__ for m in llm.engine.worker.get_model().modules() if "Attention" in type(m).__name__})
    json.dump({"tokens": [o.output_token_ids for o in outs], "attention_modules": kinds,
               "pcp_steps": getattr(runner, "pcp_steps", 0), "pcp_decode_rows": getattr(runner, "pcp_decode_rows", 0),
               "first_logits": [l for _, l in sorted(first_logits)]},
              open(os.path.join(workdir, f"result_{rank}.json"), "w"))
    if device_kind == "cuda":
        state.finish_process(llm.engine)
    state.get_world_group().barrier()
    state.destroy_distributed()


def task_pp_deepseek(rank, world, port, workdir, device_kind):
    """Randomly initialised tiny DeepSeek-style model (names seed the values, so every stage
    draws what a whole-model process draws) over ``world`` pipeline stages."""
    dev, state = setup(rank, world, port, device_kind)
    from omni_npu_b200 import SamplingParams
    from omni_npu_b200.config import ModelConfig
    from omni_npu_b200.engine.llm import LLM
    spec = json.load(open(os.path.join(workdir, "spec.json")))
    cfg = ModelConfig(dtype=torch.float32 if device_kind == "cpu" else torch.bfloat16, **spec["model"])
    llm = LLM(model=cfg, device=device_kind, pipeline_parallel_size=world, **spec["engine"])
    outs = llm.generate(spec["prompts"], SamplingParams(max_tokens=spec["max_tokens"], ignore_eos=True))
    json.dump({"tokens": [o.output_token_ids for o in outs],
               "kv_layers": len(llm.engine.worker.model_runner.kv_caches)},
              open(os.path.join(workdir, f"result_{rank}.json"), "w"))
    if device_kind == "cuda":
        from omni_npu_b200 import ops
        ops.check_status()
        state.finish_process(llm.engine)
    state.get_world_group().barrier()
    state.destroy_distributed()


def task_dcp_engine(rank, world, port, workdir, device_kind):
    """Tiny latent-attention model under tensor parallelism, with or without the KV cache sharded by
    tokens over the same ranks (decode context parallelism); spec.json says which."""
    dev, state = setup(rank, world, port, device_kind)
    from omni_npu_b200 import SamplingParams
    from omni_npu_b200.config import ModelConfig
    from omni_npu_b200.engine.llm import LLM
    spec = json.load(open(os.path.join(workdir, "spec.json")))
    cfg = ModelConfig(dtype=torch.float32 if device_kind == "cpu" else torch.bfloat16, **spec["model"])
    if spec.get("pcp"):
        # prefill steps split by tokens over the ranks; experts replicated, so that the weights are
        # those of a single process
        llm = LLM(model=cfg, device=device_kind, tensor_parallel_size=world // spec["pcp"],
                  prefill_context_parallel_size=spec["pcp"], enable_expert_parallel=bool(spec.get("ep", False)),
                  additional_config={"pcp_decode_split": bool(spec.get("pcp_decode_split", False))},
                  **spec["engine"])
    else:
        llm = LLM(model=cfg, device=device_kind, tensor_parallel_size=world,
                  decode_context_parallel_size=world if spec["dcp"] else 1, **spec["engine"])
    outs = llm.generate(spec["prompts"], SamplingParams(max_tokens=spec["max_tokens"], ignore_eos=True))
    runner = llm.engine.worker.model_runner
    json.dump({"tokens": [o.output_token_ids for o in outs], "max_blocks": runner.input_batch.max_blocks,
               "free_blocks": llm.engine.scheduler.pool.num_free, "pcp_steps": getattr(runner, "pcp_steps", 0),
               "pcp_decode_rows": getattr(runner, "pcp_decode_rows", 0)},
              open(os.path.join(workdir, f"result_{rank}.json"), "w"))
    if device_kind == "cuda":
        state.finish_process(llm.engine)
    state.get_world_group().barrier()
    state.destroy_distributed()


def task_dp_engine(rank, world, port, workdir, device_kind):
    """One engine per data-parallel rank (experts sharded over all ranks); every rank serves its
    own list of prompts, lists of different lengths."""
    dev, state = setup(rank, world, port, device_kind)
    from omni_npu_b200 import SamplingParams
    from omni_npu_b200.engine.llm import LLM
    prompts = json.load(open(os.path.join(workdir, "prompts.json")))[rank]
    kw = dict(dtype="float32") if device_kind == "cpu" else {}
    llm = LLM(model=os.path.join(workdir, "model"), device=device_kind, data_parallel_size=world,
              enable_expert_parallel=True, max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256,
              block_size=16, num_gpu_blocks=64, **kw)
    moe = [m for m in llm.engine.worker.get_model().modules() if hasattr(m, "local_experts")]
    outs = llm.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))
    json.dump({"tokens": [o.output_token_ids for o in outs], "local_experts": moe[0].local_experts,
               "dummy_steps": llm.engine.stats.get("dummy_steps", 0), "steps": llm.engine.stats["steps"]},
              open(os.path.join(workdir, f"result_{rank}.json"), "w"))
    if device_kind == "cuda":
        from omni_npu_b200 import ops
        torch.cuda.synchronize()
        ops.check_status()
        state.finish_process(llm.engine)
    state.get_world_group().barrier()
    state.destroy_distributed()


def task_server_loop(rank, world, port, workdir, device_kind):
    """The API server's engine loop under tensor parallelism: rank 0 receives the requests (as the
    HTTP handlers would submit them, at different times) and replicates them; the other ranks follow."""
    import time
    dev, state = setup(rank, world, port, device_kind)
    from omni_npu_b200 import SamplingParams
    from omni_npu_b200.engine.llm import LLM
    from omni_npu_b200.serving.api_server import EngineLoop
    prompts = json.load(open(os.path.join(workdir, "prompts.json")))
    llm = LLM(model=os.path.join(workdir, "model"), device=device_kind, dtype="float32", tensor_parallel_size=world,
              max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256, block_size=16, num_gpu_blocks=64)
    result = {"tokens": None}
    if rank == 0:
        loop = EngineLoop(llm)
        loop.KEEPALIVE_S = 0.2
        sp = SamplingParams(max_tokens=12, ignore_eos=True)
        rids = [loop.submit(prompts[0], sp)]
        time.sleep(0.3)                                   # the second and third arrive while the first decodes
        rids += [loop.submit(p, sp) for p in prompts[1:3]]
        extra = loop.submit(prompts[0], SamplingParams(max_tokens=200, ignore_eos=True))
        loop.abort(extra)                                 # an abort travels to the followers too
        outs = [loop.wait(r, timeout=120) for r in rids]
        time.sleep(0.5)                                   # a few idle keep-alive rounds
        loop.shutdown()
        result = {"tokens": [o.output_token_ids for o in outs], "steps": loop.counters["steps"]}
    else:
        EngineLoop(llm, follower=True).run_follower()
        result = {"tokens": None, "free_blocks": llm.engine.scheduler.pool.num_free,
                  "unfinished": llm.engine.has_unfinished_requests()}
    json.dump(result, open(os.path.join(workdir, f"result_{rank}.json"), "w"))
    state.get_world_group().barrier()
    state.destroy_distributed()


def task_symm(rank, world, port, workdir, device_kind):
    """Peer-memory collectives against NCCL results."""
    dev, state = setup(rank, world, port, "cuda")
    state.init_model_parallel(tp=world, device=dev)
    import torch.distributed as dist
    from omni_npu_b200 import ops
    from omni_npu_b200.parallel.symm_mem import attach_symmetric_memory
    g = state.get_tp_group()
    symm = attach_symmetric_memory(g, dev, half_bytes=96 << 20)
    res = {"max_err": {}}
    torch.manual_seed(100 + rank)
    for name, shape, mode in (("push_tiny", (1, 4096), 3), ("push", (128, 4096), 3), ("push_odd", (7, 1032), 3),
                              ("push_small_after_big", (3, 512), 3), ("push_again", (128, 4096), 3),
                              ("small_1shot", (128, 4096), 1), ("small_2shot", (128, 4096), 2),
                              ("odd", (7, 1032), 0), ("large_auto", (4096, 4096), 0),
                              ("large_1shot", (2048, 4096), 1)):
        x = torch.randn(*shape, device=dev, dtype=torch.bfloat16)
        want = x.float().clone()
        dist.all_reduce(want, group=g.device_group)
        for rep in range(3):       # repeated calls exercise the alternating halves
            got = symm.all_reduce(x, mode=mode)
        res["max_err"][name] = (got.float() - want).abs().max().item()
    # fused all-reduce + residual + RMSNorm
    x = torch.randn(96, 4096, device=dev, dtype=torch.bfloat16)
    resid = torch.randn(96, 4096, device=dev, dtype=torch.bfloat16)
    dist.broadcast(resid, src=0, group=g.device_group)
    w = torch.randn(4096, device=dev, dtype=torch.bfloat16)
    dist.broadcast(w, src=0, group=g.device_group)
    red = x.clone()
    dist.all_reduce(red, group=g.device_group)
    r_ref = resid.clone()
    y_ref = ops.fused_add_rms_norm(red, r_ref, w, 1e-6)
    r_got = resid.clone()
    y_got = symm.all_reduce_add_rms_norm(x, r_got, w, 1e-6)
    res["max_err"]["fused_norm_out"] = (y_got.float() - y_ref.float()).abs().max().item()
    # the same through the barrier-based (pull) kernel
    symm.use_ll = False
    r_pull = resid.clone()
    y_pull = symm.all_reduce_add_rms_norm(x, r_pull, w, 1e-6)
    symm.use_ll = True
    res["max_err"]["fused_norm_out_pull"] = (y_pull.float() - y_ref.float()).abs().max().item()
    res["max_err"]["fused_norm_res_pull"] = (r_pull.float() - r_ref.float()).abs().max().item()
    res["max_err"]["fused_norm_res"] = (r_got.float() - r_ref.float()).abs().max().item()
    # GEMM + all-reduce (+ residual + RMSNorm) as one kernel, against the unfused sequence
    for name, (m, n, k), with_norm in (("gemm_ar_norm", (128, 4096, 2048), True), ("gemm_ar_norm_odd", (7, 1032, 520), True),
                                       ("gemm_ar_plain", (33, 4096, 512), False), ("gemm_ar_norm_again", (128, 4096, 2048), True)):
        xa = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
        wa = torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.05
        ba = torch.randn(n, device=dev, dtype=torch.bfloat16)
        ra = torch.randn(m, n, device=dev, dtype=torch.bfloat16)
        wn = torch.randn(n, device=dev, dtype=torch.bfloat16)
        for t in (ba, ra, wn):
            dist.broadcast(t, src=0, group=g.device_group)
        part = ops.gemm(xa, wa, ba if rank == 0 else None)
        dist.all_reduce(part, group=g.device_group)
        if with_norm:
            r_ref = ra.clone()
            y_ref = ops.fused_add_rms_norm(part, r_ref, wn, 1e-6)
            r_got = ra.clone()
            y_got = symm.gemm_all_reduce(xa, wa, ba, r_got, wn, 1e-6)
            res["max_err"][name + "_res"] = (r_got.float() - r_ref.float()).abs().max().item()
        else:
            y_ref = part + ra
            y_got = symm.gemm_all_reduce(xa, wa, ba, ra, None, 0.0)
        res["max_err"][name] = (y_got.float() - y_ref.float()).abs().max().item() / max(1.0, y_ref.float().abs().max().item())
    # all-gather / reduce-scatter
    x = torch.randn(64, 512, device=dev, dtype=torch.bfloat16)
    ag_ref = torch.empty(world * 64, 512, device=dev, dtype=torch.bfloat16)
    dist.all_gather_into_tensor(ag_ref, x, group=g.device_group)
    res["max_err"]["all_gather"] = (symm.all_gather(x).float() - ag_ref.float()).abs().max().item()
    xs = torch.randn(world * 32, 512, device=dev, dtype=torch.bfloat16)
    rs_ref = torch.empty(32, 512, device=dev, dtype=torch.float32)
    dist.reduce_scatter_tensor(rs_ref, xs.float(), group=g.device_group)
    res["max_err"]["reduce_scatter"] = (symm.reduce_scatter(xs).float() - rs_ref).abs().max().item()
    # timing: decode-sized all-reduce, ours vs NCCL
    x = torch.randn(128, 4096, device=dev, dtype=torch.bfloat16)
    def timeit(fn, n=50):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n * 1e3
    res["us_symm_1MiB"] = timeit(lambda: symm.all_reduce(x))
    res["us_nccl_1MiB"] = timeit(lambda: dist.all_reduce(x, group=g.device_group))
    # the same inside a CUDA graph (no launch gaps): plain and fused with residual + RMSNorm
    def graph_time(fn, reps=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g.barrier()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for _ in range(reps):
                fn()
        torch.cuda.synchronize()
        g.barrier()
        gr.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            gr.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (5 * reps) * 1e3
    wn = torch.ones(4096, device=dev, dtype=torch.bfloat16)
    for rows in (1, 16, 128):
        xs = torch.randn(rows, 4096, device=dev, dtype=torch.bfloat16)
        rr = torch.zeros(rows, 4096, device=dev, dtype=torch.bfloat16)
        res[f"us_graph_symm_{rows}"] = graph_time(lambda: symm.all_reduce(xs, mode=1))
        res[f"us_graph_push_{rows}"] = graph_time(lambda: symm.all_reduce(xs, mode=3))
        res[f"us_graph_fused_{rows}"] = graph_time(lambda: symm.all_reduce_add_rms_norm(xs, rr, wn, 1e-6))
        res[f"us_graph_local_norm_{rows}"] = graph_time(lambda: ops.fused_add_rms_norm(xs, rr, wn, 1e-6))
    # decode-sized row-parallel projection: one kernel vs GEMM followed by the fused all-reduce
    xa = torch.randn(128, 2048, device=dev, dtype=torch.bfloat16)
    wa = torch.randn(4096, 2048, device=dev, dtype=torch.bfloat16) * 0.05
    rr = torch.zeros(128, 4096, device=dev, dtype=torch.bfloat16)
    res["us_graph_gemm_then_ar_norm"] = graph_time(lambda: symm.all_reduce_add_rms_norm(ops.gemm(xa, wa), rr, wn, 1e-6))
    res["us_graph_gemm_ar_norm_fused"] = graph_time(lambda: symm.gemm_all_reduce(xa, wa, None, rr, wn, 1e-6))
    big = torch.randn(8192, 4096, device=dev, dtype=torch.bfloat16)
    res["us_symm_64MiB"] = timeit(lambda: symm.all_reduce(big), 10)
    res["us_nccl_64MiB"] = timeit(lambda: dist.all_reduce(big, group=g.device_group), 10)
    torch.cuda.synchronize()
    ops.check_status()
    g.barrier()
    json.dump(res, open(os.path.join(workdir, f"result_{rank}.json"), "w"))
    state.destroy_distributed()


def task_nvls(rank, world, port, workdir, device_kind):
    """All-reduce through the switch (multimem) against NCCL: values, the fused residual + RMSNorm
    tail, repeated calls (alternating halves), and a size sweep timed inside CUDA graphs against the
    peer-store kernels and NCCL (NCCL left at its defaults, NVLS included, for the comparison)."""
    dev, state = setup(rank, world, port, "cuda", nccl_nvls="1")
    state.init_model_parallel(tp=world, device=dev)
    import torch.distributed as dist
    from omni_npu_b200 import ops
    from omni_npu_b200.parallel.nvls import NvlsAllReduce
    from omni_npu_b200.parallel.symm_mem import attach_symmetric_memory
    g = state.get_tp_group()
    res = {"max_err": {}, "us": {}}
    try:
        nv = NvlsAllReduce(g, dev, max_bytes=64 << 20)
    except Exception as e:
        res["unsupported"] = f"{type(e).__name__}: {e}"
        json.dump(res, open(os.path.join(workdir, f"result_{rank}.json"), "w"))
        state.destroy_distributed()
        return
    symm = attach_symmetric_memory(g, dev, half_bytes=96 << 20)
    torch.manual_seed(200 + rank)
    for name, shape, mode in (("one_tiny", (1, 4096), 1), ("one", (128, 4096), 1), ("one_odd", (7, 1032), 1),
                              ("two", (128, 4096), 2), ("two_odd", (37, 1032), 2), ("two_large", (4096, 4096), 2),
                              ("auto_large", (8192, 4096), 0), ("one_again", (128, 4096), 1)):
        x = torch.randn(*shape, device=dev, dtype=torch.bfloat16)
        want = x.float().clone()
        dist.all_reduce(want, group=g.device_group)
        for rep in range(3):
            got = nv.all_reduce(x, mode=mode)
        res["max_err"][name] = (got.float() - want).abs().max().item() / max(1.0, want.abs().max().item())
    for name, rows, mode in (("fused_one", 96, 1), ("fused_two", 96, 2), ("fused_two_large", 2048, 2)):
        x = torch.randn(rows, 4096, device=dev, dtype=torch.bfloat16)
        resid = torch.randn(rows, 4096, device=dev, dtype=torch.bfloat16)
        w = torch.randn(4096, device=dev, dtype=torch.bfloat16)
        dist.broadcast(resid, src=0, group=g.device_group)
        dist.broadcast(w, src=0, group=g.device_group)
        red = x.clone()
        dist.all_reduce(red, group=g.device_group)
        r_ref = resid.clone()
        y_ref = ops.fused_add_rms_norm(red, r_ref, w, 1e-6)
        r_got = resid.clone()
        y_got = nv.all_reduce(x, r_got, w, 1e-6, mode=mode)
        res["max_err"][name + "_out"] = (y_got.float() - y_ref.float()).abs().max().item()
        res["max_err"][name + "_res"] = (r_got.float() - r_ref.float()).abs().max().item()

    def graph_time(fn, reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g.barrier()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for _ in range(reps):
                fn()
        torch.cuda.synchronize()
        g.barrier()
        gr.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            gr.replay()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / (3 * reps) * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=g.device_group)     # max over ranks
        return round(float(t), 1)

    for rows in (1, 16, 128, 512, 2048, 8192):
        x = torch.randn(rows, 4096, device=dev, dtype=torch.bfloat16)
        nbytes = rows * 4096 * 2
        reps = 20 if rows <= 512 else 5
        row = {"nccl": graph_time(lambda: dist.all_reduce(x, group=g.device_group), reps)}
        row["nvls_one_shot"] = graph_time(lambda: nv.all_reduce(x, mode=1), reps) if nbytes <= (8 << 20) else None
        row["nvls_two_shot"] = graph_time(lambda: nv.all_reduce(x, mode=2), reps)
        if nbytes <= symm.LL_SLOT_BYTES:
            row["push"] = graph_time(lambda: symm.all_reduce(x, mode=3), reps)
        row["peer_one_shot"] = graph_time(lambda: symm.all_reduce(x, mode=1), reps) if nbytes <= (8 << 20) else None
        row["peer_two_shot"] = graph_time(lambda: symm.all_reduce(x, mode=2), reps)
        res["us"][f"{nbytes >> 10}KiB"] = row
    wn = torch.ones(4096, device=dev, dtype=torch.bfloat16)
    for rows in (16, 128):
        x = torch.randn(rows, 4096, device=dev, dtype=torch.bfloat16)
        rr = torch.zeros(rows, 4096, device=dev, dtype=torch.bfloat16)
        res["us"][f"fused_norm_{rows}rows"] = {
            "nvls_one_shot": graph_time(lambda: nv.all_reduce(x, rr, wn, 1e-6, mode=1), 20),
            "push": graph_time(lambda: symm.all_reduce_add_rms_norm(x, rr, wn, 1e-6), 20)}
    # row-parallel decode projections of a Llama-3-8B layer at this world size, 128 tokens: the
    # GEMM with the all-reduce + residual + RMSNorm pushed from its epilogue (one kernel, every rank
    # sends its tile to every other rank), against the plain GEMM followed by the all-reduce + norm
    # through the switch or by NCCL + the norm kernel
    for label, k_full in (("o_proj", 4096), ("down_proj", 14336)):
        k = k_full // world
        x = torch.randn(128, k, device=dev, dtype=torch.bfloat16) * 0.1
        ws = [torch.randn(4096, k, device=dev, dtype=torch.bfloat16) * 0.05 for _ in range(8)]
        rr = torch.zeros(128, 4096, device=dev, dtype=torch.bfloat16)
        it = [0]

        def w_next():
            it[0] += 1
            return ws[it[0] % len(ws)]

        def nccl_path():
            y = ops.gemm(x, w_next())
            dist.all_reduce(y, group=g.device_group)
            return ops.fused_add_rms_norm(y, rr, wn, 1e-6)
        row = {"gemm_then_nccl_then_norm": graph_time(nccl_path, 16),
               "gemm_then_nvls_norm": graph_time(lambda: nv.all_reduce(ops.gemm(x, w_next()), rr, wn, 1e-6, mode=1), 16)}
        if symm.can_fuse_gemm(x, ws[0]):
            row["fused_gemm_push_norm"] = graph_time(lambda: symm.gemm_all_reduce(x, w_next(), None, rr, wn, 1e-6), 16)
        res["us"][f"{label}_128x4096x{k}"] = row
    torch.cuda.synchronize()
    ops.check_status()
    g.barrier()
    json.dump(res, open(os.path.join(workdir, f"result_{rank}.json"), "w"))
    state.destroy_distributed()


def task_ep_moe(rank, world, port, workdir, device_kind):
    """Expert-parallel MoE layer (dispatch -> grouped GEMMs -> combine over peer memory, or the
    gloo all-to-all path on CPU) against the dense single-process computation."""
    dev, state = setup(rank, world, port, device_kind)
    state.init_model_parallel(tp=world, device=dev)
    from omni_npu_b200 import ops
    from omni_npu_b200.layers.moe import FusedMoE, select_experts
    from omni_npu_b200.ops import ref
    dt = torch.bfloat16 if device_kind == "cuda" else torch.float32
    E, K, H, I = 16, 4, 256, 128
    g = torch.Generator().manual_seed(42)
    full = dict(gate=torch.randn(E, H, generator=g) * 0.1, w13=torch.randn(E, 2 * I, H, generator=g) * 0.05,
                w2=torch.randn(E, H, I, generator=g) * 0.05,
                sh13=torch.randn(2 * I, H, generator=g) * 0.05, sh2=torch.randn(H, I, generator=g) * 0.05)
    layer = FusedMoE(E, K, H, I, dtype=dt, device=dev, renormalize=True, num_shared_experts=1, max_tokens=512)
    assert layer.ep_size == world and layer.local_experts == E // world
    lo = layer.expert_start
    layer.gate.weight.data.copy_(full["gate"])
    layer.w13.data.copy_(full["w13"][lo:lo + layer.local_experts])
    layer.w2.data.copy_(full["w2"][lo:lo + layer.local_experts])
    layer.shared_experts.gate_up_proj.weight.data.copy_(full["sh13"])
    layer.shared_experts.down_proj.weight.data.copy_(full["sh2"])
    errs = {}
    for t in (1, 37, 200):
        x = (torch.randn(t, H, generator=g) * 0.5).to(dt)
        xr = x.to(dt).float() if dt == torch.float32 else x
        logits = ref.gemm(xr.cpu(), full["gate"].to(dt), out_dtype=torch.float32)
        w, ids = select_experts(logits, K, renormalize=True)
        want = ref.moe_experts(xr.cpu(), full["w13"].to(dt), full["w2"].to(dt), ids, w).float()
        sh = ref.gemm(ref.gemm(xr.cpu(), full["sh13"].to(dt), swiglu=True), full["sh2"].to(dt)).float()
        want = want + sh
        for rep in range(2):
            got = layer(x.to(dev))
        errs[str(t)] = (got.float().cpu() - want).abs().max().item()
    if device_kind == "cuda":
        torch.cuda.synchronize()
        ops.check_status()
    state.get_world_group().barrier()
    json.dump({"max_err": errs}, open(os.path.join(workdir, f"result_{rank}.json"), "w"))
    if layer.buffers is not None:
        layer.buffers.close()
    if device_kind == "cuda":
        state.finish_process()
    state.destroy_distributed()


def task_pcp_moe(rank, world, port, workdir, device_kind):
    """Prefill context parallelism around a MoE layer: the ranks of the pcp group hold DIFFERENT
    tokens, the expert-parallel group spans them, and each rank gets back the MoE output of its own
    shard: dispatch and combine are the exchange, nothing is gathered around the layer."""
    dev, state = setup(rank, world, port, device_kind)
    state.init_model_parallel(tp=1, pcp=world, device=dev)
    assert state.get_pcp_group().world_size == world and state.get_tp_group().world_size == 1
    assert state.get_ep_group().world_size == world
    from omni_npu_b200 import ops
    from omni_npu_b200.layers.moe import FusedMoE, select_experts
    from omni_npu_b200.ops import ref
    dt = torch.bfloat16 if device_kind == "cuda" else torch.float32
    E, K, H, I = 16, 4, 256, 128
    g = torch.Generator().manual_seed(43)
    full = dict(gate=torch.randn(E, H, generator=g) * 0.1, w13=torch.randn(E, 2 * I, H, generator=g) * 0.05,
                w2=torch.randn(E, H, I, generator=g) * 0.05)
    layer = FusedMoE(E, K, H, I, dtype=dt, device=dev, renormalize=True, max_tokens=512)
    lo = layer.expert_start
    layer.gate.weight.data.copy_(full["gate"])
    layer.w13.data.copy_(full["w13"][lo:lo + layer.local_experts])
    layer.w2.data.copy_(full["w2"][lo:lo + layer.local_experts])
    errs = {}
    for t in (64, 203):                                      # tokens of the whole prompt batch
        x_all = (torch.randn(t, H, generator=g) * 0.5).to(dt)
        per = (t + world - 1) // world
        mine = x_all[rank * per: min(t, (rank + 1) * per)]   # this rank's shard (the last one is shorter)
        xr = mine.float() if dt == torch.float32 else mine
        logits = ref.gemm(xr.cpu(), full["gate"].to(dt), out_dtype=torch.float32)
        w, ids = select_experts(logits, K, renormalize=True)
        want = ref.moe_experts(xr.cpu(), full["w13"].to(dt), full["w2"].to(dt), ids, w).float()
        got = layer(mine.to(dev))
        assert got.shape == mine.shape
        errs[str(t)] = (got.float().cpu() - want).abs().max().item()
    if device_kind == "cuda":
        torch.cuda.synchronize()
        ops.check_status()
    state.get_world_group().barrier()
    json.dump({"max_err": errs}, open(os.path.join(workdir, f"result_{rank}.json"), "w"))
    if layer.buffers is not None:
        layer.buffers.close()
    if device_kind == "cuda":
        state.finish_process()
    state.destroy_distributed()


def task_ep_timing(rank, world, port, workdir, device_kind):
    """Device time of the expert-parallel dispatch and combine alone (CUDA events around CUDA-graph
    replays, max over ranks) for the row sizes of DeepSeek-V2-Lite and DeepSeek-V3.2, with the bytes
    that cross NVLink per rank and the fraction of the measured peer-copy rate (770 GB/s per
    direction) they amount to."""
    dev, state = setup(rank, world, port, "cuda")
    state.init_model_parallel(tp=world, device=dev)
    import torch.distributed as dist
    from omni_npu_b200 import ops
    from omni_npu_b200.layers.moe_dispatch import EpBuffers, ep_combine, ep_dispatch
    g = state.get_tp_group()
    link = 770e9
    res = {}

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g.barrier()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for _ in range(reps):
                fn()
        torch.cuda.synchronize()
        g.barrier()
        gr.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            gr.replay()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / (3 * reps) * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=g.device_group)
        return float(t)

    for label, E, K, H in (("v2lite", 64, 6, 2048), ("v32", 256, 8, 7168)):
        for T in (128, 2048):
            torch.manual_seed(11 + rank)
            x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
            w, ids = torch.topk(torch.softmax(torch.randn(T, E, device=dev), -1), K)
            ids = ids.to(torch.int32)
            w = w.float()
            row = {}
            for fp8 in (False, True):
                buf = EpBuffers(g, dev, E, H, T, K, fp8_dispatch=fp8)
                out = [None]

                def disp():
                    out[0] = ep_dispatch(None, x, ids, w, E, buf, fp8=fp8)
                t_d = timed(disp)
                rows, offs, handle = out[0]
                sent = T * K * (world - 1) / world                      # rows that leave this rank (uniform routing)
                by = sent * (H + H // 128 * 4 if fp8 else H * 2)
                key = "fp8" if fp8 else "bf16"
                row[f"dispatch_{key}_us"] = round(t_d, 1)
                row[f"dispatch_{key}_link_bytes"] = int(by)
                row[f"dispatch_{key}_frac_of_link"] = round(by / link / (t_d * 1e-6), 3)
                if not fp8:
                    y = buf.expert_y
                    y[: rows.shape[0]].copy_(rows)                       # combine reads the expert outputs in place
                    t_c = timed(lambda: ep_combine(None, y[: rows.shape[0]], handle, None, buf))
                    byc = sent * H * 2
                    row["combine_us"] = round(t_c, 1)
                    row["combine_link_bytes"] = int(byc)
                    row["combine_frac_of_link"] = round(byc / link / (t_c * 1e-6), 3)
                torch.cuda.synchronize()
                g.barrier()
                buf.close()
            res[f"{label}_T{T}"] = row
    ops.check_status()
    g.barrier()
    json.dump(res, open(os.path.join(workdir, f"result_{rank}.json"), "w"))
    state.finish_process()
    state.destroy_distributed()


def task_kv_pull(rank, world, port, workdir, device_kind):
    """Rank 0 owns a KV cache, rank 1 maps it through CUDA IPC and pulls blocks with the copy kernel."""
    dev, state = setup(rank, world, port, "cuda")
    state.init_model_parallel(tp=1, dp=world, device=dev) if False else state.init_model_parallel(tp=world, device=dev)
    from omni_npu_b200.kv_transfer.manager import KVLinkManager, make_cluster_id
    g = state.get_world_group()
    mgr = KVLinkManager(make_cluster_id("127.0.0.1", 30000 + rank, 1), 0, dev)
    torch.manual_seed(7)
    caches = [(torch.randn(64, 2, 16, 128, device=dev, dtype=torch.bfloat16),
               torch.randn(64, 2, 16, 128, device=dev, dtype=torch.bfloat16)) for _ in range(4)]
    if rank == 1:
        for k, v in caches:
            k.zero_(), v.zero_()
    export = mgr.register_memory(caches)
    exports = g.all_gather_object(export)
    res = {}
    if rank == 1:
        src_blocks, dst_blocks = [3, 9, 63, 0, 17], [5, 6, 7, 8, 60]
        ev = mgr.pull_kv(exports[0].cluster_id, 0, src_blocks, dst_blocks, refresh=lambda: exports[0])
        ev.synchronize()
        torch.manual_seed(7)
        ok = True
        for k, v in caches:
            rk = torch.randn(64, 2, 16, 128, device=dev, dtype=torch.bfloat16)
            rv = torch.randn(64, 2, 16, 128, device=dev, dtype=torch.bfloat16)
            ok &= torch.equal(k[dst_blocks], rk[src_blocks]) and torch.equal(v[dst_blocks], rv[src_blocks])
            ok &= bool(k[1].abs().sum() == 0)
        res["byte_exact"] = bool(ok)
        res["gbs_small"] = None
    # bandwidth on a pull of serving size: 48 layers x (K, V) x 512 blocks of 4 kv heads x 16 tokens x 128
    # = 96 tensors x 8 MiB = 768 MiB in the caches, 384 blocks pulled = 576 MiB over the link per pull
    mgr2 = KVLinkManager(make_cluster_id("127.0.0.1", 30100 + rank, 1), 0, dev)
    big = [(torch.zeros(512, 4, 16, 128, device=dev, dtype=torch.bfloat16),
            torch.zeros(512, 4, 16, 128, device=dev, dtype=torch.bfloat16)) for _ in range(48)]
    if rank == 0:
        for k, v in big:
            k.fill_(1.0), v.fill_(2.0)
    exports2 = g.all_gather_object(mgr2.register_memory(big))
    if rank == 1:
        n = 384
        blocks = list(range(n))
        ev = mgr2.pull_kv(exports2[0].cluster_id, 0, blocks, blocks, refresh=lambda: exports2[0])
        ev.synchronize()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0.record()
        for _ in range(5):
            ev = mgr2.pull_kv(exports2[0].cluster_id, 0, blocks, blocks)
        ev.synchronize()
        t1.record()
        torch.cuda.synchronize()
        nbytes = 5 * n * 96 * (4 * 16 * 128 * 2)
        res["gbs"] = nbytes / (t0.elapsed_time(t1) * 1e-3) / 1e9
        res["pull_mib"] = nbytes / 5 / 2**20
        res["byte_exact"] = bool(res["byte_exact"] and float(big[7][0][383].float().mean()) == 1.0
                                 and float(big[40][1][0].float().mean()) == 2.0
                                 and float(big[3][0][384].float().abs().sum()) == 0.0)
    g.barrier()
    mgr2.close()
    json.dump(res, open(os.path.join(workdir, f"result_{rank}.json"), "w"))
    g.barrier()
    mgr.close()
    state.finish_process()


def task_dcp_mla(rank, world, port, workdir, device_kind):
    """Decode context parallelism: the latent cache is sharded by tokens (token p on rank p % world);
    the merged result must equal attention over the whole cache."""
    dev, state = setup(rank, world, port, device_kind)
    state.init_model_parallel(tp=world, device=dev)
    from omni_npu_b200 import ops
    from omni_npu_b200.attention.dcp import dcp_mla_decode, local_seq_lens
    g = state.get_tp_group()
    dt = torch.bfloat16 if device_kind == "cuda" else torch.float32
    torch.manual_seed(3)
    bs, heads, b = 16, 4 * world, 3
    seq_lens = torch.tensor([37, 5, 64], dtype=torch.int32)
    nblk = 16
    full = (torch.randn(nblk, bs, 576) * 0.3).to(dt)                      # every rank builds the same global cache
    bt = torch.tensor([[1, 2, 3, 4, 5], [6, 0, 0, 0, 0], [7, 8, 9, 10, 11]], dtype=torch.int32)
    q = (torch.randn(b, heads, 576) * 0.3).to(dt)
    want = ops.mla_decode(q.reshape(b, -1), full, bt, seq_lens, b, heads, 0.1)
    # local shard: token p of sequence s sits at local position p // world of the same block-table row
    local = torch.zeros_like(full)
    flat_full, flat_local = full.view(-1, 576), local.view(-1, 576)
    for s in range(b):
        for p in range(int(seq_lens[s])):
            if p % world != rank:
                continue
            lp = p // world
            flat_local[int(bt[s, lp // bs]) * bs + lp % bs] = flat_full[int(bt[s, p // bs]) * bs + p % bs]
    hl = heads // world
    q_local = q[:, rank * hl: (rank + 1) * hl].reshape(b, -1).contiguous()
    got = dcp_mla_decode(q_local.to(dev), local.to(dev), bt.to(dev), seq_lens.to(dev), b, hl, 0.1, g)
    ref_local = want.view(b, heads, 512)[:, rank * hl: (rank + 1) * hl].reshape(b, -1)
    err = (got.float().cpu() - ref_local.float()).abs().max().item()
    assert local_seq_lens(seq_lens, world, rank).tolist() == [(int(n) - rank + world - 1) // world for n in seq_lens]
    g.barrier()
    json.dump({"max_err": err}, open(os.path.join(workdir, f"result_{rank}.json"), "w"))
    if device_kind == "cuda":
        state.finish_process()
    state.destroy_distributed()


def task_ag_gemm(rank, world, port, workdir, device_kind):
    """Column-parallel projection of a token-sharded activation as one kernel (the GEMM's TMA
    producer reads every rank's rows from its owner) against all-gather followed by a GEMM."""
    dev, state = setup(rank, world, port, "cuda")
    state.init_model_parallel(tp=world, device=dev)
    import torch.distributed as dist
    from omni_npu_b200 import ops
    from omni_npu_b200.parallel.symm_mem import attach_symmetric_memory
    g = state.get_tp_group()
    symm = attach_symmetric_memory(g, dev, half_bytes=96 << 20)
    res = {"max_err": {}}
    torch.manual_seed(7 + rank)

    def gathered(x):
        full = torch.empty(world * x.shape[0], x.shape[1], device=dev, dtype=x.dtype)
        dist.all_gather_into_tensor(full, x, group=g.device_group)
        return full

    for name, rows, n, k, swiglu, bias in (("plain", 256, 1024, 512, False, False), ("bias", 128, 768, 1024, False, True),
                                           ("swiglu", 384, 2048, 512, True, False),
                                           ("prefill", 4096 // world, 6144, 4096, False, False)):
        x = torch.randn(rows, k, device=dev, dtype=torch.bfloat16)
        w = torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.05
        b = torch.randn(n, device=dev, dtype=torch.bfloat16) if bias else None
        want = ops.gemm(gathered(x), w, b, None, None, swiglu).float()
        for rep in range(3):           # alternating staging halves; a plain collective in between
            got = symm.all_gather_gemm(x, w, b, swiglu)
            if rep == 1:
                symm.all_reduce(torch.ones(8, 64, device=dev, dtype=torch.bfloat16))
        torch.cuda.synchronize()
        res["max_err"][name] = (got.float() - want).abs().max().item()
    # row-parallel projection + reduce-scatter with the pushes inside the GEMM epilogue
    for name, m, n, k, bias in (("rs_plain", 256 * world, 1024, 512, False), ("rs_bias", 128 * world, 4096, 1024, True),
                                ("rs_prefill", 4096, 4096, 2048, False)):
        x = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
        w = torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.05
        b = torch.randn(n, device=dev, dtype=torch.bfloat16) if bias else None
        if b is not None:
            dist.broadcast(b, src=0, group=g.device_group)
        part = ops.gemm(x, w, b if rank == 0 else None).float()
        want = torch.empty(m // world, n, device=dev, dtype=torch.float32)
        dist.reduce_scatter_tensor(want, part, group=g.device_group)
        for rep in range(3):
            got = symm.gemm_reduce_scatter(x, w, b)
            if rep == 1:
                symm.all_gather_gemm(x[: 128], w)       # a different fused collective in between
        torch.cuda.synchronize()
        res["max_err"][name] = (got.float() - want).abs().max().item() / max(1.0, want.abs().max().item())
    # fused tail: + residual and RMSNorm on the reduced rows
    m, n, k = 256 * world, 1024, 512
    x = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.05
    resid = torch.randn(m // world, n, device=dev, dtype=torch.bfloat16)
    wn = (torch.rand(n, device=dev) + 0.5).bfloat16()
    dist.broadcast(wn, src=0, group=g.device_group)
    part = ops.gemm(x, w).float()
    red = torch.empty(m // world, n, device=dev, dtype=torch.float32)
    dist.reduce_scatter_tensor(red, part, group=g.device_group)
    r_ref = resid.clone()
    y_ref = ops.fused_add_rms_norm(red.bfloat16(), r_ref, wn, 1e-6)
    r_got = resid.clone()
    y_got = symm.gemm_reduce_scatter(x, w, None, r_got, wn, 1e-6)
    torch.cuda.synchronize()
    res["max_err"]["rs_norm"] = (y_got.float() - y_ref.float()).abs().max().item()
    res["max_err"]["rs_norm_residual"] = (r_got.float() - r_ref.float()).abs().max().item()
    # timing at a prefill shape: one kernel pair (stage + GEMM) vs all-gather then GEMM
    rows, n, k = 8192 // world, 6144, 4096
    x = torch.randn(rows, k, device=dev, dtype=torch.bfloat16)
    w = torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.05

    def timeit(fn, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3
    res["us_fused"] = timeit(lambda: symm.all_gather_gemm(x, w))
    res["us_symm_ag_then_gemm"] = timeit(lambda: ops.gemm(symm.all_gather(x), w))
    res["us_nccl_ag_then_gemm"] = timeit(lambda: ops.gemm(gathered(x), w))
    full = gathered(x)
    res["us_gemm_alone"] = timeit(lambda: ops.gemm(full, w))
    res["tflops_fused"] = 2.0 * rows * world * n * k / res["us_fused"] / 1e6
    # o_proj-shaped row-parallel GEMM (K sharded) + reduce-scatter
    xo = torch.randn(8192, 4096 // world, device=dev, dtype=torch.bfloat16)
    wo = torch.randn(4096, 4096 // world, device=dev, dtype=torch.bfloat16) * 0.05
    outp = torch.empty(8192 // world, 4096, device=dev, dtype=torch.bfloat16)
    res["us_rs_fused"] = timeit(lambda: symm.gemm_reduce_scatter(xo, wo))
    res["us_rs_symm_after_gemm"] = timeit(lambda: symm.reduce_scatter(ops.gemm(xo, wo)))
    res["us_rs_nccl_after_gemm"] = timeit(lambda: dist.reduce_scatter_tensor(outp, ops.gemm(xo, wo), group=g.device_group))
    res["us_rs_gemm_alone"] = timeit(lambda: ops.gemm(xo, wo))
    torch.cuda.synchronize()
    ops.check_status()
    g.barrier()
    json.dump(res, open(os.path.join(workdir, f"result_{rank}.json"), "w"))
    state.finish_process()
    state.destroy_distributed()


TASKS = {"nvls": task_nvls, "ep_timing": task_ep_timing, "dcp_engine": task_dcp_engine, "ag_gemm": task_ag_gemm, "dcp_mla": task_dcp_mla, "ep_moe": task_ep_moe, "pcp_moe": task_pcp_moe, "kv_pull": task_kv_pull, "comm": task_comm, "tp_engine": task_tp_engine, "server_loop": task_server_loop, "dp_engine": task_dp_engine, "pp_deepseek": task_pp_deepseek, "symm": task_symm}

if __name__ == "__main__":
    task, rank, world, port, workdir = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
    device_kind = sys.argv[6] if len(sys.argv) > 6 else "cpu"
    TASKS[task](rank, world, port, workdir, device_kind)
