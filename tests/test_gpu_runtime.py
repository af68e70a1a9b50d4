"""Runtime pieces on a real GPU: the sleep-mode memory pool on the CUDA virtual-memory driver calls,
and disaggregated serving through the pinned host pool."""
import time

import pytest
import torch

from omni_npu_b200 import SamplingParams
from omni_npu_b200.config import ModelConfig
from omni_npu_b200.engine.llm import LLM

pytestmark = pytest.mark.gpu


def test_sleep_releases_device_memory_and_wake_restores_the_weights():
    """Weights-tagged tensors survive a sleep / wake cycle bit for bit, everything the pool held is
    given back to the device while asleep (at least 95 % of it shows up as free memory), and the
    discarded KV tensor is usable again after the wake-up."""
    from omni_npu_b200.worker.mem_pool import B200MemAllocator
    alloc = B200MemAllocator.get_instance()
    with alloc.use_memory_pool(tag="weights"):
        w = torch.arange(64 << 20, dtype=torch.int32, device="cuda")        # 256 MiB
    with alloc.use_memory_pool(tag="kv_cache"):
        kv = torch.ones(128 << 20, dtype=torch.int32, device="cuda")         # 512 MiB
    want = w.cpu()
    torch.cuda.synchronize()
    pool_bytes = alloc.get_current_usage()
    assert pool_bytes >= (768 << 20) and alloc.get_current_usage("weights") >= (256 << 20)
    free0, _ = torch.cuda.mem_get_info()
    released = alloc.sleep(offload_tags="weights")
    free1, _ = torch.cuda.mem_get_info()
    st = alloc.stats()
    assert released == pool_bytes and st["mapped_bytes"] == 0 and st["sleeping_bytes"] == pool_bytes
    assert st["host_backup_bytes"] == alloc.get_current_usage("weights")
    assert free1 - free0 >= 0.95 * pool_bytes, (free0, free1, pool_bytes)
    mapped = alloc.wake_up()
    st = alloc.stats()
    # the tensors are touched only after the allocator reports every byte mapped again
    assert mapped == pool_bytes and st["sleeping_bytes"] == 0 and st["mapped_bytes"] == pool_bytes, alloc.last_error()
    assert torch.equal(w.cpu(), want)
    kv.fill_(3)
    assert int(kv[12345]) == 3
    del w, kv


def test_disaggregated_serving_through_the_host_pool_on_the_gpu(tmp_path, monkeypatch):
    """Prefill instance copies the prompt KV into pinned host slots and frees its GPU blocks; the
    decode instance loads the slots into its own cache and generates what one instance generates."""
    import os
    import tempfile

    from omni_npu_b200.kv_transfer import host_pool
    # shared memory, as in deployment (a mapping of a file on disk cannot be pinned)
    shm = tempfile.mkdtemp(prefix="b200_pool_test_", dir="/dev/shm") if os.path.isdir("/dev/shm") else str(tmp_path)
    monkeypatch.setattr(host_pool, "POOL_DIR", shm)
    cfg = ModelConfig(hidden_size=512, num_layers=2, num_heads=8, num_kv_heads=2, head_dim=64,
                      intermediate_size=1024, vocab_size=2048, rope_theta=10000.0,
                      max_position_embeddings=2048, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (35, 16, 50)]
    common = dict(device="cuda", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, block_size=16,
                  num_gpu_blocks=32, seed=1, enforce_eager=True, additional_config={"async_pull_kv": False})
    mono = LLM(model=cfg, **common)
    want = [o.output_token_ids for o in mono.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))]
    prefill = LLM(model=cfg, kv_transfer_config=dict(
        kv_connector="HostPoolKVConnector", kv_role="kv_producer",
        kv_connector_extra_config={"kv_port": 24521, "kv_pool_slots": 16, "kv_pool_name": "pool_g"}), **common)
    decode = LLM(model=cfg, kv_transfer_config=dict(kv_connector="OmniCacheConnector", kv_role="kv_consumer",
                                                     kv_connector_extra_config={"kv_port": 24621}), **common)
    decode.engine.worker.get_model().load_state_dict(prefill.engine.worker.get_model().state_dict())
    try:
        p_out = prefill.generate(prompts, SamplingParams(max_tokens=1, ignore_eos=True))
        conn = prefill.engine.worker.model_runner.kv_connector
        nblk = sum((len(p) + 15) // 16 for p in prompts)
        assert prefill.engine.scheduler.pool.num_free == 32 and conn.pool.num_free == 16 - nblk
        order = {}
        for i, (p, o) in enumerate(zip(prompts, p_out)):
            rid = decode.engine.add_request(p, SamplingParams(max_tokens=6, ignore_eos=True),
                                            kv_transfer_params=o.kv_transfer_params)
            order[rid] = i
        got = [None] * 3
        while decode.engine.has_unfinished_requests():
            for o in decode.engine.step():
                got[order[o.request_id]] = o.output_token_ids
        assert got == want
        deadline = time.time() + 5
        while conn.pool.num_free < 16 and time.time() < deadline:
            prefill.engine.scheduler.schedule()
            time.sleep(0.05)
        assert conn.pool.num_free == 16
    finally:
        prefill.engine.shutdown()
        decode.engine.shutdown()
        import shutil
        if shm.startswith("/dev/shm/b200_pool_test_"):
            shutil.rmtree(shm, ignore_errors=True)
