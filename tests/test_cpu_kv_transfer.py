"""Prefill/decode disaggregation on CPU: control plane, link manager, re-sharding
helpers and the full producer -> consumer life cycle through two engines."""
import time

import pytest
import torch

from omni_npu_b200 import SamplingParams
from omni_npu_b200.config import KVTransferConfig, tiny_llama
from omni_npu_b200.engine.llm import LLM
from omni_npu_b200.kv_transfer.control_plane import ControlClient, ControlServer, HeartbeatMonitor, HeartbeatThread
from omni_npu_b200.kv_transfer.manager import KVLinkManager, make_cluster_id, parse_cluster_id
from omni_npu_b200.kv_transfer.utils import TPConvertor, get_config_from_dict_or_env, get_p_start_rank


def test_cluster_id_round_trip_and_option_lookup(monkeypatch):
    cid = make_cluster_id("10.1.2.3", 14579, 8)
    assert parse_cluster_id(cid) == ("10.1.2.3", 14579, 8)
    monkeypatch.setenv("X_ENV", "from-env")
    assert get_config_from_dict_or_env({"k": "from-dict"}, "k", "X_ENV", "d") == "from-dict"
    assert get_config_from_dict_or_env({}, "k", "X_ENV", "d") == "from-env"
    assert get_config_from_dict_or_env(None, "k", "X_MISSING", "d") == "d"


def test_producer_rank_selection_and_head_resharding():
    assert [get_p_start_rank(4, 4, r) for r in range(4)] == [0, 1, 2, 3]
    assert [get_p_start_rank(2, 4, r) for r in range(4)] == [0, 0, 1, 1]
    assert [get_p_start_rank(4, 2, r) for r in range(2)] == [0, 2]
    conv = TPConvertor(num_kv_heads=8, p_tp=2, d_tp=4)
    # consumer rank 1 holds heads 2,3 = second half of producer rank 0's block
    assert conv.plan(1).sources == [(0, (2, 4), (0, 2))]
    conv = TPConvertor(num_kv_heads=8, p_tp=4, d_tp=2)
    assert conv.plan(1).sources == [(2, (0, 2), (0, 2)), (3, (0, 2), (2, 4))]
    assert TPConvertor(1, 4, 8, replicated=True).plan(5).sources == [(2, (0, 1), (0, 1))]
    assert conv.remap_blocks([7, 8, 9, 10], num_tokens=33, block_size=16) == [7, 8, 9]


def test_heartbeat_monitor_with_fake_clock():
    now = [0.0]
    m = HeartbeatMonitor(timeout_s=60, clock=lambda: now[0])
    m.beat("a")
    now[0] = 59
    assert m.alive("a") and m.expired() == []
    now[0] = 61
    assert not m.alive("a") and m.expired() == ["a"] and m.peers() == []


def test_control_plane_messages_and_lost_producer_detection():
    srv = ControlServer("127.0.0.1", 0, lambda: {"hello": "meta"})
    cli = ControlClient(srv.endpoint, "consumer-1", timeout_ms=2000)
    try:
        assert cli.get_meta() == {"hello": "meta"}
        cli.notify_pulled(["r1", "r2"])
        cli.notify_abort(["r3"])
        assert sorted(srv.take_pulled()) == ["r1", "r2", "r3"] and srv.take_pulled() == []
        assert cli.heartbeat() and srv.monitor.alive("consumer-1")
    finally:
        srv.close()
    # the producer is gone: beats fail, and after the timeout the loss is reported
    now = [0.0]
    lost = []
    cli.timeout_ms = 100
    hb = HeartbeatThread(lambda: {"p": cli}, lost.append, timeout_s=60, clock=lambda: now[0])
    hb.tick()
    assert lost == []
    now[0] = 61
    hb.tick()
    assert lost == ["p"]
    cli.close()


def test_link_manager_pull_and_layout_check():
    a = KVLinkManager(make_cluster_id("127.0.0.1", 1000, 1), 0, torch.device("cpu"))
    b = KVLinkManager(make_cluster_id("127.0.0.1", 2000, 1), 0, torch.device("cpu"))
    src = [(torch.randn(8, 2, 4, 16), torch.randn(8, 2, 4, 16)) for _ in range(3)]
    dst = [(torch.zeros(6, 2, 4, 16), torch.zeros(6, 2, 4, 16)) for _ in range(3)]
    exp = a.register_memory(src)
    b.register_memory(dst)
    b.pull_kv(exp.cluster_id, 0, [5, 1, 7], [0, 3, 2], refresh=lambda: exp)
    for (sk, sv), (dk, dv) in zip(src, dst):
        assert torch.equal(dk[[0, 3, 2]], sk[[5, 1, 7]]) and torch.equal(dv[[0, 3, 2]], sv[[5, 1, 7]])
        assert dk[1].abs().sum() == 0
    assert b.stats["blocks"] == 3 and b.is_linked(exp.cluster_id, 0)
    b.force_unlink(exp.cluster_id)
    assert not b.is_linked(exp.cluster_id, 0)
    c = KVLinkManager(make_cluster_id("127.0.0.1", 3000, 1), 0, torch.device("cpu"))
    c.register_memory([(torch.zeros(6, 2, 4, 32), torch.zeros(6, 2, 4, 32)) for _ in range(3)])
    with pytest.raises(ConnectionError):
        c.pull_kv(exp.cluster_id, 0, [0], [0], refresh=lambda: exp)
    a.close(), b.close(), c.close()


def test_disaggregated_prefill_then_decode_matches_single_engine():
    cfg = tiny_llama()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (40, 17, 33)]
    common = dict(device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, block_size=16,
                  num_gpu_blocks=32, seed=1, additional_config={"async_pull_kv": False})
    mono = LLM(model=cfg, **common)
    want = [o.output_token_ids for o in mono.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]

    prefill = LLM(model=cfg, kv_transfer_config=dict(kv_connector="P2PKVConnector", kv_role="kv_producer",
                                                      kv_port=0, kv_connector_extra_config={"kv_port": 24311}), **common)
    decode = LLM(model=cfg, kv_transfer_config=dict(kv_connector="P2PKVConnector", kv_role="kv_consumer",
                                                     kv_connector_extra_config={"kv_port": 24411}), **common)
    decode.engine.worker.get_model().load_state_dict(prefill.engine.worker.get_model().state_dict())
    try:
        p_out = prefill.generate(prompts, SamplingParams(max_tokens=1, ignore_eos=True))
        pool = prefill.engine.scheduler.pool
        assert pool.num_parked == 3, "producer must keep the blocks until they are pulled"
        for o, w in zip(p_out, want):
            assert o.output_token_ids == w[:1]
            assert o.kv_transfer_params["remote_block_ids"] and o.kv_transfer_params["remote_request_id"] == o.request_id
        # the decode instance receives the prompts plus the producers' transfer parameters
        order = {}
        for i, (p, o) in enumerate(zip(prompts, p_out)):
            rid = decode.engine.add_request(p, SamplingParams(max_tokens=8, ignore_eos=True),
                                            kv_transfer_params=o.kv_transfer_params)
            order[rid] = i
        got = [None] * 3
        while decode.engine.has_unfinished_requests():
            for o in decode.engine.step():
                got[order[o.request_id]] = o.output_token_ids
        assert got == want
        stats = decode.engine.worker.model_runner.kv_connector.manager.stats
        assert stats["pulls"] == 3 and stats["blocks"] == sum((len(p) + 15) // 16 for p in prompts)
        # acks reached the producer: one more scheduling round releases the parked blocks
        deadline = time.time() + 5
        while pool.num_parked and time.time() < deadline:
            prefill.engine.scheduler.schedule()
            time.sleep(0.05)
        assert pool.num_parked == 0 and pool.num_free == 32
    finally:
        prefill.engine.shutdown()
        decode.engine.shutdown()


def test_host_pool_slots_allocate_and_recycle(tmp_path, monkeypatch):
    from omni_npu_b200.kv_transfer import host_pool
    monkeypatch.setattr(host_pool, "POOL_DIR", str(tmp_path))
    pool = host_pool.HostKVPool("p0", 4, [64, 32], create=True)
    other = host_pool.HostKVPool("p0", 4, [64, 32], create=False)
    try:
        a = pool.alloc(3)
        assert sorted(a) == [0, 1, 2] and pool.alloc(2) is None
        pool.slots_view(1)[a[0]] = torch.arange(32, dtype=torch.uint8)
        assert torch.equal(other.slots_view(1)[a[0]], torch.arange(32, dtype=torch.uint8))    # same memory
        assert pool.slot_bytes == 96 and pool.slots_view(0).shape == (4, 64)
        pool.free(a)
        assert pool.num_free == 4
    finally:
        other.close()
        pool.close()
    assert not (tmp_path / "p0").exists()


def test_disaggregated_serving_through_the_host_pool(tmp_path, monkeypatch):
    """Prefill instance stores the prompt KV in the host pool and frees its GPU blocks at once;
    the decode instance loads the slots, generates the same tokens, and its ack recycles the slots."""
    from omni_npu_b200.kv_transfer import host_pool
    monkeypatch.setattr(host_pool, "POOL_DIR", str(tmp_path))
    cfg = tiny_llama()
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (35, 16, 50)]
    common = dict(device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, block_size=16,
                  num_gpu_blocks=32, seed=1, additional_config={"async_pull_kv": False})
    mono = LLM(model=cfg, **common)
    want = [o.output_token_ids for o in mono.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))]
    prefill = LLM(model=cfg, kv_transfer_config=dict(
        kv_connector="HostPoolKVConnector", kv_role="kv_producer",
        kv_connector_extra_config={"kv_port": 24511, "kv_pool_slots": 16, "kv_pool_name": "pool_t"}), **common)
    decode = LLM(model=cfg, kv_transfer_config=dict(kv_connector="OmniCacheConnector", kv_role="kv_consumer",
                                                     kv_connector_extra_config={"kv_port": 24611}), **common)
    decode.engine.worker.get_model().load_state_dict(prefill.engine.worker.get_model().state_dict())
    try:
        p_out = prefill.generate(prompts, SamplingParams(max_tokens=1, ignore_eos=True))
        conn = prefill.engine.worker.model_runner.kv_connector
        nblk = sum((len(p) + 15) // 16 for p in prompts)
        assert prefill.engine.scheduler.pool.num_parked == 0 and prefill.engine.scheduler.pool.num_free == 32
        assert conn.pool.num_free == 16 - nblk
        order = {}
        for i, (p, o) in enumerate(zip(prompts, p_out)):
            assert o.kv_transfer_params["kv_pool"]["pool"] == "pool_t"
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


def test_failed_kv_pull_falls_back_to_local_prefill():
    """A pull that fails on the host (injected: the link manager raises) is a per-request event:
    the decode instance computes that prompt itself, gives the same tokens, and keeps stepping."""
    cfg = tiny_llama()
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (36, 21)]
    common = dict(device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, block_size=16,
                  num_gpu_blocks=32, seed=1, additional_config={"async_pull_kv": False})
    mono = LLM(model=cfg, **common)
    want = [o.output_token_ids for o in mono.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))]
    prefill = LLM(model=cfg, kv_transfer_config=dict(kv_connector="P2PKVConnector", kv_role="kv_producer",
                                                      kv_port=0, kv_connector_extra_config={"kv_port": 24511}), **common)
    decode = LLM(model=cfg, kv_transfer_config=dict(kv_connector="P2PKVConnector", kv_role="kv_consumer",
                                                     kv_connector_extra_config={"kv_port": 24611}), **common)
    decode.engine.worker.get_model().load_state_dict(prefill.engine.worker.get_model().state_dict())
    try:
        p_out = prefill.generate(prompts, SamplingParams(max_tokens=1, ignore_eos=True))
        manager = decode.engine.worker.model_runner.kv_connector.manager
        real_pull, calls = manager.pull_kv, {"n": 0}

        def flaky_pull(*a, **kw):
            calls["n"] += 1
            if calls["n"] == 1:
                raise ConnectionError("injected: producer unreachable")
            return real_pull(*a, **kw)
        manager.pull_kv = flaky_pull
        order = {}
        for i, (p, o) in enumerate(zip(prompts, p_out)):
            order[decode.engine.add_request(p, SamplingParams(max_tokens=6, ignore_eos=True),
                                            kv_transfer_params=o.kv_transfer_params)] = i
        got, steps = [None] * 2, 0
        while decode.engine.has_unfinished_requests() and steps < 200:
            steps += 1
            for o in decode.engine.step():
                got[order[o.request_id]] = o.output_token_ids
        assert got == want
        assert decode.engine.scheduler.kv_load_failures == 1 and calls["n"] == 2
        assert decode.engine.scheduler.pool.num_free == 32
    finally:
        prefill.engine.shutdown()
        decode.engine.shutdown()
