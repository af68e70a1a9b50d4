"""Scheduler-side half of the KV connector and the block pool's parking, without engines:
which requests count as externally cached, what the per-step metadata carries, when a finished
producer request hands out transfer parameters, and how parked blocks come back (ack or expiry)."""
import types

import pytest

from omni_npu_b200.config import KVTransferConfig, tiny_llama
from omni_npu_b200.engine.block_manager import BlockPool
from omni_npu_b200.engine.llm import build_engine_config
from omni_npu_b200.engine.request import RequestStatus
from omni_npu_b200.kv_transfer import connector as conn


def _connector(role: str, async_pull: bool = False, port: int = 25011):
    cfg = build_engine_config(tiny_llama(), device="cpu", block_size=16,
                              kv_transfer_config=dict(kv_connector="P2PKVConnector", kv_role=role,
                                                      kv_connector_extra_config={"kv_port": port}),
                              additional_config={"async_pull_kv": async_pull})
    return conn.P2PKVConnector(cfg)


def _request(rid="r0", n_prompt=40, params=None, status=None):
    return types.SimpleNamespace(request_id=rid, num_prompt_tokens=n_prompt, kv_transfer_params=params,
                                 status=status, spec_token_ids=[])


REMOTE = dict(remote_block_ids=[7, 8, 9], remote_host_ip="tcp://127.0.0.1:1", remote_cluster_id="c",
              remote_request_id="p-1")


def test_external_tokens_only_for_consumers_with_remote_blocks():
    c = _connector("kv_consumer")
    try:
        assert c.get_num_new_matched_tokens(_request(params=None), 0) == (0, False)
        assert c.get_num_new_matched_tokens(_request(params={"remote_block_ids": []}), 0) == (0, False)
        # 3 remote blocks of 16 cover the 40-token prompt; tokens already computed locally are not re-counted
        assert c.get_num_new_matched_tokens(_request(params=REMOTE), 0) == (40, True)
        assert c.get_num_new_matched_tokens(_request(params=REMOTE), 16) == (24, True)
        # a longer prompt than the remote blocks hold: only what the blocks hold is external
        assert c.get_num_new_matched_tokens(_request(n_prompt=100, params=REMOTE), 0) == (48, True)
    finally:
        c.close()
    p = _connector("kv_producer", port=25012)
    try:
        assert p.get_num_new_matched_tokens(_request(params=REMOTE), 0) == (0, False)
    finally:
        p.close()


def test_step_metadata_carries_new_loads_once():
    c = _connector("kv_consumer", async_pull=False, port=25013)
    try:
        req = _request(params=REMOTE)
        c.update_state_after_alloc(req, [3, 4, 5, 6], 40)
        md = c.build_connector_meta(None)
        meta = md.requests["r0"]
        assert meta.local_block_ids == [3, 4, 5] and meta.remote_block_ids == [7, 8, 9] and meta.token_num == 40
        assert meta.remote_request_id == "p-1"
        assert c.build_connector_meta(None).requests == {}          # handed to the worker exactly once
        c.update_state_after_alloc(_request("r1", params=REMOTE), [9], 0)
        assert c.build_connector_meta(None).requests == {}          # nothing external: nothing to load
        assert not c.is_load_finished(req)                          # still pending until the worker reports
    finally:
        c.close()


def test_finished_producer_request_hands_out_transfer_parameters(monkeypatch):
    p = _connector("kv_producer", port=25014)
    try:
        done = _request("p-9", status=RequestStatus.FINISHED_LENGTH_CAPPED)
        delay, params = p.request_finished(done, [11, 12])
        assert delay == conn.BLOCK_RELEASE_DELAY_S
        assert params["remote_block_ids"] == [11, 12] and params["remote_request_id"] == "p-9"
        assert params["remote_cluster_id"] == p.cluster_id and params["remote_host_ip"].endswith(":25014")
        assert "p-9" in p.build_connector_meta(None).finished_producer
        # stopped by EOS / aborted / without blocks: nothing to transfer, blocks are freed at once
        assert p.request_finished(_request("x", status=RequestStatus.FINISHED_STOPPED), [1]) == (None, None)
        assert p.request_finished(_request("y", status=RequestStatus.FINISHED_LENGTH_CAPPED), []) == (None, None)
    finally:
        p.close()
    c = _connector("kv_consumer", port=25015)
    try:
        assert c.request_finished(_request("z", status=RequestStatus.FINISHED_LENGTH_CAPPED), [1]) == (None, None)
    finally:
        c.close()


def test_parked_blocks_return_on_ack_or_after_the_delay():
    pool = BlockPool(16, 16)
    a, b = pool.allocate(3), pool.allocate(2)
    free0 = pool.num_free
    pool.park("req-a", a, delay_s=600.0, now=100.0)
    pool.park("req-b", b, delay_s=5.0, now=100.0)
    assert pool.num_parked == 2 and pool.num_free == free0
    assert pool.expire_parked(now=104.0) == []                      # nothing is due yet
    assert pool.expire_parked(now=106.0) == ["req-b"] and pool.num_free == free0 + 2
    assert pool.release_parked("req-a") and pool.num_free == free0 + 5      # the consumer's ack
    assert not pool.release_parked("req-a")                          # a second ack is harmless
    assert pool.num_parked == 0


def test_token_interleaved_cache_resharded_to_a_wider_decode_group():
    """Prefill on 2 ranks, decode on 4: every decode rank takes each second token of one prefill rank
    out of the blocks it pulled and ends up with exactly its own tokens, in order."""
    import torch

    from omni_npu_b200.kv_transfer.utils import apply_dcp_reshard, plan_dcp_reshard
    n, pw, dw, bs, width = 37, 2, 4, 4, 3
    # producer caches: token p sits on rank p % pw at local index p // pw; its row carries p
    prod = []
    for r in range(pw):
        local = [p for p in range(n) if p % pw == r]
        nblk = -(-len(local) // bs)
        c = torch.full((nblk, bs, width), -1.0)
        for i, p in enumerate(local):
            c[i // bs, i % bs] = float(p)
        prod.append(c)
    seen = []
    for r in range(dw):
        plan = plan_dcp_reshard(n, pw, dw, r, bs)
        mine = [p for p in range(n) if p % dw == r]
        assert plan.src_rank == r % pw and plan.num_tokens == len(mine)
        pulled = prod[plan.src_rank][torch.tensor(plan.src_blocks, dtype=torch.long)]
        ids = list(range(10, 10 + -(-len(mine) // bs)))              # this rank's block ids, arbitrary
        cache = torch.full((32, bs, width), -1.0)
        apply_dcp_reshard(cache, ids, pulled, plan, bs)
        got = [cache[ids[k // bs], k % bs, 0].item() for k in range(len(mine))]
        assert got == [float(p) for p in mine]
        seen += mine
    assert sorted(seen) == list(range(n))
    # equal worlds: the identity
    plan = plan_dcp_reshard(10, 2, 2, 1, 4)
    assert plan.src_rank == 1 and plan.src_local == [0, 1, 2, 3, 4]
