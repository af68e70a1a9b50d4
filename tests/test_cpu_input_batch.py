"""Per-step input staging: rows, slots, positions, padding and the single staging buffer."""
import numpy as np
import torch

from omni_npu_b200.engine.request import Request, SamplingParams
from omni_npu_b200.engine.scheduler import ScheduledSeq
from omni_npu_b200.worker.input_batch import InputBatch, StepLayout


def _req(rid, prompt, blocks, outputs=(), **sp):
    r = Request(rid, list(prompt), SamplingParams(**sp))
    r.block_ids = list(blocks)
    r.output_token_ids = list(outputs)
    return r


def _batch():
    return InputBatch(max_num_seqs=4, max_model_len=64, block_size=4, max_num_batched_tokens=32,
                      device=torch.device("cpu"))


def test_layout_sections_do_not_overlap_and_views_alias_the_buffer():
    lay = StepLayout.make(T=8, S=4, max_blocks=16)
    starts = sorted([lay.ids, lay.pos, lay.slot, lay.seq_lens, lay.cu_q, lay.temp, lay.top_k, lay.top_p, lay.seeds,
                     lay.logits_idx, lay.next_ids, lay.bt])
    assert len(set(starts)) == len(starts) and lay.total >= lay.bt + 4 * 16
    ib = _batch()
    v = ib.views(ib.layout_for(8, 4), ib.host)
    v["ids"][0] = 77
    v["temp"][1] = 0.5
    assert ib.host_np[ib.layout_for(8, 4).ids] == 77
    assert v["seeds"].dtype == torch.int64 and v["bt"].shape == (4, 16) and v["cu_q"].numel() == 5


def test_prefill_staging_positions_slots_and_next_tokens():
    ib = _batch()
    a = _req("a", range(10, 17), blocks=[5, 2], temperature=0.7, top_k=3, top_p=0.9, seed=11)    # 7 tokens
    b = _req("b", range(30, 40), blocks=[9, 1, 4])                                                 # 10 tokens
    lay = ib.layout_for(13, 2)
    rows, max_q = ib.stage_prefill(lay, [ScheduledSeq(a, 0, 7, True), ScheduledSeq(b, 4, 6, True)])
    v = ib.views(lay, ib.host)
    assert max_q == 7 and rows.tolist() == [0, 1]
    assert v["ids"].tolist() == list(range(10, 17)) + list(range(34, 40))
    assert v["pos"].tolist() == list(range(7)) + list(range(4, 10))
    # token at position p of a sequence lives in block table[p // 4] at offset p % 4
    assert v["slot"][:7].tolist() == [5 * 4 + p for p in range(4)] + [2 * 4 + p for p in range(3)]
    assert v["slot"][7:].tolist() == [1 * 4 + p for p in range(4)] + [4 * 4, 4 * 4 + 1]
    assert v["seq_lens"][:2].tolist() == [7, 10] and v["cu_q"][:3].tolist() == [0, 7, 13]
    assert v["logits_idx"][:2].tolist() == [6, 12]
    assert v["next_ids"][:7].tolist() == list(range(11, 17)) + [-1]          # last prompt token: successor unknown
    assert abs(float(v["temp"][0]) - 0.7) < 1e-6 and int(v["top_k"][0]) == 3
    # the staged seed: the request's seed (11) mixed with the index of the token being sampled (the first)
    assert int(v["seeds"][0]) == (11 + 0x9E3779B97F4A7C15) & 0x7FFFFFFFFFFFFFFF
    assert float(v["top_p"][1]) == 1.0 and v["bt"][0, :2].tolist() == [5, 2] and v["bt"][1, :3].tolist() == [9, 1, 4]


def test_decode_staging_pads_to_the_graph_size():
    ib = _batch()
    a = _req("a", range(5), blocks=[3, 6], outputs=[41])          # 6 tokens: next position 5 -> block 6, offset 1
    b = _req("b", range(3), blocks=[7], outputs=[42, 43])          # 5 tokens: position 4 needs a second block
    b.block_ids.append(8)
    for r in (a, b):
        ib.add_request(r)
    lay = ib.layout_for(4, 4)                                      # captured batch size 4, two real sequences
    rows = ib.stage_decode(lay, [a, b])
    v = ib.views(lay, ib.host)
    assert rows.tolist() == [0, 1]
    assert v["ids"].tolist() == [41, 43, 0, 0] and v["pos"].tolist() == [5, 4, 0, 0]
    assert v["slot"].tolist() == [6 * 4 + 1, 8 * 4 + 0, -1, -1]    # padded rows write nowhere
    assert v["seq_lens"].tolist() == [6, 5, 1, 1] and v["cu_q"].tolist() == [0, 1, 2, 3, 4]
    assert v["bt"][1, :2].tolist() == [7, 8] and (v["bt"][2:] == 0).all()
    assert (v["temp"][2:] == 0).all() and (v["top_p"][2:] == 1).all()
    ib.upload(lay)
    assert ib.h2d_bytes_last == lay.total * 4 and torch.equal(ib.dev[: lay.total], ib.host[: lay.total])


def test_rows_are_compacted_when_a_request_leaves():
    ib = _batch()
    reqs = [_req(n, range(4), blocks=[i + 1], temperature=0.1 * (i + 1)) for i, n in enumerate("abc")]
    for r in reqs:
        ib.add_request(r)
    ib.remove_request("a")                                         # last row moves into the hole
    assert ib.num_rows == 2 and ib.row_of == {"c": 0, "b": 1}
    assert ib.block_table[0, 0] == 3 and abs(ib.temperature[0] - 0.3) < 1e-6
    ib.remove_request("zzz")                                       # unknown ids are ignored
    # a preempted request comes back with fewer blocks: the row follows
    reqs[1].block_ids = []
    ib.sync_blocks(1, reqs[1])
    assert ib.num_blocks[1] == 0


def test_spec_decode_staging_feeds_last_token_plus_drafts():
    ib = _batch()
    a = _req("a", range(6), blocks=[2, 3, 4], outputs=[50])        # 7 tokens so far
    lay = ib.layout_for(5, 2)
    b = _req("b", range(4), blocks=[6, 7], outputs=[60])           # 5 tokens so far
    rows, max_q = ib.stage_spec_decode(lay, [ScheduledSeq(a, 6, 3, True, [51, 52]), ScheduledSeq(b, 4, 1, True, [])])
    v = ib.views(lay, ib.host)
    assert max_q == 3 and v["ids"][:4].tolist() == [50, 51, 52, 60]
    assert v["pos"][:4].tolist() == [6, 7, 8, 4] and v["seq_lens"][:2].tolist() == [9, 5]
    assert v["slot"][:4].tolist() == [3 * 4 + 2, 3 * 4 + 3, 4 * 4 + 0, 7 * 4 + 0]
    assert v["cu_q"][:3].tolist() == [0, 3, 4] and v["logits_idx"][:2].tolist() == [2, 3]
    assert v["next_ids"][:4].tolist() == [0, 1, 2, 3]              # flat index into the [n, max_q] verified matrix
