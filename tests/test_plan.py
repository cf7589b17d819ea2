"""Execution plan: layout, block schedule with feature masks, activation-keeping modes, memory estimate, CLI."""
import pytest

from parameter_golf_b200.plan import ExecutionPlan, estimate_engine_memory, saved_slots
from parameter_golf_b200.spec import family_preset


def test_record_plan_layout_and_schedule():
    s = family_preset("record_11l")
    s.train.backend, s.train.world_size = "cuda_distributed", 8
    plan = ExecutionPlan.from_run_spec(s)
    assert plan.bank_layout.qo_bank == (22, 512, 512) and plan.bank_layout.kv_bank == (22, 256, 512)
    assert plan.bank_layout.mlp_up_bank == (11, 1536, 512) and plan.bank_layout.mlp_down_bank == (11, 512, 1536)
    assert plan.bank_layout.elems()["qo_bank"] == 22 * 512 * 512
    assert plan.grad_accum_steps == 1 and plan.micro_batch_tokens == s.train.batch_tokens // 8
    assert [x.layer for x in plan.layer_schedule] == list(range(11))
    assert [x.xsa for x in plan.layer_schedule] == [False] * 7 + [True] * 4
    assert all(x.saved for x in plan.layer_schedule)
    assert plan.layer_schedule[0].unet_role == "encoder" and plan.layer_schedule[10].unet_role == "decoder"
    assert plan.fingerprint == f"{s.fingerprint():016x}"
    lines = plan.summary_lines()
    assert any(l.startswith("plan.memory.total=") for l in lines) and "plan.bank.qo_bank=22x512x512" in lines


def test_saved_modes_follow_the_checkpoint_rule():
    sched = [(l, 0) for l in range(11)]
    assert saved_slots(sched, "edges") == [True] * 3 + [False] * 6 + [True] * 2
    assert saved_slots(sched, "inner") == [False] * 3 + [True] * 6 + [False] * 2
    assert saved_slots(sched, "none") == [False] * 11 and saved_slots(sched, "all") == [True] * 11
    rec = [(0, 0), (1, 0), (1, 1), (2, 0), (2, 1), (3, 0)]
    assert saved_slots(rec, "recurrent") == [False, True, True, True, True, False]
    assert saved_slots(rec, "edges") == [True, False, False, False, False, False]
    with pytest.raises(ValueError):
        saved_slots(sched, "some")


def test_memory_estimate_scales_and_checkpointing_shrinks_it():
    s = family_preset("record_11l")
    a = estimate_engine_memory(s, 98304)
    b = estimate_engine_memory(s, 2 * 98304)
    assert b.activations == pytest.approx(2 * a.activations, rel=1e-6) and b.params_fp32 == a.params_fp32
    assert 10 * 2 ** 30 < a.total < 40 * 2 ** 30            # the record micro-batch fits a 180 GB device several times over
    s.train.save_layer_acts = "none"
    c = estimate_engine_memory(s, 98304)
    assert c.activations < 0.35 * a.activations and c.params_fp32 == a.params_fp32
    ev = estimate_engine_memory(s, 98304, train=False)
    assert ev.grads_fp32 == 0 and ev.backward_scratch == 0 and ev.activations < a.activations


def test_plan_cli_prints_key_value_lines(capsys):
    from parameter_golf_b200.train import main
    assert main(["plan", "--family", "record_11l", "train.save_layer_acts=edges"]) == 0
    out = capsys.readouterr().out
    assert "plan.saved_mode=edges" in out and "plan.saved_blocks=5" in out and "plan.block.10.0=decoder:xsa+saved" in out


def test_preliminary_sweep_script_runs_on_cpu():
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench", "preliminary.py"), "--only", "arch"], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])
    fams = {row["family"]: row for row in out["arch"]}
    assert fams["record_11l"]["fits"] and fams["record_11l"]["params"] > 26_000_000 and fams["tiny_cpu"]["engine_gib"] < 5


def test_bank_shards_cover_every_slot_once_and_every_layer_gets_six_weight_pushes():
    """Host-side bookkeeping of the sharded optimizer: the slot ranges of the ranks tile each bank, trailing ranks may own
    nothing, and per step every layer's ready counter is bumped by exactly six slots (Q, O, K, V, up, down) whatever the
    world size: the value the QKV product of the next forward waits for."""
    from parameter_golf_b200.parallel.dist_engine import shard_range, slot_layer
    for n in (1, 3, 11, 12):
        banks = {"qo_bank": 2 * n, "kv_bank": 2 * n, "mlp_up_bank": n, "mlp_down_bank": n}
        for world in range(1, 9):
            bumps = [0] * n
            for bank, slots in banks.items():
                seen = []
                for rank in range(world):
                    s0, s1 = shard_range(slots, rank, world)
                    assert 0 <= s0 <= s1 <= slots
                    seen.extend(range(s0, s1))
                    for s in range(s0, s1):
                        bumps[slot_layer(bank, s, n)] += 1
                assert seen == list(range(slots)), (bank, world)
            assert bumps == [6] * n, (n, world, bumps)
    assert shard_range(22, 7, 8) == (21, 22) and shard_range(11, 6, 8) == (11, 11)       # the last ranks of 8 own little or nothing


def test_logit_chunk_rows_keeps_small_heads_whole_and_bounds_large_ones():
    """The output head is chunked by rows only when [T, V] passes 2^27 elements; chunks are multiples of 128 rows, at least 128,
    never more than T, and an explicit override wins."""
    from parameter_golf_b200.plan import logit_chunk_rows
    T = 98304
    assert logit_chunk_rows(T, 1024) == T                       # 100 M logits: kept whole
    r = logit_chunk_rows(T, 8192)
    assert r < T and r % 128 == 0 and r * 8192 <= 1 << 26       # 805 M logits: chunks of at most 2^26
    assert logit_chunk_rows(256, 65536) == 256                  # small batch: still whole
    assert logit_chunk_rows(T, 1024, override=1000) == 896 and logit_chunk_rows(T, 1024, override=64) == 128
    assert logit_chunk_rows(512, 1024, override=4096) == 512
