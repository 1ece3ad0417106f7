"""CPU: shard planning, and a 2-rank gloo run showing that sharded results concatenate to the unsharded result
(the CPU oracle stands in for the device kernel: the point here is the host-side partitioning and failure handling)."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np
import pytest

from fast_polynomial_transcendentals_b200 import sharding

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("n", [0, 1, 7, 8, 9, 1000, 2 ** 20 + 13])
@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_element_ranges_partition_and_stay_aligned(n, world):
    ranges = [sharding.element_range(n, r, world) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == n
    for (lo, hi), (lo2, _) in zip(ranges, ranges[1:]):
        assert hi == lo2 and lo <= hi
    for lo, hi in ranges[:-1]:
        assert hi % 8 == 0 or hi == n


def test_expert_groups_follow_the_zipf_counts():
    counts = sharding.zipf_expert_counts(131072, 64)
    assert counts.sum() == 131072 and counts.size == 64
    assert np.array_equal(counts, sharding.zipf_expert_counts(131072, 64))   # seeded, reproducible
    assert counts.max() > 4 * np.median(counts)                              # skewed
    for world in (1, 2, 4, 8):
        shards = [sharding.expert_group(counts, r, world) for r in range(world)]
        assert shards[0].first_row == 0 and shards[-1].last_row == 131072
        for a, b in zip(shards, shards[1:]):
            assert a.last_expert == b.first_expert and a.last_row == b.first_row
        assert all(s.last_expert - s.first_expert == 64 // world for s in shards)


def test_attention_blocks_keep_gqa_groups_together():
    for world in (1, 2, 4, 8):
        seen = []
        for r in range(world):
            for blk in sharding.attention_blocks(4, 32, 8, r, world):
                assert blk.first_q_head % 4 == 0 and blk.last_q_head % 4 == 0
                seen += [(blk.batch, h) for h in range(blk.first_q_head, blk.last_q_head)]
        assert seen == [(b, h) for b in range(4) for h in range(32)]
    with pytest.raises(ValueError):
        sharding.attention_blocks(1, 6, 4, 0, 1)
    with pytest.raises(ValueError):
        sharding.element_range(10, 2, 2)


WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, {root!r})
    import numpy as np, torch, torch.distributed as dist
    from fast_polynomial_transcendentals_b200 import sharding
    from oracle import oracle
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=int(sys.argv[1]), world_size=2,
                            timeout=__import__("datetime").timedelta(seconds=60))
    rank = dist.get_rank()
    if sys.argv[2] == "fail" and rank == 1:
        raise SystemExit(3)            # a rank that dies before the exchange: the other must notice and not hang
    rng = np.random.default_rng(1234)   # every rank draws the same global input from the one seed
    n = 100003
    x = rng.uniform(-8, 8, n).astype(np.float16).view(np.uint16)
    prog = oracle.find_program("SIGMOID_FWD_D3", 0)
    lo, hi = sharding.element_range(n, rank, 2)
    mine = oracle.unary(prog, x[lo:hi])
    gathered = [None, None]
    dist.all_gather_object(gathered, (lo, hi, mine.tobytes()))
    if rank == 0:
        out = np.empty(n, dtype=np.uint16)
        for a, b, raw in gathered:
            out[a:b] = np.frombuffer(raw, dtype=np.uint16)
        assert np.array_equal(out, oracle.unary(prog, x)), "sharded result differs from the unsharded one"
        print("OK")
    dist.destroy_process_group()
""")


def launch(mode, port):
    code = WORKER.format(root=str(ROOT), port=port)
    env = dict(os.environ, OMP_NUM_THREADS="2")
    return [subprocess.Popen([sys.executable, "-c", code, str(r), mode], stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                             text=True, env=env) for r in range(2)]


def test_two_gloo_ranks_concatenate_to_the_single_process_result():
    procs = launch("ok", 29731)
    outs = [p.communicate(timeout=240) for p in procs]
    assert [p.returncode for p in procs] == [0, 0], outs
    assert "OK" in outs[0][0]


def test_a_rank_that_dies_is_reported_not_waited_for_forever():
    procs = launch("fail", 29732)
    outs = [p.communicate(timeout=240) for p in procs]
    assert procs[1].returncode == 3
    assert procs[0].returncode != 0          # rank 0's collective ends with an error inside the 60 s group timeout
