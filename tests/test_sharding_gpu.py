"""GPU: shards computed separately (as the ranks of a multi-GPU job would, here one after another on one device) put
together give the unsharded result bit for bit: contiguous element ranges, expert groups of expert-sorted rows with
Zipf-distributed token counts, and (batch, kv-head group) blocks of attention addressed through strided views."""
import ctypes
import math

import numpy as np
import pytest

from fast_polynomial_transcendentals_b200 import sharding

pytestmark = pytest.mark.gpu


def stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("world", [2, 8])
def test_element_ranges_reproduce_the_whole(fpt, cuda, world):
    import torch
    n = (1 << 22) + 13
    x = (torch.rand(n, device=cuda) * 16 - 8).to(torch.float16)
    whole = torch.empty_like(x)
    fpt.call("fpt_unary", whole.data_ptr(), x.data_ptr(), n, 0, 0, 3, 0, 0, stream())
    parts = torch.full_like(x, float("nan"))
    for rank in range(world):
        lo, hi = sharding.element_range(n, rank, world)
        fpt.call("fpt_unary", parts.data_ptr() + 2 * lo, x.data_ptr() + 2 * lo, hi - lo, 0, 0, 3, 0, 0, stream())
    torch.cuda.synchronize()
    assert torch.equal(whole.view(torch.int16), parts.view(torch.int16))


@pytest.mark.parametrize("world", [2, 8])
def test_expert_groups_reproduce_the_whole(fpt, cuda, world):
    """16384 tokens, top-8 of 64 experts, intermediate 1408: rows sorted by expert, counts from the seeded Zipf(1.1)."""
    import torch
    experts, hidden = 64, 1408
    counts = sharding.zipf_expert_counts(16384 * 8, experts)
    rows = int(counts.sum())
    packed = (torch.randn(rows, 2 * hidden, device=cuda) * 1.5).to(torch.bfloat16)
    whole = torch.empty(rows, hidden, dtype=torch.bfloat16, device=cuda)
    fpt.call("fpt_swish_mul_packed", whole.data_ptr(), packed.data_ptr(), rows, hidden, 3, 1, 0, stream())
    parts = torch.full_like(whole, float("nan"))
    sizes = []
    for rank in range(world):
        shard = sharding.expert_group(counts, rank, world)
        n_rows = shard.last_row - shard.first_row
        sizes.append(n_rows)
        fpt.call("fpt_swish_mul_packed", parts.data_ptr() + 2 * hidden * shard.first_row,
                 packed.data_ptr() + 4 * hidden * shard.first_row, n_rows, hidden, 3, 1, 0, stream())
    torch.cuda.synchronize()
    assert sum(sizes) == rows and max(sizes) > min(sizes)      # Zipf: the groups are not the same size
    assert torch.equal(whole.view(torch.int16), parts.view(torch.int16))


@pytest.mark.parametrize("mode,causal,softcap", [(0, True, 50.0), (1, False, 0.0)])
def test_attention_blocks_reproduce_the_whole(fpt, cuda, mode, causal, softcap):
    import torch
    B, S, Hq, Hk, D = 2, 384, 8, 4, 128
    world = 4
    mk = lambda h: torch.randn(B, S, h, D, device=cuda).to(torch.bfloat16)
    q, k, v = mk(Hq), mk(Hk), mk(Hk)
    scale = 1.0 / math.sqrt(D)
    strides = lambda t: (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
    status = torch.zeros(1, dtype=torch.int32, device=cuda)

    def run(out, lse, qq, kk, vv):
        fpt.call("fpt_attention_fwd", out.data_ptr(), lse.data_ptr(), qq.data_ptr(), kk.data_ptr(), vv.data_ptr(), qq.shape[0], S,
                 qq.shape[2], kk.shape[2], D, strides(qq), strides(kk), strides(vv), strides(out), mode, int(causal), scale,
                 softcap, 9, status.data_ptr(), stream())

    whole = torch.empty_like(q)
    whole_lse = torch.empty(B, Hq, S, device=cuda)
    run(whole, whole_lse, q, k, v)
    parts = torch.full_like(q, float("nan"))
    parts_lse = torch.full_like(whole_lse, float("nan"))
    group = Hq // Hk
    covered = 0
    for rank in range(world):
        for blk in sharding.attention_blocks(B, Hq, Hk, rank, world):
            h0, h1 = blk.first_q_head, blk.last_q_head
            b = blk.batch
            lse = torch.empty(1, h1 - h0, S, device=cuda)      # log-sum-exp is a dense [B, H, S] plane of the call
            run(parts[b:b + 1, :, h0:h1], lse, q[b:b + 1, :, h0:h1], k[b:b + 1, :, h0 // group:h1 // group],
                v[b:b + 1, :, h0 // group:h1 // group])
            parts_lse[b, h0:h1] = lse[0]
            covered += h1 - h0
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and covered == B * Hq
    assert torch.equal(whole.view(torch.int16), parts.view(torch.int16))
    if mode != 1:
        assert torch.equal(whole_lse, parts_lse)
