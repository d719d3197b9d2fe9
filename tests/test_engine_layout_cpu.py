"""Row-block ownership layout of the sharded engine (no process group needed: the layout of every rank is computed
by every rank)."""
import torch
import torch.nn as nn

from lingua_b200.parallel.engine import BLOCK_ROWS, ParamGroup, default_scatter_filter, row_bounds


def _params():
    torch.manual_seed(0)
    return [("blk.wq.weight", nn.Parameter(torch.randn(512, 64))),
            ("blk.norm.weight", nn.Parameter(torch.randn(64))),
            ("blk.w1.weight", nn.Parameter(torch.randn(1408, 64))),   # 11 blocks: uneven over 4 and 8 ranks
            ("blk.tok_embeddings.weight", nn.Parameter(torch.randn(300, 64))),  # 2-D but not a GEMM gradient: plain
            ("blk.w2.weight", nn.Parameter(torch.randn(64, 1408))),   # fewer than 128 rows: plain
            ("blk.bias", nn.Parameter(torch.randn(7)))]


def test_row_bounds_are_monotone_block_aligned_and_cover_all_rows():
    for rows in (128, 512, 1408, 1400, 11008, 128256):
        for world in (1, 2, 3, 4, 8):
            b = row_bounds(rows, world)
            assert b[0] == 0 and b[-1] == rows and len(b) == world + 1
            assert all(x <= y for x, y in zip(b, b[1:]))
            assert all(x % BLOCK_ROWS == 0 for x in b[:-1])
            sizes = [y - x for x, y in zip(b, b[1:])]
            assert max(sizes) - min(sizes) <= 2 * BLOCK_ROWS


def test_every_element_has_exactly_one_owner_and_shards_round_trip():
    for world in (1, 2, 4, 8):
        groups = [ParamGroup("blk", list(_params()), world, r, torch.float32, torch.device("cpu"),
                             default_scatter_filter) for r in range(world)]
        g0 = groups[0]
        assert [f for f, _ in g0.params[:g0.n_mats]] == ["blk.wq.weight", "blk.w1.weight"]
        owned = torch.zeros(g0.padded, dtype=torch.int32)
        for r, g in enumerate(groups):
            assert g.segments == g0.segments and g.my_segments == g0.segments[r]
            for fo, n, so in g.my_segments:
                owned[fo:fo + n] += 1
                assert so % 8 == 0 and so + n <= g.shard_cap
        used = torch.zeros(g0.padded, dtype=torch.bool)
        for fqn, p in g0.params:
            o, n = g0.offsets[fqn]
            used[o:o + n] = True
        assert (owned[used] == 1).all(), "a parameter element is owned by no rank or by several"
        assert owned.max() <= 1
        # shards of all ranks reassemble the flat buffer
        flat = torch.arange(g0.padded, dtype=torch.float32)
        back = torch.zeros_like(flat)
        for r, g in enumerate(groups):
            g.unshard_into(back, g.shard_of(flat), r)
        assert torch.equal(back[used], flat[used])
        # the TP / replicated classes cover exactly the owned elements of the parameters
        for r, g in enumerate(groups):
            covered = sum(n for _, n, _ in g.classes())
            assert covered <= g.shard_numel and covered >= sum(n for _, n, _ in g.my_segments) - g.plain_padded
