"""Host-side logic of the vocabulary-parallel LM head, on CPU: shard bounds, the candidate layout,
and - as two gloo ranks - that gathering per-shard candidates and merging them equals the
single-device oracle for every sampling mode."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import qx_oracle as O
from quixicore_metal_b200 import parallel

MODES = {"argmax": 0, "categorical": 1, "topk": 2, "topp": 3}


@pytest.mark.parametrize("V,shards", [(128256, 1), (128256, 2), (128256, 4), (128256, 8), (4013, 3), (256, 1), (1025, 4)])
def test_vocab_shard_bounds(V, shards):
    b = parallel.vocab_shard_bounds(V, shards)
    assert len(b) == shards and b[0][0] == 0 and b[-1][1] == V
    for (a0, a1), (b0, b1) in zip(b, b[1:]):
        assert a1 == b0
    assert all(x[0] % 256 == 0 for x in b)
    tiles = [-(-(e - s) // 256) for s, e in b]
    assert max(tiles) - min(tiles) <= 1 and max(tiles) == parallel.max_shard_tiles(V, shards) or V < 256 * shards
    if V == 128256 and shards == 8:
        assert [t for t in tiles] == [63, 63, 63, 63, 63, 62, 62, 62]


def _problem(seed=5, T=4, V=4000 + 13, K=256):
    rng = np.random.default_rng(seed)
    Wq = O.synth_pack("q8_0", (0.3 * rng.standard_normal((V, K))).astype(np.float32))
    h = O.round_bf16((0.5 * rng.standard_normal((T, K))).astype(np.float32))
    bias = rng.standard_normal(V).astype(np.float32)
    return O.lm_head_logits(h, Wq, "q8_0"), bias


@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("shards", [2, 3, 8])
def test_merge_of_shard_candidates_equals_single_device(mode, shards):
    L, bias = _problem()
    m = MODES[mode]
    kw = dict(k=16, temperature=0.8, seed=42)
    want = O.lm_head_sample_from_logits(L, m, top_p=0.9, bias=bias, **kw)
    mt = parallel.max_shard_tiles(L.shape[1], shards)
    parts = [O.lm_head_shard_candidates(L[:, a:b], m, bias_local=bias[a:b], vocab_offset=a, max_tiles=mt, **kw)
             for a, b in parallel.vocab_shard_bounds(L.shape[1], shards)]
    got = O.lm_head_merge_candidates([p[0] for p in parts], [p[1] for p in parts], [p[2] for p in parts],
                                     m, top_p=0.9, **kw)
    np.testing.assert_array_equal(got, want)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, mode, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        L, bias = _problem()
        m = MODES[mode]
        kw = dict(k=16, temperature=0.8, seed=42)
        a, b = parallel.vocab_shard_bounds(L.shape[1], world)[rank]
        mt = parallel.max_shard_tiles(L.shape[1], world)
        val, idx, lse = O.lm_head_shard_candidates(L[:, a:b], m, bias_local=bias[a:b], vocab_offset=a, max_tiles=mt, **kw)
        # the exchange buffer of the device path: [values | ids (as int32 bits) | lses], one all-gather
        mine = torch.from_numpy(np.concatenate([val.ravel(), idx.ravel().view(np.float32), lse.ravel()]))
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        T, C, Ln = val.shape[0], val.shape[1], lse.shape[1]
        vals = [g[:T * C].numpy().reshape(T, C) for g in gathered]
        idxs = [g[T * C:2 * T * C].numpy().view(np.int32).reshape(T, C) for g in gathered]
        lses = [g[2 * T * C:].numpy().reshape(T, Ln) for g in gathered]
        got = O.lm_head_merge_candidates(vals, idxs, lses, m, top_p=0.9, **kw)
        want = O.lm_head_sample_from_logits(L, m, top_p=0.9, bias=bias, **kw)
        out[rank] = bool(np.array_equal(got, want))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["argmax", "topk", "topp"])
def test_two_gloo_ranks_exchange_and_merge(mode):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        out = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_rank_main, args=(r, 2, port, mode, out)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
        assert all(p.exitcode == 0 for p in procs)
        assert dict(out) == {0: True, 1: True}


def test_exchange_form_follows_the_bytes_a_rank_sends():
    """Small candidate slots travel as words that carry their step number, large ones as plain stores
    plus a flag; decode-sized partial sums use the peer all-reduce, large ones NCCL."""
    V, kk = 128256, 32
    for world in (2, 4, 8):
        tiles = parallel.max_shard_tiles(V, world)
        for T, mode, want in ((1, 0, "words"), (64, 0, "words"), (64, 2, "words"), (1, 3, "words"), (64, 3, "push")):
            C, L = parallel.candidate_layout(mode, 50 if mode == 2 else kk, tiles)
            assert parallel.candidate_exchange_form(T * (2 * C + L), world) == want, (world, T, mode)
    # the boundary: exactly 1 MB sent per rank still goes as words
    assert parallel.candidate_exchange_form((1 << 20) // 8, 2) == "words"
    assert parallel.candidate_exchange_form((1 << 20) // 8 + 4, 2) == "push"
    hidden = 8192
    assert parallel.partial_sum_over_peers(hidden * 1, 8) and parallel.partial_sum_over_peers(hidden * 8, 8)
    assert not parallel.partial_sum_over_peers(hidden * 32, 8)
    assert parallel.partial_sum_over_peers(hidden * 32, 2) and not parallel.partial_sum_over_peers(hidden * 128, 2)
    assert not parallel.partial_sum_over_peers(7, 2)          # pairs of floats per word
