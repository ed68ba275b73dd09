"""Optimizer and gradient-bucket logic that runs on the host."""
import math

import torch

from lbann_b200.ops.optim import ArenaShard, CHUNK, OWN_CHUNKS, ParameterArena
from lbann_b200.parallel.context import aligned_range, bucket_elements, plan_buckets


def test_hypergradient_adam_matches_reference_formulas():
    """src/optimizers/hypergradient_adam.cpp:137-185 restated with plain tensors."""
    torch.manual_seed(0)
    arena = ParameterArena(torch.device("cpu"))
    slot = arena.reserve("w", (5, 7))
    arena.materialise()
    slot.kind = "hypergradient_adam"
    slot.hp = {"learn_rate": 0.01, "hyper_learning_rate": 1e-3, "beta1": 0.9, "beta2": 0.99, "eps": 1e-8}
    x0 = torch.randn(5, 7)
    arena.view(arena.master, slot).copy_(x0)
    x = x0.double().clone()
    m1 = torch.zeros_like(x)
    m2 = torch.zeros_like(x)
    old = torch.zeros_like(x)
    lr, b1, b2, eps, hlr = 0.01, 0.9, 0.99, 1e-8, 1e-3
    for t in range(1, 5):
        g = torch.randn(5, 7)
        arena.view(arena.grad, slot).copy_(g)
        arena.step()
        gd = g.double()
        lr = lr + hlr * float((gd * old).sum())
        corr = math.sqrt(1 - b2 ** t) / (1 - b1 ** t)
        ge = gd + eps
        m1 = b1 * m1 + (1 - b1) * ge
        m2 = b2 * m2 + (1 - b2) * ge * ge
        old = corr * m1 / (m2.sqrt() + eps)
        x = x - lr * old
        assert torch.allclose(arena.view(arena.master, slot).double(), x, atol=1e-5)
        assert abs(slot.hp["learn_rate"] - lr) < 1e-7


def test_bucket_ranges_sit_on_16_byte_borders():
    for es in (2, 4):
        v = 16 // es
        for off, cnt in ((0, 1000), (3, 77), (1025, 4096), (5, 3)):
            a, b = aligned_range(off, cnt, es)
            assert a % v == 0 and b % v == 0 and a >= off and b <= off + cnt
        assert bucket_elements(64 << 20, es) % v == 0
        assert bucket_elements(100, es) % v == 0 and bucket_elements(100, es) >= 1 << 16


def test_bucket_plan_covers_every_trainable_slot_once():
    per = OWN_CHUNKS * CHUNK
    slots = [(0, 1000), (1024, 40000), (3 * per + 1024, 10)]
    buckets = plan_buckets(slots, 5 * per, per)
    covered = [(b.start, b.end) for b in buckets]
    assert covered == [(0, per), (per, 2 * per), (2 * per, 3 * per), (3 * per, 4 * per)][:len(covered)] or \
        all(e - s == per for s, e in covered)
    for o, c in slots:
        assert any(b.start < o + c and o < b.end for b in buckets)
    # ranges without trainable weights are not reduced
    assert all(any(b.start < o + c and o < b.end for o, c in slots) for b in buckets)


def test_shard_ownership_is_block_cyclic_and_complete():
    n = 5 * OWN_CHUNKS * CHUNK + 3 * CHUNK
    masks = [ArenaShard(r, 4, None).owner_mask(n, "cpu") for r in range(4)]
    total = torch.stack(masks).sum(0)
    assert bool((total == 1).all())          # every element has exactly one owner
    blk = OWN_CHUNKS * CHUNK
    for r, m in enumerate(masks):
        for b in range((n + blk - 1) // blk):
            assert bool(m[b * blk:(b + 1) * blk].all()) == (b % 4 == r)


def test_sharded_state_gather_restores_whole_state():
    """Each rank clears the blocks it does not own and the ranks sum: emulated with two
    arenas and a hand-made all-reduce."""
    n = 3 * OWN_CHUNKS * CHUNK
    arenas = []
    for r in range(2):
        a = ParameterArena(torch.device("cpu"))
        a.reserve("w", (n,))
        a.materialise()
        a.ensure_state1()
        a.shard = ArenaShard(r, 2, None)
        a.shard.state_whole = False
        own = a.shard.owner_mask(n, "cpu")
        a.state0.copy_(torch.where(own, torch.arange(n, dtype=torch.float32), torch.full((n,), -7.0)))
        a.state1.copy_(torch.where(own, torch.ones(n), torch.full((n,), 99.0)))
        arenas.append(a)
    pending = {}

    def make_allreduce(idx):
        def fn(t):
            pending.setdefault(idx, []).append(t)
        return fn
    for i, a in enumerate(arenas):
        a.gather_sharded_state(make_allreduce(i))
    for k in range(2):                       # the "all-reduce": sum the k-th tensor of both ranks
        s = pending[0][k] + pending[1][k]
        for i in range(2):
            pending[i][k].copy_(s)
    for a in arenas:
        assert torch.equal(a.state0, torch.arange(n, dtype=torch.float32))
        assert torch.equal(a.state1, torch.ones(n))
        assert a.shard.state_whole


def test_compact_state_pack_gather_and_commit():
    """Optimizer state kept for the owned blocks only: packing takes a rank's blocks in
    block order, the gather (unpack + sum over ranks) restores the whole tensor, views of the
    gathered copy can be written and committed back into the owned share."""
    n = 5 * OWN_CHUNKS * CHUNK - 1234                  # a ragged last block
    world = 2
    arenas = []
    for r in range(world):
        a = ParameterArena(torch.device("cpu"))
        a.reserve("w", (n // 2,))
        a.reserve("v", (n - n // 2 - 64,))
        a.materialise()
        a.ensure_state1()
        full0 = torch.arange(a.master.numel(), dtype=torch.float32)
        full1 = -full0
        a.state0.copy_(full0)
        a.state1.copy_(full1)
        a.shard = ArenaShard(r, world, None)
        before = a.state_bytes()
        a.compact_state()
        assert a.state_compact
        nblocks, mine = a._block_counts()
        assert nblocks == 5 and mine == (3 if r == 0 else 2)
        assert a.state_bytes() == 2 * 4 * mine * OWN_CHUNKS * CHUNK < 0.65 * before
        arenas.append(a)
    blk = OWN_CHUNKS * CHUNK
    assert torch.equal(arenas[1].state0[:blk], full0[blk:2 * blk])          # rank 1's first block is block 1
    pending = {}
    for i, a in enumerate(arenas):
        a.gather_sharded_state(lambda t, i=i: pending.setdefault(i, []).append(t))
    for k in range(2):
        total = pending[0][k] + pending[1][k]
        for i in range(world):
            pending[i][k].copy_(total)
    for a in arenas:
        for slot in a.slots:
            assert torch.equal(a.state_view(0, slot), a.view(full0, slot))
            assert torch.equal(a.state_view(1, slot), a.view(full1, slot))
    # a restart writes new values into the views; the commit keeps this rank's blocks of them
    a = arenas[0]
    a.state_view(0, a.slots[1]).fill_(5.0)
    want = full0.clone()
    a.view(want, a.slots[1]).fill_(5.0)
    a.commit_state()
    assert a._full_state is None
    back = a._unpack_state(a.state0)
    own = a.shard.owner_mask(want.numel(), "cpu")
    assert torch.equal(back[:a.total], torch.where(own, want, torch.zeros_like(want))[:a.total])
