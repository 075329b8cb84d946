"""Ownership partition + flat-buffer all-gather on CPU ranks (gloo, world_size 2): the owners form a
partition, views alias the flat buffer, and after step + all-gather every rank holds the same weights as a
single process stepping everything.  The step itself is played by the CPU oracle (the CUDA kernels need a
GPU); what is under test is the host-side sharding logic."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from came_b200.partition import ShardedParams, ShardedStepper, assign_owners, imbalance

SHAPES = [(64, 48), (300,), (33, 17), (128, 256), (40,), (96, 64), (16, 16)]


def test_assign_owners_is_a_balanced_partition():
    numels = [4096 * 4096] * 128 + [4096 * 11008] * 96 + [32000 * 4096] * 2 + [4096] * 65
    for w in (1, 2, 4, 8):
        owners = assign_owners(numels, w)
        assert len(owners) == len(numels) and set(owners) <= set(range(w))
        assert imbalance(numels, owners, w) < 1.02
    assert assign_owners([5, 5, 5], 2) == assign_owners([5, 5, 5], 2)      # deterministic
    with pytest.raises(ValueError):
        assign_owners([1], 0)


def test_views_alias_flat_buffer_and_are_aligned():
    sp = ShardedParams(SHAPES, torch.bfloat16, "cpu", world_size=2, rank=1)
    assert sp.flat.numel() == 2 * sp.slice_len
    seen = torch.zeros(sp.flat.numel(), dtype=torch.int32)
    for v, r in zip(sp.views, sp.owners):
        off = (v.data_ptr() - sp.flat.data_ptr()) // 2
        assert off % 128 == 0 and r * sp.slice_len <= off < (r + 1) * sp.slice_len
        seen[off:off + v.numel()] += 1
    assert int(seen.max()) == 1
    sp.views[0].fill_(3.0)
    assert float(sp.flat.float().sum()) == 3.0 * sp.views[0].numel()
    assert sorted(sp.owned) == [i for i, r in enumerate(sp.owners) if r == 1]


def test_bucketed_layout_keeps_cells_contiguous():
    sp = ShardedParams(SHAPES, torch.float32, "cpu", world_size=2, rank=0, buckets=3)
    assert len(sp.piece_len) == 3 and sp.flat.numel() == 2 * sum(sp.piece_len)
    seen = torch.zeros(sp.flat.numel(), dtype=torch.int32)
    for i, v in enumerate(sp.views):
        off = (v.data_ptr() - sp.flat.data_ptr()) // 4
        b, r = sp.bucket_of[i], sp.owners[i]
        lo = sp.bucket_off[b] + r * sp.piece_len[b]
        assert lo <= off and off + v.numel() <= lo + sp.piece_len[b]
        seen[off:off + v.numel()] += 1
    assert int(seen.max()) == 1
    assert sorted(i for b in range(3) for i in sp.owned_in_bucket(b)) == sorted(sp.owned)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import came_oracle as orc
        torch.manual_seed(0)
        init = [torch.randn(s) * 0.02 for s in SHAPES]
        grads = [torch.randn(s) * 1e-3 for s in SHAPES]
        sp = ShardedParams(SHAPES, torch.float32, "cpu", world, rank, buckets=3)
        for v, x in zip(sp.views, init):
            v.copy_(x)
        hp = orc.Hyper(weight_decay=1e-2)

        class OracleOptimizer:      # stands in for a came_b200 class on CPU ranks: steps the tensors it is given
            last_step_launches = 0

            def __init__(self, idx):
                self.idx = idx

            def step(self):
                for i in self.idx:
                    st = orc.init_state(sp.views[i], orc.CUDAFP)
                    sp.views[i].copy_(orc.step(sp.views[i].clone(), grads[i], st, hp, orc.CUDAFP))

        # each rank steps only the tensors it owns, bucket by bucket, gathering each bucket as it is done
        ShardedStepper(sp, {i: i for i in sp.owned}, OracleOptimizer).step()
        torch.save([v.clone() for v in sp.views], os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_step_then_all_gather_matches_single_process(tmp_path):
    from oracle import came_oracle as orc
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    torch.manual_seed(0)
    init = [torch.randn(s) * 0.02 for s in SHAPES]
    grads = [torch.randn(s) * 1e-3 for s in SHAPES]
    hp = orc.Hyper(weight_decay=1e-2)
    want = [orc.step(p.clone(), g, orc.init_state(p, orc.CUDAFP), hp, orc.CUDAFP) for p, g in zip(init, grads)]
    got = [torch.load(os.path.join(str(tmp_path), f"rank{r}.pt")) for r in range(world)]
    for r in range(world):
        for a, b in zip(got[r], want):
            assert torch.equal(a, b)


def test_weighted_assignment_follows_the_weights():
    owners = assign_owners([10] * 60, 4, [0.5, 1.0, 1.0, 0.5])
    load = [sum(10 for o in owners if o == r) for r in range(4)]
    assert load == [100, 200, 200, 100]
    with pytest.raises(ValueError):
        assign_owners([1, 2], 2, [1.0])
    sp = ShardedParams(SHAPES, torch.float32, "cpu", world_size=1, rank=0, buckets=3, bucket_weights=[1.0, 2.0, 1.0])
    assert sorted(i for b in range(3) for i in sp.owned_in_bucket(b)) == list(range(len(SHAPES)))


def _fallback_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import came_b200.partition as part

        real = part._lib.load()

        class Lib:      # rank 0 "exports" a handle, rank 1 cannot: the ranks must still agree on the exchange mode
            def __getattr__(self, name):
                return getattr(real, name)

            def came_b200_ipc_export(self, ptr, handle, offset):
                return part._lib.OK if rank == 0 else part._lib.E_CUDA

        part._lib.load = lambda: Lib()
        sp = ShardedParams(SHAPES, torch.float32, "cpu", world, rank, buckets=2)

        class Noop:
            last_step_launches = 0

            def __init__(self, idx):
                self.idx = idx

            def step(self):
                for i in self.idx:
                    sp.views[i].fill_(float(rank + 1))

        st = ShardedStepper(sp, {i: i for i in sp.owned}, Noop, gather_mode="auto")
        assert st.gather_mode == "nccl" and st.peer is None
        st.step()
        for v, o in zip(sp.views, sp.owners):
            assert float(v.flatten()[0]) == float(o + 1)
        with pytest.raises(RuntimeError):
            ShardedStepper(sp, {i: i for i in sp.owned}, Noop, gather_mode="peer")
        with pytest.raises(RuntimeError):      # the push mode needs the same mappings
            ShardedStepper(sp, {i: i for i in sp.owned}, Noop, gather_mode="push")
        with pytest.raises(ValueError):
            ShardedStepper(sp, {i: i for i in sp.owned}, Noop, gather_mode="bogus")
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_exchange_mode_falls_back_consistently_when_one_rank_cannot_export(tmp_path):
    """`auto`: a rank whose export fails still joins every collective of the set-up, and all ranks end in the NCCL
    (here: gloo) mode; `peer` and `push` raise on every rank."""
    world = 2
    mp.spawn(_fallback_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(os.path.join(str(tmp_path), f"ok{r}")) for r in range(world))


def _zero1_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from came_b200.partition import Zero1Step
        sp = ShardedParams(SHAPES, torch.float32, "cpu", world, rank, buckets=2)
        gflat, gviews = sp.like_flat()
        assert gflat.shape == sp.flat.shape and all(g.shape == v.shape for g, v in zip(gviews, sp.views))
        for i, g in enumerate(gviews):
            g.fill_(float((rank + 1) * (i + 1)))          # every rank's local gradient of every tensor

        class SumApplier:      # "optimizer": subtracts the (summed) gradient of the tensors it owns
            last_step_launches = 0

            def __init__(self, idx):
                self.idx = idx

            def step(self):
                for i in self.idx:
                    sp.views[i].sub_(gviews[i])

        st = ShardedStepper(sp, {i: i for i in sp.owned}, SumApplier)
        Zero1Step(st, gflat).run()
        total = sum(r + 1 for r in range(world))
        for i, v in enumerate(sp.views):
            assert torch.all(v == -float(total * (i + 1))), i      # every rank holds every tensor's update
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_zero1_sequence_reduces_steps_and_gathers(tmp_path):
    world = 2
    mp.spawn(_zero1_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(os.path.join(str(tmp_path), f"ok{r}")) for r in range(world))
