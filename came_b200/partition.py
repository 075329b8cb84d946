"""Ownership partition of a parameter set over the GPUs of one box (ZeRO-1 style) and the all-gather of
the updated weights that follows a step.

The reference is single-process (no collective anywhere in came_pytorch); this module is the one
distributed component around the step.  Tensors are independent units of the CAME step (clip RMS, row/col
means and absmax blocks are all per tensor, came_pytorch/CAME8bit.py:739-861), so each rank steps the whole
tensors it owns and no collective is needed inside the step.  Afterwards every rank needs every updated
weight: parameters live in ONE flat buffer ordered by owner, each owner's slice padded to the same length,
so a single in-place `all_gather_into_tensor` (ncclAllGather with sendbuff inside recvbuff) moves them.
"""
from __future__ import annotations

import contextlib
import math

import torch
import torch.distributed as dist

from . import _lib

PEER_STREAMS = 1    # concurrent pulls per rank in the copy-engine exchange (two measured slower at 8 GPUs: 642 vs 707 GB/s)
ALIGN_ELEMS = 128   # every tensor starts on a 256-byte boundary (bf16), keeping the 16-byte vector paths


def assign_owners(numels, world_size: int, weights=None):
    """Greedy longest-processing-time assignment of tensors to ranks by element count.
    Deterministic: ties go to the lower tensor index, then to the lower rank.  `weights` (one positive number per
    rank) asks for loads in those proportions instead of equal ones."""
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    if weights is None:
        weights = [1.0] * world_size
    if len(weights) != world_size or any(w <= 0 for w in weights):
        raise ValueError("weights must give one positive number per rank")
    order = sorted(range(len(numels)), key=lambda i: (-int(numels[i]), i))
    load = [0] * world_size
    owners = [0] * len(numels)
    for i in order:
        r = min(range(world_size), key=lambda k: ((load[k] + int(numels[i])) / weights[k], k))
        owners[i] = r
        load[r] += int(numels[i])
    return owners


def imbalance(numels, owners, world_size: int) -> float:
    """max rank load / mean rank load."""
    load = [0] * world_size
    for n, r in zip(numels, owners):
        load[r] += int(n)
    mean = sum(load) / world_size
    return max(load) / mean if mean > 0 else 1.0


class ShardedParams:
    """All parameters of a model as views into one flat buffer laid out for in-place all-gathers.

    Layout: [bucket][owner rank][that rank's tensors of the bucket, padded to the bucket's piece length].
    With one bucket this is the plain "slice per owner" layout.  With several, bucket b of every rank can be
    gathered (one contiguous in-place all-gather) while the ranks are still stepping bucket b+1.  `bucket_weights`
    sets the relative sizes of the buckets (a small first bucket starts the exchange early, a small last one
    leaves a short tail after the last step)."""

    def __init__(self, shapes, dtype: torch.dtype, device, world_size: int, rank: int, owners=None, buckets: int = 1,
                 bucket_weights=None):
        self.shapes = [tuple(s) for s in shapes]
        self.world_size, self.rank = int(world_size), int(rank)
        self.n_buckets = max(1, int(buckets))
        numels = [math.prod(s) for s in self.shapes]
        self.owners = list(owners) if owners is not None else assign_owners(numels, world_size)
        if len(self.owners) != len(self.shapes) or any(not 0 <= r < world_size for r in self.owners):
            raise ValueError("owners must give one rank in [0, world_size) per tensor")
        # inside each rank: spread its tensors over the buckets, again greedily by size
        self.bucket_of = [0] * len(self.shapes)
        for r in range(world_size):
            mine = [i for i, o in enumerate(self.owners) if o == r]
            sub = assign_owners([numels[i] for i in mine], self.n_buckets, bucket_weights)
            for i, b in zip(mine, sub):
                self.bucket_of[i] = b
        # offsets inside each (bucket, rank) cell
        fill = [[0] * world_size for _ in range(self.n_buckets)]
        local_off = []
        for n, r, b in zip(numels, self.owners, self.bucket_of):
            local_off.append(fill[b][r])
            fill[b][r] += (n + ALIGN_ELEMS - 1) // ALIGN_ELEMS * ALIGN_ELEMS
        self.piece_len = [max(max(fill[b]), ALIGN_ELEMS) for b in range(self.n_buckets)]
        self.bucket_off = [0]
        for b in range(self.n_buckets):
            self.bucket_off.append(self.bucket_off[-1] + self.piece_len[b] * world_size)
        self.slice_len = sum(self.piece_len)          # elements each rank contributes over all buckets
        self.flat = torch.zeros(self.bucket_off[-1], dtype=dtype, device=device)
        self.views = []
        for shape, n, r, b, off in zip(self.shapes, numels, self.owners, self.bucket_of, local_off):
            start = self.bucket_off[b] + r * self.piece_len[b] + off
            self.views.append(self.flat[start:start + n].view(shape))
        self.owned = [i for i, r in enumerate(self.owners) if r == rank]

    def owned_in_bucket(self, b: int):
        return [i for i in self.owned if self.bucket_of[i] == b]

    def bucket_region(self, b: int) -> torch.Tensor:
        return self.flat[self.bucket_off[b]:self.bucket_off[b + 1]]

    def my_piece(self, b: int) -> torch.Tensor:
        start = self.bucket_off[b] + self.rank * self.piece_len[b]
        return self.flat[start:start + self.piece_len[b]]

    def all_gather_bucket(self, b: int, group=None, async_op: bool = False):
        """Every rank sends its piece of bucket b and receives everybody else's, in place."""
        if self.world_size == 1:
            return None
        return dist.all_gather_into_tensor(self.bucket_region(b), self.my_piece(b), group=group, async_op=async_op)

    def all_gather(self, group=None, async_op: bool = False):
        """Gathers every bucket; with async_op returns the list of work handles."""
        works = [self.all_gather_bucket(b, group=group, async_op=async_op) for b in range(self.n_buckets)]
        return works if async_op else None

    def like_flat(self) -> tuple:
        """A second flat buffer with the same layout (for gradients) and the per-tensor views into it."""
        flat = torch.zeros_like(self.flat)
        views = []
        for v in self.views:
            start = (v.data_ptr() - self.flat.data_ptr()) // self.flat.element_size()
            views.append(flat[start:start + v.numel()].view(v.shape))
        return flat, views

    def reduce_scatter_bucket(self, flat: torch.Tensor, b: int, group=None):
        """Sums bucket b of `flat` (a buffer laid out like the parameters, e.g. every rank's local gradients) over
        the ranks; each rank receives the sum of its own piece, in place.  Backends without reduce-scatter (gloo)
        all-reduce the bucket instead."""
        if self.world_size == 1:
            return
        region = flat[self.bucket_off[b]:self.bucket_off[b + 1]]
        mine = region[self.rank * self.piece_len[b]:(self.rank + 1) * self.piece_len[b]]
        if dist.get_backend(group) == "nccl":
            dist.reduce_scatter_tensor(mine, region, op=dist.ReduceOp.SUM, group=group)
        else:
            dist.all_reduce(region, op=dist.ReduceOp.SUM, group=group)

    def gathered_bytes_per_rank(self) -> int:
        """Bytes each rank receives from its peers in one full all-gather."""
        return (self.world_size - 1) * self.slice_len * self.flat.element_size()


class PeerGather:
    """The all-gather of updated weights done with the GPUs' copy engines instead of a collective kernel: every
    rank maps the flat buffer of every peer into its own GPU's address space (CUDA IPC with peer access) and PULLS
    the peers' pieces of a bucket with plain device-to-device copies over NVLink, issued on its own GPU.  Nothing runs on the SMs, so the step of the next bucket keeps all of
    them, and a peer copy moves more bytes per second than the NCCL all-gather does here.

    Ordering between ranks comes from one-element all-reduces (NCCL, a few microseconds): a rank may read a peer's
    piece of bucket b only after the peer has finished stepping it, and nobody may start the next step (which
    rewrites its own pieces) before every peer has pulled them.  One process per GPU, all GPUs of one box visible
    to every process.  The push mode of ShardedStepper uses the same mappings the other way round: the step's kernels
    store into them, and only what they do not deliver is pulled (`pull_ranges`)."""

    def __init__(self, sharded: ShardedParams, group=None):
        import ctypes as C
        self.sharded, self.group = sharded, group
        self._lib = _lib.load()
        self.bases = [None] * sharded.world_size      # mapped allocations of the peers (to unmap)
        self.peer_ptr = [0] * sharded.world_size      # address of each peer's flat buffer in this process
        handle = C.create_string_buffer(64)
        offset = C.c_uint64(0)
        on_gpu = sharded.flat.is_cuda
        with (torch.cuda.device(sharded.flat.device) if on_gpu else contextlib.nullcontext()):
            # Every rank takes part in the collective below whatever happened to its own export: a rank that failed
            # sends None, and every rank then sees that the exchange is not available (no rank is left waiting in a
            # collective the others skipped).
            mine = None
            if self._lib.came_b200_ipc_export(sharded.flat.data_ptr(), handle, C.byref(offset)) == _lib.OK:
                mine = (handle.raw, int(offset.value))
            exported = [None] * sharded.world_size
            dist.all_gather_object(exported, mine, group=group)
            self.error = None
            if any(e is None for e in exported):
                self.error = "a rank could not export its parameter buffer"
            else:
                for r, (raw, off) in enumerate(exported):
                    if r == sharded.rank:
                        continue
                    base = C.c_void_p()
                    if self._lib.came_b200_ipc_open(raw, C.byref(base)) != _lib.OK:
                        self.error = f"mapping the buffer of rank {r} failed: " + self._lib.came_b200_last_error().decode()
                        break
                    self.bases[r] = base
                    self.peer_ptr[r] = base.value + off
        if self.error:
            return
        self.flag = torch.zeros(1, dtype=torch.float32, device=sharded.flat.device)
        # side stream(s) of the pulls; with one, a rank reads one peer at a time and the peers are visited in an order
        # rotated by rank, so that every source serves one reader at a time
        self.sides = [torch.cuda.Stream(device=sharded.flat.device) for _ in range(PEER_STREAMS)]
        self.pulled = None        # pending: "every peer has pulled my pieces of the last exchange"

    def close(self) -> None:
        for r, base in enumerate(getattr(self, "bases", [])):
            if base is not None:
                self._lib.came_b200_ipc_close(base)
                self.bases[r] = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def pull_bucket(self, b: int) -> None:
        """Enqueue (on a side stream) the copies that bring every peer's piece of bucket b into the local buffer.
        Call it after this rank's step of bucket b has been enqueued on the current stream."""
        s = self.sharded
        ready = dist.all_reduce(self.flag, group=self.group, async_op=True)   # every rank's bucket b is stepped
        for side in self.sides:
            with torch.cuda.stream(side):
                ready.wait()
        n = s.piece_len[b]
        esz = s.flat.element_size()
        with torch.cuda.device(s.flat.device):
            for k in range(1, s.world_size):
                r = (s.rank + k) % s.world_size          # start with a different peer on every rank
                lo = s.bucket_off[b] + r * n
                # issued from THIS GPU's side (its copy engine pulls): a copy issued on the source GPU from this
                # process would wait for time slices between the kernels of the process that owns that GPU
                _lib.check(self._lib.came_b200_peer_copy_async(
                    s.flat.data_ptr() + lo * esz, self.peer_ptr[r] + lo * esz, n * esz, -1,
                    self.sides[k % len(self.sides)].cuda_stream))

    def pull_ranges(self, ranges_by_rank: dict) -> None:
        """Like pull_bucket for explicit pieces: {peer rank: [(first element, elements), ...]} of the flat buffer."""
        s = self.sharded
        ready = dist.all_reduce(self.flag, group=self.group, async_op=True)   # every rank has enqueued its step
        for side in self.sides:
            with torch.cuda.stream(side):
                ready.wait()
        esz = s.flat.element_size()
        with torch.cuda.device(s.flat.device):
            for k in range(1, s.world_size):
                r = (s.rank + k) % s.world_size
                for lo, n in ranges_by_rank.get(r, ()):
                    _lib.check(self._lib.came_b200_peer_copy_async(
                        s.flat.data_ptr() + lo * esz, self.peer_ptr[r] + lo * esz, n * esz, -1,
                        self.sides[k % len(self.sides)].cuda_stream))

    def finish(self) -> None:
        """Current stream: wait for this rank's pulls.  That the peers have finished pulling FROM this rank is only
        needed before this rank's weights are rewritten: the all-reduce that says so is started here and waited
        for by `before_step`, so the end of a step does not wait for the slowest rank."""
        for side in self.sides:
            torch.cuda.current_stream().wait_stream(side)
        self.pulled = dist.all_reduce(self.flag, group=self.group, async_op=True)

    def before_step(self) -> None:
        """Current stream: the step about to be enqueued rewrites this rank's pieces; every peer must have pulled
        the previous ones."""
        if self.pulled is not None:
            self.pulled.wait()
            self.pulled = None


class ShardedStepper:
    """One optimizer per bucket over the tensors this rank owns; `step()` steps bucket after bucket and starts the
    all-gather of a bucket's updated weights as soon as its step kernels are enqueued, so that the gather of
    bucket b travels over NVLink while bucket b+1 is being stepped.  `gather_mode`: "nccl" (in-place
    all_gather_into_tensor per bucket), "peer" (copy-engine pulls over CUDA IPC mappings, see PeerGather) or "push":
    the kernel that applies a tensor's update stores the new weights into every peer's buffer as it goes (plain stores
    over NVLink into the same IPC mappings), so there is no separate exchange pass for those tensors; what the fused
    kernel does not step (1-D tensors, odd shapes) is still pulled, and one small all-reduce after the step orders
    every rank's stores before anybody reads the weights."""

    def __init__(self, sharded: ShardedParams, params_by_index: dict, make_optimizer, gather_mode: str = "nccl",
                 group=None):
        if gather_mode not in ("nccl", "peer", "push", "auto"):
            raise ValueError("gather_mode must be 'nccl', 'peer', 'push' or 'auto'")
        self.sharded, self.group = sharded, group
        self.opts = []
        for b in range(sharded.n_buckets):
            ps = [params_by_index[i] for i in sharded.owned_in_bucket(b)]
            self.opts.append(make_optimizer(ps) if ps else None)
        self.peer = None
        self.gather_mode = "nccl"
        if gather_mode != "nccl" and sharded.world_size > 1:
            # "auto": use the copy-engine exchange when every rank could map every peer, else NCCL (all ranks agree:
            # every rank runs the same two collectives whatever failed locally)
            self.peer = PeerGather(sharded, group=group)
            ok = torch.tensor([0.0 if self.peer.error else 1.0], device=sharded.flat.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if ok.item() == 1.0:
                self.gather_mode = "push" if gather_mode == "push" else "peer"
            else:
                err = self.peer.error
                self.peer.close()
                self.peer = None
                if gather_mode in ("peer", "push"):
                    raise RuntimeError(f"peer mapping of the parameter buffers failed on some rank: {err}")
        self._push_ranges = None      # push mode: {peer rank: [(first element, elements)]} still to be pulled
        if self.gather_mode == "push" and sharded.world_size - 1 > 7:
            raise ValueError("push mode serves at most 7 peers")

    def _push_args(self):
        s = self.sharded
        peers = [self.peer.peer_ptr[r] for r in range(s.world_size) if r != s.rank]
        return s.flat.data_ptr(), s.flat.numel() * s.flat.element_size(), peers

    def _set_push(self, on: bool) -> None:
        base, nbytes, peers = self._push_args()
        for o in self.opts:
            if o is not None:
                o._engine.set_push(base, nbytes, peers if on else [])

    def reset_push(self) -> None:
        """Push mode: forget which tensors the kernels deliver.  The next `step()` works it out again (a collective:
        call this on every rank) -- needed when the tensors of an optimizer, their dtypes or their alignment changed
        after the first step, since a tensor that leaves the fused kernel must be pulled from then on."""
        self._push_ranges = None

    def _setup_push(self) -> None:
        """First step in push mode (the gradients exist by now): build the plans, learn which tensors the kernels
        deliver themselves, tell the peers, and work out what is left to pull from each of them."""
        s = self.sharded
        mine = {}
        for b, o in enumerate(self.opts):
            idx = s.owned_in_bucket(b)
            if o is None:
                continue
            o.prime_for_cuda_graph()
            plans = list(o._engine.plans.values())
            flags = plans[0].pushed() if len(plans) == 1 and plans[0].n == len(idx) else [False] * len(idx)
            if not any(flags):
                flags = [False] * len(idx)
            mine.update(dict(zip(idx, flags)))
        everyone = [None] * s.world_size
        dist.all_gather_object(everyone, mine, group=self.group)
        pushed = {}
        for d in everyone:
            pushed.update(d)
        self._set_push(True)
        ranges = {}
        for i, (r, view) in enumerate(zip(s.owners, s.views)):
            if r == s.rank or pushed.get(i, False):
                continue
            lo = (view.data_ptr() - s.flat.data_ptr()) // s.flat.element_size()
            lst = ranges.setdefault(r, [])
            if lst and lst[-1][0] + lst[-1][1] == lo:
                lst[-1] = (lst[-1][0], lst[-1][1] + view.numel())
            else:
                lst.append((lo, view.numel()))
        self._push_ranges = ranges

    def step(self, gather: bool = True):
        works = []
        if self.gather_mode == "push":
            if self._push_ranges is None:
                self._setup_push()
            self.peer.before_step()
            if not gather:
                self._set_push(False)
            for opt in self.opts:
                if opt is not None:
                    opt.step()
            if not gather:
                self._set_push(True)
                return
            # one all-reduce after every rank's step kernels: the stores into this rank's buffer are complete when it
            # is; the pieces no kernel delivers are pulled behind it
            self.peer.pull_ranges(self._push_ranges)
            self.peer.finish()
            return
        if self.peer is not None:
            self.peer.before_step()
        for b, opt in enumerate(self.opts):
            if opt is not None:
                opt.step()
            if gather and self.sharded.world_size > 1:
                if self.peer is not None:
                    self.peer.pull_bucket(b)
                else:
                    works.append(self.sharded.all_gather_bucket(b, group=self.group, async_op=True))
        for w in works:
            w.wait()
        if gather and self.peer is not None:
            self.peer.finish()

    # -- sharded checkpoint: every rank saves and restores the state of the tensors it owns -------------------
    def state_dict(self) -> dict:
        """This rank's shard: the `state_dict()` of each bucket's optimizer (None where the rank owns nothing in the
        bucket) together with the ownership map it belongs to.  The weights themselves are not part of it (after a
        step every rank holds all of them in `sharded.flat`)."""
        s = self.sharded
        return {"world_size": s.world_size, "rank": s.rank, "shapes": [list(x) for x in s.shapes],
                "owners": list(s.owners), "bucket_of": list(s.bucket_of),
                "buckets": [None if o is None else o.state_dict() for o in self.opts]}

    def load_state_dict(self, sd: dict) -> None:
        s = self.sharded
        same = (sd["world_size"] == s.world_size and sd["rank"] == s.rank and sd["owners"] == list(s.owners) and
                sd["bucket_of"] == list(s.bucket_of) and [tuple(x) for x in sd["shapes"]] == s.shapes)
        if not same:
            raise ValueError("this shard was saved under a different ownership partition (world size, rank, shapes or "
                             "bucket assignment differ); re-shard it before loading")
        for o, b in zip(self.opts, sd["buckets"]):
            if (o is None) != (b is None):
                raise ValueError("bucket layout of the shard does not match")
            if o is not None:
                o.load_state_dict(b)

    def gather_only(self):
        """The exchange alone (every bucket), for timing."""
        if self.sharded.world_size == 1:
            return
        if self.peer is not None:
            self.peer.before_step()
            for b in range(self.sharded.n_buckets):
                self.peer.pull_bucket(b)
            self.peer.finish()
        else:
            self.sharded.all_gather(group=self.group)

    @property
    def last_step_launches(self) -> int:
        return sum(o.last_step_launches for o in self.opts if o is not None)


class Zero1Step:
    """The whole data-parallel optimizer sequence of one step under the ownership partition, bucket by bucket:
    reduce-scatter of the gradients (each rank receives the summed gradients of the tensors it owns), step of the owned
    tensors, all-gather of the updated weights -- optionally captured into ONE CUDA graph, so that a training step
    replays it with a single launch.  The reference has no counterpart (it is single-GPU; its `prime_for_cuda_graph`,
    came_pytorch/CAME8bit2D.py:52-72, covers the bare step of one process).

    `grad_flat` / `grad_views` come from `ShardedParams.like_flat()`: every rank writes its local gradients of ALL
    parameters there; the parameters of the optimizers must have their `.grad` set to the views of the tensors the rank
    owns.  Gradients are summed; give the optimizers' param_groups `grad_scale = 1 / world_size` for the mean (the
    scale is applied as the kernels read the gradients).  The exchange is that of the stepper: the NCCL all-gather per
    bucket (collectives are captured as graph nodes), or, for a stepper in push mode, the stores of the step's own
    kernels followed by one small all-reduce."""

    def __init__(self, stepper: "ShardedStepper", grad_flat: torch.Tensor, group=None):
        self.stepper, self.sharded, self.grad_flat, self.group = stepper, stepper.sharded, grad_flat, group
        self.graph = None

    def _run_push(self) -> None:
        """Push mode of the stepper: reduce-scatter of every bucket, the step (whose kernels store the new weights into
        the peers' buffers), one all-reduce that orders every rank's stores, the pieces no kernel delivers pulled by
        copies, one all-reduce that says everybody has pulled -- all on the current stream, so the sequence can be
        captured as it is."""
        s, st = self.sharded, self.stepper
        if st._push_ranges is None:
            st._setup_push()
        for b in range(s.n_buckets):
            s.reduce_scatter_bucket(self.grad_flat, b, group=self.group)
        for opt in st.opts:
            if opt is not None:
                opt.step()
        dist.all_reduce(st.peer.flag, group=self.group)
        esz = s.flat.element_size()
        stream = torch.cuda.current_stream(s.flat.device).cuda_stream
        with torch.cuda.device(s.flat.device):
            for r, ranges in st._push_ranges.items():
                for lo, n in ranges:
                    _lib.check(st.peer._lib.came_b200_peer_copy_async(
                        s.flat.data_ptr() + lo * esz, st.peer.peer_ptr[r] + lo * esz, n * esz, -1, stream))
        dist.all_reduce(st.peer.flag, group=self.group)

    def run(self) -> None:
        s = self.sharded
        if self.stepper.gather_mode == "push":
            self._run_push()
            return
        for b, opt in enumerate(self.stepper.opts):
            s.reduce_scatter_bucket(self.grad_flat, b, group=self.group)
            if opt is not None:
                opt.step()
            if s.world_size > 1:
                s.all_gather_bucket(b, group=self.group)

    def capture(self, warmup: int = 0) -> None:
        """Captures `run()` on a side stream.  The optimizers' states must exist (`prime_for_cuda_graph()` or earlier
        steps) and the gradient / parameter buffers must stay where they are.  `warmup` eager runs come first (they DO
        step)."""
        for opt in self.stepper.opts:
            if opt is not None:
                opt.prime_for_cuda_graph()
        if self.stepper.gather_mode == "push" and self.stepper._push_ranges is None:
            self.stepper._setup_push()      # host-side collectives: not inside the capture
        side = torch.cuda.Stream(device=self.sharded.flat.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self.run()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.run()

    def replay(self) -> None:
        """One step: re-reads the hyper-parameters from the param_groups (learning-rate schedules need no re-capture)
        and replays the captured sequence."""
        if self.graph is None:
            raise RuntimeError("capture() first")
        # The captured upload reads the staged hyper-parameter records when the graph RUNS: they may only be rewritten
        # once the previous replay has run.  Unchanged hyper-parameters need no rewrite and no wait.
        import ctypes as C
        staged = [bytes(C.string_at(C.byref(h), C.sizeof(h))) for opt in self.stepper.opts if opt is not None
                  for h in opt._hypers()]
        if staged != getattr(self, "_staged", None):
            torch.cuda.current_stream().synchronize()
            for opt in self.stepper.opts:
                if opt is not None:
                    opt.update_captured_hypers()
            self._staged = staged
        self.graph.replay()
