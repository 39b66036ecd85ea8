"""CPU, two gloo ranks: the host-side expert-parallel logic (group handling, count exchange, offsets).

Rows are moved with plain tensor indexing instead of peer stores; what is checked is that the
offset descriptors every rank derives from the gathered count table describe one consistent
lossless exchange, and that the module's group validation behaves like the reference's.
"""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import route as oroute


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, failures) -> None:
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from hyper_multicore_b200 import MegaMoeExperts

        with pytest.raises(ValueError, match="Pass ep_group explicitly"):
            MegaMoeExperts(hidden_size=64, intermediate_size=64, num_experts=8, top_k=2)
        with pytest.raises(ValueError, match="must be divisible by ep_size"):
            MegaMoeExperts(hidden_size=64, intermediate_size=64, num_experts=7, top_k=2, ep_group=dist.group.WORLD)
        module = MegaMoeExperts(hidden_size=64, intermediate_size=64, num_experts=8, top_k=2,
                                ep_group=dist.group.WORLD)
        assert module.ep_size == world and module.local_experts == 8 // world
        assert len(module.state_dict()) == 0

        experts, top_k, hidden = 8, 2, 4
        local = experts // world
        rng = np.random.default_rng(100 + rank)
        tokens = 13 + 7 * rank
        ids = np.stack([rng.choice(experts, size=top_k, replace=False) for _ in range(tokens)])
        x = torch.arange(tokens * hidden, dtype=torch.float32).reshape(tokens, hidden) + 1000 * rank
        counts = torch.from_numpy(oroute.counts(ids, experts))
        gathered = [torch.empty_like(counts) for _ in range(world)]
        dist.all_gather(gathered, counts)
        table = torch.stack(gathered).numpy()
        meta = oroute.route_metadata(table, world, rank)
        mapping, source, row_experts = oroute.permutation(ids, experts)
        routed = x[torch.from_numpy(source).long() // top_k]  # expert-major rows on the source
        # every rank publishes its routed rows and its descriptors; each owner assembles its buffer
        objects = [None] * world
        dist.all_gather_object(objects, (routed, meta, row_experts))
        capacity, _ = oroute.expert_capacity(table, world, rank)
        buffer = torch.full((capacity, hidden), -1.0)
        filled = torch.zeros(capacity, dtype=torch.int32)
        for src, (src_rows, src_meta, src_experts) in enumerate(objects):
            for j, e in enumerate(src_experts.tolist()):
                if e // local != rank:
                    continue
                dest = int(src_meta["dispatch_target_off"][e]) + (j - int(src_meta["dispatch_src_off"][e]))
                buffer[dest] = src_rows[j]
                filled[dest] += 1
        received = int(table[:, rank * local:(rank + 1) * local].sum())
        assert filled[:received].eq(1).all() and filled[received:].eq(0).all(), "dispatch is not a bijection"
        ends = meta["group_list"].tolist()
        assert ends[-1] == received
        # pull dispatch: the owner fetches segment (local expert, source) from the source's published rows at the
        # offsets the push combine uses as targets; the result must be the buffer the push dispatch built
        pulled = torch.full((capacity, hidden), -1.0)
        for le in range(local):
            for src, (src_rows, _, _) in enumerate(objects):
                start = int(meta["combine_src_off"][src * local + le])
                size = int(meta["combine_size"][src * local + le])
                first = int(meta["combine_target_off"][src * local + le])
                pulled[start:start + size] = src_rows[first:first + size]
        assert torch.equal(pulled, buffer), "pull and push dispatch disagree on the receive layout"
        # combine back: (source, local expert) segments return to the source's expert-major rows
        returned = [None] * world
        back = []
        for src in range(world):
            rows = []
            for le in range(local):
                start = int(meta["combine_src_off"][src * local + le])
                size = int(meta["combine_size"][src * local + le])
                rows.append((int(meta["combine_target_off"][src * local + le]), buffer[start:start + size]))
            back.append(rows)
        dist.all_gather_object(returned, back)
        restored = torch.full_like(routed, -2.0)
        for owner_rows in returned:
            for target, rows in owner_rows[rank]:
                restored[target:target + rows.shape[0]] = rows
        assert torch.equal(restored, routed), "combine does not return every row to its source slot"
        # failure convergence: the validity header travels with the counts, every rank validates the same
        # gathered rows and so every rank raises together (nobody goes on into a wait the other never joins)
        from hyper_multicore_b200.modules.mega_moe.route import check_gathered_rows

        def gather_rows(invalid: bool, autograd: bool, dropped: int = 0):
            counts_row = oroute.counts(ids, experts).tolist()
            if dropped:  # routes the sort dropped as out of range
                counts_row[next(i for i, c in enumerate(counts_row) if c >= dropped)] -= dropped
            payload = torch.tensor([int(invalid), tokens, int(autograd)] + counts_row, dtype=torch.int32)
            rows = [torch.empty_like(payload) for _ in range(world)]
            dist.all_gather(rows, payload)
            return [row.tolist() for row in rows]

        assert check_gathered_rows(gather_rows(False, True), top_k, experts) == table.tolist()
        with pytest.raises(ValueError, match=r"invalid inputs on EP rank\(s\) \[1\]; all ranks reject"):
            check_gathered_rows(gather_rows(rank == 1, True), top_k, experts)
        with pytest.raises(RuntimeError, match="autograd participation differs"):
            check_gathered_rows(gather_rows(False, rank == 0), top_k, experts)
        with pytest.raises(ValueError, match=r"outside that range on EP rank\(s\) \[0\]; all ranks reject"):
            check_gathered_rows(gather_rows(False, True, dropped=1 if rank == 0 else 0), top_k, experts)
        dist.barrier()
        dist.destroy_process_group()
    except BaseException as error:  # pylint: disable=broad-except
        failures.put(f"rank {rank}: {type(error).__name__}: {error}")
        raise


def test_two_rank_route_exchange_is_lossless():
    world = 2
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(rank, world, port, failures)) for rank in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    messages = []
    while not failures.empty():
        messages.append(failures.get())
    for p in procs:
        if p.is_alive():
            p.kill()
            messages.append("a rank did not finish")
    assert not messages and all(p.exitcode == 0 for p in procs), messages


def test_share_execution_resources_validation():
    """Host rules of workspace sharing (reference: hyper_multicore/modules/module.py:262-323)."""
    from hyper_multicore_b200 import MegaMoeExperts, MegaMoeNumericsOptions

    def layer(**extra):
        return MegaMoeExperts(hidden_size=64, intermediate_size=64, num_experts=4, top_k=2, **extra)

    a, b, c = layer(), layer(numerics_options=MegaMoeNumericsOptions()), layer()
    MegaMoeExperts.share_execution_resources([a, b, c])  # omitted and explicit default options are compatible
    assert a._group is b._group is c._group and len(a._group.members) == 3 and a._group.shared
    MegaMoeExperts.share_execution_resources([a, b])  # already grouped: nothing to do
    with pytest.raises(ValueError, match="at least one module"):
        MegaMoeExperts.share_execution_resources([])
    with pytest.raises(ValueError, match="duplicate"):
        MegaMoeExperts.share_execution_resources([a, a])
    with pytest.raises(TypeError, match="must be MegaMoeExperts instances"):
        MegaMoeExperts.share_execution_resources([a, object()])
    other = layer(numerics_options=MegaMoeNumericsOptions(swiglu_limit=7.0))
    with pytest.raises(ValueError, match="identical configuration"):
        MegaMoeExperts.share_execution_resources([layer(), other])
    with pytest.raises(RuntimeError, match="before first use or previous grouping"):
        MegaMoeExperts.share_execution_resources([layer(), a])
    # the workspace goes with the last member
    a._group.workspace = sentinel = type("W", (), {"closed": False, "close": lambda self: setattr(self, "closed", True)})()
    a.close()
    b.close()
    assert not sentinel.closed and not c._group.closed
    c.close()
    c.close()  # idempotent
    assert sentinel.closed and c._group.closed and c._group.workspace is None
    with pytest.raises(RuntimeError, match="closed multicore modules cannot share"):
        MegaMoeExperts.share_execution_resources([layer(), a])
