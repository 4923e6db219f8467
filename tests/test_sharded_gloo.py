"""The row-sharded Pairformer choreography on CPU ranks (gloo, world size 2 and 4).

The collectives, index bookkeeping and layouts of ``protenix_b200.sharded`` run for real; the
per-rank kernels are replaced by a plain-torch stage implementation with identical layouts
(``tests/ref_stages.py``).  The gathered result must equal the oracle's single-process block.
"""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, c_s, n_blocks, masked, q):
    for p in (os.path.dirname(HERE), HERE, os.path.join(HERE, "golden")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import protenix_b200 as px
        from golden_cases import random_mask
        from helpers import params_of, relf
        from oracle import pairformer_oracle as O
        from protenix_b200.init_utils import randomize_parameters_
        from protenix_b200.sharded import ShardedPairformer
        from ref_stages import TorchStages

        g = torch.Generator().manual_seed(7)
        z = torch.randn(n, n, 128, generator=g)
        s = torch.randn(n, c_s, generator=g) if c_s else None
        mask = random_mask(n, 3) if masked else None
        stack = randomize_parameters_(px.PairformerStack(n_blocks=n_blocks, c_s=c_s), 5).eval()
        sp = ShardedPairformer(stack, stages=TorchStages())
        z_loc = sp.shard_rows(z)
        s_out, z_loc = sp.forward(s, z_loc, mask)
        z_full = sp.gather_rows(z_loc)
        if rank == 0:
            s_ref, z_ref = O.pairformer_stack(s, z, mask, params_of(stack), n_blocks=n_blocks)
            q.put((relf(z_full, z_ref), relf(s_out, s_ref) if c_s else 0.0))
        # every rank must hold the same replicated s
        if c_s:
            ss = [torch.empty_like(s_out) for _ in range(world)]
            dist.all_gather(ss, s_out)
            assert all(torch.equal(ss[0], t) for t in ss)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n,c_s,n_blocks,masked", [(2, 16, 384, 1, True), (4, 16, 0, 2, False),
                                                        (2, 12, 384, 2, True), (4, 24, 384, 1, True)])
def test_sharded_block_equals_oracle(world, n, c_s, n_blocks, masked):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, c_s, n_blocks, masked, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    ez, es = q.get(timeout=10)
    assert ez < 2e-5 and es < 2e-5, (ez, es)


def test_sharding_rejects_indivisible_sizes():
    class _G:
        pass

    import protenix_b200 as px
    from protenix_b200.sharded import ShardedPairformer

    port = _free_port()
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        sp = ShardedPairformer(px.PairformerBlock(c_s=0), stages=object())
        sp.world = 3
        with pytest.raises(RuntimeError, match="divisible"):
            sp.shard_rows(torch.zeros(10, 10, 128))
    finally:
        dist.destroy_process_group()


def _recycle_worker(rank, world, port, n, n_cycle, q):
    for p in (os.path.dirname(HERE), HERE, os.path.join(HERE, "golden")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import protenix_b200 as px
        from golden_cases import padding_mask
        from helpers import params_of, relf
        from oracle import pairformer_oracle as O
        from protenix_b200.init_utils import randomize_parameters_
        from protenix_b200.sharded import ShardedRecyclingTrunk
        from ref_stages import TorchStages

        g = torch.Generator().manual_seed(9)
        z_init = torch.randn(n, n, 128, generator=g)
        s_init = torch.randn(n, 384, generator=g)
        mask = padding_mask(n, 2)
        trunk = randomize_parameters_(px.RecyclingTrunk(n_blocks=1, N_cycle=n_cycle), 6).eval()
        sp = ShardedRecyclingTrunk(trunk, stages=TorchStages())
        z_init_loc = sp.shard_rows(z_init)
        keep = z_init_loc.clone()
        s_out, z_loc = sp.forward(s_init, z_init_loc, mask)
        assert torch.equal(z_init_loc, keep)                      # the initial pair representation is only read
        z_full = sp.gather_rows(z_loc)
        if rank == 0:
            s_ref, z_ref = O.recycling_trunk(s_init, z_init, mask, params_of(trunk), n_blocks=1, n_cycle=n_cycle)
            q.put((relf(z_full, z_ref), relf(s_out, s_ref)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n,n_cycle", [(2, 12, 2), (4, 16, 3)])
def test_sharded_recycling_loop_equals_oracle(world, n, n_cycle):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_recycle_worker, args=(r, world, port, n, n_cycle, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    ez, es = q.get(timeout=10)
    assert ez < 2e-5 and es < 2e-5, (ez, es)
