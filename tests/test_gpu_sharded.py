"""GPU checks of the row-sharded path on one device: the rectangular (row-slab) forms of the stage
kernels against their square forms, and the whole sharded choreography with a one-rank NCCL group
against the plain module."""
import os
import socket

import pytest
import torch

import protenix_b200 as px
from golden_cases import padding_mask, random_mask
from helpers import build_module, params_of, relf
from oracle import pairformer_oracle as O
from protenix_b200 import ops
from protenix_b200.sharded import CudaStages

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("n,parts", [(48, 2), (96, 4), (120, 3)])
def test_row_slab_stages_equal_square_stages(n, parts):
    g = torch.Generator().manual_seed(n)
    z = torch.randn(n, n, 128, generator=g).to(torch.bfloat16).to(DEV)
    mask = random_mask(n, 2).to(DEV)
    blk = build_module("block", dict(c_s=0, wseed=3)).to(DEV)
    st = CudaStages()
    nl = n // parts
    a_f, b_f = st.trimul_in_proj(blk.tri_mul_out, z, mask, False)
    ai_f, bi_f = st.trimul_in_proj(blk.tri_mul_in, z, mask, True)
    q_f, k_f, v_f, bias_f, mb_f = st.triatt_in_proj(blk.tri_att_start, z, mask)
    o_f = st.triatt_flash(q_f, k_f, v_f, bias_f, mb_f)
    x_f = st.trimul_contract(a_f, b_f)
    z_mul = st.trimul_out(blk.tri_mul_out, x_f, z.clone())
    z_att = st.triatt_out(blk.tri_att_start, o_f, z.clone())
    for r in range(parts):
        rows = slice(r * nl, (r + 1) * nl)
        zs, ms = z[rows].contiguous(), mask[rows].contiguous()
        a, b = st.trimul_in_proj(blk.tri_mul_out, zs, ms, False)
        assert torch.equal(a, a_f[:, rows]) and torch.equal(b, b_f[:, rows])
        ai, bi = st.trimul_in_proj(blk.tri_mul_in, zs, ms, True)          # local rows are the k index
        assert torch.equal(ai[:, :, :nl], ai_f[:, :, rows]) and torch.equal(bi[:, :, :nl], bi_f[:, :, rows])
        assert float(ai[:, :, nl:].abs().sum()) == 0.0
        q, k, v, bias, mb = st.triatt_in_proj(blk.tri_att_start, zs, ms)
        assert torch.equal(q, q_f[rows]) and torch.equal(k, k_f[rows]) and torch.equal(v, v_f[rows])
        assert torch.equal(bias, bias_f[:, rows]) and torch.equal(mb, mb_f[rows])
        assert torch.equal(st.triatt_flash(q, k, v, bias_f, mb), o_f[rows])
        assert torch.equal(st.trimul_out(blk.tri_mul_out, x_f[:, rows].contiguous(), zs.clone()), z_mul[rows])
        assert torch.equal(st.triatt_out(blk.tri_att_start, o_f[rows].contiguous(), zs.clone()), z_att[rows])
    # the contraction on a subset of channels
    assert torch.equal(st.trimul_contract(a_f[32:48].contiguous(), b_f[32:48].contiguous()), x_f[32:48])


def test_pitched_copy_and_peer_buffer_on_one_device():
    """px_copy_2d against torch slicing, into a PeerBuffer viewed as a tensor (the multi-GPU exchanges are such copies)."""
    g = torch.Generator().manual_seed(1)
    src = torch.randn(6, 40, 24, generator=g).to(torch.bfloat16).to(DEV)          # [c][rows][ld]
    buf = ops.PeerBuffer(3 * 80 * 24 * 2, torch.device(DEV, torch.cuda.current_device()))
    dst = buf.tensor((3, 80, 24), torch.bfloat16)
    dst.zero_()
    # channels 3..5 of src become rows 40..79 of every channel of dst: one run of 40*24 elements per channel
    ops.copy_2d(buf.ptr + 40 * 24 * 2, 80 * 24 * 2, src, 3 * 40 * 24 * 2, 40 * 24 * 2, 40 * 24 * 2, 3)
    torch.cuda.synchronize()
    assert torch.equal(dst[:, 40:], src[3:]) and float(dst[:, :40].float().abs().sum()) == 0.0
    # a narrow run per row (the k-sharded exchange): columns 8..15 of every row
    ops.copy_2d(buf.ptr + 8 * 2, 24 * 2, src, 0, 24 * 2, 8 * 2, 3 * 40)
    torch.cuda.synchronize()
    assert torch.equal(dst.view(-1, 24)[:120, 8:16], src.view(-1, 24)[:120, :8])
    with pytest.raises(RuntimeError):
        ops.copy_2d(buf.ptr + 2, 48, src, 0, 48, 16, 1)                              # misaligned destination
    # the batched form: channel pair d of src -> rows 40.. of channels 0..1 of destination d (three destinations)
    bufs = [ops.PeerBuffer(2 * 80 * 24 * 2, buf.device) for _ in range(3)]
    views = [b.tensor((2, 80, 24), torch.bfloat16) for b in bufs]
    for v in views:
        v.zero_()
    ops.copy_2d_batch([b.ptr + 40 * 24 * 2 for b in bufs], src, [d * 2 * 40 * 24 * 2 for d in range(3)], 80 * 24 * 2,
                      40 * 24 * 2, 40 * 24 * 2, 2)
    torch.cuda.synchronize()
    for d, v in enumerate(views):
        assert torch.equal(v[:, 40:], src[2 * d:2 * d + 2]) and float(v[:, :40].float().abs().sum()) == 0.0
    for b in bufs:
        b.free()
    buf.free()


def test_column_slab_attention_equals_transposed_row_slab():
    """The ending node on a column slab [N i][nl j][c] (kernels' own addressing) against the starting-node kernels on
    the explicitly transposed slab."""
    n, parts = 96, 3
    nl = n // parts
    g = torch.Generator().manual_seed(7)
    z = torch.randn(n, n, 128, generator=g).to(torch.bfloat16).to(DEV)
    mask = random_mask(n, 4).to(DEV)
    blk = build_module("block", dict(c_s=0, wseed=5)).to(DEV)
    st = CudaStages()
    for r in range(parts):
        cols = slice(r * nl, (r + 1) * nl)
        zc, mc = z[:, cols].contiguous(), mask[:, cols].contiguous()              # [N i][nl j]
        zt, mt = z[:, cols].transpose(0, 1).contiguous(), mask[:, cols].t().contiguous()   # [nl j][N i]
        q, k, v, bias, mb = st.triatt_in_proj(blk.tri_att_end, zc, mc, True)
        q2, k2, v2, bias2, mb2 = st.triatt_in_proj(blk.tri_att_end, zt, mt)
        assert torch.equal(q, q2) and torch.equal(k, k2) and torch.equal(v, v2)
        assert torch.equal(bias, bias2) and torch.equal(mb, mb2)
        o = torch.randn(nl, n, 128, generator=g).to(torch.float16).to(DEV)
        out_c = st.triatt_out(blk.tri_att_end, o, zc.clone(), True)
        out_t = st.triatt_out(blk.tri_att_end, o, zt.clone())
        assert torch.equal(out_c.transpose(0, 1), out_t)


def test_sharded_path_with_one_rank_equals_module():
    import torch.distributed as dist

    from protenix_b200.sharded import ShardedPairformer

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    try:
        n = 72
        g = torch.Generator().manual_seed(4)
        z = torch.randn(n, n, 128, generator=g).to(DEV)
        s = torch.randn(n, 384, generator=g).to(DEV)
        mask = random_mask(n, 9).to(DEV)
        stack = build_module("stack", dict(n_blocks=2, c_s=384, wseed=5)).to(DEV)
        s_ref, z_ref = stack(s, z, mask)
        sp = ShardedPairformer(stack)
        s_out, z_out = sp.forward(s, sp.shard_rows(z), mask)
        assert relf(z_out, z_ref) < 1e-6 and relf(s_out, s_ref) < 1e-5
        s0, z0 = O.pairformer_stack(s.cpu(), z.cpu(), mask.cpu(), params_of(stack), n_blocks=2)
        assert relf(z_out, z0) < 2e-2 and relf(s_out, s0) < 2e-2
        # the recycling loop over the same group: row-local updates around the sharded stack
        from protenix_b200.sharded import ShardedRecyclingTrunk

        trunk = build_module("recycle", dict(n_blocks=1, c_s=384, n_cycle=2, wseed=8)).to(DEV)
        s_ref, z_ref = trunk(s, z, mask)
        st = ShardedRecyclingTrunk(trunk)
        z_init_loc = st.shard_rows(z)
        s_out, z_out = st.forward(s, z_init_loc, mask)
        assert torch.equal(z_init_loc, z)
        assert relf(z_out, z_ref) < 1e-6 and relf(s_out, s_ref) < 1e-5
    finally:
        dist.destroy_process_group()


def _nccl_worker(rank, world, port, n, q, n_blocks=2, pad=None, zdtype="bf16"):
    import sys

    here = os.path.dirname(os.path.abspath(__file__))
    for p in (os.path.dirname(here), here, os.path.join(here, "golden")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist

    from protenix_b200.sharded import ShardedPairformer

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        g = torch.Generator().manual_seed(4)
        z = torch.randn(n, n, 128, generator=g).to(torch.bfloat16 if zdtype == "bf16" else torch.float32).to(dev)
        s = torch.randn(n, 384, generator=g).to(dev)
        mask = (random_mask(n, 9) if pad is None else padding_mask(n, pad)).to(dev)
        stack = build_module("stack", dict(n_blocks=n_blocks, c_s=384, wseed=5)).to(dev)
        sp = ShardedPairformer(stack)
        try:
            s_out, z_loc = sp.forward(s, sp.shard_rows(z), mask)
            z_out = sp.gather_rows(z_loc)
            flags = ops.device_error_flags(dev, raise_on_error=False)
            if rank == 0:
                s_ref, z_ref = stack(s, z, mask)            # the single-GPU path on the same device
                finite = bool(torch.isfinite(z_out.float()).all() and torch.isfinite(s_out).all())
                q.put((relf(z_out, z_ref), relf(s_out, s_ref), bool(torch.equal(z_out, z_ref)), flags, finite))
        finally:
            sp.close()
    finally:
        dist.destroy_process_group()


def _run_ranks(world, n, **kw):
    """Spawns one process per GPU, returns rank 0's result; ranks still alive after the limit are killed, so a hung
    exchange cannot keep GPUs and IPC mappings after the test has failed."""
    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_nccl_worker, args=(r, world, port, n, q), kwargs=kw) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.kill()
        p.join(timeout=10)
    assert not hung, f"{len(hung)} rank(s) did not finish"
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    return q.get(timeout=10)


@pytest.mark.parametrize("world,n,zdtype", [(2, 136, "bf16"), (2, 144, "bf16"), (2, 144, "fp32"), (2, 136, "fp32"),
                                            (4, 192, "bf16"), (4, 192, "fp32"), (8, 256, "bf16"), (8, 256, "fp32")])
def test_sharded_over_nccl_equals_single_gpu(world, n, zdtype):
    """Gathered output of the row-sharded stack on `world` GPUs against the one-GPU stack, for both storage types of z.
    N/P = 68 goes through the all_to_all transport (the peer copies need N/P to be a multiple of 8), the other cases
    through the peer copies."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ez, es, same, flags, finite = _run_ranks(world, n, zdtype=zdtype)
    # same kernels, same per-element arithmetic: only the reduction-free re-layouts differ
    assert flags == 0 and finite
    assert ez < 1e-3 and es < 1e-3, (ez, es, same)


@pytest.mark.parametrize("world,zdtype", [(2, "fp32"), (2, "bf16"), (4, "fp32"), (8, "fp32")])
def test_sharded_block_n1536_equals_single_gpu(world, zdtype):
    """One block at N=1536 (37 trailing tokens masked) row-sharded over `world` GPUs against the same block on one GPU:
    the size the multi-GPU benchmark runs."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ez, es, same, flags, finite = _run_ranks(world, 1536, n_blocks=1, pad=37, zdtype=zdtype)
    assert flags == 0 and finite
    assert ez < 1e-3 and es < 1e-3, (ez, es, same)
