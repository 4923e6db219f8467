"""The pitched copies of the peer transport, replayed on CPU: every rank's ``put_all`` calls are executed byte by byte
into plain host buffers and the assembled buffers are compared with what the all_to_all path would deliver.  Every
exchange that the sharded path pipelines is replayed in the row (or channel) chunks it uses there."""
import pytest
import torch

from protenix_b200.sharded import ShardedPairformer


class FakeExchange:
    """Stands in for PeerExchange: one uint8 host buffer per (key, rank); put_all copies rows with the given pitches."""

    def __init__(self, world, sizes):
        self.world = world
        self.bufs = {k: [torch.zeros(v, dtype=torch.uint8) for _ in range(world)] for k, v in sizes.items()}
        self.rank = 0

    def order(self):
        return [(self.rank + 1 + i) % self.world for i in range(self.world)]

    def put_all(self, key, dst_offset, dpitch, src, src_offset_of, spitch, width, height):
        raw = src.contiguous().view(torch.uint8).reshape(-1)
        for d in self.order():
            so = src_offset_of(d)
            for v in (dst_offset, dpitch, so, spitch, width):
                assert v % 16 == 0, "the copy kernel moves 16-byte pieces"
            dst = self.bufs[key][d]
            for r in range(height):
                dst[dst_offset + r * dpitch: dst_offset + r * dpitch + width] = raw[so + r * spitch: so + r * spitch + width]


def _rank(world, rank):
    sp = object.__new__(ShardedPairformer)
    sp.world, sp.rank = world, rank
    return sp


def _ld(n):
    return (n + 7) // 8 * 8


@pytest.mark.parametrize("world,n", [(2, 32), (4, 32), (8, 64), (2, 48)])
def test_peer_copies_assemble_the_same_tensors_as_all_to_all(world, n):
    g = torch.Generator().manual_seed(world * 100 + n)
    nl, cp, ldn = n // world, 128 // world, _ld(n)
    ldm = (n + 127) // 128 * 128
    sizes = {"a": cp * n * ldn * 2, "b": cp * n * ldn * 2, "x": 128 * nl * ldn * 2, "zc": n * nl * 128 * 2,
             "zr": nl * n * 128 * 2, "bias": 4 * n * ldm * 4}
    fx = FakeExchange(world, sizes)
    bf = torch.bfloat16
    # (1) rows -> channels, rows sharded: full_a [128][N][ld]
    full = torch.randn(128, n, ldn, generator=g).to(bf)
    chunks = _rank(world, 0)._row_chunks(nl)
    assert sum(b - a for a, b in chunks) == nl and all(a % 8 == 0 for a, _ in chunks)
    for r in range(world):
        fx.rank = r
        for r0, r1 in chunks:
            _rank(world, r)._peer_rows_to_channels(fx, full[:, r * nl + r0:r * nl + r1].contiguous(), "a", False, nl, r0)
    for d in range(world):
        assert torch.equal(fx.bufs["a"][d].view(bf).view(cp, n, ldn), full[d * cp:(d + 1) * cp])
    # (2) rows -> channels, contraction index sharded: local [128][N][ld(nl)], valid columns nl
    full_k = torch.randn(128, n, n, generator=g).to(bf)
    for r in range(world):
        fx.rank = r
        for r0, r1 in chunks:
            loc = full_k[:, :, r * nl + r0:r * nl + r1].contiguous()        # [128][N][rc], rc a multiple of 8
            _rank(world, r)._peer_rows_to_channels(fx, loc, "b", True, nl, r0)
    for d in range(world):
        got = fx.bufs["b"][d].view(bf).view(cp, n, ldn)
        assert torch.equal(got[:, :, :n], full_k[d * cp:(d + 1) * cp]) and float(got[:, :, n:].float().abs().sum()) == 0.0
    # (1b), (2b) the same two exchanges sent as two channel groups per destination
    if cp >= 2:
        for k in ("a", "b"):
            for d in range(world):
                fx.bufs[k][d].zero_()
        for r in range(world):
            fx.rank = r
            for cs in ((0, cp // 2), (cp // 2, cp)):
                _rank(world, r)._peer_rows_to_channels(fx, full[:, r * nl:(r + 1) * nl].contiguous(), "a", False, nl, 0, cs)
                _rank(world, r)._peer_rows_to_channels(fx, full_k[:, :, r * nl:(r + 1) * nl].contiguous(), "b", True, nl, 0, cs)
        for d in range(world):
            assert torch.equal(fx.bufs["a"][d].view(bf).view(cp, n, ldn), full[d * cp:(d + 1) * cp])
            got = fx.bufs["b"][d].view(bf).view(cp, n, ldn)
            assert torch.equal(got[:, :, :n], full_k[d * cp:(d + 1) * cp]) and float(got[:, :, n:].float().abs().sum()) == 0.0
    # (3) channels -> rows: x [128][N][ld], rank r holds channels r*cp..
    xf = torch.randn(128, n, ldn, generator=g).to(bf)
    for r in range(world):
        fx.rank = r
        for c0, c1 in ((0, cp // 2), (cp // 2, cp)):
            _rank(world, r)._peer_channels_to_rows(fx, xf[r * cp + c0:r * cp + c1].contiguous(), c0)
    for d in range(world):
        assert torch.equal(fx.bufs["x"][d].view(bf).view(128, nl, ldn), xf[:, d * nl:(d + 1) * nl])
    # (4) row slab -> column slab and back
    z = torch.randn(n, n, 128, generator=g).to(bf)
    for r in range(world):
        fx.rank = r
        for r0, r1 in chunks:
            _rank(world, r)._peer_to_columns(fx, z[r * nl + r0:r * nl + r1].contiguous(), nl, r0)
    for d in range(world):
        assert torch.equal(fx.bufs["zc"][d].view(bf).view(n, nl, 128), z[:, d * nl:(d + 1) * nl])
    for r in range(world):
        fx.rank = r
        _rank(world, r)._peer_from_columns(fx, fx.bufs["zc"][r].view(bf).view(n, nl, 128))
    for d in range(world):
        assert torch.equal(fx.bufs["zr"][d].view(bf).view(nl, n, 128), z[d * nl:(d + 1) * nl])
    # (5) pair bias: [4][nl][ldm] of every rank -> [4][N][ldm] everywhere
    bias = torch.randn(4, n, ldm, generator=g)
    for r in range(world):
        fx.rank = r
        _rank(world, r)._peer_gather_bias(fx, bias[:, r * nl:(r + 1) * nl].contiguous())
    for d in range(world):
        assert torch.equal(fx.bufs["bias"][d].view(torch.float32).view(4, n, ldm), bias)
