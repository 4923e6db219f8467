"""Row-sharded Pairformer over the GPUs of one NVSwitch box (one process per GPU).

Rank r of P holds rows [r*N/P, (r+1)*N/P) of the pair tensor: ``z_loc`` is [N/P, N, 128].  The
single representation s and the pair mask are replicated.  Per block:

* LayerNorms, projections, gates, the transition and the residual adds are row-local.
* Triangle multiplication: the contraction is independent per channel, so after the local input
  projection a and b go from row shards to channel shards with one ``all_to_all`` each
  (each rank then contracts 128/P channels over the full N x N), and x returns with a third.
  For the incoming direction the local rows are the contraction index: the local projection
  yields a[c][i][k in local rows] and the same ``all_to_all`` assembles the k axis.
* Starting-node attention: only the pair bias [4, N, N] couples the rows: it is gathered.
* Ending-node attention: z is exchanged to column shards with an ``all_to_all`` (a distributed
  transpose), the starting-node path runs on the transposed slab, and a second ``all_to_all``
  brings the update back.
* Single branch: every rank computes the attention output of its own query rows (it holds
  their pair bias); one small ``all_gather`` assembles the [N, c_s] result.

Two transports move the slabs.  On CUDA ranks of one box (default) every exchange is a set of
pitched 2-D copies from the local tensor straight into its final place in a peer's receive buffer
(``ops.PeerBuffer``: cudaMalloc + CUDA IPC; ``px_copy_2d``: a hand-written kernel, plain 16-byte
stores over NVLink), followed by one stream-ordered 4-byte ``all_reduce`` as the fence; no
re-layout pass runs on either side, and the ending node uses the kernels' own column addressing
instead of a transposed copy.  Otherwise (CPU ranks, ``PX_PEER_EXCHANGE=0``, shapes the copies do
not cover) the same exchanges go through ``all_to_all`` plus permutes.  Compute kernels only ever
read this GPU's memory.  The choreography is written against a small stage interface so that it
can be exercised on CPU ranks (gloo) with a plain-torch stage implementation.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import ops


# ----------------------------------------------------------------------------------------------
class CudaStages:
    """Stage interface backed by the C-ABI kernels."""

    @staticmethod
    def _f(p):
        return p.detach().float()

    def standardised(self, z, eps):
        """The standardised fp16 copy of an fp32 slab (the rows the tensor core multiplies), made once per
        sub-module and handed to its projection and its output stage; None for bf16 slabs, which are used as stored."""
        return ops.standardise_rows(z, eps) if z.dtype == torch.float32 else None

    def trimul_in_proj(self, mod, z, mask, incoming, zn=None):
        f = self._f
        return ops.trimul_in_proj(z, mask, f(mod.layer_norm_in.weight), f(mod.layer_norm_in.bias),
                                  mod.linear_a_p.weight, mod.linear_a_g.weight,
                                  mod.linear_b_p.weight, mod.linear_b_g.weight, incoming,
                                  mod.layer_norm_in.eps, zn=zn)

    def trimul_contract(self, a, b):
        return ops.trimul_contract(a, b)

    def trimul_out(self, mod, x, z, zn=None):
        f = self._f
        return ops.trimul_out(x, z, f(mod.layer_norm_in.weight), f(mod.layer_norm_in.bias),
                              f(mod.layer_norm_out.weight), f(mod.layer_norm_out.bias), mod.linear_z.weight,
                              mod.linear_g.weight, mod.layer_norm_in.eps, zn=zn)

    def triatt_in_proj(self, mod, z, mask, ending=False, zn=None):
        f, m = self._f, mod.mha
        return ops.triatt_in_proj(z, mask, f(mod.layer_norm.weight), f(mod.layer_norm.bias), mod.linear.weight,
                                  m.linear_q.weight, m.linear_k.weight, m.linear_v.weight,
                                  mod.layer_norm.eps, mod.inf, ending, zn=zn)

    def triatt_flash(self, q, k, v, bias_full, mb):
        return ops.triatt_flash(q, k, v, bias_full, mb)

    def triatt_out(self, mod, o, z, ending=False, zn=None):
        f, m = self._f, mod.mha
        return ops.triatt_out(o, z, f(mod.layer_norm.weight), f(mod.layer_norm.bias), m.linear_g.weight,
                              m.linear_o.weight, mod.layer_norm.eps, ending, zn=zn)

    def add_update(self, z, upd):
        return ops.add_update_rows(z, upd)

    def transition(self, mod, z, out=None):
        f = self._f
        return ops.transition_rows(z, f(mod.layernorm1.weight), f(mod.layernorm1.bias),
                                   mod.linear_no_bias_a.weight, mod.linear_no_bias_b.weight,
                                   mod.linear_no_bias.weight, mod.layernorm1.eps, out=out)

    def pair_bias(self, mod, z, zn=None):
        b = mod.layernorm_z.bias
        return ops.pair_bias_rows(z, self._f(mod.layernorm_z.weight), None if b is None else self._f(b),
                                  mod.linear_nobias_z.weight, mod.layernorm_z.eps, zn=zn)

    def single_layer_norm(self, ln, x):
        return ln(x)

    def recycle_update(self, ln, lin, z, z_init, out):
        b = ln.bias
        return ops.recycle_update(z, z_init, self._f(ln.weight), None if b is None else self._f(b), lin.weight,
                                  ln.eps, out=out)


# ----------------------------------------------------------------------------------------------
class PeerExchange:
    """Receive buffers of this rank (a, b, x, column slab, returning rows) and the addresses of the
    same buffers on every other rank.  ``put`` writes a pitched 2-D block into a rank's buffer;
    ``fence`` orders all ranks' writes before anybody's reads."""

    def __init__(self, group, world: int, rank: int, device: torch.device, n: int, z_itemsize: int) -> None:
        self.group, self.world, self.rank, self.device = group, world, rank, device
        nl, cp, ldn = n // world, 128 // world, (n + 7) // 8 * 8
        ldm = (n + 127) // 128 * 128
        sizes = {"a": cp * n * ldn * 2, "b": cp * n * ldn * 2, "x": 128 * nl * ldn * 2,
                 "zc": n * nl * 128 * 2, "zr": nl * n * 128 * 2, "bias": 4 * n * ldm * 4,
                 "flags": 256}
        self.local: Dict[str, ops.PeerBuffer] = {k: ops.PeerBuffer(v, device) for k, v in sizes.items()}
        for k in ("a", "b", "flags"):   # pad columns [n, ld) are never written by an exchange and must read as zero
            self.local[k].tensor((sizes[k],), torch.uint8).zero_()
        self.epoch = 0                  # number of the last barrier; the same sequence on every rank
        # copies and barriers run on a stream of their own, beside the compute stream; PX_PEER_STREAM=main keeps them
        # on the compute stream (no cross-stream events, no overlap of the x return with the contraction)
        self.comm = None if os.environ.get("PX_PEER_STREAM", "comm") == "main" else torch.cuda.Stream(device=device)
        self.use_flags = os.environ.get("PX_PEER_FENCE", "flags") != "nccl"
        torch.cuda.synchronize(device)
        handles = [None] * world
        dist.all_gather_object(handles, {k: b.handle for k, b in self.local.items()}, group=group)
        self.remote: Dict[str, list] = {k: [] for k in sizes}
        for r in range(world):
            for k in sizes:
                self.remote[k].append(self.local[k].ptr if r == rank else ops.peer_open(handles[r][k], device))
        self.flag = torch.zeros(1, device=device)
        dist.barrier(group=group)

    def put_all(self, key: str, dst_offset: int, dpitch: int, src: torch.Tensor, src_offset_of, spitch: int, width: int,
                height: int) -> None:
        """One block of the same shape to every rank (one launch): rank d receives the block that starts
        ``src_offset_of(d)`` bytes into src, at ``dst_offset`` of its buffer ``key``."""
        order = self.order()
        ops.copy_2d_batch([self.remote[key][d] + dst_offset for d in order], src, [src_offset_of(d) for d in order],
                          dpitch, spitch, width, height)

    def fence(self) -> None:
        """Stream-ordered (current stream): completes on a rank only after every rank's earlier copies have completed.
        A barrier of flags in peer memory (``px_peer_barrier``); ``PX_PEER_FENCE=nccl`` selects a 4-byte all_reduce."""
        self.epoch += 1
        if self.use_flags:
            ops.peer_barrier(self.remote["flags"], self.rank, self.world, self.epoch, self.device)
        else:
            dist.all_reduce(self.flag, group=self.group)

    def send(self, fn, *keep: torch.Tensor) -> None:
        """Runs ``fn`` (copies into peer buffers) on the communication stream, after everything the compute stream has
        been given so far; the compute stream goes on.  ``keep``: tensors the copies read (their memory must not be
        reused before the copies are through)."""
        if self.comm is None:
            fn()
            return
        main = torch.cuda.current_stream(self.device)
        self.comm.wait_stream(main)
        for t in keep:
            t.record_stream(self.comm)
        with torch.cuda.stream(self.comm):
            fn()

    def join(self) -> None:
        """Barrier after the copies sent so far, on the communication stream; the compute stream waits for it."""
        if self.comm is None:
            self.fence()
            return
        main = torch.cuda.current_stream(self.device)
        self.comm.wait_stream(main)
        with torch.cuda.stream(self.comm):
            self.fence()
        main.wait_stream(self.comm)

    def mark(self) -> "torch.cuda.Event":
        """Barrier after the copies sent so far, on the communication stream only; returns the event that follows it,
        for the compute stream to wait on when it gets to the data (``wait``)."""
        stream = self.comm if self.comm is not None else torch.cuda.current_stream(self.device)
        with torch.cuda.stream(stream):
            self.fence()
            ev = torch.cuda.Event()
            ev.record(stream)
        return ev

    def wait(self, ev: "torch.cuda.Event") -> None:
        torch.cuda.current_stream(self.device).wait_event(ev)

    def close(self) -> None:
        """Unmaps the other ranks' buffers and frees this rank's (after a barrier: nobody may still be writing)."""
        if not self.local:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for k, ptrs in self.remote.items():
            for r, ptr in enumerate(ptrs):
                if r != self.rank:
                    ops.peer_close(ptr)
        for b in self.local.values():
            b.free()
        self.local, self.remote = {}, {}

    def order(self):
        """Destination ranks, starting with the next one so that the ranks do not all write to rank 0 first."""
        return [(self.rank + 1 + i) % self.world for i in range(self.world)]


# ----------------------------------------------------------------------------------------------
class ShardedPairformer:
    """Runs the blocks of a ``PairformerStack`` (or one ``PairformerBlock``) on a row-sharded z."""

    def __init__(self, module, group: Optional[dist.ProcessGroup] = None, stages=None) -> None:
        self.blocks = list(module.blocks) if hasattr(module, "blocks") else [module]
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.stages = stages if stages is not None else CudaStages()
        self._peer: Dict[tuple, PeerExchange] = {}

    def close(self) -> None:
        """Releases the peer buffers (collective: every rank of the group must call it)."""
        for px in self._peer.values():
            px.close()
        self._peer = {}

    # ---- helpers ------------------------------------------------------------------------------
    def shard_rows(self, z: torch.Tensor) -> torch.Tensor:
        n = z.shape[0]
        if n % self.world:
            raise RuntimeError(f"N={n} is not divisible by the number of ranks ({self.world}); pad with masked tokens")
        nl = n // self.world
        return z[self.rank * nl:(self.rank + 1) * nl].clone()       # private copy: the shard is updated in place

    def _all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """[world, *t.shape]: slice p is rank p's tensor."""
        t = t.contiguous()
        out = torch.empty(self.world * t.numel(), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.view(-1), group=self.group)
        return out.view((self.world,) + tuple(t.shape))

    def gather_rows(self, z_loc: torch.Tensor) -> torch.Tensor:
        return self._all_gather(z_loc).reshape((-1,) + tuple(z_loc.shape[1:]))

    def _all_to_all(self, send: torch.Tensor) -> torch.Tensor:
        """send[p] goes to rank p; returns recv with recv[p] = what rank p sent to this rank."""
        send = send.contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        return recv

    def _rows_to_channels(self, t: torch.Tensor, k_sharded: bool) -> torch.Tensor:
        """[128][rows_loc][ld] (rows sharded) -> [128/P][N][ld(N)] (channels sharded).

        With ``k_sharded`` the local tensor is [128][N][ld(N/P)]: the contraction index is the
        sharded one and the exchange concatenates it instead of the rows."""
        p = self.world
        c, r, ldl = t.shape
        cp = c // p
        recv = self._all_to_all(t.view(p, cp, r, ldl))                      # [src][cp][r][ldl]
        if not k_sharded:
            return recv.permute(1, 0, 2, 3).reshape(cp, p * r, ldl)          # rows of source p come p-th
        n = r
        nl = n // p
        full = recv[..., :nl].permute(1, 2, 0, 3).reshape(cp, n, n)          # k blocks of source p come p-th
        ldn = (n + 7) // 8 * 8
        return F.pad(full, (0, ldn - n)) if ldn != n else full.contiguous()

    def _channels_to_rows(self, x: torch.Tensor) -> torch.Tensor:
        """[128/P][N][ld] (channels sharded) -> [128][N/P][ld] (rows sharded)."""
        p = self.world
        cp, n, ldn = x.shape
        nl = n // p
        send = x.view(cp, p, nl, ldn).permute(1, 0, 2, 3)                    # [dst][cp][nl][ld]
        recv = self._all_to_all(send)                                        # [src = channel block][cp][nl][ld]
        return recv.reshape(p * cp, nl, ldn)

    def _transpose_shard(self, z_loc: torch.Tensor) -> torch.Tensor:
        """Row shard [N/P i][N j][c] of z  ->  row shard [N/P j][N i][c] of z^T (and back: an involution)."""
        p = self.world
        nl, n, c = z_loc.shape
        send = z_loc.view(nl, p, nl, c).permute(1, 0, 2, 3)                  # [dst j-block][i][j][c]
        recv = self._all_to_all(send)                                        # [src i-block][i][j][c]
        return recv.permute(2, 0, 1, 3).reshape(nl, n, c).contiguous()

    # ---- the same exchanges as direct copies into peer buffers ----------------------------------
    def _peer_for(self, z_loc: torch.Tensor) -> Optional[PeerExchange]:
        """The peer transport for this shape, or None when the all_to_all path has to be used."""
        if not (z_loc.is_cuda and isinstance(self.stages, CudaStages)) or self.world == 1:
            return None
        if os.environ.get("PX_PEER_EXCHANGE", "1") == "0":
            return None
        nl, n, _ = z_loc.shape
        if 128 % self.world or nl % 8 or n % 8:          # every copied run must be a multiple of 16 bytes
            return None
        key = (n, z_loc.element_size(), z_loc.device.index)
        if key not in self._peer:
            self._peer[key] = PeerExchange(self.group, self.world, self.rank, z_loc.device, n, z_loc.element_size())
        return self._peer[key]

    def _peer_rows_to_channels(self, px: PeerExchange, t: torch.Tensor, key: str, k_sharded: bool, nl: int,
                               r0: int = 0, csel: Optional[Tuple[int, int]] = None) -> None:
        """The copies of ``_rows_to_channels`` (no fence) for local rows [r0, r0 + rc) of this rank's nl rows:
        t [128][rc][ld] (or, ``k_sharded``, [128][N][ld(rc)]) -> buffer ``key`` [128/P][N][ld(N)].  ``csel``: only
        channels [c0, c1) of every destination's 128/P."""
        p, me = self.world, self.rank
        c, r, ldl = t.shape
        cp = c // p
        c0, c1 = csel if csel is not None else (0, cp)
        if not k_sharded:          # my rows become rows me*nl + r0.. of every channel: one run of rc*ld per channel
            px.put_all(key, ((me * nl + r0) + c0 * p * nl) * ldl * 2, p * nl * ldl * 2, t,
                       lambda d: (d * cp + c0) * r * ldl * 2, r * ldl * 2, r * ldl * 2, c1 - c0)
        else:                      # my rows are the contraction index: a run of rc per (channel, i)
            ldn = (r + 7) // 8 * 8
            px.put_all(key, (me * nl + r0) * 2 + c0 * r * ldn * 2, ldn * 2, t, lambda d: (d * cp + c0) * r * ldl * 2,
                       ldl * 2, ldl * 2, (c1 - c0) * r)

    def _peer_channels_to_rows(self, px, x: torch.Tensor, c0: int = 0) -> None:
        """x [cc][N][ld] (channels c0.. of my 128/P) -> buffer ``x`` [128][N/P][ld] of every rank: rows d*nl.. go to
        rank d."""
        p, me = self.world, self.rank
        cc, n, ldn = x.shape
        nl, cp = n // p, 128 // p
        px.put_all("x", (me * cp + c0) * nl * ldn * 2, nl * ldn * 2, x, lambda d: d * nl * ldn * 2, n * ldn * 2,
                   nl * ldn * 2, cc)

    def _peer_to_columns(self, px, z_rows: torch.Tensor, nl: int, r0: int = 0) -> None:
        """Rows [r0, r0 + rc) of the row slab [N/P i][N j][c] -> buffer ``zc`` [N i][N/P j][c] of every rank: columns
        d*nl.. go to rank d."""
        p, me = self.world, self.rank
        rc, n, c = z_rows.shape
        run = nl * c * z_rows.element_size()
        px.put_all("zc", (me * nl + r0) * run, run, z_rows, lambda d: d * run, p * run, run, rc)

    def _peer_from_columns(self, px, zc: torch.Tensor) -> None:
        """Column slab [N i][N/P j][c] -> buffer ``zr`` [N/P i][N j][c] of every rank: rows e*nl.. go to rank e."""
        p, me = self.world, self.rank
        n, nl, c = zc.shape
        run = nl * c * zc.element_size()
        px.put_all("zr", me * run, p * run, zc, lambda e: e * nl * run, run, run, nl)

    def _peer_gather_bias(self, px, bias_loc: torch.Tensor) -> None:
        """Pair bias [4][N/P u][ldm] of my rows -> rows me*nl.. of buffer ``bias`` [4][N][ldm] of every rank."""
        p, me = self.world, self.rank
        h, nl, ldm = bias_loc.shape
        run = nl * ldm * bias_loc.element_size()
        px.put_all("bias", me * run, p * run, bias_loc, lambda d: 0, run, run, h)

    # The exchanges can be pipelined against the kernels that produce their data (PX_PEER_CHUNKS > 1): the producer
    # then runs in row chunks on the compute stream, and the copies of a chunk run on the communication stream while
    # the next chunk is being computed; one barrier of flags closes each exchange.  A rank arrives at a barrier only
    # after all the compute-stream work it was given before the exchange, so a receive buffer is never overwritten
    # while its owner still reads what the previous exchange left there.  Measured on two B200s (N = 1536, fp32 z):
    # 14.43 ms per block with one chunk, 14.56 with two, 14.66 with four -- the producers are HBM-bound and the copy
    # kernel beside them only gets the room they leave, so the default is one chunk.
    def _row_chunks(self, nl: int):
        """Splits the nl local rows into pieces of multiples of 8 rows (copied runs are multiples of 16 bytes)."""
        want = max(1, int(os.environ.get("PX_PEER_CHUNKS", "1")))
        units = nl // 8
        k = max(1, min(want, units))
        cuts = [8 * (units * i // k) for i in range(k + 1)]
        return [(cuts[i], cuts[i + 1]) for i in range(k) if cuts[i + 1] > cuts[i]]

    def _tri_mul_peer(self, px: PeerExchange, mod, z_loc, mask_loc, incoming: bool, zn=None) -> None:
        """``zn``: the standardised copy of an fp32 z_loc, when the caller has it already."""
        st, p, me = self.stages, self.world, self.rank
        nl, n, _ = z_loc.shape
        cp, ldn = 128 // p, (n + 7) // 8 * 8
        if zn is None:
            zn = st.standardised(z_loc, mod.layer_norm_in.eps)
        halves = [(0, cp)] if cp < 2 else [(0, cp // 2), (cp // 2, cp)]
        a_full = px.local["a"].tensor((cp, n, ldn), torch.float16)
        b_full = px.local["b"].tensor((cp, n, ldn), torch.float16)
        if len(halves) == 2 and os.environ.get("PX_PEER_AB_HALVES", "0") == "1":
            # a and b leave in two channel groups, each closed by its own barrier on the communication stream: the
            # first group is contracted while the second is still travelling.  Measured at N = 1536, fp32 z: 7.54 ms
            # per block against 7.50 on four B200s, 13.83 against 13.52 on two (the copies slow the contraction they
            # run beside), hence off by default.
            a, b = st.trimul_in_proj(mod, z_loc, mask_loc, incoming, zn=zn)
            ready = []
            for cs in halves:
                px.send(lambda cs=cs: (self._peer_rows_to_channels(px, a, "a", incoming, nl, 0, cs),
                                       self._peer_rows_to_channels(px, b, "b", incoming, nl, 0, cs)), a, b)
                ready.append(px.mark())
            del a, b
        else:
            for r0, r1 in self._row_chunks(nl):
                a, b = st.trimul_in_proj(mod, z_loc[r0:r1], None if mask_loc is None else mask_loc[r0:r1], incoming,
                                         zn=None if zn is None else zn[r0:r1])
                px.send(lambda a=a, b=b, r0=r0: (self._peer_rows_to_channels(px, a, "a", incoming, nl, r0),
                                                  self._peer_rows_to_channels(px, b, "b", incoming, nl, r0)), a, b)
                del a, b
            px.join()
            ready = [None] * len(halves)
        for (c0, c1), ev in zip(halves, ready):     # the contraction in two channel groups: x of the first travels
            if ev is not None:                      # while the second is contracted
                px.wait(ev)
            x = st.trimul_contract(a_full[c0:c1], b_full[c0:c1])
            px.send(lambda x=x, c0=c0: self._peer_channels_to_rows(px, x, c0), x)
            del x
        px.join()
        st.trimul_out(mod, px.local["x"].tensor((128, nl, ldn), torch.float16), z_loc, zn=zn)

    def _tri_att_pair_peer(self, px: PeerExchange, start, end, z_loc, mask_loc, mask_cols) -> torch.Tensor:
        """Starting-node then ending-node attention.  The output stage of the first runs in row chunks whose rows leave
        for the column slabs of the other ranks as soon as they are final; the second works on the received column slab
        zc [N i][N/P j][c] (the kernels address it as element (u=j, t=i)) and sends the rows back.  Returns the
        updated row slab: a view of this rank's receive buffer (bf16 z: the caller's z_loc is NOT written), or z_loc
        itself with the returned update added (fp32 z)."""
        st, p, me = self.stages, self.world, self.rank
        nl, n, c = z_loc.shape
        zn = st.standardised(z_loc, start.layer_norm.eps)
        q, k, v, bias_loc, mb = st.triatt_in_proj(start, z_loc, mask_loc, zn=zn)
        h, _, ldm = bias_loc.shape
        px.send(lambda: self._peer_gather_bias(px, bias_loc), bias_loc)
        px.join()
        bias_full = px.local["bias"].tensor((h, p * nl, ldm), torch.float32)
        o = st.triatt_flash(q, k, v, bias_full, mb)
        del q, k, v
        # 16-bit tensors cross NVLink in both directions: the bf16 rows themselves, or, for an fp32 z, the standardised
        # fp16 copy on the way out and the update alone on the way back (the rows' owner adds it to its fp32 rows)
        fp32 = z_loc.dtype == torch.float32
        for r0, r1 in self._row_chunks(nl):
            st.triatt_out(start, o[r0:r1], z_loc[r0:r1], zn=None if zn is None else zn[r0:r1])
            rows = st.standardised(z_loc[r0:r1], end.layer_norm.eps) if fp32 else z_loc[r0:r1]
            px.send(lambda rows=rows, r0=r0: self._peer_to_columns(px, rows, nl, r0), rows, z_loc)
            del rows
        px.join()
        del o, zn
        zc = px.local["zc"].tensor((n, nl, c), torch.float16 if fp32 else z_loc.dtype)
        zn = None if fp32 else st.standardised(zc, end.layer_norm.eps)      # (fp32: zc already is the standardised copy)
        q, k, v, bias_loc, mb = st.triatt_in_proj(end, zc, mask_cols, True, zn=zn)
        px.send(lambda: self._peer_gather_bias(px, bias_loc), bias_loc)
        px.join()
        back = st.triatt_out(end, st.triatt_flash(q, k, v, bias_full, mb), zc, True, zn=zn)   # fp32: the update, fp16
        px.send(lambda: self._peer_from_columns(px, back), back)
        px.join()
        zr = px.local["zr"].tensor((nl, n, c), torch.float16 if fp32 else z_loc.dtype)
        if fp32:
            return st.add_update(z_loc, zr)
        return zr

    # ---- sub-modules ----------------------------------------------------------------------------
    def _tri_mul(self, mod, z_loc, mask_loc, incoming: bool) -> None:
        st = self.stages
        zn = st.standardised(z_loc, mod.layer_norm_in.eps)
        a, b = st.trimul_in_proj(mod, z_loc, mask_loc, incoming, zn=zn)
        a = self._rows_to_channels(a, k_sharded=incoming)
        b = self._rows_to_channels(b, k_sharded=incoming)
        x = st.trimul_contract(a, b)
        del a, b
        st.trimul_out(mod, self._channels_to_rows(x), z_loc, zn=zn)

    def _tri_att_rows(self, mod, z_loc, mask_loc) -> None:
        st = self.stages
        zn = st.standardised(z_loc, mod.layer_norm.eps)
        q, k, v, bias_loc, mb = st.triatt_in_proj(mod, z_loc, mask_loc, zn=zn)
        h, nl, ldm = bias_loc.shape
        bias_full = self._all_gather(bias_loc).permute(1, 0, 2, 3).reshape(h, self.world * nl, ldm)
        st.triatt_out(mod, st.triatt_flash(q, k, v, bias_full, mb), z_loc, zn=zn)

    def _single_branch(self, blk, s, bias):
        """s + AttentionPairBias(s, z) + Transition(.), query rows sharded like z; ``bias`` [H, N/P, N] is the pair
        bias of this rank's rows of the block's final z (all this branch takes from z)."""
        apb, att = blk.attention_pair_bias, blk.attention_pair_bias.attention
        nl = bias.shape[1]
        rows = slice(self.rank * nl, (self.rank + 1) * nl)
        dt = s.dtype
        x = self.stages.single_layer_norm(apb.layernorm_a, s.float().contiguous())
        n, h, d = x.shape[0], apb.n_heads, att.c_hidden
        q = F.linear(x[rows], att.linear_q.weight, att.linear_q.bias).view(nl, h, d).transpose(0, 1)
        k = F.linear(x, att.linear_k.weight).view(n, h, d).transpose(0, 1)
        v = F.linear(x, att.linear_v.weight).view(n, h, d).transpose(0, 1)
        o = F.scaled_dot_product_attention(q / math.sqrt(d), k, v, attn_mask=bias.to(q.dtype), scale=1.0)
        o = o.transpose(0, 1).reshape(nl, h * d).contiguous()
        o_full = self._all_gather(o).reshape(self.world * nl, h * d)
        o_full = o_full * torch.sigmoid(F.linear(x, att.linear_g.weight))
        s = s + F.linear(o_full, att.linear_o.weight).to(dt)
        tr = blk.single_transition
        y = self.stages.single_layer_norm(tr.layernorm1, s.float().contiguous())
        upd = F.linear(F.silu(F.linear(y, tr.linear_no_bias_a.weight)) * F.linear(y, tr.linear_no_bias_b.weight),
                       tr.linear_no_bias.weight)
        return s + upd.to(dt)

    # ---- public ---------------------------------------------------------------------------------
    @torch.no_grad()
    def forward(self, s: Optional[torch.Tensor], z_loc: torch.Tensor, pair_mask: Optional[torch.Tensor]
                ) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
        """z_loc [N/P, N, 128] is updated in place; s [N, c_s] (replicated) is returned updated."""
        nl, n, _ = z_loc.shape
        if nl * self.world != n:
            raise RuntimeError(f"z_loc has {nl} rows; expected N/P = {n}/{self.world}")
        rows = slice(self.rank * nl, (self.rank + 1) * nl)
        px = self._peer_for(z_loc)
        main = side = None
        if z_loc.is_cuda and isinstance(self.stages, CudaStages):
            from .pairformer import _side_stream

            main, side = torch.cuda.current_stream(z_loc.device), _side_stream(z_loc.device)
            side.wait_stream(main)
        mask_loc = mask_t_loc = mask_cols = None
        if pair_mask is not None:
            pair_mask = pair_mask.to(torch.float32)
            mask_loc = pair_mask[rows].contiguous()
            if px is None:
                mask_t_loc = pair_mask.t()[rows].contiguous()
            else:
                mask_cols = pair_mask[:, rows].contiguous()
        zn_final = None      # fp32 z: the standardised copy made for a block's pair bias serves the next block's first update
        for blk in self.blocks:
            if px is not None:
                zn_first = zn_final if zn_final is not None and zn_eps == blk.tri_mul_out.layer_norm_in.eps else None
                zn_final = None
                self._tri_mul_peer(px, blk.tri_mul_out, z_loc, mask_loc, incoming=False, zn=zn_first)
                del zn_first
                self._tri_mul_peer(px, blk.tri_mul_in, z_loc, mask_loc, incoming=True)
                zr = self._tri_att_pair_peer(px, blk.tri_att_start, blk.tri_att_end, z_loc, mask_loc, mask_cols)
                self.stages.transition(blk.pair_transition, zr, out=z_loc)    # reads the received rows (or z_loc itself)
            else:
                self._tri_mul(blk.tri_mul_out, z_loc, mask_loc, incoming=False)
                self._tri_mul(blk.tri_mul_in, z_loc, mask_loc, incoming=True)
                self._tri_att_rows(blk.tri_att_start, z_loc, mask_loc)
                zt = self._transpose_shard(z_loc)
                self._tri_att_rows(blk.tri_att_end, zt, mask_t_loc)
                z_loc.copy_(self._transpose_shard(zt))
                del zt
                self.stages.transition(blk.pair_transition, z_loc)
            if blk.c_s > 0 and s is not None:
                if px is not None:
                    zn_eps = blk.attention_pair_bias.layernorm_z.eps
                    zn_final = self.stages.standardised(z_loc, zn_eps)              # None for bf16 rows
                bias = self.stages.pair_bias(blk.attention_pair_bias, z_loc, zn=zn_final)   # reads the block's final z
                if side is None:
                    s = self._single_branch(blk, s, bias)
                else:               # the pair path never reads s: the rest runs beside the next block's pair path
                    bias.record_stream(side)
                    side.wait_stream(main)
                    with torch.cuda.stream(side):
                        s = self._single_branch(blk, s, bias)
        if side is not None:
            main.wait_stream(side)
            if s is not None:
                s.record_stream(main)
        return s, z_loc


class ShardedRecyclingTrunk:
    """The recycling loop of a ``RecyclingTrunk`` on a row-sharded pair representation.

    Both recycling updates are row-local (protenix/model/protenix.py:246, :287): every rank updates its own rows of z
    from its rows of z_init, s is replicated, and the stack runs through ``ShardedPairformer``.
    """

    def __init__(self, trunk, group: Optional[dist.ProcessGroup] = None, stages=None) -> None:
        self.trunk = trunk
        self.stack = ShardedPairformer(trunk.pairformer_stack, group=group, stages=stages)
        self.stages = self.stack.stages

    def shard_rows(self, z: torch.Tensor) -> torch.Tensor:
        return self.stack.shard_rows(z)

    def gather_rows(self, z_loc: torch.Tensor) -> torch.Tensor:
        return self.stack.gather_rows(z_loc)

    @torch.no_grad()
    def forward(self, s_init: torch.Tensor, z_init_loc: torch.Tensor, pair_mask: Optional[torch.Tensor] = None,
                N_cycle: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """z_init_loc [N/P, N, 128] is left untouched; returns (s [N, c_s], the rank's rows of z)."""
        t = self.trunk
        n_cycle = t.N_cycle if N_cycle is None else N_cycle
        z_loc = torch.zeros_like(z_init_loc)
        s = torch.zeros_like(s_init)
        for _ in range(n_cycle):
            z_loc = self.stages.recycle_update(t.layernorm_z_cycle, t.linear_no_bias_z_cycle, z_loc, z_init_loc, z_loc)
            x = self.stages.single_layer_norm(t.layernorm_s, s.float().contiguous())
            s = (s_init.float() + F.linear(x, t.linear_no_bias_s.weight)).to(s_init.dtype)
            s, z_loc = self.stack.forward(s, z_loc, pair_mask)
        return s, z_loc
