"""Expert-parallel MoE step: experts are sharded over the ranks of a process
group, tokens travel to the ranks that own their experts and back.

The reference ships no communication code (its host framework calls DeepEP
around `run_sonic_moe`); this module supplies the two exchanges with the
payload formats the reference's entry points accept.  On CUDA ranks that can
map each other's memory they run over NVLink peer memory (the destination
pulls its rows from the sources' quantised tokens; the forward's return is a
pull fused with the per-token reduction; dx returns as device-to-device
copies underneath the weight-gradient GEMMs; the forward reads no count back
from the device); everywhere else - CPU tensors with gloo, or the switches
below - they are `torch.distributed.all_to_all_single` calls:

  dispatch  a token is sent ONCE to every rank that owns at least one of its
            top-k experts, as e4m3 bytes + raw 1x32 ue8m0 scales (quantise before
            the wire: half the bytes of bf16), with its K local expert ids
            (-1 = not on that rank) and K probabilities
            -> `run_sonic_moe(hidden_states=e4m3, fp8_scale=scales, topk_indices with -1)`
  combine   each rank returns one bf16 row per received token (the weighted sum
            over ITS experts); the source adds the copies in ascending rank order
  backward  mirrors them: dout is dispatched as e4m3 + scales and handed to the
            down-projection backward through `Fp8CombineGradHandle`; dx and the
            score gradients return with the reverse all-to-all.

Every reduction has a fixed order, so results do not depend on timing, and
the peer-memory paths deliver rows in the order the all-to-alls would: both
give the same bits.  The planning and the all-to-all path are device-agnostic
(CPU tensors + gloo work); the FP8 payload, the peer-memory movers and the
expert compute need the CUDA kernels.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

# SONIC_MOE_EP_PEER: how the two bf16 return exchanges (forward combine, backward dx) travel.
#   "fwd" (default)  the forward's return reads the partial rows straight from the owners' memory over NVLink, fused
#                    with the per-token reduction (csrc/ep_peer.cu); the backward's (dx) travels on the communication
#                    stream, where it runs underneath the weight-gradient GEMMs (how: SONIC_MOE_EP_DX_RETURN below)
#   "1"              both read peer memory (the dx return then follows the weight gradients: nothing hides it)
#   "0"              both are NCCL all-to-alls followed by a local reduction
# Reading peer memory needs ranks that can map each other's memory (torch symmetric memory); if that fails the
# layer warns once and uses NCCL.  Measured on the reference-shape layer with NCCL dispatch and an NCCL dx return,
# first-10-step medians: 8 GPUs 5.37 ms ("fwd") against 5.55 ("0"); 2 GPUs 3.86 ("1") against 3.92 ("0").
_PEER_MODE = os.getenv("SONIC_MOE_EP_PEER", "fwd")
if _PEER_MODE not in ("0", "1", "fwd"):
    raise ValueError(f"SONIC_MOE_EP_PEER={_PEER_MODE!r}: expected '0', '1' or 'fwd'")
USE_PEER_COMBINE = _PEER_MODE in ("1", "fwd")
PEER_COMBINE_BACKWARD = _PEER_MODE == "1"
# SONIC_MOE_EP_DISPATCH=pull: the two FP8 dispatch exchanges (x in the forward, dout in the backward) are fetched by
# the destination rank straight from the sources' quantised tokens over NVLink (csrc/ep_peer.cu) - no gathered copy
# of the outgoing rows, no all-to-all, no packing of scales / ids / probabilities into a side exchange; "nccl": the
# rows are gathered and travel through NCCL all-to-alls.  Needs the same peer mapping as above.
DISPATCH = os.getenv("SONIC_MOE_EP_DISPATCH", "pull")
if DISPATCH not in ("pull", "nccl"):
    raise ValueError(f"SONIC_MOE_EP_DISPATCH={DISPATCH!r}: expected 'pull' or 'nccl'")
# SONIC_MOE_EP_SYNC_FREE=1 (default; needs the pull dispatch and the peer-memory forward return): the forward reads
# nothing back from the device.  The counts travel to the host on a side stream and are looked at when the backward's
# all-to-alls need them; until then both pull kernels take their offsets from tables built on the device and every
# buffer is sized at world x capacity rows, rows that did not arrive being masked.
SYNC_FREE = os.getenv("SONIC_MOE_EP_SYNC_FREE", "1") == "1"
# SONIC_MOE_EP_DX_RETURN=copy (default): the backward's return exchange (dx rows back to their sources) is a set of
# plain device-to-device copies into the sources' mapped buffers, issued on the communication stream - the copy
# engines move them over NVLink while the weight-gradient GEMMs keep every SM; "nccl": an all-to-all kernel, which
# shares the SMs with those GEMMs (measured on 2 GPUs: dw2 309 us under the all-to-all kernel, 233 us alone).
DX_RETURN = os.getenv("SONIC_MOE_EP_DX_RETURN", "copy")
if DX_RETURN not in ("copy", "nccl"):
    raise ValueError(f"SONIC_MOE_EP_DX_RETURN={DX_RETURN!r}: expected 'copy' or 'nccl'")


_COMM_STREAMS: dict = {}
_READBACK_STREAMS: dict = {}
_PINNED_FREE: dict = {}      # (device index, shape) -> pinned int64 host buffers no plan owns at the moment


def _readback_stream(device) -> "torch.cuda.Stream":
    """A side stream per device for small device-to-host copies that must not queue behind the compute stream."""
    key = torch.device(device).index
    st = _READBACK_STREAMS.get(key)
    if st is None:
        st = _READBACK_STREAMS[key] = torch.cuda.Stream(device=torch.device("cuda", key))
    return st


def _alloc_pinned_i64(shape):
    return torch.empty(shape, dtype=torch.int64).pin_memory()


def _pinned_take(key):
    """A pinned int64 host buffer for `key` = (device index, shape).  A plan owns its buffer from the copy of its
    counts until it has read them (or dies unread), however many plans are in flight in between - a pipeline schedule
    may run many forwards before the first backward looks at its counts."""
    free = _PINNED_FREE.setdefault(key, [])
    return free.pop() if free else _alloc_pinned_i64(key[1])


def _pinned_give(key, buf):
    """Back to the pool.  A copy into `buf` may still be in flight (a plan that died unread): the next owner's copy is
    issued on the same device's read-back stream, hence after it."""
    _PINNED_FREE.setdefault(key, []).append(buf)


def _comm_stream(device) -> "torch.cuda.Stream":
    """The one stream per device on which the expert-parallel exchanges run (same issue order on every rank)."""
    key = torch.device(device).index
    if key is None:
        key = torch.cuda.current_device()
    st = _COMM_STREAMS.get(key)
    if st is None:
        st = _COMM_STREAMS[key] = torch.cuda.Stream(device=torch.device("cuda", key))
    return st


class PeerArena:
    """A bf16 [rows, H] buffer per rank that every rank of the group has mapped.  Allocation and mapping are
    collective calls; the size is derived from quantities all ranks share."""

    def __init__(self, group, rows: int, H: int, device):
        import torch.distributed._symmetric_memory as symm
        self.rows, self.H = rows, H
        self.buf = symm.empty(rows * H, dtype=torch.bfloat16, device=device)
        self.hdl = symm.rendezvous(self.buf, group.group_name)
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        self.token = torch.zeros(1, dtype=torch.float32, device=device)
        self.group = group

    def view(self, n: int) -> torch.Tensor:
        return self.buf[: n * self.H].view(n, self.H)

    def holds(self, t: torch.Tensor) -> bool:
        return t is not None and t.is_cuda and t.data_ptr() == self.buf.data_ptr() and t.is_contiguous()

    def everyone_has_written(self):
        """Stream-ordered: returns (on the stream) once every rank's earlier work on its stream is done."""
        dist.all_reduce(self.token, group=self.group)


class ReturnArena:
    """A bf16 [rows, H] buffer per rank, mapped by all ranks, that receives the rows this rank sent out when they
    come back (in its send order): the owners copy them in with ordinary device-to-device copies."""

    def __init__(self, group, rows: int, H: int, device):
        import torch.distributed._symmetric_memory as symm
        self.rows, self.H = rows, H
        self.buf = symm.empty(rows * H, dtype=torch.bfloat16, device=device)
        self.hdl = symm.rendezvous(self.buf, group.group_name)
        self.token = torch.zeros(1, dtype=torch.float32, device=device)
        self.group = group

    def rows_of(self, rank: int, first: int, n: int) -> torch.Tensor:
        """Rows [first, first + n) of rank `rank`'s buffer as a tensor of this process."""
        return self.hdl.get_buffer(rank, (n, self.H), torch.bfloat16, first * self.H)

    def mine(self, n: int) -> torch.Tensor:
        return self.buf[: n * self.H].view(n, self.H)

    def everyone_has_written(self):
        dist.all_reduce(self.token, group=self.group)


def _align256(n: int) -> int:
    return (n + 255) // 256 * 256


class DispatchArena:
    """One byte buffer per rank, mapped by every rank of the group, from which the peers fetch what this rank sends:
    two payload slots (x in the forward, dout in the backward: e4m3 [T,H] + raw scales [T,H/32]), the tokens'
    probabilities [T,K] f32, and the send lists (token [n_send] and local expert ids [n_send,K] of every outgoing
    row).  The layout is a function of (T capacity, H, K, world) only, hence the same on all ranks."""

    def __init__(self, group, t_cap: int, H: int, K: int, world: int, device):
        import torch.distributed._symmetric_memory as symm
        self.t_cap, self.H, self.K, self.world = t_cap, H, K, world
        cap = t_cap * min(K, world)
        at = 0
        self.off_q, self.off_raw = [], []
        for _ in range(2):
            self.off_q.append(at)
            at += _align256(t_cap * H)
            self.off_raw.append(at)
            at += _align256(t_cap * (H // 32))
        self.off_probs = at
        at += _align256(t_cap * K * 4)
        self.off_tok = at
        at += _align256(cap * 4)
        self.off_idx = at
        at += _align256(cap * K * 4)
        self.off_counts = at                 # rows this rank sends to each rank, int32 [world]
        at += 256
        self.off_seg = at                    # start of each destination's segment in the send order, int32 [world+1]
        at += 256
        self.cap = cap
        self.buf = symm.empty(at, dtype=torch.uint8, device=device)
        self.hdl = symm.rendezvous(self.buf, group.group_name)
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        self.token = torch.zeros(1, dtype=torch.float32, device=device)
        self.group = group

    def fits(self, T: int, H: int, K: int, world: int) -> bool:
        return T <= self.t_cap and (H, K, world) == (self.H, self.K, self.world)

    def payload(self, slot: int, T: int):
        """(q [T,H], raw [T,H/32]) views of payload slot `slot`."""
        H = self.H
        q = self.buf[self.off_q[slot]: self.off_q[slot] + T * H].view(T, H)
        raw = self.buf[self.off_raw[slot]: self.off_raw[slot] + T * (H // 32)].view(T, H // 32)
        return q, raw

    def _i32(self, off: int, n: int):
        return self.buf[off: off + n * 4].view(torch.int32)

    def publish_lists(self, plan: "DispatchPlan", probs=None):
        """This rank's send lists (and, in the forward, its tokens' probabilities) into the mapped buffer."""
        K = self.K
        if plan.deferred:
            # no host-side count: the lists go out at their capacity together with the counts the peers need
            cap = plan.send_tok_cap.numel()
            if cap:
                self._i32(self.off_tok, cap).copy_(plan.send_tok_cap)
                self._i32(self.off_idx, cap * K).view(cap, K).copy_(plan.send_idx_cap)
            self._i32(self.off_counts, self.world).copy_(plan.md_counts)
            self._i32(self.off_seg, self.world + 1).copy_(plan.md_efo)
            if probs is not None and plan.T:
                self.buf[self.off_probs: self.off_probs + plan.T * K * 4].view(torch.float32).view(plan.T, K).copy_(
                    probs)
            return
        n = plan.n_send
        if n:
            self.buf[self.off_tok: self.off_tok + n * 4].view(torch.int32).copy_(plan.send_tok_i32)
            self.buf[self.off_idx: self.off_idx + n * K * 4].view(torch.int32).view(n, K).copy_(plan.send_idx)
        if probs is not None and plan.T:
            self.buf[self.off_probs: self.off_probs + plan.T * K * 4].view(torch.float32).view(plan.T, K).copy_(probs)

    def layout(self, slot: int):
        return (self.off_q[slot], self.off_raw[slot], self.off_tok, self.off_idx, self.off_probs)

    def everyone_has_written(self):
        """Stream-ordered: returns (on the stream) once every rank's earlier work on its stream is done."""
        dist.all_reduce(self.token, group=self.group)

    def pull(self, plan: "DispatchPlan", slot: int, with_meta: bool):
        from . import ops
        self.everyone_has_written()
        if plan.deferred:
            me = dist.get_rank(self.group)
            # rebuilt after every barrier: a later forward of the same layer may have replaced the counts
            plan.tables = ops.ep_tables(self.ptrs, me, self.off_counts, self.off_seg, self.buf.device)
            return ops.ep_dispatch_pull_dev(self.ptrs, plan.tables, me, self.layout(slot), self.H, self.K,
                                            plan.n_bound, self.buf.device, with_meta=with_meta)
        return ops.ep_dispatch_pull(self.ptrs, plan.recv_counts, plan.src_seg_off, dist.get_rank(self.group),
                                    self.layout(slot), self.H, self.K, self.buf.device, with_meta=with_meta)


class DispatchPlan:
    """Who goes where, built from the top-k indices of this rank's tokens.

    send_tok   [n_send]  token of each outgoing row, grouped by destination rank, ascending token inside
    send_idx   [n_send,K] local expert id on the destination (-1 where the slot lives elsewhere)
    send_counts / recv_counts  rows per peer (host lists)
    copy_pos / copy_off  for the source-side reductions: the outgoing rows of token t are
                         copy_pos[copy_off[t]:copy_off[t+1]], ascending destination rank
    """

    # attributes that exist only once the counts have reached the host
    _HOST_FIELDS = frozenset(("send_counts", "recv_counts", "tokens_per_local_expert", "n_send", "n_recv",
                              "first_row_at", "src_seg_off", "send_off", "max_recv_rows", "tokens_all",
                              "send_tok_i32", "send_idx", "send_rank", "send_tok", "copy_pos"))

    def __init__(self, idx: torch.Tensor, E: int, group, world: int | None = None, deferred: bool = False):
        """`deferred` (CUDA only): the counts are copied to the host on a side stream and read when first needed -
        normally at the return exchange, long after they arrived - instead of right away, so building the plan does
        not drain the GPU's work queue.  Until then only the capacity-sized device lists exist (`send_tok_cap`,
        `send_idx_cap`, `copy_pos_cap`, `md_counts`, `md_efo`)."""
        world = dist.get_world_size(group) if world is None else world
        assert E % world == 0
        T, K = idx.shape
        self.T, self.K, self.El, self.E, self.group = T, K, E // world, E, group
        self.world = world
        self.deferred = bool(deferred) and idx.is_cuda
        self._pending = None
        if idx.is_cuda:
            self._build_cuda(idx, world)
        else:
            self._build_torch(idx, world)

    def __getattr__(self, name):
        # reached only when the attribute is missing: a host-side field of a plan whose counts are still in flight
        if name in DispatchPlan._HOST_FIELDS and self.__dict__.get("_pending") is not None:
            host, ready, key = self._pending
            self._pending = None
            ready.synchronize()
            counts = host.tolist()
            _pinned_give(key, host)
            self._set_counts(counts)
            self._finish_cuda()
            return self.__dict__[name]
        raise AttributeError(name)

    def __del__(self):
        pending = self.__dict__.get("_pending")
        if pending is not None:                 # never looked at (a forward without a backward): the buffer is free
            try:
                _pinned_give(pending[2], pending[0])
            except Exception:                   # interpreter shutdown: the pool may be gone already
                pass

    def _set_counts(self, M):
        me, El, world = dist.get_rank(self.group), self.El, self.world
        self.send_counts = [int(v) for v in M[me][:world]]
        self.recv_counts = [int(M[s][me]) for s in range(world)]
        self.tokens_per_local_expert = [sum(int(M[s][world + me * El + j]) for s in range(world)) for j in range(El)]
        self.n_send, self.n_recv = sum(self.send_counts), sum(self.recv_counts)
        # where this rank's rows start inside rank r's receive order (sources ascending), and the send offsets
        self.first_row_at = [sum(int(M[s][r]) for s in range(me)) for r in range(world)]
        # where the segment addressed to this rank starts inside rank s's send order (destinations ascending)
        self.src_seg_off = [sum(int(M[s][r]) for r in range(me)) for s in range(world)]
        self.send_off = [sum(self.send_counts[:r]) for r in range(world)]
        self.max_recv_rows = max(sum(int(M[s][r]) for s in range(world)) for r in range(world))
        self.tokens_all = [int(M[s][-1]) for s in range(world)]

    def _exchange_counts(self, rows_to, pairs, world):
        """One small all-gather + ONE read-back gives every rank the whole picture: rows each rank sends to each
        other rank, routed pairs per expert (summed over sources they size the expert-sorted buffers exactly) and
        every rank's token count."""
        row = torch.cat([rows_to.reshape(-1).to(torch.int64), pairs.reshape(-1).to(torch.int64),
                         # (a fill kernel, not a host-to-device copy: a copy from pageable memory makes the host
                         # wait for everything the stream has been given)
                         torch.full((1,), self.T, dtype=torch.int64, device=rows_to.device)])
        parts = [torch.empty_like(row) for _ in range(world)]
        dist.all_gather(parts, row.contiguous(), group=self.group)
        M = torch.stack(parts)
        if not self.deferred:
            self._set_counts(M.tolist())
            return
        dev = M.device
        cur, side = torch.cuda.current_stream(dev), _readback_stream(dev)
        side.wait_stream(cur)
        key = (dev.index, tuple(M.shape))
        host = _pinned_take(key)
        with torch.cuda.stream(side):
            host.copy_(M, non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(side)
        M.record_stream(side)
        self._pending = (host, ready, key)

    def _build_cuda(self, idx, world):
        """The plan is the routing-metadata problem with destination ranks in the role of experts: one call of the
        metadata kernels on the de-duplicated destination list gives the send order (rank-major, token ascending),
        the per-rank offsets and each token's copies in ascending rank order.  Two small kernels bracket it; the
        host issues about a dozen launches and reads back once."""
        from . import ops
        T, K = self.T, self.K
        idx = idx.to(torch.int32).contiguous()
        dest_u, pairs = ops.ep_plan_dest(idx, self.E, world)
        cap = T * min(K, world)
        # the probability operand of the metadata kernels is not needed here: any f32 buffer of the right size
        md = ops.topk_metadata(dest_u, dest_u.view(torch.float32), world, alignment=1, TK_alloc=cap,
                               TKp_alloc=cap + world)
        self._idx, self._md = idx, md
        self.md_counts, self.md_efo = md["counts"], md["efo"]
        self.copy_off = md["naept"]
        if self.deferred:
            # capacity-sized lists, usable without any host-side count (rows beyond efo[world] are never read)
            self.send_tok_cap = md["x_gather_idx"][:cap]
            self.send_idx_cap, self.send_rank_cap = ops.ep_plan_send_idx(idx, self.send_tok_cap, md["efo"], cap,
                                                                         self.E, world)
            self.copy_pos_cap = md["s_reverse_scatter_idx"][:cap]
        self._exchange_counts(md["counts"], pairs, world)
        if not self.deferred:
            self._finish_cuda()

    def _finish_cuda(self):
        """The exactly-sized lists, once n_send is known on the host."""
        from . import ops
        n, md = self.n_send, self._md
        self.send_tok_i32 = md["x_gather_idx"][:n]
        if self.deferred:
            self.send_idx, self.send_rank = self.send_idx_cap[:n], self.send_rank_cap[:n]
        else:
            self.send_idx, self.send_rank = ops.ep_plan_send_idx(self._idx, self.send_tok_i32, md["efo"], n, self.E,
                                                                 self.world)
        self.send_tok = self.send_tok_i32.long()
        self.copy_pos = md["s_reverse_scatter_idx"][:n]

    def _build_torch(self, idx, world):
        """Device-agnostic construction (CPU tensors, gloo)."""
        T, K, El = self.T, self.K, self.El
        valid = idx >= 0
        dest = torch.where(valid, torch.div(idx, El, rounding_mode="floor"), torch.full_like(idx, -1))   # owning rank
        pairs = torch.bincount(idx.flatten().clamp(min=-1).long() + 1, minlength=self.E + 1)[1:]
        ranks = torch.arange(world, device=idx.device).view(world, 1, 1)
        hit = (dest.unsqueeze(0) == ranks) & valid.unsqueeze(0)                # [P,T,K]
        goes = hit.any(dim=2)                                                 # [P,T]
        pt = goes.nonzero()                                                   # rank-major, token ascending
        self.send_rank, self.send_tok = pt[:, 0], pt[:, 1]
        local = idx.unsqueeze(0) - ranks * El
        local = torch.where(hit, local, torch.full_like(local, -1))          # [P,T,K]
        self.send_idx = local[self.send_rank, self.send_tok].to(torch.int32).contiguous()
        self._exchange_counts(goes.sum(dim=1).to(torch.int64), pairs.to(torch.int64), world)
        # copies of a token, ascending rank: stable sort of the outgoing rows by token
        order = torch.sort(self.send_tok, stable=True).indices
        self.copy_pos = order.to(torch.int32).contiguous()
        off = torch.zeros(T + 1, dtype=torch.int64, device=idx.device)
        off[1:] = goes.sum(dim=0).cumsum(0)
        self.copy_off = off.to(torch.int32).contiguous()

    def a2a(self, send: torch.Tensor, reverse: bool = False, after=None) -> torch.Tensor:
        """Rows travel to their destination (or, reversed, back to their source).

        On CUDA every exchange of a plan is issued, in program order, on one communication stream.  It starts once
        `after` (an event: "the payload is complete") has happened - or, without one, once everything given to the
        current stream so far has run - and the current stream resumes when the exchange is done.  Kernels that
        were enqueued on the current stream AFTER `after` was recorded therefore run underneath the exchange: that
        is how the weight-gradient GEMMs overlap the return exchange of dx in the backward."""
        s, r = (self.recv_counts, self.send_counts) if reverse else (self.send_counts, self.recv_counts)
        send = send.contiguous()
        if not send.is_cuda:
            out = send.new_empty((sum(r),) + tuple(send.shape[1:]))
            dist.all_to_all_single(out, send, output_split_sizes=r, input_split_sizes=s, group=self.group)
            return out
        cur = torch.cuda.current_stream(send.device)
        comm = _comm_stream(send.device)
        if after is not None:
            comm.wait_event(after)
        else:
            comm.wait_stream(cur)
        with torch.cuda.stream(comm):
            out = send.new_empty((sum(r),) + tuple(send.shape[1:]))
            dist.all_to_all_single(out, send, output_split_sizes=r, input_split_sizes=s, group=self.group)
        send.record_stream(comm)
        out.record_stream(cur)
        cur.wait_stream(comm)
        return out

    def return_by_copies(self, rows: torch.Tensor, ret: "ReturnArena", after=None) -> torch.Tensor:
        """The reverse exchange of `a2a(rows, reverse=True)` as device-to-device copies: the rows received from
        source s go back into s's mapped buffer at the place they have in s's send order.  Issued on the
        communication stream after `after`; the current stream resumes once every rank's copies are done.  Returns
        this rank's buffer rows [n_send, H] (its outgoing rows, returned)."""
        cur = torch.cuda.current_stream(rows.device)
        comm = _comm_stream(rows.device)
        if after is not None:
            comm.wait_event(after)
        else:
            comm.wait_stream(cur)
        with torch.cuda.stream(comm):
            starts, at = [], 0
            for n in self.recv_counts:
                starts.append(at)
                at += n
            me, world = dist.get_rank(self.group), self.world
            for step in range(1, world + 1):
                # rank r writes to r+1 first, then r+2, ...: at any moment every destination has one writer
                s_rank = (me + step) % world
                n = self.recv_counts[s_rank]
                if n:
                    ret.rows_of(s_rank, self.src_seg_off[s_rank], n).copy_(
                        rows[starts[s_rank]:starts[s_rank] + n], non_blocking=True)
            ret.everyone_has_written()
        rows.record_stream(comm)
        cur.wait_stream(comm)
        return ret.mine(self.n_send)

    def pull_and_sum(self, arena: "PeerArena") -> torch.Tensor:
        """[T, H]: every token's partial rows read from the owning ranks' arenas and added in ascending rank order."""
        from . import ops
        arena.everyone_has_written()
        if self.deferred and self._pending is not None:
            # counts still on their way to the host: offsets come from the tables the dispatch built on the device
            return ops.ep_combine_pull_dev(arena.ptrs, self.tables, self.copy_pos_cap, self.copy_off,
                                           self.send_rank_cap, self.T, arena.H, arena.buf.device)
        return ops.ep_combine_pull(arena.ptrs, self.first_row_at, self.send_off, self.copy_pos, self.copy_off,
                                   self.send_rank, self.T, arena.H, arena.buf.device)

    def sum_copies(self, rows: torch.Tensor) -> torch.Tensor:
        """[n_send, C] -> [T, C]: add a token's copies in ascending rank order (fp32 accumulate)."""
        if rows.is_cuda and rows.dtype == torch.bfloat16 and rows.shape[1] % 8 == 0:
            from . import ops
            return ops.combine(rows.contiguous(), self.copy_pos, self.copy_off, None, self.T)
        out = torch.zeros(self.T, rows.shape[1], dtype=torch.float32, device=rows.device)
        n = (self.copy_off[1:] - self.copy_off[:-1]).long()
        for j in range(int(n.max()) if self.T else 0):
            has = n > j
            out[has] += rows[self.copy_pos[(self.copy_off[:-1].long() + j)[has]].long()].float()
        return out.to(rows.dtype)


def _pack(parts):
    """[n, *] tensors of any dtype -> one uint8 [n, total bytes] (one all-to-all instead of one per tensor)."""
    return torch.cat([p.contiguous().view(torch.uint8).reshape(p.shape[0], -1) for p in parts], dim=1)


def _unpack(buf, specs):
    """Inverse of _pack; specs = [(dtype, columns)]."""
    out, at = [], 0
    for dtype, cols in specs:
        w = cols * torch.empty((), dtype=dtype).element_size()
        out.append(buf[:, at:at + w].contiguous().view(dtype).reshape(buf.shape[0], cols))
        at += w
    return out


class _Dispatch(torch.autograd.Function):
    """x [T,H], probs [T,K] -> rows received by this rank.  FP8 payload: outputs (placeholder [N,H] carrying
    the graph, probs [N,K], e4m3 bytes [N,H], raw scales [N,H/32]); bf16 payload: (x rows, probs, None, None)."""

    @staticmethod
    def forward(ctx, x, probs, plan: DispatchPlan, fp8: bool):
        ctx.plan, ctx.x_dtype = plan, x.dtype
        K, H = plan.K, x.shape[1]
        disp = getattr(plan, "disp", None)
        if fp8 and disp is not None:
            # peers fetch this rank's rows from its quantised tokens in place; this rank fetches what is addressed to it
            from . import ops
            ops.quant_rows(x.contiguous(), raw=True, out=disp.payload(0, plan.T))
            disp.publish_lists(plan, probs.detach().float())
            q_recv, raw_recv, idx_recv, p_recv = disp.pull(plan, 0, True)
            holder = torch.empty((), dtype=x.dtype, device=x.device).expand(q_recv.shape[0], H)
            ctx.mark_non_differentiable(q_recv, raw_recv, idx_recv)
            return holder, p_recv, q_recv, raw_recv, idx_recv
        # the wide payload travels as it is (no repacking copies); scales, expert ids and probabilities share
        # one narrow exchange
        tok = plan.send_tok
        meta = [plan.send_idx, probs.float()[tok]]
        if fp8:
            from . import ops
            q, raw, _ = ops.quant_rows(x.contiguous(), raw=True)
            q_recv = plan.a2a(q[tok])
            raw_recv, idx_recv, p_recv = _unpack(plan.a2a(_pack([raw[tok]] + meta)),
                                                 [(torch.uint8, H // 32), (torch.int32, K), (torch.float32, K)])
            holder = torch.empty((), dtype=x.dtype, device=x.device).expand(plan.n_recv, H)
            ctx.mark_non_differentiable(q_recv, raw_recv, idx_recv)
            return holder, p_recv, q_recv, raw_recv, idx_recv
        x_recv = plan.a2a(x[tok])
        idx_recv, p_recv = _unpack(plan.a2a(_pack(meta)), [(torch.int32, K), (torch.float32, K)])
        ctx.mark_non_differentiable(idx_recv)
        return x_recv, p_recv, None, None, idx_recv

    @staticmethod
    def backward(ctx, dx_recv, dp_recv, _dq, _draw, _didx):
        plan = ctx.plan
        dx = dp = None
        if ctx.needs_input_grad[0] and dx_recv is not None:
            arena = getattr(plan, "arena", None) if getattr(plan, "arena_backward", True) else None
            if arena is not None:       # the choice of path must not depend on this rank's data: all ranks pull
                if dx_recv.numel() and not arena.holds(dx_recv):    # normally already where the peers read it
                    arena.view(dx_recv.shape[0]).copy_(dx_recv)
                dx = plan.pull_and_sum(arena).to(ctx.x_dtype)
            else:
                # dx_recv was complete before the weight-gradient GEMMs were enqueued: the exchange waits for that
                # moment only, so those GEMMs run underneath it
                from .functional import take_result_ready
                ready = take_result_ready(dx_recv) if dx_recv.is_cuda else None
                ret = getattr(plan, "ret", None)
                # (a bound-sized buffer of a plan with deferred counts: only the rows that arrived travel back)
                if ret is not None and dx_recv.is_cuda and dx_recv.dtype == torch.bfloat16:
                    back = plan.return_by_copies(dx_recv[:plan.n_recv], ret, after=ready)
                else:
                    back = plan.a2a(dx_recv[:plan.n_recv].contiguous(), reverse=True, after=ready)
                dx = plan.sum_copies(back).to(ctx.x_dtype)
        if ctx.needs_input_grad[1] and dp_recv is not None:
            back = plan.a2a(dp_recv[:plan.n_recv].contiguous().float(), reverse=True)
            # a slot lives on exactly one rank: every other copy contributes an exact zero
            dp = torch.zeros(plan.T, plan.K, dtype=torch.float32, device=back.device).index_add_(0, plan.send_tok, back)
        return dx, dp, None, None


class _Combine(torch.autograd.Function):
    """Per-rank partial outputs [N,H] -> out [T,H] at the source.  In backward the gradient is dispatched
    (as e4m3 + scales into `handle` when given, else as bf16 rows)."""

    @staticmethod
    def forward(ctx, o_recv, plan: DispatchPlan, handle):
        ctx.plan, ctx.handle = plan, handle
        arena = getattr(plan, "arena", None)
        if arena is not None:           # the choice of path must not depend on this rank's data: all ranks pull
            if o_recv.numel() and not arena.holds(o_recv):
                arena.view(o_recv.shape[0]).copy_(o_recv)
            return plan.pull_and_sum(arena)
        return plan.sum_copies(plan.a2a(o_recv[:plan.n_recv].contiguous(), reverse=True))

    @staticmethod
    def backward(ctx, dout):
        plan, tok = ctx.plan, ctx.plan.send_tok
        dout = dout.contiguous()
        disp = getattr(plan, "disp", None)
        if ctx.handle is not None and disp is not None:
            from . import ops
            ops.quant_rows(dout.to(torch.bfloat16), raw=True, out=disp.payload(1, plan.T))
            disp.publish_lists(plan)      # a later forward of the same layer may have replaced the lists since
            q_recv, raw_recv, _, _ = disp.pull(plan, 1, False)
            ctx.handle.put(q_recv, raw_recv)
            return (torch.empty((), dtype=dout.dtype, device=dout.device).expand(q_recv.shape[0], dout.shape[1]), None,
                    None)
        if ctx.handle is not None:
            from . import ops
            q, raw, _ = ops.quant_rows(dout.to(torch.bfloat16), raw=True)
            ctx.handle.put(plan.a2a(q[tok]), plan.a2a(raw[tok]))
            return torch.empty((), dtype=dout.dtype, device=dout.device).expand(plan.n_recv, dout.shape[1]), None, None
        return plan.a2a(dout[tok]), None, None


class ExpertParallelMoE:
    """out = EP(x, topk_idx, topk_scores, w1_local, w2_local).

    `expert_fn(rows, local_idx, probs, w1, w2, fp8_scale, handle) -> [N,H]` is the per-rank expert compute; the
    default runs `run_sonic_moe` on the FP8 payload.  Tests on CPU pass `payload="bf16"` and an fp32 stand-in."""

    def __init__(self, num_experts: int, top_k: int, group=None, payload: str = "fp8", expert_fn=None,
                 capacity_tokens: int | None = None):
        """`capacity_tokens`: the largest number of tokens any rank will ever pass in one call.  With it the mapped
        buffers are allocated on the first call and every call runs without reading counts back before its return
        exchange; without it the first call reads the counts (and sizes the buffers from them) and later calls run
        read-back-free as long as no rank's token count outgrows what the first call saw (a call that does raises)."""
        self.E, self.K, self.group, self.payload = num_experts, top_k, group, payload
        self.expert_fn = expert_fn or self._sonic_experts
        self._arena = None
        self._peer_ok = USE_PEER_COMBINE and expert_fn is None      # read at construction
        self._peer_backward = PEER_COMBINE_BACKWARD
        self._place = None
        self._disp = None
        self._disp_ok = DISPATCH == "pull" and expert_fn is None and payload == "fp8"
        self._capacity = capacity_tokens
        self._ret = None
        self._ret_ok = DX_RETURN == "copy" and expert_fn is None and payload == "fp8"
        self._sync_free = SYNC_FREE and self._disp_ok and self._peer_ok
        self._plan = None

    @property
    def last_rows_received(self) -> int:
        """Rows the last call received (waits for that call's counts if they are still on their way to the host)."""
        return 0 if self._plan is None else self._plan.n_recv

    def _grp(self):
        return self.group if self.group is not None else dist.group.WORLD

    def _make_dispatch_arena(self, t_cap: int, H: int, K: int, device):
        group = self._grp()
        world = dist.get_world_size(group)
        if not self._disp_ok or device.type != "cuda" or world < 2 or H % 128 or K > 32:
            return None
        if self._disp is None or not self._disp.fits(t_cap, H, K, world):
            try:
                self._disp = DispatchArena(group, t_cap, H, K, world, device)
            except Exception as exc:      # no peer mapping on this system: every rank fails alike
                import warnings
                warnings.warn(f"expert-parallel peer-memory dispatch unavailable ({exc!r}); using NCCL all-to-all")
                self._disp_ok, self._disp = False, None
        return self._disp

    def _make_arena(self, rows: int, H: int, device):
        if not self._peer_ok or device.type != "cuda" or dist.get_world_size(self._grp()) < 2:
            return None
        if self._arena is None or self._arena.H != H or self._arena.rows < rows:
            try:
                self._arena = PeerArena(self._grp(), rows, H, device)
            except Exception as exc:      # no peer mapping on this system: every rank fails alike
                import warnings
                warnings.warn(f"expert-parallel peer-memory combine unavailable ({exc!r}); using NCCL all-to-all")
                self._peer_ok, self._arena = False, None
        return self._arena

    def _make_return_arena(self, rows: int, H: int, device):
        if not self._ret_ok or device.type != "cuda" or dist.get_world_size(self._grp()) < 2:
            return None
        if self._ret is None or self._ret.H != H or self._ret.rows < rows:
            try:
                self._ret = ReturnArena(self._grp(), rows, H, device)
            except Exception as exc:      # no peer mapping on this system: every rank fails alike
                import warnings
                warnings.warn(f"expert-parallel return by peer copies unavailable ({exc!r}); using NCCL all-to-all")
                self._ret_ok, self._ret = False, None
        return self._ret

    def _dispatch_arena_for(self, plan: DispatchPlan, H: int, device):
        """The mapped buffer the peers fetch this rank's rows from, (re)allocated collectively when the largest token
        count of any rank (known to all ranks from the plan) outgrows it."""
        return self._make_dispatch_arena(max(plan.tokens_all), H, plan.K, device)

    def _arena_for(self, plan: DispatchPlan, H: int, device):
        """The mapped buffer for this call's partial rows, (re)allocated collectively when the largest receive
        count of any rank (known to all ranks from the plan) outgrows it."""
        # world x the largest token count: every rank sending everything to one rank always fits
        world = dist.get_world_size(self._grp())
        return self._make_arena(max(plan.max_recv_rows, world * max(plan.tokens_all)), H, device)

    def _ready_without_counts(self, T: int, H: int, K: int, device) -> bool:
        """Whether this call can run on upper-bound sizes alone: both mapped buffers exist and are large enough for
        `world x capacity` rows.  The capacity is a quantity all ranks share, so all ranks decide alike; a rank whose
        own token count exceeds it cannot go on (the peers have no way to learn that in time) and raises."""
        if not self._sync_free or device.type != "cuda":
            return False
        world = dist.get_world_size(self._grp())
        if world < 2 or H % 128 or K > 32:
            return False
        if self._disp is None and self._capacity is not None:
            # first call with a stated capacity: allocate now (collective calls, same arguments on every rank)
            if self._make_dispatch_arena(self._capacity, H, K, device) is None:
                self._sync_free = False
                return False
            if self._make_arena(world * self._capacity, H, device) is None:
                self._sync_free = False
                return False
        if self._disp is None or self._arena is None:
            return False                      # first call without a capacity: sizes come from the counts
        if (H, K, world) != (self._disp.H, self._disp.K, self._disp.world) or self._arena.H != H \
                or self._arena.rows < world * self._disp.t_cap:
            return False
        if T > self._disp.t_cap:
            raise RuntimeError(f"expert-parallel layer: {T} tokens on this rank exceed the capacity of {self._disp.t_cap} "
                               "the ranks agreed on; construct ExpertParallelMoE(capacity_tokens=...) with the largest "
                               "per-rank token count, or set SONIC_MOE_EP_SYNC_FREE=0")
        return True

    def _sonic_experts(self, rows, local_idx, probs, w1, w2, fp8_scale, handle):
        from .interface import run_sonic_moe
        plan = self._plan
        if fp8_scale is not None:
            holder, qbytes = rows
            if plan is not None and plan.deferred:
                # no counts on the host yet: expert-sorted buffers at the shape-only bound, rows that did not arrive
                # are masked (-1) and cost nothing
                return run_sonic_moe(qbytes, local_idx, probs, self.K, self.El, w1, w2, fp8=True, fp8_scale=fp8_scale,
                                     fp8_combine_grad_handle=handle, sync_free_sizing=True, grad_holder=holder,
                                     out=self._place, dx_out=self._place if self._peer_backward else None)
            # the plan's count exchange already brought the routed pairs per local expert: the expert-sorted buffers
            # are sized exactly instead of at the N*K upper bound, with no further read-back
            return run_sonic_moe(qbytes, local_idx, probs, self.K, self.El, w1, w2, fp8=True, fp8_scale=fp8_scale,
                                 fp8_combine_grad_handle=handle, tokens_per_expert=self.tokens_per_local_expert,
                                 grad_holder=holder, out=self._place,
                                 dx_out=self._place if self._peer_backward else None)
        return run_sonic_moe(rows, local_idx, probs, self.K, self.El, w1, w2, fp8=True,
                             tokens_per_expert=self.tokens_per_local_expert)

    def __call__(self, x, topk_idx, topk_scores, w1, w2):
        fp8 = self.payload == "fp8"
        T, H = x.shape
        deferred = fp8 and x.is_cuda and self._ready_without_counts(T, H, topk_idx.shape[1], x.device)
        plan = DispatchPlan(topk_idx, self.E, self.group, deferred=deferred)
        self._plan = plan
        self.El = plan.El
        if deferred:
            plan.disp, arena = self._disp, self._arena
            plan.n_bound = plan.world * self._disp.t_cap
            self.tokens_per_local_expert = None
        else:
            self.tokens_per_local_expert = plan.tokens_per_local_expert
            plan.disp = self._dispatch_arena_for(plan, H, x.device) if fp8 else None
        rows, probs, q, raw, local_idx = _Dispatch.apply(x, topk_scores, plan, fp8)
        handle = None
        if fp8:
            from .functional import Fp8CombineGradHandle
            handle = Fp8CombineGradHandle()
            rows = (rows, q)
        if not deferred:
            arena = self._arena_for(plan, H, x.device) if fp8 else None
        plan.arena = arena
        plan.arena_backward = self._peer_backward
        plan.ret = None
        if fp8 and x.is_cuda and not (arena is not None and self._peer_backward):
            # where this rank's outgoing rows land when dx comes back (sized from quantities all ranks share)
            t_cap = self._disp.t_cap if deferred else max(plan.tokens_all)
            plan.ret = self._make_return_arena(t_cap * min(plan.K, plan.world), H, x.device)
        # forward output and, later, dx of the local experts land in the mapped buffer (one region, used in turn)
        n_rows = plan.n_bound if deferred else plan.n_recv
        self._place = arena.view(n_rows) if (arena is not None and n_rows > 0) else None
        o_recv = self.expert_fn(rows, local_idx, probs, w1, w2, raw, handle)
        self._place = None
        return _Combine.apply(o_recv, plan, handle)


def parity_against_single_gpu(group=None, device=None, T=1024, H=512, I=256, K=4, experts_per_rank=8, seed=200,
                              starve_last_rank=False):
    """Self-check of the expert-parallel step on the ranks of `group` (every rank calls it): each rank draws its own
    seeded tokens, the step runs expert-parallel, and every rank then pushes ALL ranks' tokens through the
    single-GPU layer with all experts local.  Returns {tensor: (cosine, relative RMS error)} of the expert-parallel
    out / dx / dscores (this rank's tokens) and dw1 / dw2 (this rank's experts, summed over all ranks' tokens)
    against that single-GPU result.  Both sides use the same quantisation points; they differ by the bf16 rounding
    of per-rank partial sums and by the column-wise re-quantisation of the FP8 payload for the weight gradients.
    `starve_last_rank` routes every token to the experts of the other ranks, so that the last rank runs the step
    with zero received rows."""
    from . import ops
    from .interface import run_sonic_moe
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    dev = torch.device(device if device is not None else torch.device("cuda", torch.cuda.current_device()))
    E = experts_per_rank * world
    if starve_last_rank and (world < 2 or (world - 1) * experts_per_rank < K):
        raise ValueError("starve_last_rank needs at least K experts outside the last rank")

    def inputs(r):
        g = torch.Generator().manual_seed(seed + r)
        x = torch.randn(T, H, generator=g).to(torch.bfloat16)
        dy = torch.randn(T, H, generator=g).to(torch.bfloat16)
        logits = torch.randn(T, E, generator=g)
        if starve_last_rank:
            logits[:, (world - 1) * experts_per_rank:] = float("-inf")
        vals, idx = logits.topk(K, dim=-1)
        return x, dy, torch.softmax(vals, -1), idx.to(torch.int32)

    gw = torch.Generator().manual_seed(seed - 1)
    w1 = (torch.randn(E, 2 * I, H, generator=gw) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=gw) * 0.02).to(torch.bfloat16)
    El, lo = experts_per_rank, rank * experts_per_rank
    x, dy, scores, idx = inputs(rank)
    xd = x.to(dev).requires_grad_(True)
    sd = scores.to(dev).requires_grad_(True)
    w1l = w1[lo:lo + El].contiguous().to(dev).requires_grad_(True)
    w2l = w2[lo:lo + El].contiguous().to(dev).requires_grad_(True)
    # a stated capacity: the mapped buffers are allocated up front and this very first call already runs without
    # reading counts back in its forward (the layer's steady-state path)
    ep = ExpertParallelMoE(E, K, group if group is not None else dist.group.WORLD, capacity_tokens=T)
    out = ep(xd, idx.to(dev), sd, w1l, w2l)
    out.backward(dy.to(dev))
    torch.cuda.synchronize(dev)
    ops.check_status(dev)
    dw1_ref = torch.zeros(El, 2 * I, H, device=dev)
    dw2_ref = torch.zeros(El, H, I, device=dev)
    mine = None
    w1a, w2a = w1.to(dev), w2.to(dev)
    for r in range(world):
        xr, dyr, sr, ir = inputs(r)
        xa = xr.to(dev).requires_grad_(True)
        sa = sr.to(dev).requires_grad_(True)
        w1g, w2g = w1a.detach().requires_grad_(True), w2a.detach().requires_grad_(True)
        o = run_sonic_moe(xa, ir.to(dev), sa, K, E, w1g, w2g, fp8=True)
        o.backward(dyr.to(dev))
        dw1_ref += w1g.grad[lo:lo + El].float()
        dw2_ref += w2g.grad[lo:lo + El].float()
        if r == rank:
            mine = (o.detach(), xa.grad, sa.grad)
    torch.cuda.synchronize(dev)
    ops.check_status(dev)

    def st(a, b):
        a, b = a.float().flatten(), b.float().flatten()
        if float(b.norm()) == 0.0:         # nothing routed to this rank's experts: both sides must be exactly zero
            return (1.0, 0.0) if float(a.norm()) == 0.0 else (0.0, float("inf"))
        return float((a * b).sum() / (a.norm() * b.norm())), float((a - b).norm() / b.norm())

    w1_grad = w1l.grad if w1l.grad is not None else torch.zeros_like(dw1_ref)
    w2_grad = w2l.grad if w2l.grad is not None else torch.zeros_like(dw2_ref)
    res = dict(out=st(out, mine[0]), dx=st(xd.grad, mine[1]), ds=st(sd.grad, mine[2]), dw1=st(w1_grad, dw1_ref),
               dw2=st(w2_grad, dw2_ref))
    res["used_peer"] = ep._arena is not None
    res["used_pull_dispatch"] = ep._disp is not None
    res["forward_without_readback"] = bool(ep._plan is not None and ep._plan.deferred)
    res["dx_returned_by_copies"] = ep._ret is not None
    res["rows_received"] = int(ep.last_rows_received)
    return res


# per-tensor limits for `parity_against_single_gpu` (cosine above, relative RMS error below)
PARITY_LIMITS = {"out": (0.999, 0.01), "dx": (0.999, 0.01), "ds": (0.999, 0.01), "dw1": (0.999, 0.04),
                 "dw2": (0.999, 0.04)}
