"""Multi-GPU plumbing for the decode path: one process per GPU over ``torch.distributed``.

Batched decode shards by sequence and needs nothing from this module (each rank owns its sequences' arena, tables and
allocator; there is no collective in the step).  A single very long context is sharded by KV range instead: rank j holds
the j-th page-aligned slice of every sequence, every rank computes a partial ``(o, m, l)`` over its slice, and one
exchange step brings the partials to the owner, which merges them.  Exchange modes:

* ``p2p`` (default): ONE launch per rank and step (``psi_gqa_attend_exchange``).  Receive slots, arrival flags and the
  consumed word live in symmetric (peer-mapped) memory on the owner; each rank's attention launch stores its partial
  straight into its slot over NVLink and publishes its flag, and the owner's launch waits for the flags with a bound and
  merges.  Slots alternate with the step's parity and a rank stores step ``s`` only once the owner has merged step
  ``s - 2``, so nothing orders the ranks' steps but the protocol itself.
* ``p2p3``: the same data path as three launches (``psi_gqa_attend_partial`` into the slot, ``psi_gqa_signal``,
  ``psi_gqa_combine_wait`` on the owner).  One slot per rank: the caller must not start step ``s + 1`` on any rank
  before the owner has merged step ``s`` (a barrier per step).  Kept for A/B measurements.
* ``nccl``: partials are all-gathered with NCCL and merged on every rank (the portable baseline).
"""
from __future__ import annotations

from . import binding as B


class KvRangeExchange:
    def __init__(self, session, rank: int, world: int, owner: int | None = None, mode: str = "p2p", max_polls: int = 0):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.session, self.rank, self.world = session, rank, world
        self.owner = world - 1 if owner is None else owner
        self.mode = mode
        self.max_polls = max_polls
        spec = session.spec
        self.tokens, self.hq, self.d = spec.num_tokens, spec.num_q_heads, spec.head_dim
        rows = self.tokens * self.hq
        self.o_elems, self.m_elems = rows * self.d, rows
        self.per_rank = self.o_elems + 2 * self.m_elems            # f32 elements of one partial: o | m | l
        self.step_id = 0
        dev = session.device
        if mode in ("p2p", "p2p3"):
            import torch.distributed._symmetric_memory as symm
            # one allocation: 2 x `world` partial slots (one set per step parity), then `world` u32 flags and the
            # consumed word (each region 16-byte aligned)
            self.slot = (self.per_rank + 3) // 4 * 4
            self.flag_words = (world + 3) // 4 * 4
            self.recv = symm.empty(2 * world * self.slot + self.flag_words + 4, dtype=torch.float32, device=dev)
            self.recv.zero_()
            self.handle = symm.rendezvous(self.recv, dist.group.WORLD)
            self.owner_view = self.handle.get_buffer(self.owner, self.recv.shape, torch.float32)
            dist.barrier()
        elif mode == "nccl":
            self.slot = self.per_rank
            self.local = torch.zeros(self.per_rank, dtype=torch.float32, device=dev)
            self.gathered = torch.zeros(world * self.per_rank, dtype=torch.float32, device=dev)
        else:
            raise ValueError(mode)

    def _views(self, buffer, index):
        base = index * self.slot
        o = buffer[base: base + self.o_elems]
        m = buffer[base + self.o_elems: base + self.o_elems + self.m_elems]
        l = buffer[base + self.o_elems + self.m_elems: base + self.per_rank]
        return o, m, l

    def _descriptor(self) -> "B.KvExchange":
        base = self.owner_view.data_ptr()
        flags = base + 4 * 2 * self.world * self.slot
        return B.KvExchange(self.rank, self.world, self.owner, self.step_id, base, self.slot, flags,
                            flags + 4 * self.flag_words, self.max_polls)

    def step(self):
        """One decode step of the KV-range-sharded layer.  The merged output lands in ``session.out`` on the owner
        (``p2p``, ``p2p3``) or on every rank (``nccl``)."""
        s = self.session
        self.step_id += 1
        if self.mode == "p2p":
            k, v = (s.k, s.v) if s.spec.do_append else (None, None)
            s.gqa.attend_exchange(s.pages, s.table, s.spec.layer, s.q, self._descriptor(),
                                  out=s.out if self.rank == self.owner else None, k=k, v=v)
            return
        if s.spec.do_append:
            s.append()
        if self.mode == "p2p3":
            o, m, l = self._views(self.owner_view, self.rank)
            s.gqa.attend_partial(s.pages, s.table, s.spec.layer, s.q, o, m, l)
            flags = self.owner_view[2 * self.world * self.slot:]
            s.gqa.signal(flags.data_ptr() + 4 * self.rank, self.step_id)
            if self.rank == self.owner:
                parts = [self._views(self.recv, r) for r in range(self.world)]
                local_flags = self.recv[2 * self.world * self.slot:]
                s.gqa.combine_wait([p[0] for p in parts], [p[1] for p in parts], [p[2] for p in parts], self.tokens,
                                   s.out, local_flags, self.step_id, self.max_polls)
        else:
            o, m, l = self._views(self.local, 0)
            s.gqa.attend_partial(s.pages, s.table, s.spec.layer, s.q, o, m, l)
            self.dist.all_gather_into_tensor(self.gathered, self.local)
            parts = [self._views(self.gathered, r) for r in range(self.world)]
            s.gqa.combine([p[0] for p in parts], [p[1] for p in parts], [p[2] for p in parts], self.tokens, s.out)

    def partials_on_owner(self):
        """Host copies of every rank's (o, m, l) of the last step as the owner received them (for checks; owner only)."""
        if self.mode == "nccl":
            source = self.gathered
        elif self.mode == "p2p":
            half = self.world * self.slot
            source = self.recv[(self.step_id & 1) * half: (self.step_id & 1) * half + half]
        else:
            source = self.recv
        out = []
        for r in range(self.world):
            o, m, l = self._views(source, r)
            out.append((o.cpu().numpy().reshape(self.tokens, self.hq, self.d), m.cpu().numpy().reshape(self.tokens, self.hq),
                        l.cpu().numpy().reshape(self.tokens, self.hq)))
        return out
