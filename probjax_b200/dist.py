"""Sequence-sharded decode: the KV cache of every sequence is split across the
ranks of a process group, each rank runs the split-KV decode on its part, and the
per-rank ``(o, lse)`` partials are exchanged with one all-gather and combined
exactly.

The reference never shards the sequence axis (probjax/nn/sharding.py:70, 97); its
single-GPU split-KV combine (probjax/nn/pallas_kernels/kernels/
attention_splitkv.py:236-250) is the same log-sum-exp algebra applied across
ranks here.

Placement is block-cyclic by pages of ``page`` tokens: page ``p`` of a sequence
lives on rank ``p % world``, compacted in order on that rank.  With ragged lengths
a contiguous split would leave the last ranks nearly empty; block-cyclic keeps
every rank within one page of ``len / world``.  Attention over a set of keys does
not depend on their order, so a rank only needs its local valid length.

The exchange is an all-gather of one fp32 record per (sequence, query head):
``Dv`` output values plus the LSE.  Records land in this rank's own memory first
and the combine kernel reads them with ordinary loads.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import attention as _att


def local_lengths(kv_lengths: torch.Tensor, rank: int, world: int, page: int) -> torch.Tensor:
    """Valid tokens rank ``rank`` holds of sequences with global ``kv_lengths``."""
    kv_lengths = kv_lengths.to(torch.int64)
    full_pages = kv_lengths // page
    tail = kv_lengths - full_pages * page
    mine_full = (full_pages - rank + world - 1) // world  # pages p < full_pages with p % world == rank
    mine_full = torch.clamp(mine_full, min=0)
    has_tail = (full_pages % world) == rank
    return (mine_full * page + torch.where(has_tail, tail, torch.zeros_like(tail))).to(torch.int32)


def local_capacity(capacity: int, rank: int, world: int, page: int) -> int:
    """Rows rank ``rank`` needs for a cache of ``capacity`` tokens."""
    return int(local_lengths(torch.tensor([capacity]), rank, world, page)[0])


def shard_cache(cache: torch.Tensor, rank: int, world: int, page: int) -> torch.Tensor:
    """The pages of ``cache [B, cap, H, D]`` that live on ``rank``, compacted."""
    B, cap, H, D = cache.shape
    idx = torch.arange(cap, device=cache.device)
    mine = idx[(idx // page) % world == rank]
    return cache.index_select(1, mine).contiguous()


def exchange_layout(B: int, Lq: int, Hq: int, Dv: int, world: int) -> dict:
    """Offsets inside one rank's exchange buffer of ``pjx_attn_decode_sharded`` (the layout
    the header documents), ``N = B * Lq * Hq`` records per rank.

    Three-launch form: ``o(parity, rank)`` / ``lse(parity, rank)`` are float32 element offsets of
    rank ``rank``'s ``[N, Dv]`` partial outputs and ``[N]`` natural-log LSEs in the half used by
    steps of that parity; ``rank_flags`` the uint32 element offset of the per-rank flags.

    One-launch form: ``ll(parity, rank)`` is the offset, in 16-byte lines, of rank ``rank``'s ``N``
    records of ``lines`` lines each: ``Dv / 2`` lines ``{o[2i], step, o[2i+1], step}`` and one line
    ``{lse, step, 0, step}`` (values as their float32 bit patterns)."""
    N = B * Lq * Hq
    half = world * N * (Dv + 1)
    head_bytes = 2 * half * 4 + (16 + 1) * 4
    uf = (head_bytes + 15) // 16 * 16
    ll = (uf + (world + 1) * N * 4 + 15) // 16 * 16
    lines = Dv // 2 + 1
    return {
        "N": N, "half": half, "lines": lines,
        "o": lambda parity, rank: parity * half + rank * N * Dv,
        "lse": lambda parity, rank: parity * half + world * N * Dv + rank * N,
        "rank_flags": 2 * half, "unit_counters": uf // 4 + world * N,
        "ll": lambda parity, rank: ll // 16 + (parity * world + rank) * N * lines,
        "bytes": ll + 2 * world * N * lines * 16,
    }


def ll_records(o: torch.Tensor, lse: torch.Tensor, step: int) -> torch.Tensor:
    """``[N, Dv]`` float32 partial outputs and ``[N]`` LSEs as the int32 ``[N, Dv / 2 + 1, 4]`` lines of
    the one-launch exchange for step ``step`` (what a rank's kernel stores into its peers)."""
    N, Dv = o.shape
    rec = torch.full((N, Dv // 2 + 1, 4), int(step), dtype=torch.int32, device=o.device)
    bits = o.contiguous().view(torch.int32).view(N, Dv // 2, 2)
    rec[:, : Dv // 2, 0] = bits[:, :, 0]
    rec[:, : Dv // 2, 2] = bits[:, :, 1]
    rec[:, Dv // 2, 0] = lse.contiguous().view(torch.int32)
    rec[:, Dv // 2, 2] = 0
    return rec


def decode_sharded(q, k_local, v_local, kv_lengths, *, page: int, sm_scale: float, group=None,
                   return_lse: bool = False, _local_fn=None, _combine_fn=None):
    """Decode step with the KV sequence split across ``group``.

    ``q [B, Lq, Hq, D]`` is replicated; ``k_local`` / ``v_local`` are this rank's
    shards (:func:`shard_cache`); ``kv_lengths [B]`` are the *global* valid
    lengths (pass them on ``q``'s device to keep the call free of host copies).  Every rank returns the full result ``[B, Lq, Hq, Dv]`` in
    ``q.dtype`` (and the natural-log LSE ``[B, Hq, Lq]``).

    ``_local_fn`` / ``_combine_fn`` replace the two kernel calls; they exist so the
    exchange and the partition arithmetic can be exercised on CPU ranks.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    lens = local_lengths(torch.as_tensor(kv_lengths), rank, world, page).to(q.device)
    local_fn = _local_fn or (lambda q_, k_, v_, l_: _att.decode_forward(
        q_, k_, v_, kv_lengths=l_, sm_scale=sm_scale, return_lse=True, partial_f32=True))
    combine_fn = _combine_fn or (lambda o_, l_: _att.combine_partials(o_, l_, out_dtype=q.dtype))
    o_loc, lse_loc = local_fn(q, k_local, v_local, lens)  # [B,Lq,Hq,Dv] fp32, [B,Hq,Lq]
    B, Lq, Hq, Dv = o_loc.shape
    # one record per (b, t, h): Dv outputs + the LSE, rows in [B, Lq, Hq] order
    rec = torch.empty((B, Lq, Hq, Dv + 1), dtype=torch.float32, device=o_loc.device)
    rec[..., :Dv] = o_loc
    rec[..., Dv] = lse_loc.permute(0, 2, 1)
    if world > 1:
        gathered = torch.empty((world,) + tuple(rec.shape), dtype=torch.float32, device=rec.device)
        dist.all_gather([gathered[r] for r in range(world)], rec, group=group)
    else:
        gathered = rec[None]
    n = B * Lq * Hq
    o_parts = gathered[..., :Dv].reshape(world, n, Dv)
    lse_parts = gathered[..., Dv].reshape(world, n)
    o, lse = combine_fn(o_parts, lse_parts)
    o = o.reshape(B, Lq, Hq, Dv)
    if return_lse:
        return o, lse.reshape(B, Lq, Hq).permute(0, 2, 1).contiguous()
    return o


class ShardedDecoder:
    """Repeated decode steps over one sequence-sharded cache with every buffer
    allocated once: the local split-KV decode writes its fp32 partial and LSE, two
    ``all_gather_into_tensor`` calls land all ranks' partials in local memory, and the
    combine kernel writes the result.  With ``use_graph`` the four launches of a
    step are captured in one CUDA graph (a decode step is a few tens of
    microseconds, so launch overhead matters).

    ``kv_lengths`` are the global valid lengths; call :meth:`set_lengths` when they
    change.  ``q`` is read from the tensor passed at construction (copy new queries
    into ``decoder.q``).
    """

    def __init__(self, q, k_local, v_local, kv_lengths, *, page: int, sm_scale: float, group=None,
                 use_graph: bool = False):
        from . import _lib

        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.page, self.sm_scale = page, float(sm_scale)
        self.q, self.k, self.v = q.contiguous(), k_local.contiguous(), v_local.contiguous()
        dev = q.device
        B, Lq, Hq, D = q.shape
        self.cap, Hkv, Dv = self.k.shape[1], self.k.shape[2], self.v.shape[3]
        self.shape = (B, Lq, Hq, Hkv, D, Dv)
        n = B * Lq * Hq
        self.o_loc = torch.empty((n, Dv), dtype=torch.float32, device=dev)
        self.lse_loc = torch.empty((B, Hq, Lq), dtype=torch.float32, device=dev)
        self.o_all = torch.empty((self.world, n, Dv), dtype=torch.float32, device=dev)
        self.lse_all = torch.empty((self.world, n), dtype=torch.float32, device=dev)
        self.out = torch.empty((B, Lq, Hq, Dv), dtype=q.dtype, device=dev)
        self.lse = torch.empty((n,), dtype=torch.float32, device=dev)
        self.lens = torch.empty((B,), dtype=torch.int32, device=dev)
        self.set_lengths(kv_lengths)
        L = _lib.lib()
        need = L.pjx_attn_decode_workspace_bytes(B, Lq, Hq, Hkv, Dv, self.cap, 0)
        self.ws = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
        self._L, self._dt = L, _att._DTYPES[q.dtype]
        self.graph = None
        if use_graph:
            self._capture()

    def set_lengths(self, kv_lengths):
        self.lens.copy_(local_lengths(torch.as_tensor(kv_lengths), self.rank, self.world, self.page))

    def _step(self):
        from . import _lib

        B, Lq, Hq, Hkv, D, Dv = self.shape
        dev = self.q.device
        stream = torch.cuda.current_stream(dev).cuda_stream
        rc = self._L.pjx_attn_decode_splitkv(
            self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.lens.data_ptr(), self.o_loc.data_ptr(),
            self.lse_loc.data_ptr(), B, Lq, Hq, Hkv, D, Dv, self.cap, self._dt, self.sm_scale, 0, 1,
            self.ws.data_ptr(), self.ws.numel(), stream)
        _lib.check(rc)
        lse_rows = self.lse_loc.reshape(-1) if Lq == 1 else self.lse_loc.permute(0, 2, 1).reshape(-1)
        if self.world > 1:
            dist.all_gather_into_tensor(self.o_all.view(-1), self.o_loc.view(-1), group=self.group)
            dist.all_gather_into_tensor(self.lse_all.view(-1), lse_rows.contiguous(), group=self.group)
        else:
            self.o_all[0].copy_(self.o_loc)
            self.lse_all[0].copy_(lse_rows)
        rc = self._L.pjx_attn_combine(self.o_all.data_ptr(), self.lse_all.data_ptr(), self.world, B * Lq * Hq, Dv,
                                      self.out.data_ptr(), self.lse.data_ptr(), self._dt, stream)
        _lib.check(rc)

    def _capture(self):
        side = torch.cuda.Stream(self.q.device)
        side.wait_stream(torch.cuda.current_stream(self.q.device))
        with torch.cuda.stream(side):
            for _ in range(3):
                self._step()
        torch.cuda.current_stream(self.q.device).wait_stream(side)
        torch.cuda.synchronize(self.q.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._step()
        self.graph = graph

    def __call__(self, return_lse: bool = False):
        if self.graph is not None:
            self.graph.replay()
        else:
            self._step()
        if return_lse:
            B, Lq, Hq = self.shape[:3]
            return self.out, self.lse.reshape(B, Lq, Hq).permute(0, 2, 1)
        return self.out


class FusedShardedDecoder:
    """Sequence-sharded decode whose exchange is done by the kernels themselves
    (``pjx_attn_decode_sharded``): peer stores over NVLink into every rank's
    exchange buffer plus a flag, no library collective on the data path.  The
    exchange buffers are one torch symmetric-memory allocation per rank, mapped
    into every process of ``group``.

    One process per GPU; every rank must construct the decoder and call it the same
    number of times.  ``decoder.q`` holds the queries of the step.
    """

    def __init__(self, q, k_local, v_local, kv_lengths, *, page: int, sm_scale: float, group=None,
                 block_table=None, overlap_steps: bool = False):
        """``overlap_steps``: consecutive calls are issued back to back on one stream and nothing
        between them writes ``q``, the caches or the lengths (``PJX_DECODE_OVERLAP_PREVIOUS``): a step
        then streams its cache while the previous step's exchange is still draining.

        ``block_table`` (``int32 [B, max_pages]``) switches to a paged local cache: ``k_local`` /
        ``v_local`` are then page pools ``[num_pages, page_size, Hkv, D]`` and row ``b`` of the table
        names, in order, the pool pages that hold this rank's share of sequence ``b`` (the pool page
        size is the cache's own and must be a multiple of 64; ``page`` stays the sharding granule)."""
        import ctypes

        from . import _lib

        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.page, self.sm_scale = page, float(sm_scale)
        self.flags = 1 if overlap_steps else 0
        self.q, self.k, self.v = q.contiguous(), k_local.contiguous(), v_local.contiguous()
        dev = q.device
        B, Lq, Hq, D = q.shape
        self.block_table = None
        if block_table is not None:
            self.block_table = torch.as_tensor(block_table).to(device=dev, dtype=torch.int32).contiguous()
            if self.block_table.dim() != 2 or self.block_table.shape[0] != B:
                raise ValueError(f"block_table must be [B={B}, max_pages], got {tuple(self.block_table.shape)}")
            self.pool_page = self.k.shape[1]
        self.cap = self.k.shape[1] if block_table is None else self.block_table.shape[1] * self.k.shape[1]
        Hkv, Dv = self.k.shape[2], self.v.shape[3]
        self.shape = (B, Lq, Hq, Hkv, D, Dv)
        self.out = torch.empty((B, Lq, Hq, Dv), dtype=q.dtype, device=dev)
        self.lse = torch.empty((B, Hq, Lq), dtype=torch.float32, device=dev)
        self.lens = torch.empty((B,), dtype=torch.int32, device=dev)
        self.set_lengths(kv_lengths)
        L = _lib.lib()
        self.ws = torch.empty(max(L.pjx_attn_decode_workspace_bytes(B, Lq, Hq, Hkv, Dv, self.cap, 0), 256),
                              dtype=torch.uint8, device=dev)
        nbytes = L.pjx_attn_decode_sharded_buffer_bytes(B, Lq, Hq, Dv, self.world)
        if nbytes == 0:
            raise ValueError(f"unsupported exchange geometry (world={self.world})")
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm

            self.xbuf = symm.empty(nbytes, dtype=torch.uint8, device=dev)
            self.xbuf.zero_()
            torch.cuda.synchronize(dev)
            self._handle = symm.rendezvous(self.xbuf, group if group is not None else dist.group.WORLD)
            ptrs = [int(x) for x in self._handle.buffer_ptrs]
            dist.barrier(group)  # every rank has zeroed its flags before anyone publishes
        else:
            self.xbuf = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
            ptrs = [self.xbuf.data_ptr()]
        self._ptrs = (ctypes.c_void_p * self.world)(*ptrs)
        self._status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._L, self._dt, self.step = L, _att._DTYPES[q.dtype], 0

    def set_lengths(self, kv_lengths):
        self.lens.copy_(local_lengths(torch.as_tensor(kv_lengths), self.rank, self.world, self.page))

    def __call__(self, return_lse: bool = False):
        from . import _lib

        B, Lq, Hq, Hkv, D, Dv = self.shape
        self.step += 1
        stream = torch.cuda.current_stream(self.q.device).cuda_stream
        if self.block_table is not None:
            rc = self._L.pjx_attn_decode_sharded_paged(
                self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.block_table.data_ptr(),
                self.lens.data_ptr(), self.out.data_ptr(), self.lse.data_ptr(), B, Lq, Hq, Hkv, D, Dv, self.pool_page,
                self.block_table.shape[1], self._dt, self.sm_scale, 0, self.ws.data_ptr(), self.ws.numel(), self.rank,
                self.world, self._ptrs, self.step, self.flags, self._status.data_ptr(), stream)
        else:
            rc = self._L.pjx_attn_decode_sharded(
                self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.lens.data_ptr(), self.out.data_ptr(),
                self.lse.data_ptr(), B, Lq, Hq, Hkv, D, Dv, self.cap, self._dt, self.sm_scale, 0,
                self.ws.data_ptr(), self.ws.numel(), self.rank, self.world, self._ptrs, self.step, self.flags,
                self._status.data_ptr(), stream)
        _lib.check(rc)
        return (self.out, self.lse) if return_lse else self.out

    def check_status(self):
        """Synchronise and raise if a wait on a peer's flag expired."""
        from . import _lib

        rc = self._L.pjx_read_status(self._status.data_ptr(), torch.cuda.current_stream(self.q.device).cuda_stream)
        if rc:
            self._status.zero_()
        _lib.check(rc)
