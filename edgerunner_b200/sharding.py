"""Multi-GPU partitioning of the decode path (one process per GPU, torch.distributed for the plumbing).

Attention is independent per (sequence, kv-head group, layer), so the path shards without any reduction:

* by sequence   -- rank r owns sequences [r*B/G, (r+1)*B/G): no communication at all;
* by kv head    -- rank r owns kv heads [r*Hkv/G, (r+1)*Hkv/G) and the q heads that attend to them; its cache
                   holds only those heads.  Per layer batch the ranks exchange their [B, Hq/G, 128] output
                   slices with one all-gather (NCCL over NVLink on GPUs, gloo in the CPU tests).

The reference is single-device (no collective call sites anywhere), so this module has no counterpart there.
"""
import torch
import torch.distributed as dist


def split_range(total, world, rank):
    """Contiguous, balanced [begin, end) of `total` items for `rank` of `world`."""
    base, rem = divmod(int(total), int(world))
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


class HeadShard:
    """kv-head sharding: which kv heads / q heads a rank owns."""

    def __init__(self, num_heads, num_kv_heads, world, rank):
        if num_kv_heads % world:
            raise ValueError("num_kv_heads %d is not divisible by world size %d" % (num_kv_heads, world))
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.group = num_heads // num_kv_heads
        self.world, self.rank = world, rank
        self.kv_begin, self.kv_end = split_range(num_kv_heads, world, rank)
        self.q_begin, self.q_end = self.kv_begin * self.group, self.kv_end * self.group
        self.local_kv_heads = self.kv_end - self.kv_begin
        self.local_heads = self.q_end - self.q_begin

    def slice_q(self, q):
        """q: [..., num_heads, head_dim] -> this rank's heads."""
        return q[..., self.q_begin:self.q_end, :]

    def slice_kv(self, kv):
        return kv[..., self.kv_begin:self.kv_end, :]


def all_gather_heads(local_out, group=None):
    """local_out: [..., local_heads, head_dim] (same shape on every rank) -> [..., world*local_heads, head_dim],
    rank slices concatenated along the head axis in rank order."""
    world = dist.get_world_size(group)
    if world == 1:
        return local_out
    local_out = local_out.contiguous()
    parts = [torch.empty_like(local_out) for _ in range(world)]
    dist.all_gather(parts, local_out, group=group)
    return torch.cat(parts, dim=-2)


def max_over_ranks(value, device=None, group=None):
    """Max of a python float over ranks (used for device-timed benchmark durations)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


class _DeviceSpan:
    """A raw device allocation dressed for torch.as_tensor (CUDA array interface), float32."""

    def __init__(self, ptr, shape):
        self.__cuda_array_interface__ = {"shape": tuple(int(x) for x in shape), "typestr": "<f4", "data": (int(ptr), False),
                                         "version": 2, "strides": None}


class HeadShardedDecoder:
    """One rank's side of a decode stack whose kv heads are split over the ranks of a node.

    The rank's `cache` holds `shard.local_kv_heads` kv heads; `step` appends one token per sequence, runs attention for
    the rank's query heads and leaves every rank holding the outputs of ALL heads as `[layers, batch, num_heads, 128]`:

    * exchange "p2p"  -- the decode kernel's merge epilogue stores each finished row into that buffer on this GPU and, by
      plain peer stores, on every other GPU (buffers shared through CUDA IPC, er_peer_buffer_*); a 4-byte all-reduce
      enqueued behind the launch is the only collective (it orders "all ranks' launches are complete");
    * exchange "nccl" -- each rank computes its slice, one NCCL all-gather, one re-layout kernel.  Used when the IPC
      mapping is refused, and as the plain-library baseline of the fused path.

    world == 1 degenerates to an ordinary decode step.
    """

    def __init__(self, cache, layers, batch, num_heads, num_kv_heads, world, rank, exchange="p2p", group=None):
        import ctypes as C
        from ._lib import check, lib
        self.cache, self.layers, self.batch = cache, layers, batch
        self.num_heads, self.world, self.rank, self.group = num_heads, world, rank, group
        self.shard = HeadShard(num_heads, num_kv_heads, world, rank)
        self._own_ptr, self._opened = None, []
        self._host_full, self._with_self, self.host_rows = None, None, None
        self.exchange = "none" if world == 1 else exchange
        dev = torch.device("cuda", torch.cuda.current_device())
        nfull = layers * batch * num_heads * 128
        if self.exchange == "p2p":
            own, handle = C.c_void_p(), (C.c_uint8 * 64)()
            ok = lib().er_peer_buffer_create(nfull * 4, C.byref(own), handle) == 0
            handles = [None] * world
            dist.all_gather_object(handles, bytes(handle) if ok else None, group=group)
            peers = []
            if ok and all(h is not None for h in handles):
                for r, h in enumerate(handles):
                    if r == rank:
                        continue
                    p = C.c_void_p()
                    if lib().er_peer_buffer_open((C.c_uint8 * 64).from_buffer_copy(h), C.byref(p)) != 0:
                        ok = False
                        break
                    peers.append(p.value)
                    self._opened.append(p.value)
            else:
                ok = False
            agree = torch.tensor([1 if ok else 0], device=dev)
            dist.all_reduce(agree, op=dist.ReduceOp.MIN, group=group)
            self._own_ptr = own.value
            if int(agree.item()) == 1:
                self.full = torch.as_tensor(_DeviceSpan(own.value, (layers, batch, num_heads, 128)), device=dev)
                self._peer_array = (C.c_void_p * max(len(peers), 1))(*peers)
                self._num_peers = len(peers)
                self._flag = torch.zeros(1, device=dev)
                self._set_sharding(True)
            else:
                self.p2p_refused = lib().er_last_error_string().decode()
                self._release_peer_buffers()
                self.exchange = "nccl"
        if self.exchange == "nccl":
            hl = self.shard.local_heads
            self.out_local = torch.empty((layers, batch, hl, 128), device=dev)
            self.gathered = torch.empty((world, layers, batch, hl, 128), device=dev)
            self.full = torch.empty((layers, batch, num_heads, 128), device=dev)
        elif self.exchange == "none":
            self.full = torch.empty((layers, batch, num_heads, 128), device=dev)

    def _set_sharding(self, with_peers):
        from ._lib import check, lib
        check(lib().er_kv_set_output_sharding(self.cache.handle, self.num_heads, self.shard.q_begin, self._peer_array,
                                              self._num_peers if with_peers else 0))

    def step(self, q_local, k_local, v_local, params, stream=None, exchange=True):
        """q_local: [layers, batch, local_heads, 128]; k_local / v_local: [layers, batch, local_kv_heads, 128] (this rank's
        heads).  Returns the [layers, batch, num_heads, 128] outputs (valid on `stream` after the call's work).
        exchange=False runs the rank's own compute only (timing the exchange's share)."""
        from ._lib import check, lib, ptr, stream_ptr
        hl = self.shard.local_heads
        if self.exchange == "nccl":
            self.cache.decode_step(q_local, k_local, v_local, self.out_local, hl, params, stream=stream)
            if exchange:
                dist.all_gather_into_tensor(self.gathered, self.out_local, group=self.group)
                check(lib().er_relayout_head_shards(ptr(self.gathered), ptr(self.full), self.world, self.layers * self.batch, hl,
                                                    stream_ptr(stream)))
        elif self.exchange == "p2p":
            self.cache.decode_step(q_local, k_local, v_local, self.full, hl, params, stream=stream)
            if exchange:
                dist.all_reduce(self._flag, group=self.group)      # "every rank's launch, and with it its peer stores, is complete"
        else:
            self.cache.decode_step(q_local, k_local, v_local, self.full, hl, params, stream=stream)
        return self.full

    def step_host(self, hq_local, hk_local, hv_local, hout_local, params, stream=None):
        """The same step from pinned host memory: this rank's q / k / v slices come straight out of `hq_local`, `hk_local`,
        `hv_local` (the decode kernel pulls the rows itself on float16 caches), the exchange runs on the device, and the rank's
        own heads `[layers, batch, local_heads, 128]` land in the pinned `hout_local` -- the ranks' host buffers together hold
        the step's result once (`hout_local` may be None: `self.host_rows` then names the rows where they are).  Returns the device
        tensor of all heads (valid on the stream after the exchange).

        p2p exchange: the launch writes its rows to a pinned full-width host buffer (`out`), to its own device buffer and to the
        peers' (all as "peer" addresses), and reports to a host word, so the call returns as soon as the rank's own rows are in
        host memory -- no device-to-host copy, no stream synchronisation; the 4-byte all-reduce that orders the peers' stores
        stays on the stream for the device-side consumers."""
        hl = self.shard.local_heads
        if self.exchange == "p2p":
            import ctypes as C
            from ._lib import check, lib
            if self._host_full is None:
                self._host_full = torch.empty((self.layers, self.batch, self.num_heads, 128), dtype=torch.float32).pin_memory()
                ptrs = [self._peer_array[i] for i in range(self._num_peers)] + [self._own_ptr]
                self._with_self = (C.c_void_p * len(ptrs))(*ptrs)
            check(lib().er_kv_set_output_sharding(self.cache.handle, self.num_heads, self.shard.q_begin, self._with_self, self._num_peers + 1))
            try:
                self.cache.decode_step_host(hq_local, hk_local, hv_local, self._host_full, hl, params, stream=stream)
            finally:
                self._set_sharding(True)
            dist.all_reduce(self._flag, group=self.group)
            self.host_rows = self._host_full[:, :, self.shard.q_begin:self.shard.q_end]     # the rank's heads, in place
            if hout_local is not None:
                hout_local.copy_(self.host_rows)      # host to host, for callers that want them contiguous
            return self.full
        target = self.out_local if self.exchange == "nccl" else self.full
        self.cache.decode_step_host(hq_local, hk_local, hv_local, target, hl, params, stream=stream)
        if self.exchange == "nccl":
            from ._lib import check, lib, ptr, stream_ptr
            dist.all_gather_into_tensor(self.gathered, self.out_local, group=self.group)
            check(lib().er_relayout_head_shards(ptr(self.gathered), ptr(self.full), self.world, self.layers * self.batch, hl,
                                                stream_ptr(stream)))
            hout_local.copy_(self.out_local, non_blocking=True)
        else:
            hout_local.copy_(self.full, non_blocking=True)
        (stream if stream is not None and not isinstance(stream, int) else torch.cuda.current_stream()).synchronize()
        self.host_rows = hout_local
        return self.full

    def set_peer_stores(self, enabled):
        """p2p exchange only: drop / restore the peer stores (the rank then fills its own buffer only)."""
        if self.exchange == "p2p":
            self._set_sharding(bool(enabled))

    def _release_peer_buffers(self):
        from ._lib import lib
        for p in self._opened:
            lib().er_peer_buffer_close(p)
        self._opened = []
        if dist.is_initialized() and self.world > 1:
            dist.barrier(group=self.group)          # nobody frees a buffer a peer still has mapped
        if self._own_ptr:
            lib().er_peer_buffer_destroy(self._own_ptr)
            self._own_ptr = None

    def close(self):
        if self.exchange == "p2p":
            from ._lib import lib
            torch.cuda.synchronize()
            lib().er_kv_set_output_sharding(self.cache.handle, 0, 0, None, 0)
            self.full = None
            self._release_peer_buffers()
            self.exchange = "closed"


def head_sharded_reference(er, make_cache, fill_cache, q, k, v, params, world, steps=1):
    """All `world` shards of a kv-head-sharded decode computed one after the other on THIS GPU (one cache per shard, the
    same shapes and therefore the same CTA work split as the real ranks) and concatenated: what the exchange must deliver,
    bit for bit.  make_cache(local_kv_heads) -> KVCache; fill_cache(cache, shard); q: [steps, L, B, H, 128],
    k / v: [steps, L, B, Hkv, 128] device tensors.  Returns [steps, L, B, H, 128]."""
    S, L, B, H, _ = q.shape
    Hkv = k.shape[3]
    outs = torch.empty_like(q)
    for r in range(world):
        shard = HeadShard(H, Hkv, world, r)
        cache = make_cache(shard.local_kv_heads)
        fill_cache(cache, shard)
        o = torch.empty((L, B, shard.local_heads, 128), device=q.device)
        for s in range(S):
            cache.decode_step(shard.slice_q(q[s]).contiguous(), shard.slice_kv(k[s]).contiguous(), shard.slice_kv(v[s]).contiguous(),
                              o, shard.local_heads, params)
            outs[s, :, :, shard.q_begin:shard.q_end] = o
        torch.cuda.synchronize()
        cache.close()
    return outs


def small_paged_case(er, seed=3, layers=2, batch=5, num_heads=32, num_kv_heads=8, lo=40, hi=400, page_size=16, steps=2, theta=5.0e5):
    """A Llama-3.1-8B-shaped (32 query / 8 kv heads) ragged batch in 16-token pages with a seeded random block table, small
    enough for a CPU check: returns a dict with the inputs (numpy / torch, identical on every rank) and two callbacks,
    make_cache(local_kv_heads) and fill_cache(cache, shard), that build and pre-fill a cache holding a kv-head slice."""
    import numpy as np
    rng = np.random.Generator(np.random.PCG64(seed))
    lens = [int(x) for x in rng.integers(lo, hi + 1, size=batch)]
    cap = (max(lens) + steps + 15) // 16 * 16
    pages = sum((n + steps + page_size - 1) // page_size for n in lens)
    order = rng.permutation(pages)

    def f16(shape):
        return rng.standard_normal(shape, dtype=np.float32).astype(np.float16).astype(np.float32)

    k0 = [[f16((n, num_kv_heads, 128)) for n in lens] for _ in range(layers)]
    v0 = [[f16((n, num_kv_heads, 128)) for n in lens] for _ in range(layers)]
    q = torch.as_tensor(f16((steps, layers, batch, num_heads, 128))).cuda()
    k = torch.as_tensor(f16((steps, layers, batch, num_kv_heads, 128))).cuda()
    v = torch.as_tensor(f16((steps, layers, batch, num_kv_heads, 128))).cuda()
    params = er.step_params(rope_theta=theta)

    def make_cache(local_kv_heads):
        # the persistent kernel on both sides of a comparison: launches that write sharded rows always use it, and a
        # bit-for-bit check needs the same summation order
        c = er.KVCache(cap, layers, local_kv_heads, 128, er.Precision.float16, max_batch=batch, layout=er.Layout.paged,
                       page_size=page_size, num_pages=pages, decode_kernel=1)
        alloc = er.BlockTableAllocator(pages, page_size, free_order=order)
        for b, n in enumerate(lens):
            c.set_block_table(b, alloc.ensure(b, n + steps))
        return c

    def fill_cache(cache, shard):
        for l in range(layers):
            for b, n in enumerate(lens):
                cache.write_rows(l, b, 0, n, torch.as_tensor(np.ascontiguousarray(k0[l][b][:, shard.kv_begin:shard.kv_end])).cuda(),
                                 torch.as_tensor(np.ascontiguousarray(v0[l][b][:, shard.kv_begin:shard.kv_end])).cuda(), params)
        torch.cuda.synchronize()

    return dict(lens=lens, k0=k0, v0=v0, q=q, k=k, v=v, params=params, make_cache=make_cache, fill_cache=fill_cache,
                layers=layers, batch=batch, num_heads=num_heads, num_kv_heads=num_kv_heads, steps=steps, theta=theta)


def verify_exchange(er, world, rank, exchange, group=None):
    """Runs the small paged case through HeadShardedDecoder on `world` ranks and checks, on every rank, that the exchanged
    [layers, batch, heads, 128] outputs equal -- bit for bit -- the shards computed one after the other on this rank's own
    GPU (head_sharded_reference).  Returns the exchange actually used ("p2p" may fall back to "nccl")."""
    case = small_paged_case(er)
    want = head_sharded_reference(er, case["make_cache"], case["fill_cache"], case["q"], case["k"], case["v"], case["params"], world,
                                  steps=case["steps"])
    shard = HeadShard(case["num_heads"], case["num_kv_heads"], world, rank)
    cache = case["make_cache"](shard.local_kv_heads)
    case["fill_cache"](cache, shard)
    dec = HeadShardedDecoder(cache, case["layers"], case["batch"], case["num_heads"], case["num_kv_heads"], world, rank, exchange, group)
    used = dec.exchange
    for s in range(case["steps"]):
        ql, kl, vl = (shard.slice_q(case["q"][s]).contiguous(), shard.slice_kv(case["k"][s]).contiguous(),
                      shard.slice_kv(case["v"][s]).contiguous())
        if s + 1 < case["steps"]:
            full = dec.step(ql, kl, vl, case["params"])
        else:   # the last step from pinned host memory: same rows on the device, the rank's own heads on the host
            hq, hk, hv = (x.cpu().pin_memory() for x in (ql, kl, vl))
            hout = torch.empty(ql.shape, dtype=torch.float32).pin_memory()
            full = dec.step_host(hq, hk, hv, hout, case["params"])
            if not torch.equal(hout, want[s][:, :, shard.q_begin:shard.q_end].cpu()):
                raise AssertionError("rank %d: host rows of step_host (%s) differ from the per-shard reference" % (rank, used))
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=group)
        if not torch.equal(full, want[s]):
            bad = (full != want[s]).nonzero()
            raise AssertionError("rank %d: exchanged outputs (%s) differ from the per-shard reference at step %d, first index %s" %
                                 (rank, used, s, bad[0].tolist()))
        if world > 1:
            dist.barrier(group=group)      # nobody starts the next step (and overwrites a peer's buffer) while a rank still compares
    assert cache.device_status() == 0
    dec.close()
    cache.close()
    return used
