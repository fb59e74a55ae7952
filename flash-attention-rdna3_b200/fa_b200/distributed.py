"""Multi-GPU use of the attention path: one process per GPU, ``torch.distributed`` for the plumbing.

The reference is single-GPU (no communication code anywhere in fa_rdna3); two modes are added here.

1. Batch x head partition (dense, varlen, decode): every (batch, kv-head group) is independent, so ranks
   take disjoint slices and nothing is exchanged. :func:`partition_batch_heads` gives the slices.

2. KV-sharded long-context paged decode: rank r owns the pages of logical blocks r, r + G, r + 2G, ...
   of every sequence (block-cyclic, so ragged context lengths stay balanced), holds the whole query, runs
   the paged kernel over its blocks only and produces a partial ``(O_r fp32, LSE_r)``, written by the kernel
   straight into this rank's slot of the gather buffer. One in-place all-gather of ``batch * heads *
   (head_dim + 1)`` floats per rank brings the partials into local memory and the LSE-weighted merge
   (``fa_combine``, the rule of fa_rdna3/kernels/decode.py:101-122) reads the gathered slots where they lie, on
   every rank: two kernels of the local decode, one collective, one merge kernel, no copies in between.
   Shards without keys contribute ``LSE = -inf`` and are ignored by the merge.

The collective only ever reads local memory: partials are gathered by NCCL first and merged afterwards.

Between the GPUs of one node the gather needs no collective at all (`transport="push"`, the default where it can be
set up): every rank keeps its gather buffer in memory that the other ranks have mapped through CUDA IPC, the local
kernels write this rank's partial into its own slot, and `fa_peer_merge` copies that slot into every peer's buffer with
ordinary stores over NVLink, raises a flag there, waits (bounded) for the peers' flags on its own buffer and merges.
Only stores cross the link, nothing reads peer memory, no TMA or multicast instruction is involved. Two buffers
alternate between calls so that a fast rank cannot overwrite a slot a slow rank is still merging.
"""
import ctypes as C
import math

import torch

from . import _lib
from .interface import (_DTYPE_CODE, _paged_balanced_slots, _paged_launch, _paged_splits_b200,
                        _paged_tensor_core_ok, _status_word, _stream)
from ._validation import validate_inference_only, validate_paged_inputs, validate_softmax_scale


def partition_batch_heads(batch, kv_heads, world_size, rank):
    """Contiguous range [start, stop) of flattened (batch, kv_head) groups owned by `rank`.

    Groups are dealt as evenly as possible; the first ``total % world_size`` ranks get one extra."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError("rank must satisfy 0 <= rank < world_size")
    total = batch * kv_heads
    base, extra = divmod(total, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_dense_by_heads(query, key, value, world_size, rank):
    """Slices of (batch, heads, seq, dim) tensors for `rank` when the partition falls on whole kv heads of
    every batch entry (kv_heads % world_size == 0): returns (q, k, v) views, no copies."""
    kv_heads = key.shape[1]
    if kv_heads % world_size != 0:
        raise ValueError("kv heads must divide evenly over the ranks for a head-sliced view")
    per = kv_heads // world_size
    group = query.shape[1] // kv_heads
    ks = slice(rank * per, (rank + 1) * per)
    qs = slice(rank * per * group, (rank + 1) * per * group)
    return query[:, qs], key[:, ks], value[:, ks]


def _merge_partials_cuda(gathered_o, gathered_lse, out_dtype):
    """gathered_o (G, rows, D) fp32, gathered_lse (G, rows) fp32 on the GPU; rows and the D elements of a row are
    contiguous, the stride between shards is free (the two may be views of one gather buffer)."""
    lib = _lib.load()
    G, rows, D = gathered_o.shape
    out = torch.empty(rows, D, dtype=out_dtype, device=gathered_o.device)
    p = _lib.CombineParams()
    p.out_dtype, p.rows, p.head_dim, p.num_splits = _DTYPE_CODE[out_dtype], rows, D, G
    p.o_partial, p.o_split_stride, p.o_row_stride = gathered_o.data_ptr(), gathered_o.stride(0), gathered_o.stride(1)
    p.lse_partial, p.lse_split_stride, p.lse_row_stride = (gathered_lse.data_ptr(), gathered_lse.stride(0),
                                                           gathered_lse.stride(1))
    p.out, p.out_row_stride = out.data_ptr(), D
    with torch.cuda.device(out.device):
        _lib.check(lib.fa_combine(C.byref(p), _stream(out.device)))
    return out


def _gather_buffer(world, rows, head_dim, device):
    """One buffer for the all-gather: shard r's slot holds its (rows, head_dim) partial followed by its rows LSEs,
    padded to a multiple of four floats so that every slot starts 16-byte aligned. Returns (flat, o, lse) where o is
    the (world, rows, head_dim) view and lse the (world, rows) view of the same memory."""
    slot = -(-(rows * (head_dim + 1)) // 4) * 4
    flat = torch.empty((world, slot), dtype=torch.float32, device=device)
    o = flat[:, :rows * head_dim].view(world, rows, head_dim)
    lse = flat[:, rows * head_dim:rows * (head_dim + 1)]
    return flat, o, lse


class _PeerGather:
    """Gather buffers of all ranks of `group` for partials of (rows, head_dim), mapped into this process: two sets of
    `world` slots and `world` flags per rank, in one allocation per rank that the others open through CUDA IPC."""

    def __init__(self, world, rank, rows, head_dim, device, group):
        """Collective: every rank of `group` runs the same three collectives whatever fails locally (a failure is kept
        in `self.error` and reported by the caller's vote), so no rank is left waiting in one of them."""
        import torch.distributed as dist
        from torch.multiprocessing.reductions import reduce_tensor

        self.world, self.rank, self.rows, self.head_dim = world, rank, rows, head_dim
        self.slot = -(-(rows * (head_dim + 1)) // 4) * 4
        self.set_floats = world * self.slot
        flag_floats = -(-world // 4) * 4
        self.flag_offset = [2 * self.set_floats + s * flag_floats for s in range(2)]
        probe_offset = 2 * self.set_floats + 2 * flag_floats
        self.calls, self.error, self.peers = 0, None, []
        mine = torch.device(device).index
        rebuild = args = None
        try:
            # [set 0 slots][set 1 slots][set 0 flags][set 1 flags][probe words]; zero-initialised: no flag is raised
            self.local = torch.zeros(2 * self.set_floats + 3 * flag_floats, dtype=torch.float32, device=device)
            rebuild, args = reduce_tensor(self.local)
        except Exception as exc:
            self.error = f"{type(exc).__name__}: {exc}"
        everyone = [None] * world
        dist.all_gather_object(everyone, (mine, args), group=group)                       # collective 1
        if self.error is None and any(a is None for _, a in everyone):
            self.error = "a peer could not export its buffer"
        if self.error is None:
            try:
                lib = _lib.load()
                with torch.cuda.device(device):
                    for r, (owner, peer_args) in enumerate(everyone):
                        if r == rank:
                            self.peers.append(self.local)
                            continue
                        _lib.check(lib.fa_enable_peer_access(owner))
                        # An IPC handle is mapped into the address space of the device that is current when it is
                        # opened, and the kernels that store through it run on THIS rank's GPU: open it as memory of
                        # this device (argument 6 of the rebuild call is the device index), not of the owner's as a
                        # consumer on the same GPU would.
                        peer_args = list(peer_args)
                        peer_args[6] = mine
                        self.peers.append(rebuild(*peer_args))
                    # Before any kernel stores through these mappings, prove them with copies the driver validates:
                    # every rank writes its number into its word of every peer's probe area ...
                    stamp = torch.full((1,), float(rank + 1), dtype=torch.float32, device=device)
                    for r, t in enumerate(self.peers):
                        if r != rank:
                            t[probe_offset + rank:probe_offset + rank + 1].copy_(stamp)
                    torch.cuda.synchronize(device)
            except Exception as exc:
                self.error = f"{type(exc).__name__}: {exc}"
        dist.barrier(group=group)                                                          # collective 2
        if self.error is None:
            # ... and finds the peers' numbers in its own
            seen = self.local[probe_offset:probe_offset + world].tolist()
            missing = [r for r in range(world) if r != rank and seen[r] != float(r + 1)]
            if missing:
                self.error = f"the buffer of this rank did not receive the stores of rank(s) {missing}"

    def views(self, which):
        """(o, lse) views of this rank's own slot in set `which`, where the local kernels write the partial."""
        base = which * self.set_floats + self.rank * self.slot
        mine = self.local[base:base + self.slot]
        return (mine[:self.rows * self.head_dim].view(self.rows, self.head_dim),
                mine[self.rows * self.head_dim:self.rows * (self.head_dim + 1)])

    def merge(self, which, epoch, out_dtype, device):
        lib = _lib.load()
        out = torch.empty(self.rows, self.head_dim, dtype=out_dtype, device=device)
        p = _lib.PeerMergeParams()
        p.world, p.rank, p.out_dtype, p.rows, p.head_dim = self.world, self.rank, _DTYPE_CODE[out_dtype], self.rows, self.head_dim
        p.epoch, p.slot_floats = epoch, self.slot
        for r, t in enumerate(self.peers):
            p.peer_base[r] = t.data_ptr() + which * self.set_floats * 4
            p.peer_flags[r] = t.data_ptr() + self.flag_offset[which] * 4
        p.out, p.out_row_stride = out.data_ptr(), self.head_dim
        p.status = _status_word(device).data_ptr()
        with torch.cuda.device(device):
            _lib.check(lib.fa_peer_merge(C.byref(p), _stream(device)))
        return out


_peer_gathers = {}
_push_unavailable = set()


def _peer_gather(world, rank, rows, head_dim, device, group):
    """The cached _PeerGather for this problem, or None when the ranks cannot all set one up (every rank then takes the
    NCCL path: the decision is taken together, one object all-gather per new problem shape)."""
    import torch.distributed as dist

    key = (id(group), world, rank, rows, head_dim, torch.device(device).index)
    if key in _peer_gathers:
        return _peer_gathers[key]
    if id(group) in _push_unavailable:
        return None
    made = _PeerGather(world, rank, rows, head_dim, device, group)   # no IPC here, no peer path, ...: made.error
    votes = [None] * world
    dist.all_gather_object(votes, made.error, group=group)                              # collective 3
    if any(v is not None for v in votes):
        _push_unavailable.add(id(group))
        import warnings
        warnings.warn("fa_b200: peer-store merge unavailable, using the NCCL all-gather: "
                      + "; ".join(f"rank {r}: {v}" for r, v in enumerate(votes) if v is not None), RuntimeWarning)
        return None
    _peer_gathers[key] = made
    return made


def release_peer_buffers(group=None):
    """Collective: drops the mappings of the peers' gather buffers, then (after a barrier) this rank's own buffers, so
    that no process ends while another still maps its memory. Call it before destroying the process group."""
    import torch.distributed as dist

    held = list(_peer_gathers.values())
    _peer_gathers.clear()
    for g in held:
        g.peers = []
    import gc
    gc.collect()
    torch.cuda.ipc_collect()   # hands the released mappings back to their producers
    torch.cuda.synchronize()
    if dist.is_available() and dist.is_initialized():
        dist.barrier(group=group)
    del held


def paged_decode_kv_sharded(query, k_cache, v_cache, block_table, context_lens, softmax_scale=None, *,
                            group=None, max_context_len=None, num_splits=None, check_ranks_agree=True,
                            transport=None, _local_partial=None, _merge=None):
    """Paged decode with the KV pages of each sequence sharded block-cyclically over the ranks of `group`.

    Every rank passes the full ``query``, ``block_table`` and ``context_lens`` and its own page pool
    (only the pages of its logical blocks are read). Returns the merged ``(batch, q_heads, head_dim)``
    result on every rank. ``check_ranks_agree=False`` skips the exchange of problem shapes that guards against
    ranks describing different problems (an object all-gather through the host, the only synchronising step of a
    call). ``transport``: "push" (peer stores between the GPUs of one node, no collective), "nccl" (one all-gather) or
    None: push where it can be set up, else NCCL - all ranks must pass the same value.
    ``_local_partial`` / ``_merge`` replace the CUDA kernels in CPU tests of the protocol.
    """
    import torch.distributed as dist

    if not dist.is_available() or not dist.is_initialized():
        raise RuntimeError("paged_decode_kv_sharded needs an initialised torch.distributed process group")
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if _local_partial is None:
        validate_paged_inputs(query, k_cache, v_cache, block_table, context_lens)
        validate_inference_only(query, k_cache, v_cache)
    validate_softmax_scale(softmax_scale)
    batch, q_heads, head_dim = query.shape
    scale = 1.0 / math.sqrt(head_dim) if softmax_scale is None else float(softmax_scale)

    # every rank must describe the same problem; a mismatch would corrupt the merge silently
    if check_ranks_agree:
        meta = [batch, q_heads, head_dim, int(block_table.shape[1]), int(k_cache.shape[1])]
        all_meta = [None] * world
        dist.all_gather_object(all_meta, meta, group=group)
        if any(m != meta for m in all_meta):
            raise ValueError(f"ranks disagree on the decode problem: {all_meta}")

    rows = batch * q_heads
    if transport not in (None, "push", "nccl"):
        raise ValueError('transport must be None, "push" or "nccl"')
    peer = None
    if _local_partial is None and transport != "nccl" and world > 1 and world <= _lib.FA_MAX_PEERS:
        peer = _peer_gather(world, rank, rows, head_dim, query.device, group)
        if peer is None and transport == "push":
            raise RuntimeError("paged_decode_kv_sharded: the peer-store transport could not be set up on every rank")
    if peer is not None:
        which, epoch = peer.calls % 2, peer.calls // 2 + 1
        peer.calls += 1
        mine_o, mine_lse = peer.views(which)
    else:
        flat, g_o, g_lse = _gather_buffer(world, rows, head_dim, query.device)
        mine_o, mine_lse = g_o[rank], g_lse[rank]
    if _local_partial is None:
        sm_count = torch.cuda.get_device_properties(query.device).multi_processor_count
        capacity = block_table.shape[1] * k_cache.shape[1]
        local_ctx = -(-(capacity if max_context_len is None else min(capacity, int(max_context_len))) // world)
        kv_heads = k_cache.shape[2]
        tensor_core = _paged_tensor_core_ok(query, head_dim, q_heads, kv_heads, k_cache.shape[1], scale)
        balance = False
        if num_splits is not None:
            splits = int(num_splits)
        else:
            splits = _paged_splits_b200(batch, kv_heads, q_heads // kv_heads, k_cache.shape[1], block_table.shape[1],
                                        sm_count, local_ctx, tensor_core=tensor_core)
            if tensor_core and splits > 1 and batch <= min(256, sm_count):
                balance = True
                splits = _paged_balanced_slots(kv_heads, k_cache.shape[1], block_table.shape[1], sm_count, local_ctx)
        # the local kernels write this rank's partial straight into its slot of the gather buffer
        _paged_launch(query, k_cache, v_cache, block_table, context_lens, scale, splits, first_block=rank,
                      block_step=world, want_lse=True, out_f32=True, balance=balance,
                      out_buffers=(mine_o.view(batch, q_heads, head_dim), mine_lse.view(batch, q_heads)))
    else:
        o_r, lse_r = _local_partial(query, k_cache, v_cache, block_table, context_lens, scale, rank, world)
        g_o[rank].copy_(o_r.reshape(rows, head_dim))
        g_lse[rank].copy_(lse_r.reshape(rows))
    if peer is not None:   # stores into the peers' buffers, flags, bounded wait, merge: no collective
        return peer.merge(which, epoch, query.dtype, query.device).reshape(batch, q_heads, head_dim)
    dist.all_gather_into_tensor(flat.view(-1), flat[rank], group=group)   # in place: the input is this rank's slot
    merge = _merge_partials_cuda if _merge is None else _merge
    return merge(g_o, g_lse, query.dtype).reshape(batch, q_heads, head_dim)
