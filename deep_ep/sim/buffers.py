"""CPU (gloo) stand-ins for the native runtimes of `BucketBuffer`, `PPBuffer` and `EngramBuffer`.

They make the Python layer of those buffers (sessions, alias checks, argument validation, hooks) run and be tested
without a GPU, the same way `deep_ep.sim.ep.SimEPRuntime` does for `EPBuffer`. Semantics follow the native runtimes
(`csrc/buffers/{bucket,pp,engram}.hpp`, which in turn follow the reference's `csrc/buffers/bucket.hpp:23-153`,
`pp.hpp:14-92`, `engram.hpp:19-212`); data moves with `torch.distributed` collectives on CPU tensors.
"""
from typing import Callable, List, Optional

import torch
import torch.distributed as dist


class SimContext:
    """What the Python layer reads from a native `Context`."""

    def __init__(self, rank_idx: int, num_ranks: int, context_idx: int = 0):
        self.rank_idx, self.num_ranks, self.context_idx = rank_idx, num_ranks, context_idx
        self.num_workspace_bytes = self.num_gpu_buffer_bytes = self.num_rdma_storage_bytes = 0
        self.peers_ready = True

    def get_physical_domain_size(self):
        return 1, self.num_ranks

    def get_logical_domain_size(self):
        return 1, self.num_ranks

    def has_multicast(self) -> bool:
        return False

    def status_code(self) -> int:
        return 0


class _NoEvent:
    """Stands where a CUDA event would be: everything has already happened when a CPU call returns."""

    def current_stream_wait(self) -> None:
        pass


def _bytes_of(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(-1).view(torch.uint8)


def _gather_bytes(t: torch.Tensor, group: dist.ProcessGroup) -> List[torch.Tensor]:
    mine = _bytes_of(t).clone()
    parts = [torch.empty_like(mine) for _ in range(group.size())]
    dist.all_gather(parts, mine, group=group)
    return parts


class SimBucketRuntime:
    """`all_gather` / `reduce` of registered tensors over CPU process groups."""

    MAX_BUCKETS = 64

    def __init__(self, groups: List[dist.ProcessGroup], num_bytes: int):
        self.groups = groups
        self.storage = torch.zeros(num_bytes, dtype=torch.uint8)
        self.contexts = [SimContext(g.rank(), g.size(), i) for i, g in enumerate(groups)]
        self.main_context = self.contexts[0]
        self.destroyed = False

    def _offset(self, t: torch.Tensor) -> int:
        return t.data_ptr() - self.storage.data_ptr()

    def all_gather(self, srcs, dsts, context_idx: int, num_sms: int):
        assert not self.destroyed and 0 <= context_idx < len(self.groups)
        assert srcs and len(srcs) <= self.MAX_BUCKETS and (not dsts or len(dsts) == len(srcs))
        group = self.groups[context_idx]
        rank, size, total = group.rank(), group.size(), self.storage.numel()
        gathered = []
        for i, src in enumerate(srcs):
            assert src.is_contiguous() and src.numel() > 0
            shard = src.nbytes
            src_off = self._offset(src)
            bucket = src_off - rank * shard                     # in place: src is my shard of the gathered tensor
            if dsts:
                dst = dsts[i]
                assert dst.is_contiguous() and dst.dtype == src.dtype and dst.nbytes == size * shard
                bucket = self._offset(dst)
            assert 0 <= bucket <= total and shard <= (total - bucket) // size, \
                'all-gather outputs must belong to this BucketBuffer'
            assert src_off == bucket + rank * shard or src_off + shard <= bucket or src_off >= bucket + size * shard, \
                'a source may only overlap the output as this rank\'s own shard'
            for r, part in enumerate(_gather_bytes(src, group)):
                self.storage[bucket + r * shard:bucket + (r + 1) * shard] = part
            gathered.append(self.storage.narrow(0, bucket, size * shard).view(src.dtype))
        return _NoEvent(), (lambda: gathered), num_sms

    def reduce(self, srcs, context_idx: int, num_sms: int, scale: float, all_reduce: bool):
        assert not self.destroyed and srcs and len(srcs) <= self.MAX_BUCKETS
        group = self.groups[context_idx]
        rank, size = group.rank(), group.size()
        results = []
        for src in srcs:
            off = self._offset(src)
            assert src.is_contiguous() and 0 <= off and off + src.nbytes <= self.storage.numel(), \
                'reduced tensors must belong to this BucketBuffer'
            assert off % 16 == 0 and src.nbytes % (size * 16) == 0, \
                'reduced tensors must start on a 16-byte boundary and split into 16-byte aligned shards'
            assert src.dtype in (torch.bfloat16, torch.float16, torch.float32)
            flat = src.view(-1)
            acc = torch.zeros(flat.numel(), dtype=torch.float32)
            for part in _gather_bytes(flat, group):                 # fp32 sum in rank order, one rounding
                acc += part.view(src.dtype).float()
            out = (acc * scale).to(src.dtype)
            m = flat.numel() // size
            if all_reduce:
                flat.copy_(out)
                results.append(src)
            else:
                flat[rank * m:(rank + 1) * m] = out[rank * m:(rank + 1) * m]
                results.append(flat.narrow(0, rank * m, m))
        return results, _NoEvent(), num_sms

    def print_memory_usage(self) -> None:
        print(f'[sim] bucket storage: {self.storage.numel()} bytes')

    def destroy(self) -> None:
        assert not self.destroyed
        for g in self.groups:
            dist.barrier(g)
        self.storage, self.destroyed = None, True


class SimPPRuntime:
    """Ring neighbours exchange tensors with point-to-point messages; sends are posted without waiting for the receiver."""

    def __init__(self, group: dist.ProcessGroup, num_max_tensor_bytes: int, num_max_inflight_tensors: int):
        self.group = group
        self.rank_idx, self.num_ranks = group.rank(), group.size()
        self.num_max_tensor_bytes, self.num_max_inflight = num_max_tensor_bytes, num_max_inflight_tensors
        self.context = self.main_context = SimContext(self.rank_idx, self.num_ranks)
        self.storage = torch.zeros(0, dtype=torch.uint8)
        self._pending = {}          # destination -> list of (work handle, buffer kept alive)
        self.destroyed = False

    def _check(self, x: torch.Tensor, peer: int) -> None:
        assert not self.destroyed and x.is_contiguous() and 0 < x.nbytes <= self.num_max_tensor_bytes
        assert peer in ((self.rank_idx + 1) % self.num_ranks, (self.rank_idx - 1) % self.num_ranks), \
            'only the previous or the next rank of the ring can be addressed'

    def send(self, x: torch.Tensor, dst: int, num_sms: int) -> None:
        self._check(x, dst)
        pending = self._pending.setdefault(dst, [])
        while len(pending) >= self.num_max_inflight:                 # credit: at most that many sends run ahead
            pending.pop(0)[0].wait()
        payload = _bytes_of(x).clone()
        pending.append((dist.isend(payload, dist.get_global_rank(self.group, dst), group=self.group), payload))

    def recv(self, x: torch.Tensor, src: int, num_sms: int) -> None:
        self._check(x, src)
        payload = torch.empty(x.nbytes, dtype=torch.uint8)
        dist.recv(payload, dist.get_global_rank(self.group, src), group=self.group)
        x.view(-1).view(torch.uint8).copy_(payload)

    def print_memory_usage(self) -> None:
        print(f'[sim] pp ring: {self.num_max_inflight} x {self.num_max_tensor_bytes} bytes per direction')

    def destroy(self) -> None:
        assert not self.destroyed
        for pending in self._pending.values():
            for work, _ in pending:
                work.wait()
        dist.barrier(self.group)
        self.destroyed = True


class SimEngramRuntime:
    """Every rank keeps a copy of all shards (gathered at `write`); `fetch` indexes them locally."""

    def __init__(self, group: dist.ProcessGroup, num_gpu_bytes: int, num_rdma_storage_bytes: int):
        self.group = group
        self.rank_idx, self.num_ranks = group.rank(), group.size()
        self.context = self.main_context = SimContext(self.rank_idx, self.num_ranks)
        self.num_gpu_bytes, self.num_rdma_storage_bytes = num_gpu_bytes, num_rdma_storage_bytes
        self.config = None
        self.tables: List[torch.Tensor] = []
        self.sf_tables: Optional[List[torch.Tensor]] = None
        self.destroyed = False

    def set_config(self, num_entries_per_layer, hidden, elem_size, num_max_tokens, num_entries_per_token, num_sf_packs) -> None:
        assert not self.destroyed
        dist.barrier(self.group)
        storage = sum(num_entries_per_layer) * hidden * elem_size
        recv = len(num_entries_per_layer) * num_max_tokens * num_entries_per_token * hidden * elem_size
        sf = sum(num_entries_per_layer) * num_sf_packs * 2
        assert storage <= self.num_rdma_storage_bytes, 'table shards do not fit the storage region'
        assert recv + sf <= self.num_gpu_bytes, 'receive region too small for this configuration'
        self.config = (list(num_entries_per_layer), hidden, elem_size, num_max_tokens, num_entries_per_token, num_sf_packs)

    def write(self, storages, sfs) -> None:
        assert self.config is not None, 'call set_config first'
        entries, hidden, elem_size, _, _, packs = self.config
        assert len(storages) == len(entries) and (sfs is not None) == (packs > 0)
        self.tables = []
        for n, t in zip(entries, storages):
            assert t.dim() == 2 and tuple(t.shape) == (n, hidden) and t.element_size() == elem_size and t.is_contiguous()
            parts = _gather_bytes(t, self.group)
            self.tables.append(torch.cat(parts).view(self.num_ranks * n, hidden * elem_size))
        self.sf_tables = None
        if sfs is not None:
            self.sf_tables = []
            for n, sf in zip(entries, sfs):
                assert tuple(sf.shape) == (self.num_ranks * n, packs) and sf.element_size() == 2 and sf.is_contiguous()
                shard = sf.view(torch.int16)[self.rank_idx * n:(self.rank_idx + 1) * n]       # each rank contributes its slice
                self.sf_tables.append(torch.cat(_gather_bytes(shard, self.group)).view(torch.int16).view(self.num_ranks * n, packs))
        dist.barrier(self.group)

    def fetch(self, indices: torch.Tensor, num_qps: int, use_col_major_sf: bool) -> List[Callable]:
        assert self.config is not None and self.tables, 'call set_config and write first'
        entries, hidden, elem_size, num_max_tokens, per_token, packs = self.config
        assert indices.dim() == 3 and indices.dtype == torch.int32 and indices.is_contiguous() and num_qps == 0
        num_layers, num_tokens, p = indices.shape
        assert num_layers == len(entries) and num_tokens <= num_max_tokens and p == per_token
        dtype = torch.float8_e4m3fn if packs > 0 else torch.bfloat16
        hooks = []
        for layer in range(num_layers):
            idx = indices[layer].long()
            safe = idx.clamp(min=0).view(-1)
            rows = self.tables[layer][safe].view(num_tokens, per_token, hidden * elem_size).clone()
            rows[idx < 0] = 0                                        # skipped entries: contents unspecified, zero here
            fetched = rows.view(num_tokens, per_token * hidden * elem_size).view(dtype)
            if packs == 0:
                hooks.append(lambda fetched=fetched: fetched)
                continue
            sf = self.sf_tables[layer][safe].view(num_tokens, per_token * packs)
            if use_col_major_sf:
                sf = sf.t().contiguous().t()                         # strides (1, num_tokens)
            hooks.append(lambda fetched=fetched, sf=sf: (fetched, sf))
        return hooks

    def print_memory_usage(self) -> None:
        print(f'[sim] engram: {self.num_gpu_bytes} receive bytes, {self.num_rdma_storage_bytes} storage bytes')

    def destroy(self) -> None:
        assert not self.destroyed
        dist.barrier(self.group)
        self.tables, self.sf_tables, self.destroyed = [], None, True
