"""Sharding of the decode path across GPUs: by request, by KV head, or both.

Every (request, KV head) segment is independent through the whole decode path (block tables, page
summaries, page selection, attention), so the ranks form a grid of ``request_shards x head_shards``:
a rank holds some requests and, of those, a contiguous range of KV heads.  Nothing crosses GPUs on the
hot path in either direction.

* Requests are dealt out by total page count (longest-processing-time-first greedy), which is what the
  per-step cost is proportional to.
* A rank that owns heads ``[lo, hi)`` keeps a KV pool of ``hi - lo`` heads per page
  (``[pages, hi - lo, page_size, head_dim]``, the layout of the reference's ``cache/triton_kernels/set_kv.py:28-33``
  with its head count replaced by the local one) and calls the whole path with ``num_kv_heads = hi - lo`` and the
  query heads ``[lo * group, hi * group)``.  Segment ``s = request * heads + head`` and row ``page * heads + head``
  (``csrc/utils_sglang.cu:291-307`` of the reference) then number the local heads, so no kernel takes a head
  range: a head shard is the same program on a narrower pool.  This is also what a tensor-parallel serving
  engine hands each rank.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple


@dataclass(frozen=True)
class Shard:
    """What one rank holds: ascending global request ids and the KV heads ``[head_lo, head_hi)`` of each."""
    requests: Tuple[int, ...]
    head_lo: int
    head_hi: int

    @property
    def num_heads(self) -> int:
        return self.head_hi - self.head_lo


def head_range(num_kv_heads: int, head_shards: int, index: int) -> Tuple[int, int]:
    """Heads of head shard ``index`` out of ``head_shards`` equal contiguous ranges."""
    if head_shards < 1 or num_kv_heads % head_shards != 0:
        raise ValueError(f"{num_kv_heads} KV heads cannot be split into {head_shards} equal shards")
    if not 0 <= index < head_shards:
        raise ValueError(f"head shard {index} out of range for {head_shards} shards")
    per = num_kv_heads // head_shards
    return index * per, (index + 1) * per


def shard_grid(page_counts: Sequence[int], num_kv_heads: int, world_size: int, head_shards: int = 1) -> List[Shard]:
    """One `Shard` per rank for a ``(world_size / head_shards) x head_shards`` grid.

    Rank ``r`` is request shard ``r // head_shards`` and head shard ``r % head_shards`` (the ranks that share
    requests are neighbours).  Deterministic, so every rank computes the same grid without communication."""
    if world_size < 1 or head_shards < 1 or world_size % head_shards != 0:
        raise ValueError(f"{world_size} ranks cannot form a grid with {head_shards} head shards")
    parts = balance_requests(page_counts, world_size // head_shards)
    return [Shard(tuple(parts[r // head_shards]), *head_range(num_kv_heads, head_shards, r % head_shards))
            for r in range(world_size)]


def choose_head_shards(page_counts: Sequence[int], num_kv_heads: int, world_size: int) -> int:
    """The number of head shards (a common divisor of ``world_size`` and ``num_kv_heads``) with the lightest
    heaviest rank, load = pages x heads; ties go to fewer head shards (fewer, longer lists per rank)."""
    best, best_load = 1, None
    for t in range(1, min(world_size, num_kv_heads) + 1):
        if world_size % t or num_kv_heads % t:
            continue
        parts = balance_requests(page_counts, world_size // t)
        load = max(sum(int(page_counts[i]) for i in part) for part in parts) * (num_kv_heads // t)
        if best_load is None or load < best_load:
            best, best_load = t, load
    return best


def slice_heads(x, num_kv_heads: int, head_lo: int, head_hi: int, group: int = 1):
    """The rows of heads ``[head_lo, head_hi)`` of a tensor whose leading dimension is ``n * num_kv_heads * group``
    in (n, head, group-member) order: a paged cache ``[pages * heads, ...]`` (``group = 1``), a page-summary cache,
    or queries / outputs ``[bs * heads, group, dim]``.  Returns a contiguous copy (this is a re-sharding step, not
    part of the decode path)."""
    n = x.shape[0] // (num_kv_heads * group)
    if n * num_kv_heads * group != x.shape[0]:
        raise ValueError("leading dimension is not a multiple of the head count")
    v = x.reshape(n, num_kv_heads, group, *x.shape[1:])[:, head_lo:head_hi]
    return v.reshape(n * (head_hi - head_lo) * group, *x.shape[1:]).contiguous()


def local_row_to_global(rows, num_kv_heads: int, shard: "Shard"):
    """Rows ``page * local_heads + local_head`` of a head shard as rows ``page * num_kv_heads + head`` of the
    unsharded pool (for comparing selections; works on tensors and arrays)."""
    hl = shard.num_heads
    return (rows // hl) * num_kv_heads + shard.head_lo + rows % hl


def balance_requests(page_counts: Sequence[int], world_size: int) -> List[List[int]]:
    """Assign request ids to ``world_size`` ranks, heaviest first onto the lightest rank.

    Returns one ascending list of request ids per rank.  Deterministic: ties go to the lower
    request id / lower rank, so every rank computes the same assignment without communication.
    """
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    order = sorted(range(len(page_counts)), key=lambda i: (-int(page_counts[i]), i))
    load = [0] * world_size
    out: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda k: (load[k], k))
        out[r].append(i)
        load[r] += int(page_counts[i])
    return [sorted(x) for x in out]


_DTYPE_CODES = [torch_name for torch_name in ("float32", "bfloat16", "float16", "int32", "int64", "int16", "uint8")]


def gather_for_verification(local: dict, group=None, dtype=None) -> dict:
    """Collect per-request results from every rank (verification only; never on the hot path).

    ``local`` maps a global request id to a tensor (any shape, any device).  Every rank gets back the
    union.  Tensors are moved through ``torch.distributed.all_gather`` after padding to a common length,
    so the call works on NCCL (device tensors over NVLink) and on gloo (CPU tensors) alike.
    ``dtype``: the payload dtype, the same on every rank.  When it is not given the ranks agree on one first
    (a rank that holds no request has nothing to infer it from), and a disagreement raises on every rank.
    """
    import torch
    import torch.distributed as dist

    if not dist.is_available() or not dist.is_initialized():
        return dict(local)
    world = dist.get_world_size(group)
    backend = dist.get_backend(group)
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    ids = sorted(local)
    # header: per request (id, numel, ndim, dims...) as int64; payload: flattened values as one dtype
    if dtype is None:
        # agree on the payload dtype: code of the local dtype (or -1 for "nothing to send"), max over ranks
        mine = _DTYPE_CODES.index(str(next(iter(local.values())).dtype).replace("torch.", "")) if local else -1
        codes = [torch.zeros(1, dtype=torch.int64, device=dev) for _ in range(world)]
        dist.all_gather(codes, torch.tensor([mine], dtype=torch.int64, device=dev), group=group)
        seen = {int(c.item()) for c in codes} - {-1}
        if len(seen) > 1:
            raise TypeError("gather_for_verification: ranks hold different dtypes; pass dtype= explicitly")
        dtype = getattr(torch, _DTYPE_CODES[seen.pop()]) if seen else torch.float32
    header, chunks = [], []
    for i in ids:
        t = local[i]
        assert t.dtype == dtype, "gather_for_verification: one dtype per call"
        header += [i, t.numel(), t.dim(), *t.shape]
        chunks.append(t.reshape(-1).to(dev))
    head = torch.tensor(header, dtype=torch.int64, device=dev)
    body = torch.cat(chunks) if chunks else torch.zeros(0, dtype=dtype, device=dev)
    sizes = torch.tensor([head.numel(), body.numel()], dtype=torch.int64, device=dev)
    all_sizes = [torch.zeros_like(sizes) for _ in range(world)]
    dist.all_gather(all_sizes, sizes, group=group)
    max_h = int(max(s[0] for s in all_sizes))
    max_b = int(max(s[1] for s in all_sizes))
    head_p = torch.zeros(max(1, max_h), dtype=torch.int64, device=dev)
    head_p[: head.numel()] = head
    body_p = torch.zeros(max(1, max_b), dtype=dtype, device=dev)
    body_p[: body.numel()] = body
    heads = [torch.zeros_like(head_p) for _ in range(world)]
    bodies = [torch.zeros_like(body_p) for _ in range(world)]
    dist.all_gather(heads, head_p, group=group)
    dist.all_gather(bodies, body_p, group=group)
    out = {}
    for r in range(world):
        h = heads[r][: int(all_sizes[r][0])].tolist()
        b = bodies[r][: int(all_sizes[r][1])]
        pos, off = 0, 0
        while pos < len(h):
            rid, numel, ndim = h[pos], h[pos + 1], h[pos + 2]
            shape = h[pos + 3: pos + 3 + ndim]
            out[rid] = b[off: off + numel].reshape(shape).cpu()
            pos += 3 + ndim
            off += numel
    return out
