"""Request-level sharding across GPUs.

Every (request, KV head) segment is independent through the whole decode path, so requests are
simply dealt out to ranks; nothing crosses GPUs on the hot path.  Balance is by total page count
(longest-processing-time-first greedy), which is what the per-step cost is proportional to.
"""
from __future__ import annotations

from typing import List, Sequence


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
