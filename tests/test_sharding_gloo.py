"""The multi-rank path on CPU: two gloo ranks shard a ragged batch by request, each computes its shard
(with the oracle standing in for the GPU kernels), results are gathered for verification and must equal
the single-process result.  No collective is used anywhere but in that gather."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
SEQ = [1024, 5000, 333, 16, 2500, 700, 64, 4100]
H, G, D, P, K = 2, 2, 64, 16, 8


def _selection_for(requests):
    """Oracle selection + attention output for a subset of requests, keyed by global request id."""
    from oracle import vortex_oracle as vo

    sel, out = {}, {}
    for r in requests:
        prob = vo.make_paged_problem(1000 + r, [SEQ[r]], H, G, D, P)   # a request's data depends on its id only
        plan = vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], P, H, K, 1, 1, 64, 16)
        vo.forward_indexer(prob["q"], prob["centroids"], plan, K, 1, 1)
        sel[r] = torch.as_tensor(plan["sparse_kv_indices"].astype(np.int64))
        out[r] = vo.decode_gqa(prob["q"], prob["k"], prob["v"], plan["sparse_kv_indptr"], plan["sparse_kv_indices"],
                               plan["kv_last_page_len"]).float()
    return sel, out


def _worker(rank, world, port, q):
    for p in (str(ROOT), str(ROOT / "vortex_torch-dev_b200")):
        sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from vortex_torch.runtime import balance_requests, gather_for_verification

    pages = [(s + P - 1) // P for s in SEQ]
    parts = balance_requests(pages, world)            # every rank computes the same assignment
    sel, out = _selection_for(parts[rank])
    all_sel = gather_for_verification(sel)
    all_out = gather_for_verification(out)
    if rank == 0:
        q.put((parts, {k: v.numpy() for k, v in all_sel.items()}, {k: v.numpy() for k, v in all_out.items()}))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_matches_single_process():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29000 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    parts, sel, out = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(parts[0] + parts[1]) == list(range(len(SEQ)))
    want_sel, want_out = _selection_for(range(len(SEQ)))
    assert sorted(sel) == list(range(len(SEQ)))
    for r in range(len(SEQ)):
        np.testing.assert_array_equal(sel[r], want_sel[r].numpy())
        np.testing.assert_array_equal(out[r], want_out[r].numpy())


def _worker_sparse(rank, world, port, q):
    for p in (str(ROOT), str(ROOT / "vortex_torch-dev_b200")):
        sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from vortex_torch.runtime import balance_requests, gather_for_verification

    pages = [(s + P - 1) // P for s in SEQ[:2]]        # two requests on three ranks: one rank holds nothing
    parts = balance_requests(pages, world)
    sel, out = _selection_for(parts[rank])
    all_sel = gather_for_verification(sel)               # the empty rank has to learn the dtype from the others
    all_out = gather_for_verification(out, dtype=torch.float32)
    if rank == 0:
        q.put((parts, {k: v.numpy() for k, v in all_sel.items()}, {k: v.numpy() for k, v in all_out.items()}))
    dist.barrier()
    dist.destroy_process_group()


def test_more_ranks_than_requests():
    """A rank without requests takes part in the verification gather with the payload dtype of the others."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31000 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker_sparse, args=(r, 3, port, q)) for r in range(3)]
    for p in procs:
        p.start()
    parts, sel, out = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(len(x) for x in parts) == [0, 1, 1]
    want_sel, want_out = _selection_for(range(2))
    for r in range(2):
        np.testing.assert_array_equal(sel[r], want_sel[r].numpy())
        assert sel[r].dtype == np.int64
        np.testing.assert_array_equal(out[r], want_out[r].numpy())


# ----------------------------------------------------------------------------- KV-head split
HS_SEQ = [1024, 5000, 333, 2500]
HS_H = 4


def _head_shard_result(requests, shard):
    """Oracle selection + attention for ``requests`` on the KV heads of ``shard`` only: the rank's pool, summaries
    and queries are the head slices of the unsharded ones, and the path runs with the local head count."""
    from oracle import vortex_oracle as vo
    from vortex_torch.runtime import local_row_to_global, slice_heads

    sel, out = {}, {}
    hl = shard.num_heads
    for r in requests:
        prob = vo.make_paged_problem(2000 + r, [HS_SEQ[r]], HS_H, G, D, P)
        k, v, c = (slice_heads(prob[n], HS_H, shard.head_lo, shard.head_hi) for n in ("k", "v", "centroids"))
        qq = slice_heads(prob["q"], HS_H, shard.head_lo, shard.head_hi)
        plan = vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], P, hl, K, 1, 1, 64, 16)
        vo.forward_indexer(qq, c, plan, K, 1, 1)
        rows = torch.as_tensor(plan["sparse_kv_indices"].astype(np.int64))
        # key: (request, first head) packed into one id; value: selection in the unsharded pool's row numbering
        sel[r * HS_H + shard.head_lo] = local_row_to_global(rows, HS_H, shard)
        out[r * HS_H + shard.head_lo] = vo.decode_gqa(qq, k, v, plan["sparse_kv_indptr"], plan["sparse_kv_indices"],
                                                      plan["kv_last_page_len"]).float()
    return sel, out


def _worker_heads(rank, world, port, q):
    for p in (str(ROOT), str(ROOT / "vortex_torch-dev_b200")):
        sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from vortex_torch.runtime import gather_for_verification, shard_grid

    pages = [(s + P - 1) // P for s in HS_SEQ]
    grid = shard_grid(pages, HS_H, world, head_shards=2)      # every rank computes the same grid
    sel, out = _head_shard_result(grid[rank].requests, grid[rank])
    all_sel = gather_for_verification(sel)
    all_out = gather_for_verification(out)
    if rank == 0:
        q.put((grid, {k: v.numpy() for k, v in all_sel.items()}, {k: v.numpy() for k, v in all_out.items()}))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_head_split_matches_single_process():
    """Two ranks, each with half the KV heads of every request: the union equals the unsharded result bit for bit."""
    from oracle import vortex_oracle as vo

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 33000 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker_heads, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    grid, sel, out = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [(g.head_lo, g.head_hi) for g in grid] == [(0, 2), (2, 4)]
    assert all(g.requests == tuple(range(len(HS_SEQ))) for g in grid)
    for r in range(len(HS_SEQ)):
        prob = vo.make_paged_problem(2000 + r, [HS_SEQ[r]], HS_H, G, D, P)
        plan = vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], P, HS_H, K, 1, 1, 64, 16)
        vo.forward_indexer(prob["q"], prob["centroids"], plan, K, 1, 1)
        want_out = vo.decode_gqa(prob["q"], prob["k"], prob["v"], plan["sparse_kv_indptr"], plan["sparse_kv_indices"],
                                 plan["kv_last_page_len"]).float().numpy()
        sip = plan["sparse_kv_indptr"]
        for lo in (0, 2):   # heads lo, lo+1 of request r are segments lo, lo+1 of the unsharded plan
            np.testing.assert_array_equal(sel[r * HS_H + lo], plan["sparse_kv_indices"][sip[lo]:sip[lo + 2]])
            np.testing.assert_array_equal(out[r * HS_H + lo], want_out[lo:lo + 2])
