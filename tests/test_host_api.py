"""Host-side logic that needs no GPU: registry, loader, format-tagged tensors, contexts, the profile pass,
the sharding helper, and that the C-ABI library exports every symbol the header declares."""
import re
import textwrap
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def test_cabi_exports_every_declared_symbol():
    from vortex_torch import _cabi

    header = (ROOT / "include" / "vortex_b200.h").read_text()
    declared = sorted(set(re.findall(r"\b(vtx_[a-z0-9_]+)\s*\(", header)))
    assert declared, "no declarations found in the header"
    for name in declared:
        assert hasattr(_cabi.lib, name), f"{name} declared in include/vortex_b200.h but not exported"
    assert set(_cabi.EXPORTED) == set(declared)
    assert _cabi.version() >= 100
    assert _cabi.status_string(0) == "ok" and "invalid" in _cabi.status_string(1)


def test_no_cpu_fallback():
    from vortex_torch import _cabi

    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _cabi.ptr(torch.zeros(4))


def test_registry_and_loader(tmp_path):
    from vortex_torch.flow import build_vflow, register, vFlow
    from vortex_torch.flow import registry
    from vortex_torch.flow.loader import FlowInitError, FlowLoadError

    assert {"block_sparse_attention", "gqa_block_sparse_attention", "gqa_quest_sparse_attention"} <= set(registry.list_keys())
    with pytest.raises(registry.RegistryError, match="must inherit"):
        register("not_a_flow")(int)
    with pytest.raises(registry.RegistryError, match="already exists"):
        register("block_sparse_attention")(registry.get("block_sparse_attention"))
    with pytest.raises(FlowLoadError, match="not found"):
        build_vflow("does_not_exist")
    with pytest.raises(FlowLoadError, match="does not exist"):
        build_vflow("block_sparse_attention", None, str(tmp_path / "missing.py"))
    with pytest.raises(FlowInitError, match="mismatch"):
        build_vflow("block_sparse_attention", {"bogus": 1})
    f = tmp_path / "user_flow.py"
    f.write_text(textwrap.dedent('''
        from vortex_torch.flow import vFlow, register
        @register("tmp_user_flow")
        class F(vFlow):
            def __init__(self, k=3):
                super().__init__(); self.k = k
            def forward_indexer(self, q, o, cache, ctx): pass
            def forward_cache(self, cache, loc, ctx): pass
            def create_cache(self, page_size, head_dim): return {"s": (2, head_dim)}
    '''))
    flow = build_vflow("tmp_user_flow", {"k": 5}, str(f))
    assert flow.k == 5 and isinstance(flow, vFlow)
    meta = flow.get_cache_meta_info(16, 128)
    assert meta == {"s": (2, 128), "k": (16, 128), "v": (16, 128)}
    assert flow.get_token_ratio(16, 128) == pytest.approx(2.0 + 2 / 16)
    bad = tmp_path / "bad_flow.py"
    bad.write_text("raise ValueError('boom')")
    with pytest.raises(FlowLoadError, match="boom"):
        build_vflow("tmp_user_flow", None, str(bad))


def test_vtensor_rules():
    from vortex_torch.abs import FORMAT, as_vtensor, vTensor

    a = as_vtensor(torch.randn(2, 3), FORMAT.RAGGED)
    b = as_vtensor(torch.ones(2, 3), FORMAT.RAGGED)
    assert isinstance(a + 2.0, vTensor) and (a + 2.0)._format == FORMAT.RAGGED
    assert (a * b)._format == FORMAT.RAGGED
    with pytest.raises(RuntimeError, match="plain torch.Tensor"):
        _ = a + torch.randn(2, 3)
    with pytest.raises(RuntimeError, match="mismatch"):
        _ = a + as_vtensor(torch.randn(2, 3), FORMAT.PAGED)
    assert as_vtensor(a, FORMAT.PAGED) is a and a._format == FORMAT.PAGED
    import pickle
    c = pickle.loads(pickle.dumps(b))
    assert isinstance(c, vTensor) and c._format == FORMAT.RAGGED and torch.equal(torch.Tensor(c), torch.Tensor(b))


def test_lazy_group_mean_is_invisible():
    from vortex_torch.abs import FORMAT, as_vtensor
    from vortex_torch.abs.tensor import lazy_group_mean_source, materialize

    q = as_vtensor(torch.randn(5, 4, 16), FORMAT.BATCHED)
    real = q.mean(dim=1, keepdim=True)
    q._vtx_allow_lazy_mean = True
    lazy = q.mean(dim=1, keepdim=True)
    assert lazy_group_mean_source(lazy) is q and lazy.shape == real.shape
    assert torch.equal(torch.Tensor(lazy * 1.0), torch.Tensor(real))           # any torch op sees the real mean
    assert torch.equal(torch.Tensor(materialize(lazy)), torch.Tensor(real))
    calls = []
    import vortex_torch.abs.tensor as vt
    orig = vt.materialize
    vt.materialize = lambda x: (calls.append(1), orig(x))[1]
    try:  # shape / placement queries must not compute the mean
        assert lazy.dim() == 3 and lazy.shape[1] == 1 and lazy.device == q.device and lazy.dtype == q.dtype
        lazy.data_ptr(), lazy.size(0), lazy.is_contiguous()
        assert calls == []
    finally:
        vt.materialize = orig
    assert lazy_group_mean_source(q.mean(dim=2, keepdim=True)) is None           # other reductions are untouched
    assert lazy_group_mean_source(q.mean(dim=1)) is None


def test_profile_pass_allocates_and_detects_fusion():
    from vortex_torch.runtime import VortexDecodeRuntime
    from vortex_torch.utils import Mode

    rt = VortexDecodeRuntime(2, 16, 8, 128, num_pages=32, max_bs=3, context_len=512, device="cpu")
    assert rt.ictx.mode == Mode.execute and rt.cctx.mode == Mode.execute
    assert rt.ictx.max_num_pages_per_request == 32 and rt.ictx.max_num_pages == 32 * 3 * 8
    assert rt.flow.gemv.output_buffer.shape == (32 * 3 * 8, 1, 1)
    assert rt.ictx._aux_total_bytes == 32 * 3 * 8 * 2 and rt.ictx._aux_total_flops == 128
    assert rt.flow.gemv._fused_consumer is rt.flow.output_func and rt.flow.gemv._x_is_group_mean
    assert not rt.flow.gemv._score_read_elsewhere  # shape checks in the profile pass do not count as reads
    assert rt.ictx.missing() == [] and rt.cctx.missing() == []
    with pytest.raises(RuntimeError, match="already called"):
        rt.ictx.create(rt.backend, rt.model_runner)
    assert rt.flow.run_indexer_virtual(2, 16, 128, device="cpu") == 128


def test_every_shipped_flow_can_be_built():
    from vortex_torch.flow import build_vflow

    for name in ("block_sparse_attention", "gqa_block_sparse_attention", "gqa_quest_sparse_attention"):
        build_vflow(name)  # every operator of the shipped flows can be constructed


def test_balance_requests():
    from vortex_torch.runtime import balance_requests

    pages = [64, 2048, 100, 1500, 900, 31, 777, 1200]
    for w in (1, 2, 4, 8):
        parts = balance_requests(pages, w)
        assert sorted(sum(parts, [])) == list(range(len(pages)))
        loads = [sum(pages[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(pages)
    assert balance_requests(pages, 2) == balance_requests(pages, 2)


def test_gqa_chain_is_recognised_and_stand_alone_use_needs_the_gpu():
    from vortex_torch.abs import FORMAT, as_vtensor
    from vortex_torch.indexer import Context, GeMM, Max, Softmax
    from vortex_torch.runtime import ServerArgs, VortexDecodeRuntime

    rt = VortexDecodeRuntime(2, 8, 2, 128, num_pages=32, max_bs=2, context_len=256, device="cpu",
                             server_args=ServerArgs(vortex_module_name="gqa_block_sparse_attention"))
    f = rt.flow
    assert f.output_func._gqa_chain == (f.gemm, f.softmax, f.max_op)
    assert f.output_func.chain_intact() and f.gemm._runs_fused() and f.max_op._runs_fused()
    assert f.gemm.output_buffer.shape == (rt.ictx.max_num_pages, 1, 4) and f.max_op.output_buffer.shape[1:] == (1, 1)
    # a GeMM whose result does not end in a fused chain runs its own kernel: on CPU tensors that is an error
    # (there is no CPU fallback), never a silent no-op
    ctx = Context()
    ctx.max_num_pages = 8
    g = GeMM()
    bf = torch.bfloat16
    out = g.profile(as_vtensor(torch.zeros(1, 2, 16, dtype=bf), FORMAT.BATCHED),
                    as_vtensor(torch.zeros(4, 1, 16, dtype=bf), FORMAT.PAGED), ctx)
    assert out.shape == (8, 1, 2) and not g._runs_fused()
    sm = Softmax(dim=0, scale=0.5)
    sm.profile(out, ctx)
    mx = Max(dim=2)
    assert mx.profile(out, ctx).shape == (8, 1, 1)
    rt.ictx.set_batch_size(1)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        g.execute(torch.zeros(1, 2, 16, dtype=bf), torch.zeros(4, 1, 16, dtype=bf), rt.ictx)
    with pytest.raises(NotImplementedError, match="bfloat16"):
        GeMM().profile(as_vtensor(torch.zeros(1, 2, 16), FORMAT.BATCHED), as_vtensor(torch.zeros(4, 1, 16), FORMAT.PAGED),
                       ctx)


def test_head_shards_and_grid():
    from vortex_torch.runtime import (Shard, choose_head_shards, head_range, local_row_to_global, shard_grid,
                                      slice_heads)

    assert [head_range(8, 4, i) for i in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    with pytest.raises(ValueError):
        head_range(8, 3, 0)
    with pytest.raises(ValueError):
        head_range(8, 2, 2)
    pages = [100, 7, 64, 2048, 33, 900]
    grid = shard_grid(pages, 8, 8, head_shards=4)
    assert len(grid) == 8 and all(isinstance(g, Shard) for g in grid)
    # ranks 0-3 share the requests of request shard 0 and split its heads; every (request, head) has one owner
    assert grid[0].requests == grid[3].requests and grid[4].requests == grid[7].requests
    owners = {}
    for rank, g in enumerate(grid):
        for r in g.requests:
            for hd in range(g.head_lo, g.head_hi):
                assert (r, hd) not in owners
                owners[(r, hd)] = rank
    assert len(owners) == len(pages) * 8
    with pytest.raises(ValueError):
        shard_grid(pages, 8, 8, head_shards=3)
    # one huge request: splitting heads is the only way to spread it
    assert choose_head_shards([4096, 10, 10], 8, 8) == 8
    # many equal requests: request sharding alone is already even, fewer head shards win the tie
    assert choose_head_shards([64] * 64, 8, 8) == 1
    x = torch.arange(3 * 4 * 2).view(3 * 4, 2)            # 3 pages x 4 heads
    y = slice_heads(x, 4, 1, 3)
    assert y.shape == (6, 2) and torch.equal(y[:, 0], torch.tensor([2, 4, 10, 12, 18, 20]))
    qx = torch.arange(2 * 4 * 3).view(2 * 4, 3, 1)        # queries [bs*H, G, D]
    assert torch.equal(slice_heads(qx, 4, 2, 4), qx.view(2, 4, 3, 1)[:, 2:4].reshape(4, 3, 1))
    sh = Shard((0,), 2, 4)
    rows = torch.tensor([0, 1, 2, 3, 9])                  # page*2 + local head
    assert local_row_to_global(rows, 8, sh).tolist() == [2, 3, 10, 11, 35]


@pytest.mark.parametrize("G", [1, 3, 5, 8, 16])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_unfused_group_mean_follows_the_canonical_order(G, dtype):
    """The mean a flow sees when nothing is fused (any group size) is the oracle's, bit for bit, also where the
    order of the fp32 sum matters (values spread over 30 binades)."""
    from oracle import vortex_oracle as vo
    from vortex_torch.abs import FORMAT, as_vtensor
    from vortex_torch.abs.tensor import materialize

    g = torch.Generator().manual_seed(G)
    q = (torch.randn(6, G, 64, generator=g) * torch.exp2(torch.randint(-15, 15, (6, G, 64), generator=g).float())).to(dtype)
    want = vo.q_group_mean(q)
    eager = as_vtensor(q.clone(), FORMAT.BATCHED).mean(dim=1, keepdim=True)
    assert torch.equal(torch.Tensor(eager).view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                       want.view(torch.int16 if dtype == torch.bfloat16 else torch.int32))
    lazy_src = as_vtensor(q.clone(), FORMAT.BATCHED)
    lazy_src._vtx_allow_lazy_mean = True
    lazy = lazy_src.mean(dim=1, keepdim=True)
    assert torch.equal(torch.Tensor(materialize(lazy)), torch.Tensor(eager))
