"""The vFlow plugin API end to end on the GPU: user-visible calls only, checked against the oracle."""
import math
import textwrap

import numpy as np
import pytest
import torch

from oracle import vortex_oracle as vo

pytestmark = pytest.mark.gpu


def _runtime(prob, seq, L, H, G, D, P, K, bos, eos, dtype, flow=None, skip=(0,)):
    from vortex_torch.runtime import ServerArgs, VortexDecodeRuntime

    sa = ServerArgs(page_size=P, vortex_topk_val=K, vortex_page_reserved_bos=bos, vortex_page_reserved_eos=eos,
                    vortex_layers_skip=list(skip), vortex_max_seq_lens=int(max(seq)))
    pages = prob["k"].shape[0] // H
    rt = VortexDecodeRuntime(L, H * G, H, D, num_pages=pages, max_bs=len(seq), context_len=int(max(seq)),
                             server_args=sa, dtype=dtype, flow=flow)
    rt.model_runner.req_to_token_pool.req_to_token.copy_(torch.as_tensor(prob["req_to_token"]))
    return rt


@pytest.mark.parametrize("dtype,seq", [(torch.float32, [4096]), (torch.bfloat16, [2048, 1000, 8192, 300])])
def test_runtime_step_matches_oracle(dtype, seq):
    """Two layers (layer 0 dense, layer 1 sparse), the new token closes a page when seq % P == 0."""
    L, H, G, D, P, K, bos, eos = 2, 8, 2, 128, 16, 30, 1, 1
    prob = vo.make_paged_problem(7, seq, H, G, D, P, dtype=dtype)
    rt = _runtime(prob, seq, L, H, G, D, P, K, bos, eos, dtype)
    bs = len(seq)
    g = torch.Generator().manual_seed(1)
    # caches hold everything except the newest token of each request; the step writes it
    loc = torch.as_tensor([int(prob["req_to_token"][r, seq[r] - 1]) for r in range(bs)], dtype=torch.int64)
    ks, vs, cents, qs, nks, nvs = [], [], [], [], [], []
    for l in range(L):
        pl = vo.make_paged_problem(100 + l, seq, H, G, D, P, dtype=dtype)
        k, v, cent = pl["k"], pl["v"], pl["centroids"]
        nk = torch.stack([k[(loc[r] // P) * H + torch.arange(H), loc[r] % P] for r in range(bs)])
        nv = torch.stack([v[(loc[r] // P) * H + torch.arange(H), loc[r] % P] for r in range(bs)])
        k0, v0, c0 = k.clone(), v.clone(), cent.clone()
        for r in range(bs):
            rows = (loc[r] // P) * H + torch.arange(H)
            k0[rows, loc[r] % P] = 0
            v0[rows, loc[r] % P] = 0
            c0[rows] = 0  # the centroid of a page closed by this step must come from forward_cache
        rt.pool.buffers[l]["k"].copy_(k0)
        rt.pool.buffers[l]["v"].copy_(v0)
        rt.pool.buffers[l]["centroids"].copy_(c0)
        ks.append(k); vs.append(v); cents.append(cent)
        qs.append(torch.randn(bs, H * G, D, generator=g).to(dtype)); nks.append(nk); nvs.append(nv)
    outs = [torch.empty(bs, H * G, D, dtype=dtype, device="cuda") for _ in range(L)]
    rt.flow.gemv.output_buffer.fill_(-7.0)
    rt.step(torch.as_tensor(prob["seq_lens"]).cuda(), torch.as_tensor(prob["req_indices"]).cuda(),
            [q.cuda() for q in qs], [x.cuda() for x in nks], [x.cuda() for x in nvs], loc.cuda(), outs)
    torch.cuda.synchronize()
    ref = vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], P, H, K, bos, eos, 64, 16)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    for l in range(L):
        assert torch.equal(rt.pool.buffers[l]["k"].cpu(), ks[l])
        full = [r for r in range(bs) if seq[r] % P == 0]
        for r in full:
            rows = (loc[r] // P) * H + torch.arange(H)
            assert torch.equal(rt.pool.buffers[l]["centroids"].cpu()[rows], cents[l][rows])
        qv = qs[l].view(bs * H, G, D)
        if l == 0:
            want = vo.decode_gqa(qv, ks[l], vs[l], ref["dense_kv_indptr"], ref["dense_kv_indices"], ref["kv_last_page_len"])
        else:
            plan = {k_: v_.copy() for k_, v_ in ref.items()}
            vo.forward_indexer(qv, cents[l], plan, K, bos, eos)
            ns = int(plan["sparse_kv_indptr"][-1])
            np.testing.assert_array_equal(rt.backend.kv_indices_decode[1].cpu().numpy()[:ns], plan["sparse_kv_indices"])
            want = vo.decode_gqa(qv, ks[l], vs[l], plan["sparse_kv_indptr"], plan["sparse_kv_indices"], plan["kv_last_page_len"])
        got = outs[l].view(bs * H, G, D).cpu().float()
        assert bool(((got - want.float()).abs() <= tol * want.float().abs().clamp(min=1)).all())
    # the fused indexer path was taken: the GeMV never wrote its score buffer
    assert rt.flow.gemv._fused_consumer is rt.flow.output_func and not rt.flow.gemv._score_read_elsewhere
    assert bool((rt.flow.gemv.output_buffer == -7.0).all())


def test_user_flow_file_runs_unfused_when_scores_are_read(tmp_path):
    """A user flow that touches the scores with a torch op must fall back to GeMV + topK, same selection."""
    from vortex_torch.flow import build_vflow

    src = textwrap.dedent('''
        import torch
        from vortex_torch.flow import vFlow, register
        from vortex_torch.indexer import GeMV, topK
        from vortex_torch.cache import Mean as CMean

        @register("probe_reads_scores")
        class Probe(vFlow):
            def __init__(self, shift=0.0):
                super().__init__()
                self.gemv, self.output_func, self.reduction, self.shift = GeMV(), topK(), CMean(dim=1), shift
                self.seen = None
            def forward_indexer(self, q, o, cache, ctx):
                score = self.gemv(q.mean(dim=1, keepdim=True), cache["centroids"], ctx=ctx)
                self.seen = score.abs().sum()            # plain torch read of the scores
                self.output_func(score, o, ctx=ctx)
            def forward_cache(self, cache, loc, ctx):
                self.reduction(cache["k"], cache["centroids"], loc=loc, ctx=ctx)
            def create_cache(self, page_size, head_dim):
                return {"centroids": (1, head_dim)}
    ''')
    f = tmp_path / "probe_flow.py"
    f.write_text(src)
    flow = build_vflow("probe_reads_scores", {"shift": 1.0}, str(f))
    seq, L, H, G, D, P, K = [2048, 900], 1, 4, 2, 128, 16, 10
    prob = vo.make_paged_problem(3, seq, H, G, D, P)
    rt = _runtime(prob, seq, L, H, G, D, P, K, 1, 1, torch.bfloat16, flow=flow, skip=())
    assert flow.gemv._score_read_elsewhere
    for name in ("k", "v", "centroids"):
        rt.pool.buffers[0][name].copy_(prob[name])
    rt.plan(torch.as_tensor(prob["seq_lens"]).cuda(), torch.as_tensor(prob["req_indices"]).cuda())
    q = prob["q"].cuda()
    flow.forward_indexer(q, rt.backend.kv_indices_decode[1].view(-1, 1, 1), rt.pool.buffers[0], ctx=rt.ictx)
    ref = vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], P, H, K, 1, 1, 64, 16)
    vo.forward_indexer(prob["q"], prob["centroids"], ref, K, 1, 1)
    ns = int(ref["sparse_kv_indptr"][-1])
    np.testing.assert_array_equal(rt.backend.kv_indices_decode[1].cpu().numpy()[:ns], ref["sparse_kv_indices"])
    assert float(flow.seen) > 0


def test_vortex_torch_C_shim_signatures():
    """The pybind-module names of the reference, called with its positional argument order."""
    import vortex_torch_C as C

    P, H, K, bos, eos = 16, 2, 4, 1, 1
    prob = vo.make_paged_problem(1, [700, 40], H, 2, 128, P)
    ref = vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], P, H, K, bos, eos, 64, 16)
    i32 = dict(dtype=torch.int32, device="cuda")
    S = 2 * H
    dip, sip = torch.zeros(S + 1, **i32), torch.zeros(S + 1, **i32)
    din, sin_ = torch.zeros(4096, **i32), torch.full((256,), -1, **i32)
    last = torch.zeros(S, **i32)
    w = [torch.zeros(512, **i32) for _ in range(3)] + [torch.zeros(1, **i32), torch.zeros(1, **i32)]
    C.sglang_plan_decode(torch.as_tensor(prob["seq_lens"]).cuda(), dip, din, sip, sin_, last,
                         torch.as_tensor(prob["req_to_token"]).cuda(), torch.as_tensor(prob["req_indices"]).cuda(),
                         *w, P, H, K, bos, eos, 64, 16)
    np.testing.assert_array_equal(dip.cpu().numpy(), ref["dense_kv_indptr"])
    scores = vo.forward_indexer(prob["q"], prob["centroids"], ref, K, bos, eos)
    C.topk_output(scores.cuda(), dip, sip, din, sin_, S, K, bos, eos, 64)
    ns = int(ref["sparse_kv_indptr"][-1])
    np.testing.assert_array_equal(sin_.cpu().numpy()[:ns], ref["sparse_kv_indices"])


@pytest.mark.parametrize("flow_name", ["block_sparse_attention", "gqa_block_sparse_attention",
                                       "gqa_quest_sparse_attention"])
def test_graphed_step_with_programmatic_launch_matches_eager(flow_name):
    """The CUDA-graph replay of a step, kernels chained by programmatic dependent launch (with and without the
    early prologue of the layer kernel), gives the eager results bit for bit over repeated replays, for each of
    the three shipped flows."""
    from vortex_torch.flow import build_vflow
    from vortex_torch.runtime import GraphedDecodeStep

    seq, L, H, G, D, P, K = [2048, 1000, 4096, 300], 4, 8, 2, 128, 16, 30
    prob = vo.make_paged_problem(17, seq, H, G, D, P)
    rt = _runtime(prob, seq, L, H, G, D, P, K, 1, 1, torch.bfloat16, flow=build_vflow(flow_name))
    for l in range(L):
        pl = vo.make_paged_problem(200 + l, seq, H, G, D, P)
        for name, buf in rt.pool.buffers[l].items():
            # k, v and whatever page summaries the flow keeps (seeded with something page-shaped)
            buf.copy_(pl[name] if name in pl else pl["centroids"] * (1.5 if "max" in name else 0.5))
    bs = len(seq)
    step = GraphedDecodeStep(rt, bs)
    step.seq_lens.copy_(torch.as_tensor(prob["seq_lens"]))
    step.req_indices.copy_(torch.as_tensor(prob["req_indices"]))
    step.loc.copy_(torch.as_tensor([int(prob["req_to_token"][r, seq[r] - 1]) for r in range(bs)]))
    step.q.normal_(); step.new_k.normal_(); step.new_v.normal_()
    step.replay()  # eager: no graph yet
    torch.cuda.synchronize()
    want_out, want_sel = step.out.clone(), rt.backend.kv_indices_decode[1].clone()
    for pdl in (0, 1, 2):
        step.graph = None
        step.capture(programmatic_launch=pdl)
        for _ in range(5):
            step.out.zero_()
            rt.backend.kv_indices_decode[1].fill_(-1)
            step.replay()
        torch.cuda.synchronize()
        assert torch.equal(step.out, want_out), f"graph replay differs (programmatic_launch={pdl})"
        ns = int(rt.backend.kv_indptr_decode[1][bs * H].item())
        assert torch.equal(rt.backend.kv_indices_decode[1][:ns], want_sel[:ns])


def test_host_pipeline_graph_matches_device_path():
    """run_from_host through the overlapped copy/compute graph returns what the device-resident replay gives."""
    from vortex_torch.runtime import GraphedDecodeStep

    seq, L, H, G, D, P, K = [2048, 1000, 4096], 4, 8, 2, 128, 16, 30
    prob = vo.make_paged_problem(19, seq, H, G, D, P)
    rt = _runtime(prob, seq, L, H, G, D, P, K, 1, 1, torch.bfloat16)
    for l in range(L):
        pl = vo.make_paged_problem(300 + l, seq, H, G, D, P)
        for name in ("k", "v", "centroids"):
            rt.pool.buffers[l][name].copy_(pl[name])
    bs = len(seq)
    step = GraphedDecodeStep(rt, bs)
    h = step.host_buffers()
    g = torch.Generator().manual_seed(0)
    h["seq_lens"].copy_(torch.as_tensor(prob["seq_lens"]))
    h["req_indices"].copy_(torch.as_tensor(prob["req_indices"]))
    h["loc"].copy_(torch.as_tensor([int(prob["req_to_token"][r, seq[r] - 1]) for r in range(bs)]))
    for n in ("q", "new_k", "new_v"):
        h[n].copy_(torch.randn(h[n].shape, generator=g).bfloat16())
    want = step.run_from_host().clone()      # plain copies + eager kernels
    for pdl in (0, 2):
        step.capture_host_pipeline(programmatic_launch=pdl)
        for _ in range(3):
            h["out"].zero_()
            got = step.run_from_host()
        assert torch.equal(got, want), f"host pipeline differs (programmatic_launch={pdl})"


@pytest.mark.parametrize("fuse", [True, False])
def test_gqa_block_sparse_flow_through_runtime(fuse, monkeypatch):
    """The shipped gqa_block_sparse_attention flow (GeMM -> Softmax -> Max -> topK; CMean) run by the
    runtime: selections bit-exact with the oracle's restatement of that flow, attention within tolerance.
    With fusion on, every sparse layer must be ONE launch (token write + selection + attention)."""
    from vortex_torch import _cabi
    from vortex_torch.flow import build_vflow

    fused_calls = []
    real = _cabi.sparse_layer_fused

    def counting(*args, **kwargs):
        fused_calls.append(kwargs.get("gqa_softmax_scale"))
        return real(*args, **kwargs)

    monkeypatch.setattr(_cabi, "sparse_layer_fused", counting)

    seq, L, H, G, D, P, K, bos, eos = [2048, 1000, 4096, 300], 2, 8, 2, 128, 16, 30, 1, 1
    prob = vo.make_paged_problem(37, seq, H, G, D, P)
    flow = build_vflow("gqa_block_sparse_attention")
    rt = _runtime(prob, seq, L, H, G, D, P, K, bos, eos, torch.bfloat16, flow=flow)
    rt.fuse_attention = fuse
    assert flow.output_func._gqa_chain is not None
    for l in range(L):
        for name in ("k", "v", "centroids"):
            rt.pool.buffers[l][name].copy_(prob[name])
    bs = len(seq)
    loc = torch.as_tensor([int(prob["req_to_token"][r, seq[r] - 1]) for r in range(bs)], dtype=torch.int64)
    nk = torch.stack([prob["k"][(loc[r] // P) * H + torch.arange(H), loc[r] % P] for r in range(bs)]).cuda()
    nv = torch.stack([prob["v"][(loc[r] // P) * H + torch.arange(H), loc[r] % P] for r in range(bs)]).cuda()
    q = prob["q"].view(bs, H * G, D).cuda()
    outs = [torch.empty_like(q) for _ in range(L)]
    rt.step(torch.as_tensor(prob["seq_lens"]).cuda(), torch.as_tensor(prob["req_indices"]).cuda(), [q] * L, [nk] * L,
            [nv] * L, loc.cuda(), outs)
    torch.cuda.synchronize()
    plan = vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], P, H, K, bos, eos, 64, 16)
    assert fused_calls == ([pytest.approx(0.09)] * (L - 1) if fuse else []), fused_calls
    vo.forward_indexer_gqa(prob["q"], prob["centroids"], plan, K, bos, eos, scale=0.09)
    ns = int(plan["sparse_kv_indptr"][-1])
    np.testing.assert_array_equal(rt.backend.kv_indices_decode[1].cpu().numpy()[:ns], plan["sparse_kv_indices"])
    want = vo.decode_gqa(prob["q"], prob["k"], prob["v"], plan["sparse_kv_indptr"], plan["sparse_kv_indices"],
                         plan["kv_last_page_len"])
    got = outs[1].view(bs * H, G, D).float().cpu()
    assert bool(((got - want.float()).abs() <= 2e-2 * want.float().abs().clamp(min=1)).all())


@pytest.mark.parametrize("fuse", [True, False])
def test_gqa_quest_flow_through_runtime(fuse, monkeypatch):
    """The shipped gqa_quest_sparse_attention flow (CMax/CMin caches; Multiply x2 -> Maximum -> Sum -> Max ->
    topK) run by the runtime: envelopes of the page the step closes exact, selections bit-exact with the oracle.
    With fusion on, every sparse layer must be ONE launch (token write + both envelopes + selection + attention)."""
    from vortex_torch import _cabi
    from vortex_torch.flow import build_vflow

    fused_calls = []
    real = _cabi.sparse_layer_fused

    def counting(*args, **kwargs):
        fused_calls.append((kwargs.get("quest_min") is not None, kwargs.get("new_k") is not None or len(args) > 17))
        return real(*args, **kwargs)

    monkeypatch.setattr(_cabi, "sparse_layer_fused", counting)

    seq, L, H, G, D, P, K, bos, eos = [2048, 1000, 4096, 300], 2, 8, 2, 128, 16, 30, 1, 1
    prob = vo.make_paged_problem(38, seq, H, G, D, P)
    kf = prob["k"].float()
    cmax, cmin = kf.max(1, keepdim=True).values.bfloat16(), kf.min(1, keepdim=True).values.bfloat16()
    flow = build_vflow("gqa_quest_sparse_attention")
    rt = _runtime(prob, seq, L, H, G, D, P, K, bos, eos, torch.bfloat16, flow=flow)
    rt.fuse_attention = fuse
    assert flow.output_func._quest_chain is not None
    bs = len(seq)
    loc = torch.as_tensor([int(prob["req_to_token"][r, seq[r] - 1]) for r in range(bs)], dtype=torch.int64)
    closing_rows = torch.cat([(loc[r] // P) * H + torch.arange(H) for r in range(bs) if seq[r] % P == 0])
    for l in range(L):
        rt.pool.buffers[l]["k"].copy_(prob["k"]); rt.pool.buffers[l]["v"].copy_(prob["v"])
        c0, c1 = cmax.clone(), cmin.clone()
        c0[closing_rows] = 0; c1[closing_rows] = 0      # must be produced by forward_cache during the step
        rt.pool.buffers[l]["max"].copy_(c0); rt.pool.buffers[l]["min"].copy_(c1)
    nk = torch.stack([prob["k"][(loc[r] // P) * H + torch.arange(H), loc[r] % P] for r in range(bs)]).cuda()
    nv = torch.stack([prob["v"][(loc[r] // P) * H + torch.arange(H), loc[r] % P] for r in range(bs)]).cuda()
    q = prob["q"].view(bs, H * G, D).cuda()
    outs = [torch.empty_like(q) for _ in range(L)]
    rt.step(torch.as_tensor(prob["seq_lens"]).cuda(), torch.as_tensor(prob["req_indices"]).cuda(), [q] * L, [nk] * L,
            [nv] * L, loc.cuda(), outs)
    torch.cuda.synchronize()
    assert fused_calls == ([(True, True)] * (L - 1) if fuse else []), fused_calls
    assert torch.equal(rt.pool.buffers[1]["max"].cpu()[closing_rows], cmax[closing_rows])
    assert torch.equal(rt.pool.buffers[1]["min"].cpu()[closing_rows], cmin[closing_rows])
    plan = vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], P, H, K, bos, eos, 64, 16)
    vo.forward_indexer_quest(prob["q"], cmax, cmin, plan, K, bos, eos)
    ns = int(plan["sparse_kv_indptr"][-1])
    np.testing.assert_array_equal(rt.backend.kv_indices_decode[1].cpu().numpy()[:ns], plan["sparse_kv_indices"])
    want = vo.decode_gqa(prob["q"], prob["k"], prob["v"], plan["sparse_kv_indptr"], plan["sparse_kv_indices"],
                         plan["kv_last_page_len"])
    got = outs[1].view(bs * H, G, D).float().cpu()
    assert bool(((got - want.float()).abs() <= 2e-2 * want.float().abs().clamp(min=1)).all())


@pytest.mark.parametrize("op,alpha,beta", [(0, 0.0, 0.0), (0, 0.5, -2.0), (1, 0.0, -1.0), (1, 0.3, 0.7), (2, 0.0, -1.0),
                                           (3, 0.0, 1.0), (3, 0.7, -1.3), (4, 1.5, 0.3)])
def test_elementwise_kernel_matches_oracle(op, alpha, beta):
    """vtx_elementwise on the packed rows of a RAGGED tensor: bit-exact with the oracle, rows past the packed
    count untouched, odd element counts (tail path) included."""
    from vortex_torch import _cabi

    g = torch.Generator().manual_seed(5 + op)
    for S, C, D, rows in ((4096, 1, 1, 3001), (1024, 2, 3, 777), (64, 1, 8, 64)):
        x = (torch.randn(S, C, D, generator=g) * 4).bfloat16()
        x[0, 0, 0] = 300.0
        x[1 % S, 0, 0] = -300.0
        out = torch.full((S, C, D), 7.0, dtype=torch.bfloat16, device="cuda")
        count = torch.tensor([rows], dtype=torch.int32, device="cuda")
        _cabi.elementwise(x.cuda(), out, count, op, alpha, beta)
        want = vo.elementwise(x[:rows], op, alpha, beta)
        got = out.cpu()
        assert torch.equal(got[:rows].view(torch.int16), want.view(torch.int16)), (op, S, C, D)
        assert bool((got[rows:] == 7.0).all())


def test_user_flow_with_elementwise_between_gemv_and_topk(tmp_path):
    """GeMV -> Abs -> topK as a user flow: the scores are written, transformed by the elementwise kernel and
    selected by the stand-alone top-k; selections equal the oracle's on |score|."""
    from vortex_torch.flow import build_vflow

    src = textwrap.dedent('''
        from vortex_torch.flow import vFlow, register
        from vortex_torch.indexer import GeMV, topK, Abs
        from vortex_torch.cache import Mean as CMean

        @register("probe_abs_scores")
        class Probe(vFlow):
            def __init__(self):
                super().__init__()
                self.gemv, self.act, self.output_func, self.reduction = GeMV(), Abs(), topK(), CMean(dim=1)
            def forward_indexer(self, q, o, cache, ctx):
                score = self.gemv(q.mean(dim=1, keepdim=True), cache["centroids"], ctx=ctx)
                self.output_func(self.act(score, ctx=ctx), o, ctx=ctx)
            def forward_cache(self, cache, loc, ctx):
                self.reduction(cache["k"], cache["centroids"], loc=loc, ctx=ctx)
            def create_cache(self, page_size, head_dim):
                return {"centroids": (1, head_dim)}
    ''')
    f = tmp_path / "probe_abs_flow.py"
    f.write_text(src)
    flow = build_vflow("probe_abs_scores", {}, str(f))
    seq, L, H, G, D, P, K = [2048, 900], 1, 4, 2, 128, 16, 10
    prob = vo.make_paged_problem(4, seq, H, G, D, P)
    rt = _runtime(prob, seq, L, H, G, D, P, K, 1, 1, torch.bfloat16, flow=flow, skip=())
    assert flow.gemv._score_read_elsewhere
    for name in ("k", "v", "centroids"):
        rt.pool.buffers[0][name].copy_(prob[name])
    rt.plan(torch.as_tensor(prob["seq_lens"]).cuda(), torch.as_tensor(prob["req_indices"]).cuda())
    flow.forward_indexer(prob["q"].cuda(), rt.backend.kv_indices_decode[1].view(-1, 1, 1), rt.pool.buffers[0],
                         ctx=rt.ictx)
    ref = vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], P, H, K, 1, 1, 64, 16)
    eff_bs = prob["q"].shape[0]
    scores = vo.gemv_scores(vo.q_group_mean(prob["q"]), prob["centroids"], ref["dense_kv_indptr"],
                            ref["dense_kv_indices"], eff_bs, K, 1, 1)
    vo.topk_select(vo.elementwise(scores.view(-1, 1, 1), 3, 0.0, 1.0).view(-1), ref["dense_kv_indptr"],
                   ref["sparse_kv_indptr"], ref["dense_kv_indices"], ref["sparse_kv_indices"], eff_bs, K, 1, 1)
    ns = int(ref["sparse_kv_indptr"][-1])
    np.testing.assert_array_equal(rt.backend.kv_indices_decode[1].cpu().numpy()[:ns], ref["sparse_kv_indices"])


@pytest.mark.parametrize("op,alpha,beta", [(0, 1.0, 1.0), (1, 1.0, 1.0), (2, 1.0, 1.0), (2, 0.3, -1.7), (3, 1.0, 1.0)])
def test_elementwise_binary_kernel_matches_oracle(op, alpha, beta):
    """vtx_elementwise_binary on packed rows, same-shape and broadcast inner dims: bit-exact with the oracle."""
    from vortex_torch import _cabi

    g = torch.Generator().manual_seed(11 + op)
    for S, xs, ys, rows in ((2048, (1, 1), (1, 1), 1999), (512, (2, 8), (2, 8), 300), (512, (2, 8), (1, 8), 512),
                            (256, (4, 1), (1, 16), 77)):
        x = (torch.randn(S, *xs, generator=g) * 3).bfloat16()
        y = (torch.randn(S, *ys, generator=g) * 3).bfloat16()
        oc, od = max(xs[0], ys[0]), max(xs[1], ys[1])
        out = torch.full((S, oc, od), 7.0, dtype=torch.bfloat16, device="cuda")
        count = torch.tensor([rows], dtype=torch.int32, device="cuda")
        _cabi.elementwise_binary(x.cuda(), y.cuda(), out, count, op, alpha, beta)
        want = vo.elementwise_binary(x[:rows], y[:rows], op, alpha, beta)
        got = out.cpu()
        assert torch.equal(got[:rows].view(torch.int16), want.view(torch.int16)), (op, xs, ys)
        assert bool((got[rows:] == 7.0).all())


def test_user_flow_adding_two_score_sets(tmp_path):
    """Two GeMV score sets (group mean against the centroids, first query head against the centroids) combined by
    Add and selected by topK: a flow outside the shipped ones, run through the plugin API."""
    from vortex_torch.flow import build_vflow

    src = textwrap.dedent('''
        from vortex_torch.flow import vFlow, register
        from vortex_torch.indexer import GeMV, topK, Add
        from vortex_torch.cache import Mean as CMean

        @register("probe_two_scores")
        class Probe(vFlow):
            def __init__(self):
                super().__init__()
                self.g0, self.g1, self.add, self.output_func, self.reduction = GeMV(), GeMV(), Add(0.5, 2.0), topK(), CMean(dim=1)
            def forward_indexer(self, q, o, cache, ctx):
                a = self.g0(q.mean(dim=1, keepdim=True), cache["centroids"], ctx=ctx)
                b = self.g1(q[:, :1].contiguous(), cache["centroids"], ctx=ctx)
                self.output_func(self.add(a, b, ctx=ctx), o, ctx=ctx)
            def forward_cache(self, cache, loc, ctx):
                self.reduction(cache["k"], cache["centroids"], loc=loc, ctx=ctx)
            def create_cache(self, page_size, head_dim):
                return {"centroids": (1, head_dim)}
    ''')
    f = tmp_path / "probe_two_scores.py"
    f.write_text(src)
    flow = build_vflow("probe_two_scores", {}, str(f))
    seq, L, H, G, D, P, K = [2048, 900], 1, 4, 2, 128, 16, 10
    prob = vo.make_paged_problem(6, seq, H, G, D, P)
    rt = _runtime(prob, seq, L, H, G, D, P, K, 1, 1, torch.bfloat16, flow=flow, skip=())
    for name in ("k", "v", "centroids"):
        rt.pool.buffers[0][name].copy_(prob[name])
    rt.plan(torch.as_tensor(prob["seq_lens"]).cuda(), torch.as_tensor(prob["req_indices"]).cuda())
    flow.forward_indexer(prob["q"].cuda(), rt.backend.kv_indices_decode[1].view(-1, 1, 1), rt.pool.buffers[0],
                         ctx=rt.ictx)
    ref = vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], P, H, K, 1, 1, 64, 16)
    eff_bs = prob["q"].shape[0]
    args = (ref["dense_kv_indptr"], ref["dense_kv_indices"], eff_bs, K, 1, 1)
    sa = vo.gemv_scores(vo.q_group_mean(prob["q"]), prob["centroids"], *args)
    sb = vo.gemv_scores(prob["q"][:, :1].contiguous(), prob["centroids"], *args)
    comb = vo.elementwise_binary(sa.view(-1, 1, 1), sb.view(-1, 1, 1), 2, 0.5, 2.0).view(-1)
    vo.topk_select(comb, ref["dense_kv_indptr"], ref["sparse_kv_indptr"], ref["dense_kv_indices"],
                   ref["sparse_kv_indices"], eff_bs, K, 1, 1)
    ns = int(ref["sparse_kv_indptr"][-1])
    np.testing.assert_array_equal(rt.backend.kv_indices_decode[1].cpu().numpy()[:ns], ref["sparse_kv_indices"])
