"""Cache-side operators in every layout (PAGED / RAGGED operands and outputs) against the CPU oracle, bit for bit:
reductions (Mean / Max / Min / L2Norm over rows or columns), unary and binary elementwise, GeMM; and the operator
classes driven the way a flow's forward_cache drives them."""
import pytest
import torch

from oracle import vortex_oracle as vo
from vortex_torch import _cabi

pytestmark = pytest.mark.gpu

P, H, PAGES, NNZ = 16, 3, 20, 14


def _loc(seed=0):
    g = torch.Generator().manual_seed(seed)
    closing = torch.randperm(PAGES, generator=g)[:9] * P + (P - 1)
    other = torch.randperm(PAGES, generator=g)[:NNZ - 9] * P + 5
    return torch.cat([closing, other])[torch.randperm(NNZ, generator=g)]


def _operand(ragged, r, c, seed):
    rows = NNZ * H if ragged else PAGES * H
    return torch.randn(rows, r, c, generator=torch.Generator().manual_seed(seed)).bfloat16()


def _eq(a, b):
    return torch.equal(a.cpu().view(torch.int16), b.view(torch.int16))


@pytest.mark.parametrize("x_ragged", [False, True])
@pytest.mark.parametrize("out_ragged", [False, True])
@pytest.mark.parametrize("dim", [1, 2])
@pytest.mark.parametrize("kind", [vo.REDUCE_MEAN, vo.REDUCE_MAX, vo.REDUCE_MIN, vo.REDUCE_L2NORM])
def test_cache_reduce_every_layout(kind, dim, x_ragged, out_ragged):
    loc = _loc(1)
    x = _operand(x_ragged, P, 40, 2)
    shape = ((NNZ if out_ragged else PAGES) * H,) + ((1, 40) if dim == 1 else (P, 1))
    want = torch.full(shape, 3.0, dtype=torch.bfloat16)
    got = want.cuda()
    _cabi.cache_reduce(x.cuda(), got, loc.cuda(), H, P, dim, kind, x_ragged=x_ragged, out_ragged=out_ragged)
    vo.cache_reduce(x, want, loc, P, H, dim, kind, x_ragged=x_ragged, out_ragged=out_ragged)
    assert _eq(got, want)


def test_cache_reduce_agrees_with_the_tuned_mean_kernel():
    loc = _loc(3)
    x = _operand(False, P, 128, 4)
    a = torch.zeros(PAGES * H, 1, 128, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros_like(a)
    _cabi.cmean(x.cuda(), a, loc.cuda(), H, P)
    _cabi.cache_reduce(x.cuda(), b, loc.cuda(), H, P, 1, vo.REDUCE_MEAN)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


@pytest.mark.parametrize("layout", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("op,alpha,beta", [(0, 0.25, -1.0), (1, 0.5, 2.0), (2, 0.0, -1.0), (3, -0.75, 1.5), (4, 2.0, 0.5)])
def test_cache_elementwise_every_layout(op, alpha, beta, layout):
    loc = _loc(5)
    x = _operand(layout[0], 4, 24, 6)
    want = torch.full(((NNZ if layout[1] else PAGES) * H, 4, 24), 3.0, dtype=torch.bfloat16)
    got = want.cuda()
    _cabi.cache_elementwise(x.cuda(), got, loc.cuda(), H, P, op, alpha, beta, x_ragged=layout[0], out_ragged=layout[1])
    vo.cache_elementwise(x, want, loc, P, H, op, alpha, beta, x_ragged=layout[0], out_ragged=layout[1])
    assert _eq(got, want)


@pytest.mark.parametrize("layout", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("op,alpha,beta", [(0, 1, 1), (1, 1, 1), (2, 0.37, -2.5), (3, 1, 1)])
def test_cache_binary_every_layout(op, alpha, beta, layout):
    loc = _loc(7)
    x, y = _operand(layout[0], 4, 24, 8), _operand(layout[0], 1, 24, 9)
    want = torch.full(((NNZ if layout[1] else PAGES) * H, 4, 24), 3.0, dtype=torch.bfloat16)
    got = want.cuda()
    _cabi.cache_binary(x.cuda(), y.cuda(), got, loc.cuda(), H, P, op, alpha, beta, in_ragged=layout[0],
                       out_ragged=layout[1])
    vo.cache_binary(x, y, want, loc, P, H, op, alpha, beta, in_ragged=layout[0], out_ragged=layout[1])
    assert _eq(got, want)


@pytest.mark.parametrize("layout", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("nx,ny,k", [(16, 4, 128), (3, 5, 20)])
def test_cache_gemm_every_layout(nx, ny, k, layout):
    loc = _loc(11)
    x, y = _operand(layout[0], nx, k, 12), _operand(layout[0], ny, k, 13)
    want = torch.full(((NNZ if layout[1] else PAGES) * H, ny, nx), 3.0, dtype=torch.bfloat16)
    got = want.cuda()
    _cabi.cache_gemm(x.cuda(), y.cuda(), got, loc.cuda(), H, P, in_ragged=layout[0], out_ragged=layout[1])
    vo.cache_gemm(x, y, want, loc, P, H, in_ragged=layout[0], out_ragged=layout[1])
    assert _eq(got, want)


def test_cache_operator_classes_through_a_context():
    """The operator objects as a flow's forward_cache would use them: profile with tagged tensors, then execute."""
    from vortex_torch.abs import FORMAT, as_vtensor
    from vortex_torch.cache import Abs, GeMM, L2Norm, Maximum
    from vortex_torch.runtime import ServerArgs, VortexDecodeRuntime

    rt = VortexDecodeRuntime(1, H * 2, H, 128, num_pages=PAGES, max_bs=NNZ, context_len=PAGES * P,
                             server_args=ServerArgs(page_size=P, vortex_topk_val=4))
    ctx = rt.cctx
    loc = _loc(17)
    k = _operand(False, P, 128, 18).cuda()
    proj = _operand(False, 4, 128, 19).cuda()
    norms = torch.zeros(PAGES * H, P, 1, dtype=torch.bfloat16, device="cuda")
    ops = dict(l2=L2Norm(dim=2), mm=GeMM(), ab=Abs(), mx=Maximum())
    ctx.profile()
    t = lambda x: as_vtensor(x, FORMAT.PAGED)
    o1 = ops["l2"](t(k), t(norms), loc=loc.cuda(), ctx=ctx)
    o2 = ops["mm"](t(k), t(proj), None, loc=loc.cuda(), ctx=ctx)          # RAGGED buffer [max_new_tokens*H, 4, P]
    o3 = ops["ab"](o2, None, loc=loc.cuda(), ctx=ctx)
    o4 = ops["mx"](o2, o3, None, loc=loc.cuda(), ctx=ctx)
    assert o1._format == FORMAT.PAGED and o2._format == o3._format == o4._format == FORMAT.RAGGED
    assert tuple(o2.shape[1:]) == (4, P)
    ctx.execute()
    ops["l2"](k, norms, loc=loc.cuda(), ctx=ctx)
    mm = ops["mm"](k, proj, None, loc=loc.cuda(), ctx=ctx)
    ab = ops["ab"](mm, None, loc=loc.cuda(), ctx=ctx)
    mx = ops["mx"](mm, ab, None, loc=loc.cuda(), ctx=ctx)
    want_n = vo.cache_reduce(k.cpu(), torch.zeros(PAGES * H, P, 1, dtype=torch.bfloat16), loc, P, H, 2, vo.REDUCE_L2NORM)
    assert _eq(norms, want_n)
    rows = mm.shape[0]
    want_mm = vo.cache_gemm(k.cpu(), proj.cpu(), torch.zeros(rows, 4, P, dtype=torch.bfloat16), loc, P, H,
                            out_ragged=True)
    want_ab = vo.cache_elementwise(want_mm, torch.zeros_like(want_mm), loc, P, H, 3, 0.0, 1.0, x_ragged=True,
                                   out_ragged=True)
    want_mx = vo.cache_binary(want_mm, want_ab, torch.zeros_like(want_mm), loc, P, H, 0, in_ragged=True, out_ragged=True)
    touched = [r for _, r in vo._cache_items(loc, P, H)]
    assert _eq(mm[touched], want_mm[touched]) and _eq(ab[touched], want_ab[touched]) and _eq(mx[touched], want_mx[touched])


@pytest.mark.parametrize("alpha", [0.0, -1.0, 0.3, float("-inf")])
def test_cache_fill_in_place(alpha):
    """Fill(alpha): triggered blocks become bf16(alpha) even where they held NaN or inf; the others keep their bits."""
    from vortex_torch.abs import FORMAT, as_vtensor
    from vortex_torch.cache.fill import Fill
    from vortex_torch.runtime import ServerArgs, VortexDecodeRuntime

    rt = VortexDecodeRuntime(1, H * 2, H, 128, num_pages=PAGES, max_bs=NNZ, context_len=PAGES * P,
                             server_args=ServerArgs(page_size=P, vortex_topk_val=4))
    ctx = rt.cctx
    loc = _loc(23)
    x = _operand(False, 3, 40, 24)
    x[::2, 0, 0] = float("nan")
    x[1::2, 1, 1] = float("inf")
    want = vo.cache_fill(x.clone(), loc, P, H, alpha)
    xd = x.cuda()
    op = Fill(alpha)
    ctx.profile()
    assert op(as_vtensor(xd, FORMAT.PAGED), loc=loc.cuda(), ctx=ctx)._format == FORMAT.PAGED
    ctx.execute()
    assert op(xd, loc=loc.cuda(), ctx=ctx) is xd
    assert _eq(xd, want)
    assert len(list(vo._cache_items(loc, P, H))) == 9 * H
