"""Prefill-side helpers (planners and chunk-wise transposes) against the oracle and, when the cross-check
extension is built, against the reference project's own CUDA kernels - bit for bit in both cases."""
import numpy as np
import pytest
import torch

import vortex_torch_C as C
from oracle import build_ref
from oracle import vortex_oracle as vo

pytestmark = pytest.mark.gpu

CASES = [dict(cached=[40, 7, 128, 1, 300], inp=[8, 7, 100, 1, 33], P=4, H=2),
         dict(cached=[4096, 17, 513], inp=[4096, 17, 1], P=16, H=8),
         dict(cached=[100 + 3 * i for i in range(300)], inp=[1 + (i % 5) for i in range(300)], P=16, H=2)]


def _inputs(c):
    prob = vo.make_paged_problem(3, c["cached"], c["H"], 1, 8, c["P"], dtype=torch.float32)
    bs = len(c["cached"])
    order = np.random.default_rng(1).permutation(bs)
    r2t = np.zeros_like(prob["req_to_token"])
    r2t[order] = prob["req_to_token"]
    return r2t, order.astype(np.int64)


def _run_plan(mod, c, r2t, ridx):
    dev, i32 = "cuda", dict(dtype=torch.int32, device="cuda")
    bs, H, P = len(c["cached"]), c["H"], c["P"]
    n = (np.asarray(c["cached"]) + P - 1) // P
    out = dict(kv_indptr=torch.full((bs * H + 1,), -1, **i32), kv_indices=torch.full((int(n.sum()) * H,), -1, **i32),
               qo_ragged=torch.full((bs + 1,), -1, **i32), qo_paged=torch.full((bs * H + 1,), -1, **i32),
               last=torch.full((bs * H,), -1, **i32), table=torch.zeros(sum(c["inp"]), dtype=torch.uint16, device=dev))
    mod.sglang_plan_prefill(torch.tensor(c["cached"], **i32), out["kv_indptr"], out["kv_indices"],
                            torch.tensor(c["inp"], **i32), out["qo_ragged"], out["qo_paged"], out["last"],
                            torch.as_tensor(r2t, **i32), torch.as_tensor(ridx, device=dev), out["table"], P, H)
    torch.cuda.synchronize()
    return out


@pytest.fixture(scope="module")
def ref():
    return build_ref.load() if build_ref.built_module_path() is not None else None


@pytest.mark.parametrize("c", CASES, ids=lambda c: f"bs{len(c['cached'])}P{c['P']}H{c['H']}")
def test_plan_prefill(c, ref):
    r2t, ridx = _inputs(c)
    mine = _run_plan(C, c, r2t, ridx)
    want = vo.plan_prefill(c["cached"], c["inp"], r2t, ridx, c["P"], c["H"])
    for mk, wk in (("kv_indptr", "dense_kv_indptr"), ("kv_indices", "dense_kv_indices"), ("qo_ragged", "qo_indptr_ragged"),
                   ("qo_paged", "qo_indptr_paged"), ("last", "kv_last_page_len")):
        np.testing.assert_array_equal(mine[mk].cpu().numpy(), want[wk], err_msg=mk)
    np.testing.assert_array_equal(mine["table"].cpu().view(torch.int16).numpy().view(np.uint16), want["batch_table"])
    if ref is not None and len(c["cached"]) <= 1024:
        theirs = _run_plan(ref, c, r2t, ridx)
        for k in mine:
            assert torch.equal(mine[k].view(torch.int16) if mine[k].dtype == torch.uint16 else mine[k],
                               theirs[k].view(torch.int16) if theirs[k].dtype == torch.uint16 else theirs[k]), k


@pytest.mark.parametrize("c", CASES[:2], ids=lambda c: f"bs{len(c['cached'])}P{c['P']}H{c['H']}")
def test_plan_prefill_fa3(c, ref):
    r2t, ridx = _inputs(c)
    bs, H, P = len(c["cached"]), c["H"], c["P"]
    cached_seg = np.repeat(np.asarray(c["cached"], dtype=np.int32), H)
    cu = np.zeros(bs * H + 1, dtype=np.int32)
    cu[1:] = np.cumsum(np.repeat(np.asarray(c["inp"], dtype=np.int32), H))
    stride = int((max(c["cached"]) + P - 1) // P) + 2
    ntok = sum(c["inp"])
    want = vo.plan_prefill_fa3(cached_seg, cu, r2t, ridx, P, H, stride, ntok)
    res = {}
    for name, mod in (("mine", C), ("ref", ref)):
        if mod is None:
            continue
        pt = torch.full((bs * H, stride), -1, dtype=torch.int32, device="cuda")
        bt = torch.zeros(ntok, dtype=torch.uint16, device="cuda")
        mod.sglang_plan_prefill_fa3(torch.as_tensor(cached_seg).cuda(), torch.as_tensor(cu).cuda(),
                                    torch.as_tensor(r2t, dtype=torch.int32).cuda(), torch.as_tensor(ridx).cuda(), pt, bt, P, H)
        torch.cuda.synchronize()
        res[name] = (pt.cpu().numpy(), bt.cpu().view(torch.int16).numpy().view(np.uint16))
    np.testing.assert_array_equal(res["mine"][0], want["page_table"])
    np.testing.assert_array_equal(res["mine"][1], want["batch_table"])
    if "ref" in res:
        np.testing.assert_array_equal(res["mine"][0], res["ref"][0])
        np.testing.assert_array_equal(res["mine"][1], res["ref"][1])


@pytest.mark.parametrize("lens,H,G,D", [([5, 1, 17, 64], 8, 2, 128), ([300, 2], 2, 4, 64), ([33], 4, 1, 20)])
def test_chunkwise_transposes(lens, H, G, D, ref):
    g = torch.Generator().manual_seed(0)
    N = sum(lens)
    indptr = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    table = torch.repeat_interleave(torch.arange(len(lens)), torch.tensor(lens)).to(torch.int16).view(torch.uint16)
    x = torch.randn(N, H * G, D, generator=g).bfloat16()
    lse = torch.randn(N * H, G, generator=g)
    hm = C.Chunkwise_NH2HN_Transpose(x.cuda(), indptr.cuda(), table.cuda(), H * G, H, D)
    assert torch.equal(hm.cpu(), vo.chunkwise_nh2hn(x, indptr.tolist(), H))
    back, lse_tm = C.Chunkwise_HN2NH_Transpose(hm, lse.cuda(), indptr.cuda(), table.cuda(), H * G, H, D)
    assert torch.equal(back.cpu(), x)                                           # round trip
    assert torch.equal(lse_tm.cpu(), vo.chunkwise_hn2nh(lse, indptr.tolist(), H))
    back3 = C.Chunkwise_HN2NH_Transpose_FA3(hm, indptr.cuda(), table.cuda(), H * G, H, D)
    assert torch.equal(back3.cpu(), x)
    if ref is not None and D % 4 == 0:
        r_hm = ref.Chunkwise_NH2HN_Transpose(x.cuda(), indptr.cuda(), table.cuda(), H * G, H, D)
        r_back, r_lse = ref.Chunkwise_HN2NH_Transpose(r_hm, lse.cuda(), indptr.cuda(), table.cuda(), H * G, H, D)
        r_back3 = ref.Chunkwise_HN2NH_Transpose_FA3(r_hm, indptr.cuda(), table.cuda(), H * G, H, D)
        torch.cuda.synchronize()
        assert torch.equal(hm, r_hm) and torch.equal(back, r_back) and torch.equal(lse_tm, r_lse) and torch.equal(back3, r_back3)
