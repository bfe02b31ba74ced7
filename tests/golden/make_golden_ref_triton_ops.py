"""Generate golden vectors from the reference project's Triton kernels of the two other shipped flows,
run on CPU under the Triton interpreter.

    TRITON_INTERPRET=1 python tests/golden/make_golden_ref_triton_ops.py tests/golden/ref_triton_ops.npz

Imports the reference package from its checkout (with an empty stand-in for its CUDA-only extension
module) and runs the explicit-argument twins of its kernels:
  `_mm_bpr`                 indexer/triton_kernels/matmul_impl.py           (GeMM of gqa_block_sparse_attention)
  `_softmax_inplace_r`      indexer/triton_kernels/softmax_impl.py          (Softmax(dim=0, scale))
  `_reduce_rr`              indexer/triton_kernels/reduce_impl.py           (Max / Min / Mean / Sum / L2Norm, dim 1 and 2)
  `_elementwise_binary_bpr` indexer/triton_kernels/elementwise_binary_impl.py (Multiply, Maximum, Minimum on BATCHED x PAGED)
  `_elementwise_binary_rrr` same file                                       (Maximum, Minimum, Multiply on RAGGED x RAGGED)
  `_reduce_pp`              cache/triton_kernels/reduce_impl.py             (cache Max / Min / Mean / L2Norm, dim 1)
Inputs are fp32 tensors holding bf16-representable values (the interpreter mishandles bf16 inputs); kernels
that cast their result to bf16 still round it, kernels that rely on bf16 arithmetic (the elementwise ones)
return the unrounded fp32 value, which the tests round once.  Reductions run in numpy's order, so sums pin
the oracle to within one bf16 ulp, maxima / minima / products exactly.
"""
import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"
REF = os.environ.get("VORTEX_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference"))
sys.path.insert(0, REF)
stub = types.ModuleType("vortex_torch_C")
for n in ["sglang_plan_decode", "sglang_plan_prefill", "sglang_plan_decode_fa3", "sglang_plan_prefill_fa3",
          "Chunkwise_NH2HN_Transpose", "Chunkwise_HN2NH_Transpose", "Chunkwise_HN2NH_Transpose_FA3", "topk_output"]:
    setattr(stub, n, None)
sys.modules["vortex_torch_C"] = stub

import numpy as np  # noqa: E402
import torch  # noqa: E402
import vortex_torch  # noqa: E402,F401  (the reference package)
from vortex_torch.cache.triton_kernels.reduce_impl import _reduce_pp  # noqa: E402
from vortex_torch.indexer.triton_kernels.elementwise_binary_impl import (  # noqa: E402
    _elementwise_binary_bpr, _elementwise_binary_rrr)
from vortex_torch.indexer.triton_kernels.matmul_impl import _mm_bpr  # noqa: E402
from vortex_torch.indexer.triton_kernels.reduce_impl import _reduce_rr  # noqa: E402
from vortex_torch.indexer.triton_kernels.softmax_impl import _softmax_inplace_r  # noqa: E402
from vortex_torch.utils import ElementwiseBinaryOpType, ReduceType  # noqa: E402

# The interpreter of Triton 3.6 has no builder for bf16 constants, which the elementwise kernels create for
# alpha and beta (`tl.full((), alpha, dtype=tl.bfloat16)`) whatever the operator.  The operators recorded
# here (Mul, Maximum, Minimum) never read them, so a float32 constant in their place changes nothing.
from triton.runtime import interpreter as _interp  # noqa: E402

if not hasattr(_interp.InterpreterBuilder, "get_bf16"):
    _interp.InterpreterBuilder.get_bf16 = _interp.InterpreterBuilder.get_fp32


def main(out_path):
    assert vortex_torch.__file__.startswith(REF), "the reference package must be the one imported here"
    g = torch.Generator().manual_seed(777)
    bf = lambda t: t.bfloat16().float()
    i32 = lambda x: torch.tensor(x, dtype=torch.int32)
    out = {}
    # ---- layout of a small step: 3 segments with 14, 300 and 9 pages; bos = eos = 1, topk 4; candidates
    # 12, 298 and 7; workloads are chunks of at most 8 candidates starting behind the bos page
    bos, eos, topk, chunk, G, D = 1, 1, 4, 8, 4, 128
    seg_pages = [14, 300, 9]
    indptr = np.concatenate([[0], np.cumsum(seg_pages)]).astype(np.int32)
    total = int(indptr[-1])
    table_rows = 400
    indices = torch.randperm(table_rows, generator=g)[:total].to(torch.int32)
    wq, woff, wlen = [], [], []
    for s, n in enumerate(seg_pages):
        c = n - bos - eos
        if c <= topk:
            continue
        for o in range(0, c, chunk):
            wq.append(s); woff.append(int(indptr[s]) + bos + o); wlen.append(min(chunk, c - o))
    wn = i32([len(wq)])
    wq, woff, wlen = i32(wq), i32(woff), i32(wlen)
    out.update(indptr=indptr, indices=indices.numpy(), wq=wq.numpy(), woff=woff.numpy(), wlen=wlen.numpy(),
               bos=np.asarray(bos), eos=np.asarray(eos), topk=np.asarray(topk))
    # ---- GeMM (mm_bpr): o[row, 0, g] = y[row] . x[seg, g]
    x = bf(torch.randn(3, G, D, generator=g))
    y = bf(torch.randn(table_rows, 1, D, generator=g))
    mm = torch.zeros(total, 1, G)
    _mm_bpr(x, y, mm, indices, wq, woff, wlen, wn, chunk, 2)
    out.update(q=x.numpy(), table=y.numpy(), mm_out=mm.numpy())
    # ---- Softmax(dim=0, scale) in place over the candidates of every segment with more than topk of them
    sm = mm.clone()
    _softmax_inplace_r(sm, 0, torch.from_numpy(indptr), 0.09, bos, eos, topk, 3)
    out.update(softmax_scale=np.asarray(0.09, dtype=np.float32), softmax_out=sm.numpy())
    # ---- RAGGED reductions: Max over the heads (dim 2), then the whole family on a [*, G, 16] tensor
    mx = torch.zeros(total, 1, 1)
    _reduce_rr(sm, mx, 2, ReduceType.Max, woff, wlen, wn, chunk, 1)
    out.update(max_dim2_out=mx.numpy())
    r = bf(torch.randn(total, G, 16, generator=g))
    out.update(reduce_in=r.numpy())
    for name, rt in (("mean", ReduceType.Mean), ("max", ReduceType.Max), ("min", ReduceType.Min),
                     ("l2norm", ReduceType.L2Norm), ("sum", ReduceType.Sum)):
        o1 = torch.zeros(total, 1, 16)
        _reduce_rr(r, o1, 1, rt, woff, wlen, wn, chunk, 1)
        o2 = torch.zeros(total, G, 1)
        _reduce_rr(r, o2, 2, rt, woff, wlen, wn, chunk, 1)
        out[f"reduce_{name}_dim1"] = o1.numpy()
        out[f"reduce_{name}_dim2"] = o2.numpy()
    # ---- Multiply / Maximum / Minimum of BATCHED q with PAGED rows -> RAGGED [*, G, D]
    # (kept for the two short segments and the first 24 rows of the long one: the fixture stays small)
    keep = np.concatenate([np.arange(indptr[0], indptr[1]), np.arange(indptr[1], indptr[1] + 24),
                           np.arange(indptr[2], indptr[3])])
    out["bpr_rows"] = keep
    for name, op in (("mul", ElementwiseBinaryOpType.Mul), ("max", ElementwiseBinaryOpType.Maximum),
                     ("min", ElementwiseBinaryOpType.Minimum)):
        o = torch.zeros(total, G, D)
        _elementwise_binary_bpr(x, y, o, indices, wq, woff, wlen, wn, chunk, op, 1.0, 1.0, 1)
        out[f"bpr_{name}_out"] = o.numpy()[keep]
    # ---- RAGGED x RAGGED with broadcasting of the inner dims
    a = bf(torch.randn(total, G, 16, generator=g))
    b = bf(torch.randn(total, 1, 16, generator=g))
    out.update(rrr_a=a.numpy(), rrr_b=b.numpy())
    for name, op in (("mul", ElementwiseBinaryOpType.Mul), ("max", ElementwiseBinaryOpType.Maximum),
                     ("min", ElementwiseBinaryOpType.Minimum)):
        o = torch.zeros(total, G, 16)
        _elementwise_binary_rrr(a, b, o, woff, wlen, wn, chunk, op, 1.0, 1.0, 1)
        out[f"rrr_{name}_out"] = o.numpy()
    # ---- cache-side page reductions over the token axis
    pages, H, P = 12, 2, 16
    k = bf(torch.randn(pages * H, P, D, generator=g))
    loc = torch.tensor([15, 47, 40, 191, 100, 111], dtype=torch.int64)
    out.update(cache_k=k.numpy(), cache_loc=loc.numpy(), cache_H=np.asarray(H), cache_P=np.asarray(P))
    for name, rt in (("mean", ReduceType.Mean), ("max", ReduceType.Max), ("min", ReduceType.Min),
                     ("l2norm", ReduceType.L2Norm)):
        o = torch.zeros(pages * H, 1, D)
        _reduce_pp(k, o, loc, H, P, 1, rt)
        out[f"cache_{name}_out"] = o.numpy()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k: v.shape for k, v in out.items() if hasattr(v, "shape") and v.ndim})


if __name__ == "__main__":
    main(sys.argv[1])
