"""Generate golden vectors from the reference project's own Triton kernels, run on CPU.

    TRITON_INTERPRET=1 python tests/golden/make_golden_ref_triton.py tests/golden/ref_triton_kernels.npz

Imports the reference package from its checkout (with an empty stand-in for its CUDA-only extension
module) and runs, under the Triton interpreter, the three Triton kernels of the decode path:
`mv_bpr_kernel` (indexer/triton_kernels/mv_impl.py), `reduce_pp_kernel` with Mean
(cache/triton_kernels/reduce_impl.py) and `set_kv_buffer_kernel` (cache/triton_kernels/set_kv.py).
Inputs are fp32 tensors holding bf16-representable values: the interpreter mishandles bf16 inputs, and
with fp32 inputs the kernels still round their outputs to bf16.  The reduction order of the interpreter
is numpy's, not a GPU's, so these vectors pin the oracle to within one bf16 ulp, not bit for bit.
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
from vortex_torch.cache.triton_kernels.set_kv import set_kv_buffer_launcher  # noqa: E402
from vortex_torch.indexer.triton_kernels.mv_impl import mv_bpr_kernel  # noqa: E402
from vortex_torch.utils import ReduceType  # noqa: E402


def main(out_path):
    assert vortex_torch.__file__.startswith(REF), "the reference package must be the one imported here"
    g = torch.Generator().manual_seed(2024)
    pages, H, P, D = 24, 2, 16, 128
    bf = lambda t: t.bfloat16().float()
    k = bf(torch.randn(pages * H, P, D, generator=g))
    # ---- CMean (reduce_pp, Mean, dim=1)
    cent = torch.zeros(pages * H, 1, D)
    loc = torch.tensor([15, 47, 40, 383, 200, 207, 95], dtype=torch.int64)
    _reduce_pp(k, cent, loc, H, P, 1, ReduceType.Mean)
    # ---- set_kv
    kc, vc = torch.zeros(pages * H, P, D), torch.zeros(pages * H, P, D)
    nk, nv = bf(torch.randn(9, H, D, generator=g)), bf(torch.randn(9, H, D, generator=g))
    sloc = torch.tensor([0, 17, 33, 100, 383, 250, 64, 65, 15], dtype=torch.int64)
    set_kv_buffer_launcher(kc, vc, nk, nv, sloc, P)
    # ---- GeMV (mv_bpr): 3 segments over a shared centroid table, two workload chunks each
    cents = bf(torch.randn(pages * H, 1, D, generator=g))
    x = bf(torch.randn(3, 1, D, generator=g))
    indices = torch.randperm(pages * H, generator=g)[:36].to(torch.int32)
    wq = torch.tensor([0, 0, 1, 1, 2, 2], dtype=torch.int32)
    woff = torch.tensor([0, 8, 12, 20, 24, 32], dtype=torch.int32)
    wlen = torch.tensor([8, 4, 8, 4, 8, 4], dtype=torch.int32)
    wn = torch.tensor([6], dtype=torch.int32)
    scores = torch.zeros(36, 1, 1)
    mv_bpr_kernel[(2,)](x, cents, scores, indices, wq, woff, wlen, wn, 8, D)
    np.savez_compressed(
        out_path, k=k.numpy(), cmean_loc=loc.numpy(), cmean_out=cent.numpy(), setkv_new_k=nk.numpy(),
        setkv_new_v=nv.numpy(), setkv_loc=sloc.numpy(), setkv_k=kc.numpy(), setkv_v=vc.numpy(),
        mv_centroids=cents.numpy(), mv_x=x.numpy(), mv_indices=indices.numpy(), mv_wq=wq.numpy(),
        mv_woff=woff.numpy(), mv_wlen=wlen.numpy(), mv_scores=scores.numpy(), H=np.asarray(H), P=np.asarray(P))
    print("wrote", out_path)


if __name__ == "__main__":
    main(sys.argv[1])
