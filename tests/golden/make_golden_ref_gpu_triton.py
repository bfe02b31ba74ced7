"""Record what the reference project's own GPU kernels compute on bf16 inputs (run on a B200).

    VORTEX_REFERENCE_DIR=<checkout of the reference> python tests/golden/make_golden_ref_gpu_triton.py <output.npz>

Imports the reference package from its checkout with, in place of its pybind module, the cross-check
extension built by oracle/build_ref.py (the reference's csrc/topk.cu and csrc/utils_sglang.cu compiled for
sm_100), JIT-compiles its Triton kernels for the GPU at hand and runs, on a seeded bf16 batch of the config-2
shape (8 KV heads, group 2, head_dim 128, page 16, top-k 30 + 1 + 1):
  `mv_bpr_kernel`     indexer/triton_kernels/mv_impl.py      (the GeMV of block_sparse_attention)
  `topk_output`       csrc/topk.cu                           (on the reference's own scores)
  `reduce_pp_kernel`  cache/triton_kernels/reduce_impl.py    (cache Mean: the reference sums in bf16)
The inputs come from `oracle.make_paged_problem(seed, ...)`, so the file only needs to hold the outputs: the
reference's scores (bf16 bit patterns) and selected rows, and its centroids for a few completed pages.
tests/test_golden.py compares the CPU oracle with them and reports how often the two agree.
"""
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import build_ref  # noqa: E402
from oracle import vortex_oracle as vo  # noqa: E402

REF = os.environ.get("VORTEX_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference"))
SEED, SEQ, H, G, D, P, K, BOS, EOS, CHUNK = 71, [8192, 8192, 5000, 700], 8, 2, 128, 16, 30, 1, 1, 64


def main(out_path):
    ext = build_ref.load()
    assert ext is not None, "build oracle/_ref first (python oracle/build_ref.py)"
    sys.modules["vortex_torch_C"] = ext
    sys.path.insert(0, REF)
    import vortex_torch  # the reference package
    assert os.path.realpath(vortex_torch.__file__).startswith(os.path.realpath(REF))
    from vortex_torch.cache.triton_kernels.reduce_impl import _reduce_pp
    from vortex_torch.indexer.triton_kernels.mv_impl import mv_bpr_kernel
    from vortex_torch.utils import ReduceType

    dev, i32 = "cuda", dict(dtype=torch.int32, device="cuda")
    prob = vo.make_paged_problem(SEED, SEQ, H, G, D, P)
    plan = vo.plan_decode(prob["seq_lens"], prob["req_to_token"], prob["req_indices"], P, H, K, BOS, EOS, CHUNK, 16)
    S = len(SEQ) * H
    dip = torch.as_tensor(plan["dense_kv_indptr"], **i32)
    sip = torch.as_tensor(plan["sparse_kv_indptr"], **i32)
    din = torch.as_tensor(plan["dense_kv_indices"], **i32)
    nw = int(plan["winfo_num_workloads"][0])
    wq = torch.as_tensor(plan["winfo_q_indices"][:nw], **i32)
    woff = torch.as_tensor(plan["winfo_kv_offsets"][:nw], **i32)
    wlen = torch.as_tensor(plan["winfo_kv_lens"][:nw], **i32)
    wn = torch.tensor([nw], **i32)
    cent = prob["centroids"].to(dev)
    # ---- GeMV: x = grouped-query mean (torch's own mean, as the reference flow computes it)
    q = prob["q"].to(dev)
    x = q.mean(dim=1, keepdim=True)
    scores = torch.zeros(int(dip[-1]), 1, 1, dtype=torch.bfloat16, device=dev)
    num_sms = torch.cuda.get_device_properties(0).multi_processor_count
    mv_bpr_kernel[(4 * num_sms,)](x, cent, scores, din, wq, woff, wlen, wn, CHUNK, D, num_warps=8, num_stages=2)
    # ---- top-k on the reference's scores
    sel = torch.as_tensor(plan["sparse_kv_indices"], **i32).clone()
    max_pages = (max(SEQ) + P - 1) // P
    ext.topk_output(scores, dip, sip, din, sel, S, K, BOS, EOS, max_pages)
    # ---- cache Mean on a few completed pages of request 0
    k = prob["k"].to(dev)
    loc = torch.as_tensor([int(prob["req_to_token"][0, t]) for t in (15, 31, 4095, 8191, 100)], dtype=torch.int64,
                          device=dev)
    cm = torch.zeros_like(cent)
    _reduce_pp(k, cm, loc, H, P, 1, ReduceType.Mean)
    torch.cuda.synchronize()
    rows = torch.nonzero(cm.abs().sum(dim=(1, 2)) > 0).view(-1)
    np.savez_compressed(
        out_path, seed=np.asarray(SEED), seq=np.asarray(SEQ), H=np.asarray(H), G=np.asarray(G), D=np.asarray(D),
        P=np.asarray(P), K=np.asarray(K), bos=np.asarray(BOS), eos=np.asarray(EOS), chunk=np.asarray(CHUNK),
        q_mean_bits=x.view(torch.int16).cpu().numpy(), scores_bits=scores.view(torch.int16).cpu().numpy().reshape(-1),
        selected=sel.cpu().numpy(), cmean_loc=loc.cpu().numpy(), cmean_rows=rows.cpu().numpy(),
        cmean_bits=cm[rows].view(torch.int16).cpu().numpy(), gpu=np.asarray(torch.cuda.get_device_name(0)))
    print("wrote", out_path)

if __name__ == "__main__":
    main(sys.argv[1])
