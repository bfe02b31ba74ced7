"""Generate golden vectors from the reference project's own CUDA kernels (run on a GPU box).

    python tests/golden/make_golden_ref_gpu.py <output.npz>

Needs the cross-check extension built by oracle/build_ref.py (the reference's csrc/topk.cu and
csrc/utils_sglang.cu compiled for sm_100).  For a few seeded cases it records the inputs and what the
reference's `sglang_plan_decode`, `sglang_plan_decode_fa3` and `topk_output` wrote; the committed file
`tests/golden/ref_cuda_kernels.npz` is this script's output and pins the CPU oracle in
tests/test_golden.py without a GPU.
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import build_ref  # noqa: E402
from oracle import vortex_oracle as vo  # noqa: E402

CASES = [
    dict(seq=[9, 18, 40, 64], P=4, H=2, K=1, bos=1, eos=1, mc=2),
    dict(seq=[24, 16, 100], P=4, H=1, K=1, bos=1, eos=2, mc=4),
    dict(seq=[1, 2, 3, 4, 5, 600, 77, 16, 1023, 31], P=16, H=4, K=3, bos=0, eos=1, mc=8),
    dict(seq=[2048, 17, 512, 513, 900], P=16, H=2, K=30, bos=1, eos=1, mc=64),
]


def main(out_path):
    ref = build_ref.load()
    assert ref is not None, "build oracle/_ref first (python oracle/build_ref.py)"
    dev, i32 = "cuda", dict(dtype=torch.int32, device="cuda")
    blob = {"n_cases": np.asarray(len(CASES))}
    for ci, c in enumerate(CASES):
        prob = vo.make_paged_problem(40 + ci, c["seq"], c["H"], 1, 8, c["P"], dtype=torch.float32)
        seq = torch.as_tensor(prob["seq_lens"], **i32)
        r2t = torch.as_tensor(prob["req_to_token"], **i32)
        ridx = torch.as_tensor(prob["req_indices"], dtype=torch.int64, device=dev)
        n = (np.asarray(c["seq"], dtype=np.int64) + c["P"] - 1) // c["P"]
        S, budget = len(c["seq"]) * c["H"], c["K"] + c["bos"] + c["eos"]
        nd, ns = int(n.sum()) * c["H"], int(np.minimum(n, budget).sum()) * c["H"]
        stride = int(n.max()) + 3
        dip, sip = torch.full((S + 1,), -1, **i32), torch.full((S + 1,), -1, **i32)
        din, sin_ = torch.full((nd,), -1, **i32), torch.full((ns,), -1, **i32)
        last = torch.full((S,), -1, **i32)
        w = [torch.full((nd + S,), -1, **i32) for _ in range(3)] + [torch.full((1,), -1, **i32) for _ in range(2)]
        ref.sglang_plan_decode(seq, dip, din, sip, sin_, last, r2t, ridx, *w, c["P"], c["H"], c["K"], c["bos"],
                               c["eos"], c["mc"], 1)
        t = [torch.full((S, stride), -1, **i32), torch.full((S,), -1, **i32),
             torch.full((S, stride), -1, **i32), torch.full((S,), -1, **i32)]
        d2 = [torch.full_like(x, -1) for x in (dip, din, sip, sin_)]
        w2 = [torch.full_like(x, -1) for x in w]
        ref.sglang_plan_decode_fa3(seq, d2[0], d2[1], d2[2], d2[3], *t, r2t, ridx, *w2, c["P"], c["H"], c["K"],
                                   c["bos"], c["eos"], c["mc"], 1)
        g = torch.Generator().manual_seed(100 + ci)
        vals = torch.tensor([-1.0, 0.0, -0.0, 2.5, 0.125, 7.0, -3.5])
        scores = torch.where(torch.rand(nd, generator=g) < 0.5, vals[torch.randint(0, 7, (nd,), generator=g)],
                             torch.randn(nd, generator=g) * 5).bfloat16()
        sel = sin_.clone()
        ref.topk_output(scores.cuda(), dip, sip, din, sel, S, c["K"], c["bos"], c["eos"], int(n.max()))
        torch.cuda.synchronize()
        pre = f"c{ci}_"
        for k, v in c.items():
            blob[pre + "cfg_" + k] = np.asarray(v)
        blob[pre + "req_to_token"] = prob["req_to_token"]
        blob[pre + "req_indices"] = prob["req_indices"]
        nw = int(w[3].item())
        for name, ten in (("dense_kv_indptr", dip), ("dense_kv_indices", din), ("sparse_kv_indptr", sip),
                          ("sparse_kv_indices", sin_), ("kv_last_page_len", last), ("winfo_q_indices", w[0][:nw]),
                          ("winfo_kv_offsets", w[1][:nw]), ("winfo_kv_lens", w[2][:nw]), ("winfo_num_workloads", w[3]),
                          ("winfo_chunk_size", w[4]), ("dense_page_table", t[0]), ("dense_cache_seqlens", t[1]),
                          ("sparse_page_table", t[2]), ("sparse_cache_seqlens", t[3]), ("topk_selected", sel)):
            blob[pre + name] = ten.cpu().numpy()
        blob[pre + "scores_bf16_bits"] = scores.view(torch.int16).numpy()
    np.savez_compressed(out_path, **blob)
    print("wrote", out_path)


if __name__ == "__main__":
    main(sys.argv[1])
