"""Generate ``ops_golden.npz``: seeded inputs and the outputs PyTorch eager gives for them.

PyTorch eager is what every test of the reference compares its kernels with
(tests/test_jit_ops.py there), so these vectors pin the CPU oracle to the same yardstick.
bf16 tensors are stored as fp32 (exactly representable).  Run: python tests/golden/gen_op_golden.py
"""
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

HERE = Path(__file__).resolve().parent


def main():
    g = torch.Generator().manual_seed(0)
    rn = lambda *s: torch.randn(*s, generator=g)
    out = {}
    # GEMM family (shapes of the reference tests plus ragged ones)
    A, B, Cm = rn(17, 9), rn(9, 13), rn(17, 13)
    out.update(mm_A=A, mm_B=B, mm_out=A @ B)
    out.update(addmm_C=Cm, addmm_out=torch.addmm(Cm, A, B, alpha=0.5, beta=2.0))
    bias = rn(13)
    out.update(addmm_bias=bias, addmm_bias_out=torch.addmm(bias, A, B))
    A3, B3 = rn(5, 17, 9), rn(5, 9, 13)
    out.update(bmm_A=A3, bmm_B=B3, bmm_out=torch.bmm(A3, B3))
    # softmax / mean
    X = rn(8, 5, 33) * 3
    out.update(softmax_X=X, softmax_out=torch.softmax(X, -1), mean_out=X.mean(-1, keepdim=True))
    # attention: biased (the reference's form), and causal grouped-query
    Q, K, V, bia = rn(2, 3, 8, 16), rn(2, 3, 10, 16), rn(2, 3, 10, 12), rn(2, 3, 8, 10)
    o = F.scaled_dot_product_attention(Q, K, V, attn_mask=bia, scale=0.3)
    lse = torch.logsumexp(Q @ K.transpose(-1, -2) * 0.3 + bia, -1)
    out.update(sdpa_Q=Q, sdpa_K=K, sdpa_V=V, sdpa_bias=bia, sdpa_out=o, sdpa_lse=lse)
    Qg, Kg, Vg = rn(2, 4, 6, 16), rn(2, 2, 9, 16), rn(2, 2, 9, 16)
    mask = torch.ones(6, 9, dtype=torch.bool).tril(diagonal=9 - 6)
    og = F.scaled_dot_product_attention(Qg, Kg.repeat_interleave(2, 1), Vg.repeat_interleave(2, 1), attn_mask=mask)
    out.update(gqa_Q=Qg, gqa_K=Kg, gqa_V=Vg, gqa_out=og)
    # data movement
    inp = rn(4, 3, 6)
    idx = torch.randint(0, 6, (4, 3, 5), generator=g)
    out.update(gather_inp=inp, gather_idx=idx, gather_out=torch.gather(inp, 2, idx))
    idx0 = torch.randint(0, 4, (3, 3, 6), generator=g)
    out.update(gather0_idx=idx0, gather0_out=torch.gather(inp, 0, idx0))
    perm = torch.stack([torch.randperm(6, generator=g) for _ in range(12)]).reshape(4, 3, 6)
    src = rn(4, 3, 6)
    out.update(scatter_idx=perm, scatter_src=src, scatter_out=inp.clone().scatter_(2, perm, src))
    a, b = rn(4, 3, 6), rn(4, 5, 6)
    out.update(cat_a=a, cat_b=b, cat_out=torch.cat([a, b], 1))
    m2 = torch.rand(9, 9, generator=g) > 0.5
    i0 = torch.randint(-9, 9, (2, 1, 5, 1), generator=g)
    i1 = torch.randint(0, 9, (1, 1, 1, 5), generator=g)
    out.update(index_self=m2, index_i0=i0, index_i1=i1, index_out=m2[i0, i1])
    ids = torch.randint(0, 1000, (6, 40), generator=g)
    pos = torch.randint(0, 40, (7,), generator=g)
    out.update(index2_self=ids, index2_pos=pos, index2_out=ids[:, pos])
    stop = torch.randint(0, 1000, (50,), generator=g)
    out.update(isin_test=stop, isin_out=torch.isin(ids, stop))
    # topk with many ties: stable descending sort defines the tie order
    tk = torch.randint(0, 8, (5, 64), generator=g).float()
    sv, si = torch.sort(tk, dim=-1, descending=True, stable=True)
    out.update(topk_X=tk, topk_vals=sv[:, :10], topk_idx=si[:, :10])
    tk2 = rn(3, 500)
    v2, i2 = torch.topk(tk2, 50)
    out.update(topk2_X=tk2, topk2_vals=v2, topk2_idx=i2)
    # maps
    E = rn(3, 5, 7)
    E2 = rn(3, 5, 7).abs() + 0.5
    out.update(map_X=E, map_Y=E2, map_silu=F.silu(E), map_rsqrt=torch.rsqrt(E2), map_pow=E2 ** 1.5,
               map_add_alpha=torch.add(E, E2, alpha=2.0), map_div=E / E2, map_sub_scalar=E - 1.5,
               map_le=(E <= 0.0), map_gelu=F.gelu(E),
               map_where=torch.where(E > 0, E, E2))
    # whole-tensor folds
    bl = torch.rand(1000, generator=g) > 0.001
    iv = torch.randint(-10**12, 10**12, (777,), generator=g)
    out.update(fold_bool=bl, fold_all=bl.all(), fold_any=bl.any(), fold_i64=iv, fold_max=iv.max())
    np.savez_compressed(HERE / "ops_golden.npz", **{k: (v.numpy() if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in out.items()})
    print(f"{len(out)} arrays written")


if __name__ == "__main__":
    main()
