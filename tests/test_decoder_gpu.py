"""The kuiops-only decoder against HuggingFace's Llama in PyTorch eager with the same weights
(tiny config): logits of prefill and of a decode step within the bf16 bar, and equal greedy
tokens where the top-2 margin is not within rounding."""
import numpy as np
import pytest
import torch

from _util import to_np
from oracle import kuiops_oracle as O

pytestmark = pytest.mark.gpu


def _hf_twin(dec):
    from transformers import LlamaConfig, LlamaForCausalLM
    c = dec.cfg
    hf = LlamaConfig(hidden_size=c.d_model, intermediate_size=c.d_ff, num_hidden_layers=c.n_layers,
                     num_attention_heads=c.n_heads, num_key_value_heads=c.n_kv_heads, head_dim=c.head_dim,
                     vocab_size=c.vocab, rms_norm_eps=c.eps, rope_theta=c.rope_theta, max_position_embeddings=512,
                     tie_word_embeddings=False, attention_bias=False, mlp_bias=False)
    m = LlamaForCausalLM(hf).to(torch.bfloat16).cuda().eval()
    hq, hk, hd = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim, c.head_dim
    with torch.no_grad():
        m.model.embed_tokens.weight.copy_(dec.embed)
        m.lm_head.weight.copy_(dec.lm_head)
        m.model.norm.weight.copy_(dec.norm_f)
        for L, H in zip(dec.layers, m.model.layers):
            H.self_attn.q_proj.weight.copy_(L["wqkv"][:hq])
            H.self_attn.k_proj.weight.copy_(L["wqkv"][hq:hq + hk])
            H.self_attn.v_proj.weight.copy_(L["wqkv"][hq + hk:])
            H.self_attn.o_proj.weight.copy_(L["wo"])
            H.mlp.gate_proj.weight.copy_(L["wgu"][0::2])      # rows are interleaved gate, up, gate, up ...
            H.mlp.up_proj.weight.copy_(L["wgu"][1::2])
            H.mlp.down_proj.weight.copy_(L["wd"])
            H.input_layernorm.weight.copy_(L["n1"])
            H.post_attention_layernorm.weight.copy_(L["n2"])
    return m


def test_decoder_matches_hf_llama(cuda):
    from kuillm_b200.decoder import Decoder, DecoderConfig
    dec = Decoder(DecoderConfig.tiny(), device="cuda", seed=0, init_std=0.05)
    twin = _hf_twin(dec)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 1000, (3, 17), generator=g).cuda()
    dec.alloc_cache(3, 40)
    logits = dec.prefill(ids)
    with torch.no_grad():
        ref = twin(ids, use_cache=True)
    rel = O.rel_frobenius(to_np(logits), to_np(ref.logits[:, -1]))
    assert rel < 3e-2, rel
    nxt = ref.logits[:, -1].argmax(-1)
    step = dec.decode_step(nxt)
    with torch.no_grad():
        ref2 = twin(nxt[:, None], past_key_values=ref.past_key_values, use_cache=True)
    rel2 = O.rel_frobenius(to_np(step), to_np(ref2.logits[:, -1]))
    assert rel2 < 3e-2, rel2
    # the element-wise bar, against the same weights evaluated in fp32 by PyTorch eager
    twin32 = twin.float()
    with torch.no_grad():
        r32 = twin32(ids, use_cache=True)
        r32b = twin32(nxt[:, None], past_key_values=r32.past_key_values, use_cache=True)
    for got, want in ((logits, r32.logits[:, -1]), (step, r32b.logits[:, -1])):
        err = O.max_rel_err(to_np(got), to_np(want))
        assert err <= 2e-2, f"max relative error {err:.3e} against the fp32 model"


def test_generate_is_deterministic_and_cache_consistent(cuda):
    from kuillm_b200.decoder import Decoder, DecoderConfig
    dec = Decoder(DecoderConfig.tiny(), device="cuda", seed=1, init_std=0.05)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 1000, (2, 12), generator=g).cuda()
    dec.alloc_cache(2, 32)
    a = dec.generate(ids, 6)
    dec.length = 0
    b = dec.generate(ids, 6)
    assert torch.equal(a, b)
    dec.length = 0
    c = dec.generate(ids, 6, use_graph=True)          # captured decode step, device-side counters
    assert torch.equal(a, c)
    dec.length = 0
    assert torch.equal(a, dec.generate(ids, 6, use_graph=True))   # replaying the same graph again
    # decoding token by token equals prefilling the longer prompt (cache append is consistent)
    dec.length = 0
    full = torch.cat([ids, a[:, :3]], 1)
    l_full = dec.prefill(full)
    dec.length = 0
    dec.prefill(ids)
    for t in range(3):
        l_step = dec.decode_step(a[:, t].contiguous())
    assert O.rel_frobenius(to_np(l_step), to_np(l_full)) < 3e-2


def test_sampled_generation_repeats_and_respects_its_filters(cuda):
    """Sampled decoding through the fused sampler: the same seed repeats the generation, another seed
    does not, top_k = 1 is greedy, and every sampled token lies in the top-k of the logits it was drawn from."""
    from kuipy import _ffi
    from kuillm_b200.decoder import Decoder, DecoderConfig
    dec = Decoder(DecoderConfig.tiny(), device="cuda", seed=1, init_std=0.05)
    ids = torch.randint(0, 1000, (3, 10), generator=torch.Generator().manual_seed(2)).cuda()
    dec.alloc_cache(3, 32)
    samp = dict(temperature=0.9, top_k=20, top_p=0.9, seed=123)
    a = dec.generate(ids, 8, sampling=samp)
    dec.length = 0
    assert torch.equal(a, dec.generate(ids, 8, sampling=samp))
    dec.length = 0
    assert not torch.equal(a, dec.generate(ids, 8, sampling=dict(samp, seed=124)))
    dec.length = 0
    greedy = dec.generate(ids, 8)
    dec.length = 0
    assert torch.equal(greedy, dec.generate(ids, 8, sampling=dict(temperature=0.7, top_k=1, top_p=1.0, seed=5)))
    dec.length = 0
    logits = dec.prefill(ids).float()
    tok = dec.sample_token(logits.to(dec.cfg.dtype), **samp)
    top = logits.topk(20, dim=-1).indices
    assert all(int(tok[r]) in set(top[r].tolist()) for r in range(3))
    assert _ffi.tc_error() == 0


def test_rope_prefill_sized_call_equals_row_chunks(cuda):
    """A prefill-sized call shares each row's sines and cosines over eight heads; small calls compute
    them per head.  Same arithmetic, so the packed rows and both caches must agree bit for bit."""
    from kuipy import _ffi
    hq, hk, d, seqs, per = 16, 8, 128, 10, 1024
    rows = seqs * per
    g = torch.Generator().manual_seed(11)
    qkv = torch.randn(rows, (hq + 2 * hk) * d, generator=g).bfloat16().cuda()
    pos = torch.arange(per).repeat(seqs).cuda()
    kc1, vc1 = (torch.zeros(seqs, hk, per, d, dtype=torch.bfloat16, device="cuda") for _ in range(2))
    kc2, vc2 = torch.zeros_like(kc1), torch.zeros_like(vc1)
    big = qkv.clone()
    _ffi.rope_qkv(big, hq, hk, d, pos, 5e5, kc1, vc1, rows_per_seq=per)
    small = qkv.clone()
    for s0 in range(0, rows, 64):                    # 64 rows at a time: the per-head form
        seq = s0 // per
        _ffi.rope_qkv(small[s0:s0 + 64], hq, hk, d, pos[s0:s0 + 64], 5e5, kc2[seq:seq + 1], vc2[seq:seq + 1], rows_per_seq=per)
    assert torch.equal(big, small) and torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    assert not torch.equal(big, qkv)


@pytest.mark.parametrize("M,hq,hk,K", [(32, 32, 8, 4096), (5, 4, 2, 1024), (128, 8, 8, 2048), (32, 16, 4, 4096), (32, 4, 1, 4096)])
def test_qkv_projection_with_rope_epilogue_equals_two_kernels(cuda, M, hq, hk, K):
    """The fused projection + rotary embedding + cache append must reproduce gemm followed by
    rope_qkv bit for bit: packed rows and both caches."""
    from kuipy import _ffi
    d, cap = 128, 64
    g = torch.Generator().manual_seed(21)
    A = torch.randn(M, K, generator=g).bfloat16().cuda()
    W = (torch.randn((hq + 2 * hk) * d, K, generator=g) / K ** 0.5).bfloat16().cuda()
    pos = torch.randint(0, cap, (M,), generator=g).cuda()
    kc1, vc1 = (torch.zeros(M, hk, cap, d, dtype=torch.bfloat16, device="cuda") for _ in range(2))
    kc2, vc2 = torch.zeros_like(kc1), torch.zeros_like(vc1)
    ref = _ffi.gemm(A, W, trans_b=True)
    plain = ref.clone()
    _ffi.rope_qkv(ref, hq, hk, d, pos, 5e5, kc1, vc1, rows_per_seq=1)
    out = _ffi.gemm_rope_qkv(A, W, hq, hk, d, pos, 5e5, kc2, vc2, rows_per_seq=1)
    assert out is not None, "the shape is meant to take the fused kernel"
    assert torch.equal(out, ref) and torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    assert not torch.equal(out, plain) and _ffi.tc_error() == 0
    # too little K for the split-K placement: the caller is told to run the two kernels
    small = _ffi.gemm_rope_qkv(A[:, :128].contiguous(), W[:, :128].contiguous(), hq, hk, d, pos, 5e5, kc2, vc2, rows_per_seq=1)
    assert small is None



def _fold_config():
    from kuillm_b200.decoder import DecoderConfig
    # head dimension 128 and a model width of 512: the shapes the fused projections (rotary epilogue, folded norms) take
    return DecoderConfig.tiny(d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, d_ff=1024)


def test_folded_norms_match_the_unfused_layer_sequence(cuda):
    """Decode steps with both RMSNorms of a layer folded into the GEMMs around them (five launches per
    layer) against the plain sequence norm -> projection on the same weights, with norm weights that
    are not all ones (folded into the projection columns first): logits within the bf16 bar, the same
    launch count difference the fold promises, and deterministic."""
    from kuipy import _ffi
    from kuillm_b200.decoder import Decoder
    cfg = _fold_config()
    g = torch.Generator().manual_seed(5)
    decs = []
    for fold in (True, False):
        dec = Decoder(cfg, device="cuda", seed=3, init_std=0.05)
        gw = torch.Generator().manual_seed(9)
        for L in dec.layers:
            L["n1"].copy_((1 + 0.2 * torch.randn(cfg.d_model, generator=gw)).to(cfg.dtype))
            L["n2"].copy_((1 + 0.2 * torch.randn(cfg.d_model, generator=gw)).to(cfg.dtype))
        if fold:
            dec.fold_norm_weights()
            assert all(bool((L["n1"] == 1).all()) and bool((L["n2"] == 1).all()) for L in dec.layers)
        else:
            dec.fold_norm = False                          # norm weights stay in the norm kernels, projections unchanged
        dec.alloc_cache(4, 48)
        decs.append(dec)
    ids = torch.randint(0, cfg.vocab, (4, 20), generator=g).cuda()
    # The yardstick for both forms is the same model in fp32 (PyTorch eager, the unfolded weights): the folded form
    # may not be further from it than the plain sequence is (it skips one rounding; its folded weights round
    # differently), and both stay within the bf16 bar of a whole model.
    twin32 = _hf_twin(decs[1]).float()
    lf, lu = decs[0].prefill(ids), decs[1].prefill(ids)
    with torch.no_grad():
        ref = twin32(ids, use_cache=True)
    want = ref.logits[:, -1]
    e_f, e_u = O.max_rel_err(to_np(lf), to_np(want)), O.max_rel_err(to_np(lu), to_np(want))
    assert e_f <= max(2e-2, 1.25 * e_u), (e_f, e_u)
    tok = want.argmax(-1)
    past = ref.past_key_values
    for _ in range(3):
        n0 = _ffi.launch_count()
        a = decs[0].decode_step(tok)
        n_fold = _ffi.launch_count() - n0
        n0 = _ffi.launch_count()
        b = decs[1].decode_step(tok)
        n_plain = _ffi.launch_count() - n0
        with torch.no_grad():
            ref = twin32(tok[:, None], past_key_values=past, use_cache=True)
        want, past = ref.logits[:, -1], ref.past_key_values
        e_f, e_u = O.max_rel_err(to_np(a), to_np(want)), O.max_rel_err(to_np(b), to_np(want))
        assert e_f <= max(2e-2, 1.25 * e_u), (e_f, e_u)
        assert O.rel_frobenius(to_np(a), to_np(want)) < 3e-2
        assert n_plain - n_fold == 2 * cfg.n_layers - 1, (n_plain, n_fold)      # every norm but the first and the final one is gone
        tok = want.argmax(-1)
    # same step twice from the same state: same bits (the tile partials are summed in a fixed order)
    first = decs[0].decode_step(tok)
    decs[0].length -= 1                                    # rewind: the same position again rewrites the same cache row
    assert torch.equal(first, decs[0].decode_step(tok))
    assert _ffi.tc_error() == 0


def test_folded_norm_gemm_pair_against_the_oracle(cuda):
    """kuiops_gemm_residual_ssq + kuiops_gemm_swiglu_rms against the fp64 oracle of
    r' = r + A W^T;  y = swiglu(rmsnorm(r') V^T): the residual as stored, the per-tile sums of squares,
    and the activation within the bf16 bar; ragged row counts and a width that is not a whole tile."""
    from kuipy import _ffi
    g = torch.Generator().manual_seed(11)
    for (M, K, N, F) in ((32, 1024, 512, 768), (5, 512, 320, 256), (128, 2048, 1024, 512)):
        A = torch.randn(M, K, generator=g).bfloat16().cuda()
        W = (torch.randn(N, K, generator=g) / K ** 0.5).bfloat16().cuda()
        r = torch.randn(M, N, generator=g).bfloat16().cuda()
        V = (torch.randn(2 * F, N, generator=g) / N ** 0.5).bfloat16().cuda()       # gate / up rows interleaved
        resid = r.clone()
        tiles = _ffi.ssq_tiles(N)
        ssq = torch.full((tiles, M), float("nan"), device="cuda")
        assert _ffi.gemm_residual_ssq(A, W, resid, ssq)
        want_r = to_np(r).astype(np.float64) + to_np(A).astype(np.float64) @ to_np(W).astype(np.float64).T
        assert O.max_rel_err(to_np(resid), want_r) <= 2e-2
        stored = to_np(resid).astype(np.float64)
        pad = np.zeros((M, tiles * 128))
        pad[:, :N] = stored ** 2
        want_ssq = pad.reshape(M, tiles, 128).sum(-1).T
        np.testing.assert_allclose(to_np(ssq), want_ssq, rtol=1e-5)
        act = _ffi.gemm_swiglu_rms(resid, V, ssq, 1e-5)
        assert act is not None
        h = stored / np.sqrt((stored ** 2).mean(-1, keepdims=True) + 1e-5)
        gu = h @ to_np(V).astype(np.float64).T
        gate, up = gu[:, 0::2], gu[:, 1::2]
        want = gate / (1 + np.exp(-gate)) * up
        assert O.max_rel_err(to_np(act), want) <= 2e-2
        # the same through the plain kernels: norm, then the fused gate|up projection
        plain = _ffi.gemm_swiglu(_ffi.rmsnorm(resid, torch.ones(N, device="cuda", dtype=torch.bfloat16), 1e-5), V)
        assert O.max_rel_err(to_np(act), to_np(plain).astype(np.float64)) <= 2e-2
    assert _ffi.tc_error() == 0
