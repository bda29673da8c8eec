"""A Llama-shaped decoder built only from kuiops kernels: the whole-model harness of the library.

The reference runs HuggingFace ``model.generate`` under its dispatch mode (infer.py:135-148) and
so pays one Python dispatch per aten op.  This harness issues the same operator sequence
directly through the C ABI (embedding, RMSNorm, fused QKV GEMM, rotary + KV append, attention,
output GEMM, SwiGLU MLP, final norm, vocabulary GEMM, arg-max), with a static KV cache instead
of the per-token ``cat`` along the sequence axis.  It exists to measure decode + prefill
throughput on the Llama-3-8B shape and to check the operator library end to end; it is not a
model zoo.  Every compute op inside ``prefill`` / ``decode_step`` is a kuiops kernel; PyTorch is
used for buffers, the position / length bookkeeping tensors, copies between static buffers, and
CUDA-graph capture of the decode step.

Parallel forms: batch data-parallel is "one Decoder per rank on its slice of the batch, no
collective"; tensor-parallel splits QKV / gate-up by output columns and O / down by input rows
across ``tp`` ranks with one all-reduce after each row-split GEMM (two per layer): NCCL, or for
decode-sized steps the fused form (``enable_fused_allreduce``) in which the GEMM epilogue stores
its partial product into every rank's memory and the following RMSNorm sums the partials.
"""
from dataclasses import dataclass

import torch

from .kuipy import _ffi


@dataclass
class DecoderConfig:
    n_layers: int = 32
    d_model: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    d_ff: int = 14336
    vocab: int = 128256
    eps: float = 1e-5
    rope_theta: float = 5e5
    dtype: torch.dtype = torch.bfloat16

    @staticmethod
    def llama3_8b():
        return DecoderConfig()

    @staticmethod
    def tiny(**kw):
        base = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, d_ff=512, vocab=1000)
        base.update(kw)
        return DecoderConfig(**base)

    def params(self):
        per_layer = (self.d_model * (self.n_heads + 2 * self.n_kv_heads) * self.head_dim
                     + self.n_heads * self.head_dim * self.d_model + 3 * self.d_model * self.d_ff + 2 * self.d_model)
        return self.n_layers * per_layer + 2 * self.vocab * self.d_model + self.d_model


def shard_out_features(t, n_blocks_total, block, rank, size):
    """Rows [rank, rank + 1) / size of a [out, in] weight, in whole blocks of `block` output
    features (a head's rows for Q / K / V, single rows for gate / up): the column-parallel split."""
    per = n_blocks_total // size
    return t[rank * per * block:(rank + 1) * per * block].contiguous()


def shard_in_features(t, width_per_rank, rank):
    """Columns of a [out, in] weight that multiply this rank's slice of the activations (O and
    down projections): the row-parallel split whose partial products are summed by all-reduce."""
    return t[:, rank * width_per_rank:(rank + 1) * width_per_rank].contiguous()


def dp_slice(batch, rank, size):
    """Sequences [lo, hi) of a global batch that rank `rank` of `size` data-parallel ranks serves."""
    per = (batch + size - 1) // size
    lo = min(rank * per, batch)
    return lo, min(lo + per, batch)


class Decoder:
    """Weights are stored as [out_features, in_features] (the Linear layout), i.e. the
    ``trans_b`` operand form of ``kuiops_gemm``, so no transpose is ever materialised."""

    def __init__(self, cfg: DecoderConfig, device="cuda", seed=0, tp_rank=0, tp_size=1, tp_group=None,
                 init_std=0.02):
        self.cfg, self.device = cfg, torch.device(device)
        self.tp_rank, self.tp_size, self.tp_group = tp_rank, tp_size, tp_group
        assert cfg.n_heads % tp_size == 0 and cfg.n_kv_heads % tp_size == 0 and cfg.d_ff % tp_size == 0
        assert cfg.vocab % tp_size == 0
        self.hq, self.hk = cfg.n_heads // tp_size, cfg.n_kv_heads // tp_size
        self.ff = cfg.d_ff // tp_size
        g = torch.Generator(device=self.device).manual_seed(seed)
        d, hd, dt = cfg.d_model, cfg.head_dim, cfg.dtype

        def w(*shape):
            return (torch.randn(*shape, generator=g, device=self.device, dtype=torch.float32) * init_std).to(dt)

        # every rank draws the full-size tensors from the same seed and keeps its shard, so a
        # tensor-parallel run holds exactly the weights of the single-GPU run
        def shard_rows(t, n_blocks_total, block):
            return shard_out_features(t, n_blocks_total, block, tp_rank, tp_size)

        self.embed = w(cfg.vocab, d)
        self.layers = []
        for _ in range(cfg.n_layers):
            wq, wk, wv = w(cfg.n_heads * hd, d), w(cfg.n_kv_heads * hd, d), w(cfg.n_kv_heads * hd, d)
            wo = w(d, cfg.n_heads * hd)
            wg, wu, wd = w(cfg.d_ff, d), w(cfg.d_ff, d), w(d, cfg.d_ff)
            layer = dict(
                wqkv=torch.cat([shard_rows(wq, cfg.n_heads, hd), shard_rows(wk, cfg.n_kv_heads, hd),
                                shard_rows(wv, cfg.n_kv_heads, hd)], 0).contiguous(),
                wo=shard_in_features(wo, self.hq * hd, tp_rank),
                # gate and up rows interleaved (2j = gate_j, 2j + 1 = up_j): the layout of the fused
                # GEMM + SwiGLU epilogue
                wgu=torch.stack([shard_rows(wg, cfg.d_ff, 1), shard_rows(wu, cfg.d_ff, 1)], 1).reshape(2 * self.ff, d).contiguous(),
                wd=shard_in_features(wd, self.ff, tp_rank),
                n1=torch.ones(d, device=self.device, dtype=dt), n2=torch.ones(d, device=self.device, dtype=dt))
            del wq, wk, wv, wo, wg, wu, wd
            self.layers.append(layer)
        self.norm_f = torch.ones(d, device=self.device, dtype=dt)
        # vocabulary-parallel head: a rank scores vocab / tp consecutive token ids; the greedy step only
        # exchanges each rank's best (value, id) pair per sequence instead of streaming the whole head on every rank
        self.lm_head = w(cfg.vocab, d)
        if tp_size > 1:
            self.lm_head = shard_out_features(self.lm_head, cfg.vocab, 1, tp_rank, tp_size).clone()   # a copy: the slice would keep all rows alive
        self.vocab_lo = tp_rank * (cfg.vocab // tp_size)
        self.k_cache = self.v_cache = None
        self.cap = 0
        self.length = 0
        self.exchange, self.exchange_rows = None, 0
        # decode-sized steps on one GPU run the RMSNorms inside the GEMMs around them (kuiops_gemm_residual_ssq /
        # *_rms): the norm weights live in the columns of the consuming projections
        self.fold_norm = True
        self.fold_norm_weights()
        # tensor-parallel prefills of at least this many rows hide their all-reduces behind compute (two halves
        # of the batch walk the layers in lockstep)
        self.overlap_min_rows = 4096
        # SMs the GEMMs of such a prefill leave to the summing kernel.  Measured at 4 ranks (prefill of 32 x 2048):
        # the overlap only pays when at least as many SMs stay free as the library's kernel has CTAs (32 by
        # default: 294 ms against 308 ms without overlap and 309 - 322 ms with fewer SMs free); at 2 ranks the
        # sums are too short to pay for the SMs
        self.overlap_sm_reserve = 32 if tp_size >= 4 else 0

    def fold_norm_weights(self):
        """Multiply each layer's norm weights into the columns of the projection that consumes the
        normalised rows (n1 into the packed QKV weight, n2 into gate|up) and leave unit norm weights
        behind: the same function, in the form the folded-norm GEMMs need.  Idempotent; to be called
        again after norm weights have been assigned (a checkpoint loader)."""
        with torch.no_grad():
            for L in self.layers:
                for norm, weight in (("n1", "wqkv"), ("n2", "wgu")):
                    g = L[norm]
                    if not bool((g == 1).all()):
                        L[weight] = (L[weight].float() * g.float()[None, :]).to(L[weight].dtype).contiguous()
                        g.fill_(1.0)

    # ---- state ---------------------------------------------------------------------------
    def alloc_cache(self, batch, capacity):
        shape = (self.cfg.n_layers, batch, self.hk, capacity, self.cfg.head_dim)
        self.k_cache = torch.zeros(shape, device=self.device, dtype=self.cfg.dtype)
        self.v_cache = torch.zeros(shape, device=self.device, dtype=self.cfg.dtype)
        self.cap, self.length, self.batch = capacity, 0, batch

    def enable_fused_allreduce(self, max_rows=128):
        """Tensor-parallel groups only: map every rank's receive area (kuillm_b200.peer) so that steps
        of at most `max_rows` rows replace the two NCCL all-reduces of a layer by the push epilogue
        of the row-split GEMMs plus the gathering norm.  Larger steps (prefill) keep NCCL."""
        if self.tp_size <= 1:
            return None
        from .peer import PeerExchange
        self.exchange_rows = min(int(max_rows), 128)
        self.exchange = PeerExchange(self.tp_group, self.device, self.exchange_rows, self.cfg.d_model, self.cfg.dtype)
        return self.exchange

    def _allreduce(self, t):
        if self.tp_size > 1:
            torch.distributed.all_reduce(t, group=self.tp_group)
        return t

    # ---- one forward over `seq` new positions per sequence -------------------------------------
    def _forward(self, ids, positions, seq, last_only=True, kv_lens=None):
        """kv_lens: device int64 [B] key counts; when given the attention reads the whole cache
        capacity bounded by them, so the launch arguments do not depend on the step."""
        cfg = self.cfg
        B = ids.shape[0]
        hd, hq, hk = cfg.head_dim, self.hq, self.hk
        rows = B * seq
        x = _ffi.embedding(self.embed, ids.reshape(-1))                  # [rows, d]
        resid = None
        start, end = self.length, self.length + seq
        # decode-sized steps of a tensor-parallel group: the row-split projections push their partial
        # products straight into every rank's receive area and the norm that follows sums them
        ex = self.exchange if (self.tp_size > 1 and self.exchange is not None and rows <= self.exchange_rows) else None
        # one GPU, decode-sized step: both norms of a layer run inside the GEMMs around them (five launches per
        # layer instead of seven).  ssq_a / ssq_b hold the per-tile sums of squares of the residual rows that the
        # O and down projections leave for the projections that follow them.
        fold = (self.fold_norm and self.tp_size == 1 and rows <= 128 and hd == 128 and cfg.dtype in (torch.bfloat16, torch.float16)
                and cfg.d_model % 8 == 0)
        if fold:
            tiles = _ffi.ssq_tiles(cfg.d_model)
            ssq_a = torch.empty((tiles, rows), dtype=torch.float32, device=self.device)
            ssq_b = torch.empty((tiles, rows), dtype=torch.float32, device=self.device)
        folded_resid = False                    # True once resid holds the running sum and ssq_a its squares
        for li, L in enumerate(self.layers):
            qkv = None
            if folded_resid:
                qkv = _ffi.gemm_rope_qkv_rms(resid, L["wqkv"], hq, hk, hd, positions, cfg.rope_theta, ssq_a, cfg.eps,
                                             self.k_cache[li], self.v_cache[li], rows_per_seq=seq)
                if qkv is None:
                    raise RuntimeError("kuiops: the folded-norm QKV projection refused a shape its producer accepted")
            elif resid is None:
                h = _ffi.rmsnorm(x, L["n1"], cfg.eps)
                resid = x
            elif ex is not None:
                h = _ffi.rmsnorm_gather(ex, rows, L["n1"], cfg.eps, resid)
            else:
                h = _ffi.rmsnorm(x, L["n1"], cfg.eps, residual=resid)      # resid += x ; h = norm(resid)
            # decode-sized steps: projection, rotary embedding and cache append in one launch
            if qkv is None:
                qkv = _ffi.gemm_rope_qkv(h, L["wqkv"], hq, hk, hd, positions, cfg.rope_theta, self.k_cache[li], self.v_cache[li],
                                         rows_per_seq=seq) if rows <= 128 and hd == 128 else None
            if qkv is None:
                qkv = _ffi.gemm(h, L["wqkv"], trans_b=True)              # [rows, (hq + 2 hk) * hd]
                _ffi.rope_qkv(qkv, hq, hk, hd, positions, cfg.rope_theta, self.k_cache[li], self.v_cache[li], rows_per_seq=seq)
            W = qkv.shape[1]
            q4 = qkv.as_strided((B, hq, seq, hd), (seq * W, hd, W, 1))
            attn = torch.empty((rows, hq * hd), device=self.device, dtype=cfg.dtype)
            o4 = attn.as_strided((B, hq, seq, hd), (seq * hq * hd, hd, hq * hd, 1))
            if start == 0:
                # prefill: keys and values of this call are still in the packed projection
                k4 = qkv.as_strided((B, hk, seq, hd), (seq * W, hd, W, 1), hq * hd)
                v4 = qkv.as_strided((B, hk, seq, hd), (seq * W, hd, W, 1), (hq + hk) * hd)
            elif kv_lens is not None:
                k4, v4 = self.k_cache[li], self.v_cache[li]
            else:
                k4 = self.k_cache[li][:, :, :end]
                v4 = self.v_cache[li][:, :, :end]
            _ffi.sdpa(q4, k4, v4, is_causal=True, need_lse=False, out=o4, kv_lens=kv_lens)
            if fold and (folded_resid or _ffi.gemm_residual_ssq(attn, L["wo"], resid, ssq_b)):
                if folded_resid:
                    _ffi.gemm_residual_ssq(attn, L["wo"], resid, ssq_b)          # resid += attn Wo^T, squares -> ssq_b
                act = _ffi.gemm_swiglu_rms(resid, L["wgu"], ssq_b, cfg.eps)      # norm 2 inside the gate|up projection
                if act is None or not _ffi.gemm_residual_ssq(act, L["wd"], resid, ssq_a):
                    raise RuntimeError("kuiops: the folded-norm MLP refused a shape its attention half accepted")
                folded_resid = True
                continue
            fold = False                         # the shape does not suit the folded kernels: plain sequence from here on
            if ex is not None:
                _ffi.gemm_push(attn, L["wo"], trans_b=True, exchange=ex)
                h2 = _ffi.rmsnorm_gather(ex, rows, L["n2"], cfg.eps, resid)
                act = _ffi.gemm_swiglu(h2, L["wgu"])
                _ffi.gemm_push(act, L["wd"], trans_b=True, exchange=ex)   # summed by the next norm
                continue
            o = self._allreduce(_ffi.gemm(attn, L["wo"], trans_b=True))
            h2 = _ffi.rmsnorm(o, L["n2"], cfg.eps, residual=resid)
            act = _ffi.gemm_swiglu(h2, L["wgu"])
            x = self._allreduce(_ffi.gemm(act, L["wd"], trans_b=True))
        self.length = end
        last = torch.arange(seq - 1, rows, seq, device=self.device) if (last_only and seq > 1) else None
        if ex is not None:
            # the last projection's partials are still in the exchange: sum and normalise every row,
            # then keep the rows that feed the vocabulary GEMM
            hf = _ffi.rmsnorm_gather(ex, rows, self.norm_f, cfg.eps, resid)
            if last is not None:
                hf = _ffi.index(hf, 0, [last])
        elif folded_resid:
            if last is not None:
                resid = _ffi.index(resid, 0, [last])                     # only the last position of each sequence feeds the vocabulary GEMM
            hf = _ffi.rmsnorm(resid, self.norm_f, cfg.eps)               # resid already holds the last projection's sum
        else:
            if last is not None:
                # only the last position of each sequence feeds the vocabulary GEMM
                x = _ffi.index(x, 0, [last])
                resid = _ffi.index(resid, 0, [last])
            hf = _ffi.rmsnorm(x, self.norm_f, cfg.eps, residual=resid)
        return _ffi.gemm(hf, self.lm_head, trans_b=True)                 # [B or rows, vocab / tp]: this rank's token ids

    def _full_logits(self, local):
        """[rows, vocab] logits on every rank from the ranks' vocabulary shards (tensor parallel only)."""
        if self.tp_size == 1:
            return local
        rows, per = local.shape
        parts = torch.empty((self.tp_size, rows, per), dtype=local.dtype, device=self.device)
        torch.distributed.all_gather_into_tensor(parts, local.contiguous(), group=self.tp_group)
        return parts.permute(1, 0, 2).reshape(rows, self.tp_size * per)

    def next_token(self, local):
        """Greedy token of every row from this rank's shard of the logits.  Tensor parallel: each rank
        takes the arg-max of its shard, the ranks exchange (value, token id) pairs - two small
        all-gathers instead of the whole vocabulary - and every rank picks the largest value, the
        lowest rank (= lowest token id) winning ties, exactly as the arg-max over the full row does."""
        idx = _ffi.argmax_lastdim(local)
        if self.tp_size == 1:
            return idx
        B = idx.shape[0]
        val = _ffi.gather(local, 1, idx.reshape(B, 1)).reshape(B)
        if self.vocab_lo:
            _ffi.add_i64_(idx, self.vocab_lo)
        vals = torch.empty((self.tp_size, B), dtype=val.dtype, device=self.device)
        idxs = torch.empty((self.tp_size, B), dtype=torch.int64, device=self.device)
        torch.distributed.all_gather_into_tensor(vals, val, group=self.tp_group)
        torch.distributed.all_gather_into_tensor(idxs, idx, group=self.tp_group)
        best = _ffi.argmax_lastdim(vals.t().contiguous())                # [B]: the rank that holds the row's maximum
        return _ffi.gather(idxs.t().contiguous(), 1, best.reshape(B, 1)).reshape(B)

    def sample_token(self, local, temperature=0.7, top_k=50, top_p=0.8, seed=0, offset=0):
        """One sampled token per row: temperature, top-k and top-p filters and the draw in one fused call
        (kuiops_sample_topk_topp_f32) over the full fp32 logits.  Every rank of a tensor-parallel group
        draws from the same stream position and so picks the same token."""
        logits = _ffi.cast(self._full_logits(local), torch.float32)
        return _ffi.sample_topk_topp(logits, temperature, top_k, top_p, seed=seed, offset=offset)

    def _forward_tp_overlap(self, ids, positions, seq):
        """Prefill of a tensor-parallel group with the sums over ranks hidden behind compute.  The batch
        is cut into two halves of sequences that walk the layers in lockstep: while one half's partial
        products are being summed (NCCL, asynchronously, on the library's own stream) the other half
        computes its attention or MLP block.  Same kernels and the same two all-reduces per layer and
        half as the plain form; only the order of launches differs."""
        # the GEMMs are persistent grids over every SM: without free SMs the summing kernel would only run
        # between them, and nothing would overlap
        old_reserve = _ffi.gemm_set_sm_reserve(self.overlap_sm_reserve)
        try:
            return self._forward_tp_overlap_body(ids, positions, seq)
        finally:
            _ffi.gemm_set_sm_reserve(old_reserve)

    def _forward_tp_overlap_body(self, ids, positions, seq):
        import torch.distributed as dist
        cfg = self.cfg
        B = ids.shape[0]
        hd, hq, hk = cfg.head_dim, self.hq, self.hk
        hb = B // 2
        pos2 = positions.view(B, seq)
        halves = []
        for h in range(2):
            sl = slice(h * hb, (h + 1) * hb)
            halves.append(dict(sl=sl, rows=hb * seq, pos=pos2[sl].reshape(-1).contiguous(), resid=None, work=None,
                               x=_ffi.embedding(self.embed, ids[sl].reshape(-1))))
        for li, L in enumerate(self.layers):
            for st in halves:                                   # attention block; ends with an asynchronous sum over ranks
                if st["work"] is not None:
                    st["work"].wait()                            # the previous layer's down projection, summed
                if st["resid"] is None:
                    h = _ffi.rmsnorm(st["x"], L["n1"], cfg.eps)
                    st["resid"] = st["x"]
                else:
                    h = _ffi.rmsnorm(st["x"], L["n1"], cfg.eps, residual=st["resid"])
                qkv = _ffi.gemm(h, L["wqkv"], trans_b=True)
                _ffi.rope_qkv(qkv, hq, hk, hd, st["pos"], cfg.rope_theta, self.k_cache[li][st["sl"]], self.v_cache[li][st["sl"]],
                              rows_per_seq=seq)
                W = qkv.shape[1]
                q4 = qkv.as_strided((hb, hq, seq, hd), (seq * W, hd, W, 1))
                k4 = qkv.as_strided((hb, hk, seq, hd), (seq * W, hd, W, 1), hq * hd)
                v4 = qkv.as_strided((hb, hk, seq, hd), (seq * W, hd, W, 1), (hq + hk) * hd)
                attn = torch.empty((st["rows"], hq * hd), device=self.device, dtype=cfg.dtype)
                o4 = attn.as_strided((hb, hq, seq, hd), (seq * hq * hd, hd, hq * hd, 1))
                _ffi.sdpa(q4, k4, v4, is_causal=True, need_lse=False, out=o4)
                st["o"] = _ffi.gemm(attn, L["wo"], trans_b=True)
                st["work"] = dist.all_reduce(st["o"], group=self.tp_group, async_op=True)
            for st in halves:                                   # MLP block; ends the same way
                st["work"].wait()
                h2 = _ffi.rmsnorm(st["o"], L["n2"], cfg.eps, residual=st["resid"])
                act = _ffi.gemm_swiglu(h2, L["wgu"])
                st["x"] = _ffi.gemm(act, L["wd"], trans_b=True)
                st["work"] = dist.all_reduce(st["x"], group=self.tp_group, async_op=True)
        outs = []
        for st in halves:
            st["work"].wait()
            last = torch.arange(seq - 1, st["rows"], seq, device=self.device)
            x, resid = _ffi.index(st["x"], 0, [last]), _ffi.index(st["resid"], 0, [last])
            outs.append(_ffi.gemm(_ffi.rmsnorm(x, self.norm_f, cfg.eps, residual=resid), self.lm_head, trans_b=True))
        self.length += seq
        return torch.cat(outs, 0)

    def prefill(self, ids, local_logits=False):
        B, S = ids.shape
        assert self.k_cache is not None and S <= self.cap and self.length == 0
        positions = torch.arange(S, device=self.device).repeat(B)
        if self.tp_size > 1 and B % 2 == 0 and B * S >= self.overlap_min_rows and B * S > self.exchange_rows:
            out = self._forward_tp_overlap(ids, positions, S)
        else:
            out = self._forward(ids, positions, S)
        return out if local_logits else self._full_logits(out)

    def decode_step(self, ids, local_logits=False):
        B = ids.shape[0]
        positions = torch.full((B,), self.length, device=self.device, dtype=torch.int64)
        out = self._forward(ids.reshape(B, 1), positions, 1)
        return out if local_logits else self._full_logits(out)

    # ---- captured decode step -----------------------------------------------------------------
    def _graph_step(self):
        """One self-advancing decode step on static buffers: token in -> logits -> arg-max ->
        token out, then the token is fed back and the device-side counters move on."""
        B = self._tok.shape[0]
        logits = self._forward(self._tok.reshape(B, 1), self._pos, 1, kv_lens=self._kvlen)
        self.length -= 1                        # the host counter is advanced by the caller per replay
        nxt = self.next_token(logits)
        self._tok_out.copy_(nxt)
        self._tok.copy_(nxt)
        _ffi.add_i64_(self._pos, 1)
        _ffi.add_i64_(self._kvlen, 1)

    def capture_decode(self, batch):
        """Capture the decode step in a CUDA graph (launch-bound otherwise: ~290 kernels per token)."""
        dev = self.device
        self._tok = torch.zeros(batch, dtype=torch.int64, device=dev)
        self._tok_out = torch.zeros(batch, dtype=torch.int64, device=dev)
        self._pos = torch.zeros(batch, dtype=torch.int64, device=dev)
        self._kvlen = torch.ones(batch, dtype=torch.int64, device=dev)
        saved = self.length
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):                  # warm-up on the capture stream: scratch buffers get allocated here
                # it runs at the last cache slot, which is rewritten before any real step reads it,
                # so a cache that already holds a prompt stays intact
                self.length = self.cap - 1
                self._pos.fill_(self.cap - 1)
                self._kvlen.fill_(self.cap)
                self._graph_step()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self._graph = torch.cuda.CUDAGraph()
        self.length = 1
        n0 = _ffi.launch_count()
        with torch.cuda.graph(self._graph, stream=side):
            self._graph_step()
        self.graph_launches = _ffi.launch_count() - n0      # kuiops kernels replayed per captured step
        self.length = saved
        return self._graph

    def decode_graph(self, first_tok, steps, out=None):
        """Run `steps` captured decode steps starting from token `first_tok` at the current length."""
        B = first_tok.shape[0]
        if out is None:
            out = torch.empty((B, steps), dtype=torch.int64, device=self.device)
        self._tok.copy_(first_tok)
        self._pos.fill_(self.length)
        self._kvlen.fill_(self.length + 1)
        for t in range(steps):
            self._graph.replay()
            out[:, t].copy_(self._tok_out)
            self.length += 1
        return out

    def generate(self, ids, new_tokens, use_graph=False, sampling=None):
        """Greedy decoding, or sampled decoding when `sampling` is a dict of sample_token's arguments
        (temperature, top_k, top_p, seed; token t of the generation draws at stream offset 4 t);
        returns the [B, new_tokens] generated ids."""
        if sampling is not None:
            kw = dict(sampling)
            out = [self.sample_token(self.prefill(ids, local_logits=True), offset=0, **kw)]
            for t in range(1, new_tokens):
                out.append(self.sample_token(self.decode_step(out[-1], local_logits=True), offset=4 * t, **kw))
            return torch.stack(out, 1)
        tok = self.next_token(self.prefill(ids, local_logits=True))
        if use_graph and new_tokens > 1:
            if getattr(self, "_graph", None) is None or self._tok.shape[0] != ids.shape[0]:
                self.capture_decode(ids.shape[0])
            rest = self.decode_graph(tok, new_tokens - 1)
            return torch.cat([tok[:, None], rest], 1)
        out = [tok]
        for _ in range(new_tokens - 1):
            tok = self.next_token(self.decode_step(tok, local_logits=True))
            out.append(tok)
        return torch.stack(out, 1)
