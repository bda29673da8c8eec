"""CPU restatement of what each kuiops operator computes.  TEST INFRASTRUCTURE ONLY.

Nothing in the product imports this module: it is the checker used by ``tests/``, by
``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference`` legs of
``bench.py``.  The product path fails loudly when the CUDA library is missing instead of
falling back to anything here.

Where the reference states an operator's meaning itself (the F* specifications of the data
movement kernels, the wrapper conventions) the function below restates that text in numpy loops
or index arithmetic and cites it.  Where the arithmetic lives in the external, un-vendored
Kuiper repository (GEMM, softmax, attention, maps: see the ``open`` lines cited per function)
the restatement follows the published definition of the aten op, which is also what every test
of the reference compares against (tests/test_jit_ops.py:58,93,150,187,227,270,309,394 there).
Parity pin: ``tests/test_oracle_golden.py`` checks every function here against
``tests/golden/ops_golden.npz``, produced by ``tests/golden/gen_op_golden.py`` from PyTorch
eager (the reference tests' own oracle), and the comparator against the reference's
``kuipy._verify_compare`` outputs recorded in ``tests/golden/verify_golden.json``.  For topk,
isin, index, reduce and causal / grouped-query attention the reference has neither kernel nor
test: parity unpinned by the reference; those are pinned by PyTorch semantics only.
"""
import math

import numpy as np

# ---------------------------------------------------------------------------------------------
# data movement: restated from the F* specifications
# ---------------------------------------------------------------------------------------------


def gather(inp: np.ndarray, dim: int, idx: np.ndarray) -> np.ndarray:
    """out[x] = inp[x with x[dim] := idx[x]] for every cell x of idx
    (kuiops/gather/Kuiops.Gather.fsti:25-36, kernel body Kuiops.Gather.fst:93-99)."""
    assert inp.ndim == idx.ndim
    out = np.empty(idx.shape, dtype=inp.dtype)
    for x in np.ndindex(*idx.shape):
        src = list(x)
        j = int(idx[x])
        assert 0 <= j < inp.shape[dim], "index outside the gathered axis"
        src[dim] = j
        out[x] = inp[tuple(src)]
    return out


def gather_fast(inp, dim, idx):
    """Vectorised form of ``gather`` for sizes the loop cannot finish; equal by construction
    (numpy's take_along_axis on the leading idx-shaped block of inp)."""
    sl = tuple(slice(0, idx.shape[d]) if d != dim else slice(None) for d in range(inp.ndim))
    return np.take_along_axis(inp[sl], idx, axis=dim)


def scatter(self_: np.ndarray, dim: int, idx: np.ndarray, src: np.ndarray) -> np.ndarray:
    """out = copy of self; out[i with i[dim] := idx[i]] = src[i] for every cell i of src, visited
    in row-major order (kuiops/scatter/Kuiops.Scatter.fsti:29-52; the kernel needs the index map
    to be injective, :36-41, so the visiting order cannot matter for valid inputs)."""
    assert idx.shape == src.shape and self_.ndim == src.ndim
    out = self_.copy()
    for i in np.ndindex(*src.shape):
        dst = list(i)
        j = int(idx[i])
        assert 0 <= j < self_.shape[dim]
        dst[dim] = j
        out[tuple(dst)] = src[i]
    return out


def scatter_fast(self_, dim, idx, src):
    out = self_.copy()
    sl = tuple(slice(0, src.shape[d]) if d != dim else slice(None) for d in range(out.ndim))
    np.put_along_axis(out[sl], idx, src, axis=dim)
    return out


def cat(tensors, dim: int) -> np.ndarray:
    """Output cell x comes from the input whose range along `dim` contains x[dim], at that
    coordinate minus the range start (binary form: kuiops/cat/Kuiops.Cat.fsti:40-60, fcat in
    Kuiops.Cat.fst:150-186; n-ary is the fold of the binary form)."""
    first = tensors[0]
    shape = list(first.shape)
    shape[dim] = sum(t.shape[dim] for t in tensors)
    out = np.empty(shape, dtype=first.dtype)
    start = 0
    for t in tensors:
        sl = [slice(None)] * out.ndim
        sl[dim] = slice(start, start + t.shape[dim])
        out[tuple(sl)] = t
        start += t.shape[dim]
    return out


def index(self_: np.ndarray, first_dim: int, indices) -> np.ndarray:
    """aten.index.Tensor with index tensors on the adjacent dims starting at first_dim: the
    broadcast index shape replaces those dims; negative indices wrap (signature recorded in the
    reference's KERNELS.md:67; no reference kernel)."""
    bshape = np.broadcast_shapes(*[i.shape for i in indices])
    ib = [np.broadcast_to(i, bshape) for i in indices]
    pre, post = self_.shape[:first_dim], self_.shape[first_dim + len(indices):]
    out = np.empty(tuple(pre) + tuple(bshape) + tuple(post), dtype=self_.dtype)
    for p in np.ndindex(*pre):
        for b in np.ndindex(*bshape):
            coord = []
            for k, i in enumerate(ib):
                v = int(i[b])
                ext = self_.shape[first_dim + k]
                if v < 0:
                    v += ext
                assert 0 <= v < ext
                coord.append(v)
            out[p + b] = self_[p + tuple(coord)]
    return out


def isin(elements: np.ndarray, test_elements: np.ndarray, invert: bool = False) -> np.ndarray:
    """Membership of each element in the test set (KERNELS.md:56-57; no reference kernel)."""
    members = set(int(v) for v in np.asarray(test_elements).reshape(-1))
    flat = np.fromiter((int(v) in members for v in elements.reshape(-1)), dtype=bool, count=elements.size)
    out = flat.reshape(elements.shape)
    return ~out if invert else out


def topk(x: np.ndarray, k: int):
    """Largest-k per row, sorted by value descending and, among equal values, index ascending;
    NaN ranks above +inf (aten.topk signature in KERNELS.md:58; no reference kernel; the tie
    rule is the stable descending sort)."""
    rows = x.reshape(-1, x.shape[-1])
    vals = np.empty((rows.shape[0], k), dtype=x.dtype)
    idxs = np.empty((rows.shape[0], k), dtype=np.int64)
    for r in range(rows.shape[0]):
        row = rows[r]
        key = np.where(np.isnan(row), np.inf, row).astype(np.float64)
        nan_rank = np.isnan(row).astype(np.int64)
        # lexsort: last key is primary.  primary: NaN first, then value descending, then index
        order = np.lexsort((np.arange(row.size), -key, -nan_rank))[:k]
        idxs[r] = order
        vals[r] = row[order]
    return vals.reshape(x.shape[:-1] + (k,)), idxs.reshape(x.shape[:-1] + (k,))


def reduce_fold(op: str, a: np.ndarray):
    """Exact left-to-right fold of the flat tensor under an associative f
    (kuiops/reduce/Kuiops.HReducePoly.Exact.fsti:26-46): all / any over bool, max."""
    flat = a.reshape(-1)
    if op == "all":
        acc = True
        for v in flat:
            acc = acc and bool(v)
        return np.bool_(acc)
    if op == "any":
        acc = False
        for v in flat:
            acc = acc or bool(v)
        return np.bool_(acc)
    if op == "max":
        acc = flat[0]
        for v in flat[1:]:
            if np.isnan(acc):
                break
            if np.isnan(v) or v > acc:
                acc = v
        return acc
    raise ValueError(op)


# ---------------------------------------------------------------------------------------------
# floating point operators (fp64 accumulation, compared within the stated tolerances)
# ---------------------------------------------------------------------------------------------


def mm(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    """C[M,N] = A[M,K] B[K,N] (Klas.GEMM.* opened at kuiops/mm/Kuiops.Mm.Inst.fst.j2:9-15)."""
    return A.astype(np.float64) @ B.astype(np.float64)


def addmm(C: np.ndarray, A: np.ndarray, B: np.ndarray, alpha=1.0, beta=1.0) -> np.ndarray:
    """beta*C + alpha*(A B) with C broadcast over rows when 1-D
    (kuiops/addmm/wrapper_addmm.cu.j2:7-24, Kuiops.Addmm.Inst.fst.j2:11-12)."""
    return beta * C.astype(np.float64) + alpha * (A.astype(np.float64) @ B.astype(np.float64))


def bmm(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    """C[b] = A[b] B[b] (kuiops/bmm/Kuiops.Bmm.fst:13-23)."""
    return np.einsum("bmk,bkn->bmn", A.astype(np.float64), B.astype(np.float64))


def softmax_lastdim(X: np.ndarray) -> np.ndarray:
    """exp(x - max) / sum over the last axis (Klas.RowSoftmax, kuiops/softmax/Kuiops.Softmax.Inst.fst.j2:8-11)."""
    x = X.astype(np.float64)
    z = np.exp(x - x.max(axis=-1, keepdims=True))
    return z / z.sum(axis=-1, keepdims=True)


def cumsum_lastdim(X: np.ndarray) -> np.ndarray:
    """aten.cumsum over the last axis (backlog in the reference, KERNELS.md:68-90; semantics are
    torch.cumsum's).  Floats are accumulated in float64 and rounded once; int64 wraps."""
    if np.issubdtype(X.dtype, np.floating):
        return np.cumsum(X.astype(np.float64), axis=-1).astype(X.dtype)
    return np.cumsum(X, axis=-1, dtype=X.dtype)


def sort_lastdim(X: np.ndarray, descending: bool = False):
    """aten.sort over the last axis, stable (backlog in the reference, KERNELS.md:68-90; semantics
    are torch.sort(stable=True)'s): NaN is the largest value, -0 equals +0, equal values keep their
    original order.  Returns (values, int64 indices)."""
    rows = X.reshape(-1, X.shape[-1])
    vals = np.empty_like(rows)
    idxs = np.empty(rows.shape, dtype=np.int64)
    for r in range(rows.shape[0]):
        row = rows[r]
        nan = np.isnan(row)
        key = np.where(nan, 0.0, row).astype(np.float64)
        pos = np.arange(row.size)
        # lexsort: the last key is the primary one
        order = np.lexsort((pos, -key, ~nan)) if descending else np.lexsort((pos, key, nan))
        idxs[r] = order
        vals[r] = row[order]
    return vals.reshape(X.shape), idxs.reshape(X.shape)


def philox4x32_10(counter, key):
    """Philox4x32 with 10 rounds (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11):
    the published algorithm, restated.  counter: 4 uint32, key: 2 uint32 -> 4 uint32."""
    c = [int(x) & 0xFFFFFFFF for x in counter]
    k = [int(x) & 0xFFFFFFFF for x in key]
    for _ in range(10):
        p0, p1 = 0xD2511F53 * c[0], 0xCD9E8D57 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & 0xFFFFFFFF, p1 & 0xFFFFFFFF, ((p0 >> 32) ^ c[3] ^ k[1]) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        k = [(k[0] + 0x9E3779B9) & 0xFFFFFFFF, (k[1] + 0xBB67AE85) & 0xFFFFFFFF]
    return c


def multinomial(P: np.ndarray, num_samples: int, seed: int, offset: int) -> np.ndarray:
    """Categorical draws with replacement from the rows of a non-negative fp32 matrix: the
    specification the kuiops kernel states for itself (the reference has no multinomial kernel,
    only the backlog entry KERNELS.md:68-90; PyTorch's draws use a private stream and agree in
    distribution only).  u(row, j) = (x0 >> 8) * 2^-24 with x = Philox4x32-10((offset_lo,
    offset_hi, row, j), (seed_lo, seed_hi)); the index inverts the row's running fp32 sum taken in
    a fixed order: 4 elements per lane left to right, a Hillis-Steele scan over the 32 lanes of a
    128-element group, groups left to right inside each of 32 segments, segments left to right;
    at every level the first entry with weight whose running sum exceeds the target, else the last
    entry with weight."""
    f32 = np.float32
    rows = P.reshape(-1, P.shape[-1]).astype(f32)
    m, n = rows.shape
    groups = -(-n // 128)
    gpw = -(-groups // 32)
    out = np.zeros((m, num_samples), dtype=np.int64)
    for r in range(m):
        a = np.zeros(groups * 128, dtype=f32)
        a[:n] = rows[r]
        a[~(a >= 0) | np.isinf(a)] = 0
        a = a.reshape(groups, 32, 4)
        e = np.empty_like(a)                                  # running sums inside a lane
        e[..., 0] = a[..., 0]
        for j in range(1, 4):
            e[..., j] = e[..., j - 1] + a[..., j]
        own = e[..., 3]
        incl = own.copy()                                     # Hillis-Steele over the 32 lanes
        for o in (1, 2, 4, 8, 16):
            up = np.zeros_like(incl)
            up[:, o:] = incl[:, :-o]
            nxt = incl + up
            nxt[:, :o] = incl[:, :o]
            incl = nxt.astype(f32)
        excl = np.zeros_like(incl)
        excl[:, 1:] = incl[:, :-1]
        gsum = incl[:, 31]
        seg_sum = np.zeros(32, dtype=f32)
        for w in range(32):
            s = f32(0)
            for k in range(min(w * gpw, groups), min(w * gpw + gpw, groups)):
                s = f32(s + gsum[k])
            seg_sum[w] = s
        prefix = np.zeros(33, dtype=f32)
        for w in range(32):
            prefix[w + 1] = f32(prefix[w] + seg_sum[w])
        total = prefix[32]
        for j in range(num_samples):
            x = philox4x32_10((offset & 0xFFFFFFFF, (offset >> 32) & 0xFFFFFFFF, r, j), (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
            u = f32(x[0] >> 8) * f32(2.0 ** -24)
            t = f32(u * total)
            w, last = -1, -1
            for q in range(32):
                if seg_sum[q] > 0:
                    last = q
                    if prefix[q + 1] > t:
                        w = q
                        break
            if w < 0:
                w = last
            if w < 0:
                out[r, j] = 0
                continue
            tw = f32(t - prefix[w])
            run, hit, hit_run, lastk, last_run = f32(0), -1, f32(0), -1, f32(0)
            for k in range(min(w * gpw, groups), min(w * gpw + gpw, groups)):
                if gsum[k] > 0:
                    lastk, last_run = k, run
                    if f32(run + gsum[k]) > tw:
                        hit, hit_run = k, run
                        break
                run = f32(run + gsum[k])
            if hit < 0:
                hit, hit_run = lastk, last_run
            has = own[hit] > 0
            over = has & ((hit_run + incl[hit]).astype(f32) > tw)
            lane = int(np.argmax(over)) if over.any() else int(np.nonzero(has)[0][-1])
            choice, lastnz = -1, -1
            for i in range(4):
                if a[hit, lane, i] > 0:
                    lastnz = i
                    if choice < 0 and f32(hit_run + f32(excl[hit, lane] + e[hit, lane, i])) > tw:
                        choice = i
            if choice < 0:
                choice = lastnz
            out[r, j] = hit * 128 + lane * 4 + choice
    return out.reshape(P.shape[:-1] + (num_samples,))


def mean_lastdim(X: np.ndarray) -> np.ndarray:
    """sum_j (x[i,j] / n), keepdim: the division is part of the pre-map
    (kuiops/mean/Kuiops.Mean.fsti:25-32)."""
    x = X.astype(np.float64)
    return (x / x.shape[-1]).sum(axis=-1, keepdims=True)


def sdpa(Q, K, V, bias=None, scale=None, is_causal=False):
    """out = softmax(scale * Q K^T + bias, causal mask bottom-right aligned) V, and
    lse = log sum exp of the masked scores (kuiops/sdpa/Kuiops.Sdpa.fst.1:13-27 for the biased,
    unmasked form and the host-side bias convention at kuipy/kuiops.py:673-677; LSE check at
    tests/test_jit_ops.py:191-193).  Q (n,h,l,e), K (n,h_kv,s,e), V (n,h_kv,s,ev)."""
    Q, K, V = Q.astype(np.float64), K.astype(np.float64), V.astype(np.float64)
    n, h, l, e = Q.shape
    hkv, s = K.shape[1], K.shape[2]
    g = h // hkv
    if scale is None:
        scale = 1.0 / math.sqrt(e)
    Kx, Vx = np.repeat(K, g, axis=1), np.repeat(V, g, axis=1)
    sc = np.einsum("nhle,nhse->nhls", Q, Kx) * scale
    if bias is not None:
        sc = sc + np.broadcast_to(bias.astype(np.float64), sc.shape)
    if is_causal:
        i = np.arange(l)[:, None]
        j = np.arange(s)[None, :]
        sc = np.where(j <= i + (s - l), sc, -np.inf)
    mx = sc.max(axis=-1, keepdims=True)
    mx = np.where(np.isfinite(mx), mx, 0.0)
    p = np.exp(sc - mx)
    den = p.sum(axis=-1, keepdims=True)
    with np.errstate(divide="ignore", invalid="ignore"):
        lse = (np.log(den) + mx)[..., 0]
        out = np.einsum("nhls,nhse->nhle", np.where(den > 0, p / den, 0.0), Vx)
    return out, lse


_MAPS = {
    "silu": lambda x, c0, c1: x / (1.0 + np.exp(-x)),          # x * 1/(1+exp(-x)), Kuiops.Elementwise.fsti
    "neg": lambda x, c0, c1: -x,
    "rsqrt": lambda x, c0, c1: 1.0 / np.sqrt(x),
    "cos": lambda x, c0, c1: np.cos(x),
    "sin": lambda x, c0, c1: np.sin(x),
    "pow": lambda x, c0, c1: np.power(x, c0),
    "square": lambda x, c0, c1: x * x,
    "add": lambda x, c0, c1: x + c1 * c0,
    "mul": lambda x, c0, c1: x * c0,
    "sub": lambda x, c0, c1: x - c1 * c0,
    "div": lambda x, c0, c1: x / c0,
    "gelu": lambda x, c0, c1: 0.5 * x * (1.0 + np.vectorize(math.erf)(x / math.sqrt(2.0))),
}


def map_op(op: str, X: np.ndarray, other=0.0, alpha=1.0) -> np.ndarray:
    """Elementwise map; ``other`` is a scalar or a same-shape array
    (kuiops/elementwise/Kuiops.Elementwise.fsti, lambdas built at kuipy/kuiops.py:292-296)."""
    x = X.astype(np.float64)
    o = other.astype(np.float64) if isinstance(other, np.ndarray) else float(other)
    with np.errstate(all="ignore"):
        return _MAPS[op](x, o, float(alpha))


def compare_scalar(op: str, X: np.ndarray, c: float) -> np.ndarray:
    return {"eq": X == c, "le": X <= c, "lt": X < c}[op]


def where(cond, a, b):
    return np.where(cond.astype(bool), a, b)


def rmsnorm(x, w, eps, residual=None):
    """Llama RMSNorm: h = x (+ residual); y = w * (h * rsqrt(mean(h^2) + eps)) with fp32 statistics."""
    h = x.astype(np.float64) + (residual.astype(np.float64) if residual is not None else 0.0)
    y = h / np.sqrt((h * h).mean(axis=-1, keepdims=True) + eps)
    return y * w.astype(np.float64), h


def rope(x, positions, theta):
    """Rotate-half rotary embedding on x (rows, heads, d) at integer positions (rows,)."""
    rows, heads, d = x.shape
    half = d // 2
    inv = theta ** (-np.arange(half, dtype=np.float64) * 2.0 / d)
    ang = positions.astype(np.float64)[:, None] * inv[None, :]
    cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    x = x.astype(np.float64)
    lo, hi = x[..., :half], x[..., half:]
    return np.concatenate([lo * cos - hi * sin, hi * cos + lo * sin], axis=-1)


# ---------------------------------------------------------------------------------------------
# comparators
# ---------------------------------------------------------------------------------------------


def rel_frobenius(out: np.ndarray, ref: np.ndarray) -> float:
    """||out - ref|| / (||ref|| + 1e-12) over positions where both are finite: the reference's
    verify-mode metric (kuipy/__init__.py:193-224)."""
    o, r = out.astype(np.float64), ref.astype(np.float64)
    ok = np.isfinite(o) & np.isfinite(r)
    if not ok.any():
        return 0.0
    return float(np.linalg.norm((o - r)[ok]) / (np.linalg.norm(r[ok]) + 1e-12))


def max_rel_err(out: np.ndarray, ref: np.ndarray) -> float:
    """max |out - ref| / max |ref|: the "max relative error" of the bf16 GEMM / attention bar."""
    o, r = out.astype(np.float64), ref.astype(np.float64)
    scale = np.abs(r).max()
    return float(np.abs(o - r).max() / (scale if scale > 0 else 1.0))


def sample_topk_topp(logits: np.ndarray, temperature: float, top_k: int, top_p: float, seed: int, offset: int):
    """The specification kuiops_sample_topk_topp_f32 states for itself (the reference has no sampler; its driver
    samples through HuggingFace's temperature / top-k / top-p warpers, infer.py:139-143).  Returns (token ids,
    probability of the token under the filtered distribution, margin): margin[row] is the relative distance of
    the draw's threshold to the nearest running sum, or 0 when ranks that carry weight sit within rounding of
    the nucleus cut; a restatement whose exp differs in the last bit can only disagree where the margin is of
    that order."""
    f32 = np.float32
    rows = logits.reshape(-1, logits.shape[-1]).astype(f32)
    m, n = rows.shape
    k = min(int(top_k), n)
    ids = np.zeros(m, dtype=np.int64)
    prob = np.zeros(m, dtype=f32)
    margin = np.zeros(m, dtype=np.float64)
    inv_t = f32(1.0) / f32(temperature)
    for r in range(m):
        v, idx = topk(rows[r:r + 1], k)
        v, idx = v[0].astype(f32), idx[0]
        with np.errstate(all="ignore"):
            e = np.exp(((v - v[0]) * inv_t).astype(f32)).astype(f32)
        e[0] = 1
        e[~(e >= 0) | np.isinf(e)] = 0
        a = np.zeros(1024, dtype=f32)
        a[:k] = e
        a = a.reshape(8, 32, 4)
        run = np.empty_like(a)
        run[..., 0] = a[..., 0]
        for j in range(1, 4):
            run[..., j] = (run[..., j - 1] + a[..., j]).astype(f32)
        incl = run[..., 3].copy()
        for o in (1, 2, 4, 8, 16):
            nxt = incl.copy()
            nxt[:, o:] = (incl[:, o:] + incl[:, :-o]).astype(f32)
            incl = nxt
        lane_excl = np.zeros_like(incl)
        lane_excl[:, 1:] = incl[:, :-1]
        base = np.zeros(9, dtype=f32)
        for g in range(8):
            base[g + 1] = f32(base[g] + incl[g, 31])
        total = base[8]
        before = (base[:8, None] + lane_excl).astype(f32)                  # [8, 32]
        excl = np.empty_like(a)
        excl[..., 0] = before
        for j in range(1, 4):
            excl[..., j] = (before + run[..., j - 1]).astype(f32)
        incl_r = (before[..., None] + run).astype(f32).reshape(-1)
        excl, a_flat = excl.reshape(-1), a.reshape(-1)
        cut = f32(f32(top_p) * total)
        keep = (np.arange(1024) < k) & ((np.arange(1024) == 0) | (excl < cut))
        R = int(keep.sum())
        K = incl_r[R - 1]
        x = philox4x32_10((offset & 0xFFFFFFFF, (offset >> 32) & 0xFFFFFFFF, r, 0), (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
        u = f32(x[0] >> 8) * f32(2.0 ** -24)
        t = f32(u * K)
        cand = np.nonzero((np.arange(1024) < R) & (a_flat > 0))[0]
        over = cand[incl_r[cand] > t]
        pick = int(over[0]) if len(over) else int(cand[-1])
        ids[r] = idx[pick]
        prob[r] = a_flat[pick] / K if K > 0 else 1.0
        scale = max(float(total), 1e-30)
        # ranks whose membership a last-bit difference could flip only matter by the weight they carry
        near_cut = np.abs(excl[1:k].astype(np.float64) - float(cut)) <= 1e-6 * scale
        d_cut = 1.0 if float(a_flat[1:k][near_cut].astype(np.float64).sum()) <= 4e-6 * scale else 0.0
        d_pick = np.abs(incl_r[:R].astype(np.float64) - float(t)).min() / scale
        margin[r] = min(d_cut, d_pick)
    return ids.reshape(logits.shape[:-1]), prob.reshape(logits.shape[:-1]), margin.reshape(logits.shape[:-1])
